// Host layer behind include/hb200.h: context, resident weights and
// activations, the dtype -> kernel table, the recorded batch, and the
// host-buffer entry points that mirror the reference's call shapes.
//
// Mirrors, at whole-matrix granularity:
//   ThreadPool::par_dot_rows / par_dot_rows_batched / par_quantize  hearth-llm/src/pool.rs:467-618
//   LlamaModel::matmul / matmul_batch dtype table                  hearth-llm/src/model/matmul.rs:152-343, :606-672
//   GpuCompute residency and begin_batch/end_batch                 hearth-compute/src/lib.rs:104, :206-251
// Errors never cross the boundary as exceptions: every entry point is
// wrapped in a catch-all and returns a status code.
#include <cuda.h>

#include <algorithm>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <vector>

#include "../../include/hb200.h"
#include "common.cuh"

using namespace hb200;

// ------------------------------------------------------------------ errors --

namespace hb200 {
static thread_local std::string g_last_error;
void set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
}
int bound_device();
}  // namespace hb200

#define HB_GUARD_BEGIN try {
// First statement of every entry point that takes a weight, an activation or a batch: the object's device slot
// becomes the current one.
#define HB_USE(obj)                                   \
    do {                                              \
        if (obj) {                                    \
            const int _rc = use_slot((obj)->slot);    \
            if (_rc) return _rc;                      \
        }                                             \
    } while (0)
#define HB_GUARD_END                                          \
    }                                                         \
    catch (const std::bad_alloc&) {                           \
        set_error("host allocation failed");                  \
        return HB200_ERR_TOO_LARGE;                           \
    }                                                         \
    catch (...) {                                             \
        set_error("unexpected C++ exception");                \
        return HB200_ERR_CUDA;                                \
    }

// ----------------------------------------------------------------- objects --

#include "objects.h"

struct BatchEntry {
    hb200_weight_t w;
    hb200_act_t a;
    size_t seq_len;
    float* out;
    size_t ld_out;
};
struct BatchGroup {  // one launch
    int kind, m;
    FlatRec* recs_dev = nullptr;   // per CTA a run of segments (whole panels, or a part of a panel cut between two CTAs), each with its op
    int* seg_begin_dev = nullptr;  // grid + 1
    float* carry_dev = nullptr;    // running sums handed from the CTA before a cut to the CTA after it
    int* cflags_dev = nullptr;     // per carry slot: arrivals of writer warps so far (eight per launch)
    unsigned epoch = 0;            // launches of this group so far (wraps; the kernels compare differences)
    int grid = 0;
    int n_items = 0;  // panels
    int n_segs = 0;   // segments of the plan
};
struct hb200_batch {
    std::vector<BatchEntry> entries;
    std::vector<BatchGroup> groups;
    std::vector<BatchEntry> kquant;  // K-quant ops launch on their own
    std::vector<BatchEntry> tensor;       // ops for the prefill tensor-core kernel (see dot_path)
    std::vector<BatchEntry> tensor_rows;  // ops for the few-token tensor-core kernel
    struct TcGroup { int kind = 0; bool rows = false; TcMat* mats_dev = nullptr; int* chunks_dev = nullptr; int n_tiles = 0, grid = 0; };
    std::vector<TcGroup> tc_groups;  // one persistent launch per weight kind
    struct KqGroup { int kind = 0, mt = 0; KqMat* mats_dev = nullptr; int* chunks_dev = nullptr; int n_items = 0, grid = 0; };
    std::vector<KqGroup> kq_groups;  // K-quant ops: one launch per (kind, tokens per pass)
    // host-input path: distinct activations in order of first use, a staging buffer for their f32 rows
    std::vector<hb200_act_t> acts;
    std::vector<size_t> act_seq;       // rows used of each
    std::vector<size_t> act_offset;    // float offset of each inside x_stage
    size_t input_floats = 0;
    float* x_stage = nullptr;
    QuantDesc* qdescs_dev = nullptr;
    int q_max_chunks = 0, q_max_seq = 0, n_qacts = 0;
    bool has_kquant_inputs = false;
    int slot = 0;           // device slot the batch (and every weight and activation in it) lives in
    PeerTable peers = {};   // n > 1: outputs go to every rank's buffer
    size_t peer_area_floats = 0;  // two output areas this far apart, written in turn (0: one area)
    int epoch = 0;
    bool sealed = false;
    // Pipelined host path: the ops in the order they were added, and sub-batches over contiguous runs of them, each
    // with the activations it is the first to use and the span of output floats it writes.
    std::vector<std::pair<int, size_t>> order;  // (0: entries, 1: kquant; index in that list)
    bool is_child = false;
    struct Segment {
        hb200_batch* ops = nullptr;
        size_t act_lo = 0, act_hi = 0;   // activations first used here: indices into acts
        int q_lo = 0, q_hi = 0;          // their descriptors in qdescs_dev
        const float* out_lo = nullptr;   // device span [out_lo, out_hi) written by these ops
        const float* out_hi = nullptr;
    };
    std::vector<Segment> segments;
    std::vector<cudaEvent_t> seg_in, seg_done;
};

namespace {

struct Context {
    bool ready = false;
    int device = -1;
    int sm_count = 0;
    cudaStream_t stream = nullptr;  // used by the host-buffer calls
    // scratch for the host-buffer calls, grown on demand
    uint8_t* d_in = nullptr;
    size_t d_in_bytes = 0;
    uint8_t* d_out = nullptr;
    size_t d_out_bytes = 0;
    hb200_act_t act = nullptr;                // the one in use, an entry of `acts`
    std::map<size_t, hb200_act_t> acts;       // by width
    int* d_status = nullptr;  // device word set by kernels whose bounded waits expire
    cudaEvent_t ev_inputs = nullptr;  // orders a step's compute behind the stream that produced its device-resident inputs
    void* d_argmax = nullptr;  // ticket + partial results of the argmax kernel, then one result word
    uint8_t* d_terms = nullptr;  // per-block terms of the two-phase f32-activation matvec
    size_t d_terms_bytes = 0;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;  // the pipelined host path: uploads and readbacks beside the compute stream
};
// One context per device slot.  hb200_init binds slot 0; hb200_init_multi binds slots 0 .. n-1 (normally to devices
// 0 .. n-1) so that ONE host thread - the shape of the reference's dispatcher, hearth-llm/src/pool.rs:398-425 - can
// drive every GPU of the box.  Every object remembers the slot it was created in, and every call on an object makes
// that slot (and its CUDA device) current first; calls without an object act on the current slot.
Context g_ctx_pool[MAX_PEERS];
int g_n_slots = 0;   // slots bound (0 before any init)
int g_cur = 0;       // the current slot
#define g_ctx (g_ctx_pool[g_cur])

// Makes `slot` and its device current.  Objects of a context that has been shut down are refused.
int use_slot(int slot) {
    if (slot < 0 || slot >= MAX_PEERS || !g_ctx_pool[slot].ready) {
        set_error("the object belongs to device slot %d, which is not initialised", slot);
        return HB200_ERR_NOT_INITIALIZED;
    }
    if (slot != g_cur || g_n_slots > 1) {
        g_cur = slot;
        HB_CUDA(cudaSetDevice(g_ctx_pool[slot].device));
    }
    return 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;

// Tensor maps over an activation's int8 plane: [max_seq rows][ld_q bytes], 128-byte swizzle, boxes of 128 rows x 128
// bytes (prefill kernel) and 32 rows x 128 bytes (few-token kernel).
static int encode_one_qmap(hb200_act* a, unsigned char* host, void** dev, cuuint32_t box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)a->ld_q, (cuuint64_t)a->max_seq};
    const cuuint64_t strides[1] = {(cuuint64_t)a->ld_q};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode_tiled(reinterpret_cast<CUtensorMap*>(host), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->q, dims, strides, box,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return HB200_ERR_CUDA; }
    if (!*dev) HB_CUDA(cudaMalloc(dev, 128));
    HB_CUDA(cudaMemcpy(*dev, host, 128, cudaMemcpyHostToDevice));
    return 0;
}
int encode_qmap(hb200_act* a) {
    if (!g_encode_tiled) { a->has_qmap = false; return 0; }
    static_assert(sizeof(CUtensorMap) <= sizeof(a->qmap), "tensor map storage");
    int rc;
    if ((rc = encode_one_qmap(a, a->qmap, &a->qmap_dev, 128))) return rc;
    if ((rc = encode_one_qmap(a, a->qmap32, &a->qmap32_dev, GEMM_TCR_TOK_TILE))) return rc;
    a->has_qmap = true;
    return 0;
}

int kind_of(int dtype) {
    switch (dtype) {
        case HB200_Q1_0: case HB200_Q1_0_G128: case HB200_Q1_0_G128_LEGACY: return KIND_Q1;
        case HB200_Q2_0: case HB200_PQ2_0: return KIND_Q2;
        case HB200_PTQ1_0: return KIND_Q2;  // re-coded to 2-bit codes at upload
        case HB200_Q8_0: return KIND_Q8;
        case HB200_Q4_K: return KIND_Q4K;
        case HB200_Q6_K: return KIND_Q6K;
        default: return KIND_NONE;
    }
}

int need_ctx() {
    if (!g_ctx.ready) {
        set_error("hb200_init has not succeeded in this process");
        return HB200_ERR_NOT_INITIALIZED;
    }
    return 0;
}

int grow(uint8_t** p, size_t* have, size_t want) {
    if (*have >= want) return 0;
    if (*p) HB_CUDA(cudaFree(*p));
    *p = nullptr;
    *have = 0;
    size_t sz = want + want / 4 + 4096;
    HB_CUDA(cudaMalloc(p, sz));
    *have = sz;
    return 0;
}

void fill_op(DotOp& op, const hb200_weight* w, const hb200_act* a, size_t tok0, float* out, size_t ld_out, int32_t* iout) {
    op.bits = w->bits;
    op.scales = w->scales;
    op.aq = a->q + tok0 * (size_t)a->ld_q;
    op.ad = a->d + tok0 * (size_t)a->ld_b;
    op.asum = a->sums + tok0 * (size_t)a->ld_b;
    op.out = out ? out + tok0 * ld_out : nullptr;
    op.iout = iout;
    op.n_rows = (int)w->n_rows;
    op.nb = w->nb;
    op.n_sub = w->n_sub;
    op.ld_out = (int)ld_out;
    op.ld_q = a->ld_q;
    op.ld_b = a->ld_b;
}

int check_pair(const hb200_weight* w, const hb200_act* a, size_t seq_len, size_t ld_out) {
    if (!w || !a) { set_error("null weight or activation handle"); return HB200_ERR_NULL; }
    if (a->slot != w->slot) { set_error("the weight lives in device slot %d, the activation in slot %d", w->slot, a->slot); return HB200_ERR_BAD_SHAPE; }
    if (a->n_cols != w->n_cols) {
        set_error("dim mismatch: weight has %zu columns, activation %zu", w->n_cols, a->n_cols);
        return HB200_ERR_BAD_SHAPE;
    }
    if (seq_len > a->max_seq) { set_error("seq_len %zu exceeds the activation's capacity %zu", seq_len, a->max_seq); return HB200_ERR_BAD_SHAPE; }
    if (ld_out < w->n_rows) { set_error("ld_out %zu is smaller than n_rows %zu", ld_out, w->n_rows); return HB200_ERR_BAD_SHAPE; }
    return 0;
}

}  // namespace

namespace {

// Which kernel a Q8_0-activation op runs on: the streaming dp4a kernel (even passes of at most four tokens), the few-token
// tensor-core kernel (rows on the MMA's M side) or the prefill tensor-core kernel (tokens on the M side).
enum DotPath { PATH_DP4A = 0, PATH_TC_ROWS = 1, PATH_TC = 2 };
DotPath dot_path(const hb200_weight* w, const hb200_act* a, size_t seq_len) {
    if (!a->has_qmap || w->nb <= 0 || (w->kind != KIND_Q1 && w->kind != KIND_Q2)) return PATH_DP4A;
    if (gemm_tcr_wanted(w->kind, seq_len)) return PATH_TC_ROWS;
    if (gemm_tc_wanted(w->kind, seq_len)) return PATH_TC;
    return PATH_DP4A;
}

// Tokens of the next streaming-kernel pass when `left` remain: the fewest passes of at most GEMV_MAX_M tokens, as even
// as possible (5 = 3 + 2, 9 = 3 + 3 + 3): a pass costs a fixed part plus a part per token, and the fixed part of a
// one-token pass is the dearest.  Every token's result is independent of how the passes are cut.
size_t dp4a_pass_tokens(size_t left) {
    const size_t passes = (left + GEMV_MAX_M - 1) / GEMV_MAX_M;
    return (left + passes - 1) / passes;
}

int dot_rows_launch(const hb200_weight* w, const hb200_act* a, size_t seq_len, float* out, size_t ld_out, cudaStream_t st) {
    if (w->kind == KIND_Q4K || w->kind == KIND_Q6K) {
        set_error("K-quant weights take f32 activations; use hb200_matmul_f32[_dev]");
        return HB200_ERR_UNSUPPORTED;
    }
    // Prefill-sized token counts of a 1-/2-bit weight go to the tensor cores; fewer run as passes of the streaming dp4a kernel.
    const DotPath path = dot_path(w, a, seq_len);
    if (path == PATH_TC_ROWS)
        return launch_gemm_tcr(w->kind, a->qmap32_dev, w->bits, w->scales, a->d, a->ld_b, (int)w->n_rows, w->nb, (int)seq_len, out,
                               (int)ld_out, g_ctx.sm_count, g_ctx.d_status, st);
    if (path == PATH_TC)
        return launch_gemm_tc(w->kind, a->qmap_dev, w->bits, w->scales, a->d, a->ld_b, (int)w->n_rows, w->nb, (int)seq_len, out,
                              (int)ld_out, g_ctx.sm_count, g_ctx.d_status, st);
    for (size_t tok0 = 0, m = 0; tok0 < seq_len; tok0 += m) {
        m = dp4a_pass_tokens(seq_len - tok0);
        DotOp op;
        fill_op(op, w, a, tok0, out, ld_out, nullptr);
        int grid = g_ctx.sm_count * gemv_dp4a_ctas_per_sm(w->kind, (int)m);
        if (grid > w->n_panels) grid = w->n_panels;
        const int rc = launch_gemv_dp4a(w->kind, (int)m, false, nullptr, grid, w->n_panels, &op, st);
        if (rc) return rc;
    }
    return 0;
}

// After a synchronising call: turn a device-side wait expiry into an error code, and clear it.
int check_device_status() {
    int h = 0;
    HB_CUDA(cudaMemcpy(&h, g_ctx.d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (h != 0) {
        cudaMemset(g_ctx.d_status, 0, sizeof(int));
        // 1..9: mbarrier waits of the tensor-core kernels; 40: bulk copy of x in the eight-token K-quant kernel; 50: carry
        // of a panel cut between two CTAs (decode matvec); 100 + r: peer rank r's flag
        set_error("a bounded wait inside a kernel expired (code %d); results of that call are invalid", h);
        return HB200_ERR_TIMEOUT;
    }
#ifdef HB200_BOUNDS
    // the bounds-checked build: indices outside their buffers were counted (and skipped) by the kernels
    int (*const fetch[])(int*, int*) = {bounds_fetch_dp4a, bounds_fetch_kquant, bounds_fetch_quantize, bounds_fetch_producers};
    const char* const unit[] = {"gemv_dp4a.cu", "kquant.cu", "quantize.cu", "producers.cu"};
    for (int i = 0; i < 4; i++) {
        int site = 0, count = 0;
        const int rc = fetch[i](&site, &count);
        if (rc) return rc;
        if (count) {
            set_error("bounds-checked build: %d accesses of %s fell outside their buffers and were skipped, the first at site %d", count, unit[i], site);
            return HB200_ERR_CUDA;
        }
    }
#endif
    return 0;
}


// The activation the host-buffer calls stage their input in: one per width, kept for the life of the context (a
// model alternates between a handful of widths - d_model, the FFN width - so nothing is allocated or freed after the
// first call of each), replaced only when a call brings more tokens than it holds.
int ensure_ctx_act(size_t seq_len, size_t n_cols) {
    if (g_ctx.act && g_ctx.act->n_cols == n_cols && g_ctx.act->max_seq >= seq_len) return 0;
    g_ctx.act = nullptr;
    auto it = g_ctx.acts.find(n_cols);
    if (it != g_ctx.acts.end() && it->second->max_seq >= seq_len) { g_ctx.act = it->second; return 0; }
    if (it != g_ctx.acts.end()) { hb200_act_free(it->second); g_ctx.acts.erase(it); }
    if (g_ctx.acts.size() >= 16) {  // a caller cycling through many widths: keep the cache bounded
        for (auto& kv : g_ctx.acts) hb200_act_free(kv.second);
        g_ctx.acts.clear();
    }
    hb200_act_t fresh = nullptr;
    const int rc = hb200_act_create(seq_len, n_cols, &fresh);
    if (rc) return rc;
    g_ctx.acts[n_cols] = fresh;
    g_ctx.act = fresh;
    return 0;
}

}  // namespace

// --------------------------------------------------------------- lifecycle --

namespace hb200 {
int bound_device() { return g_ctx.ready ? g_ctx.device : -1; }
int use_slot_of(int slot) { return use_slot(slot); }
}  // namespace hb200

// Binds slot `slot` to CUDA device `device`: stream, status word, scratch, per-device kernel attributes.
static int init_slot(int slot, int device) {
    Context& c = g_ctx_pool[slot];
    if (c.ready) {
        if (c.device == device) return HB200_OK;
        set_error("slot %d is already bound to device %d", slot, c.device);
        return HB200_ERR_BAD_SHAPE;
    }
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0) {
        set_error("no CUDA device: %s", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
        return HB200_ERR_NO_DEVICE;
    }
    if (device < 0 || device >= n) { set_error("device %d out of range (0..%d)", device, n - 1); return HB200_ERR_NO_DEVICE; }
    cudaDeviceProp prop;
    HB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library contains sm_100a code only", device, prop.major, prop.minor);
        return HB200_ERR_NO_DEVICE;
    }
    HB_CUDA(cudaSetDevice(device));
    const int before = g_cur;
    g_cur = slot;
    HB_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    c.device = device;
    c.sm_count = prop.multiProcessorCount;
    int rc;
    if ((rc = gemv_dp4a_prepare())) return rc;
    if ((rc = kquant_prepare())) return rc;
    if ((rc = gemm_tc_prepare())) return rc;
    if ((rc = gemm_tcr_prepare())) return rc;
    if ((rc = producers_prepare())) return rc;
    if (!g_encode_tiled) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e2 = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e2 != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
            set_error("cuTensorMapEncodeTiled is not available from this driver");
            return HB200_ERR_CUDA;
        }
        g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    }
    HB_CUDA(cudaMalloc(&c.d_status, sizeof(int)));
    HB_CUDA(cudaMemset(c.d_status, 0, sizeof(int)));
    HB_CUDA(cudaMalloc(&c.d_argmax, argmax_scratch_bytes() + 256));
    HB_CUDA(cudaMemset(c.d_argmax, 0, argmax_scratch_bytes() + 256));
    c.ready = true;
    if (slot + 1 > g_n_slots) g_n_slots = slot + 1;
    g_cur = before;
    return HB200_OK;
}

extern "C" int hb200_init(int device) {
    HB_GUARD_BEGIN
    const int rc = init_slot(0, device);
    if (rc) return rc;
    return use_slot(g_n_slots > 1 ? g_cur : 0);
    HB_GUARD_END
}

extern "C" int hb200_init_slots(const int* devices, int n_slots) {
    HB_GUARD_BEGIN
    if (!devices) { set_error("null device list"); return HB200_ERR_NULL; }
    if (n_slots < 1 || n_slots > MAX_PEERS) { set_error("%d device slots: between 1 and %d", n_slots, MAX_PEERS); return HB200_ERR_BAD_SHAPE; }
    int rc;
    for (int i = 0; i < n_slots; i++)
        if ((rc = init_slot(i, devices[i]))) return rc;
    // every device may store into every other device's memory (plain peer stores of the row-sharded batches)
    for (int i = 0; i < n_slots; i++)
        for (int j = 0; j < n_slots; j++) {
            if (devices[i] == devices[j]) continue;
            int can = 0;
            HB_CUDA(cudaDeviceCanAccessPeer(&can, devices[i], devices[j]));
            if (!can) { set_error("device %d cannot access device %d", devices[i], devices[j]); return HB200_ERR_UNSUPPORTED; }
            HB_CUDA(cudaSetDevice(devices[i]));
            cudaError_t e = cudaDeviceEnablePeerAccess(devices[j], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (e != cudaSuccess) { set_error("cudaDeviceEnablePeerAccess(%d -> %d) failed: %s", devices[i], devices[j], cudaGetErrorString(e)); return HB200_ERR_CUDA; }
        }
    return use_slot(0);
    HB_GUARD_END
}

extern "C" int hb200_init_multi(int n_devices) {
    int devices[MAX_PEERS];
    for (int i = 0; i < MAX_PEERS; i++) devices[i] = i;
    if (n_devices < 1 || n_devices > MAX_PEERS) { set_error("%d devices: between 1 and %d", n_devices, MAX_PEERS); return HB200_ERR_BAD_SHAPE; }
    return hb200_init_slots(devices, n_devices);
}

extern "C" int hb200_set_slot(int slot) {
    HB_GUARD_BEGIN
    return use_slot(slot);
    HB_GUARD_END
}

extern "C" int hb200_slot_count(void) { return g_n_slots; }

extern "C" int hb200_shutdown(void) {
    HB_GUARD_BEGIN
    for (int slot = 0; slot < MAX_PEERS; slot++) {
        Context& c = g_ctx_pool[slot];
        if (!c.ready) continue;
        cudaSetDevice(c.device);
        cudaDeviceSynchronize();
        for (auto& kv : c.acts) hb200_act_free(kv.second);
        c.acts.clear();
        c.act = nullptr;
        if (c.d_in) cudaFree(c.d_in);
        if (c.d_out) cudaFree(c.d_out);
        if (c.d_status) cudaFree(c.d_status);
        if (c.ev_inputs) cudaEventDestroy(c.ev_inputs);
        if (c.d_argmax) cudaFree(c.d_argmax);
        if (c.d_terms) cudaFree(c.d_terms);
        if (c.stream) cudaStreamDestroy(c.stream);
        if (c.copy_in) cudaStreamDestroy(c.copy_in);
        if (c.copy_out) cudaStreamDestroy(c.copy_out);
        c = Context();
    }
    g_n_slots = 0;
    g_cur = 0;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" const char* hb200_last_error(void) { return g_last_error.c_str(); }
extern "C" int hb200_sm_count(void) { return g_ctx.ready ? g_ctx.sm_count : 0; }

extern "C" int hb200_measure_i8_peak(double* tops) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (!tops) { set_error("null output"); return HB200_ERR_NULL; }
    if ((rc = measure_i8_peak(g_ctx.sm_count, g_ctx.d_status, g_ctx.stream, tops))) return rc;
    return check_device_status();
    HB_GUARD_END
}

// ---------------------------------------------------------------- geometry --

extern "C" size_t hb200_block_size(int dtype) {
    switch (kind_of(dtype)) {
        case KIND_Q1: case KIND_Q2: return 128;
        case KIND_Q8: return 32;
        case KIND_Q4K: case KIND_Q6K: return 256;
        default: return 0;
    }
}
extern "C" size_t hb200_block_bytes(int dtype) {
    if (dtype == HB200_PTQ1_0) return 28;
    switch (kind_of(dtype)) {
        case KIND_Q1: return 18;
        case KIND_Q2: case KIND_Q8: return 34;
        case KIND_Q4K: return 144;
        case KIND_Q6K: return 210;
        default: return 0;
    }
}
extern "C" size_t hb200_byte_size(int dtype, size_t n_cols) {
    const size_t bs = hb200_block_size(dtype);
    if (!bs) return 0;
    return ((n_cols + bs - 1) / bs) * hb200_block_bytes(dtype);
}

extern "C" const char* hb200_selected_kernel(int dtype, size_t seq_len) {
    const int kind = kind_of(dtype);
    if (seq_len == 0) return "none";
    switch (kind) {
        case KIND_Q1: return gemm_tcr_wanted(kind, seq_len) ? "gemm_tcgen05_i8_rows_q1_0" : (gemm_tc_wanted(kind, seq_len) ? "gemm_tcgen05_i8_q1_0" : "gemv_dp4a_q1_0");
        case KIND_Q2: return gemm_tcr_wanted(kind, seq_len) ? "gemm_tcgen05_i8_rows_q2_0" : (gemm_tc_wanted(kind, seq_len) ? "gemm_tcgen05_i8_q2_0" : "gemv_dp4a_q2_0");
        case KIND_Q8: return "gemv_dp4a_q8_0";
        case KIND_Q4K: return "kquant_gemv_q4_k_f32";
        case KIND_Q6K: return "kquant_gemv_q6_k_f32";
        default: return "none";
    }
}

// hearth_quant::dispatch_report (hearth-quant/src/lib.rs:449-473): for every distinct format of the list, the runs
// of token counts served by one kernel, found by asking hb200_selected_kernel (the last run is open-ended).
namespace {
const char* dtype_name(int dtype) {  // GgmlDType::name (hearth-gguf/src/ggml.rs:178-224)
    switch (dtype) {
        case HB200_Q8_0: return "Q8_0";
        case HB200_Q4_K: return "Q4_K";
        case HB200_Q6_K: return "Q6_K";
        case HB200_Q1_0: return "Q1_0";
        case HB200_Q2_0: return "Q2_0";
        case HB200_Q1_0_G128: case HB200_Q1_0_G128_LEGACY: return "Q1_0_G128";
        case HB200_PQ2_0: return "PQ2_0";
        case HB200_PTQ1_0: return "PTQ1_0";
        default: return nullptr;
    }
}
struct KernelRun { size_t lo, hi; const char* kernel; };  // hi == 0: open-ended
std::vector<KernelRun> kernel_runs(int dtype) {
    std::vector<KernelRun> runs;
    const size_t probe_to = (size_t)GEMM_TCR_MAX_TOKENS + 2;  // beyond the last threshold nothing changes
    for (size_t m = 1; m <= probe_to; m++) {
        const char* k = hb200_selected_kernel(dtype, m);
        if (runs.empty() || strcmp(runs.back().kernel, k) != 0) runs.push_back({m, m, k});
        else runs.back().hi = m;
    }
    runs.back().hi = 0;
    return runs;
}
std::vector<int> distinct_formats(const int* dtypes, size_t n) {
    std::vector<int> out;
    for (size_t i = 0; i < n; i++) {
        const char* nm = dtype_name(dtypes[i]);
        if (!nm || kind_of(dtypes[i]) == KIND_NONE) continue;
        bool seen = false;
        for (int d : out) seen = seen || strcmp(dtype_name(d), nm) == 0;
        if (!seen) out.push_back(dtypes[i]);
    }
    return out;
}
std::string lower(const char* s) {
    std::string r(s);
    for (char& c : r) if (c >= 'A' && c <= 'Z') c = (char)(c - 'A' + 'a');
    return r;
}
int emit_text(const std::string& text, char* buf, size_t cap, size_t* needed) {
    if (needed) *needed = text.size();
    if (!buf || cap < text.size() + 1) {
        set_error("text of %zu bytes does not fit a buffer of %zu", text.size() + 1, cap);
        return HB200_ERR_TOO_LARGE;
    }
    memcpy(buf, text.c_str(), text.size() + 1);
    return HB200_OK;
}
std::string device_name() {
    if (!g_ctx.ready) return "none";
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, g_ctx.device) != cudaSuccess) return "unknown";
    return prop.name;
}
std::string range_text(const KernelRun& r) {
    char t[48];
    if (r.hi == 0) snprintf(t, sizeof(t), "%zu+", r.lo);
    else if (r.hi == r.lo) snprintf(t, sizeof(t), "%zu", r.lo);
    else snprintf(t, sizeof(t), "%zu-%zu", r.lo, r.hi);
    return t;
}
}  // namespace

extern "C" int hb200_dispatch_report(const int* dtypes, size_t n_dtypes, char* json, size_t cap, size_t* needed) {
    HB_GUARD_BEGIN
    if (!dtypes && n_dtypes) { set_error("null dtype list"); return HB200_ERR_NULL; }
    std::string js = "{\"device\": \"" + device_name() + "\", \"sm\": \"" + (g_ctx.ready ? "10.0" : "none") + "\", \"sm_count\": " +
                     std::to_string(g_ctx.ready ? g_ctx.sm_count : 0) + ", \"kernels\": {";
    bool first = true;
    for (int d : distinct_formats(dtypes, n_dtypes)) {
        js += std::string(first ? "" : ", ") + "\"" + lower(dtype_name(d)) + "\": [";
        first = false;
        const std::vector<KernelRun> runs = kernel_runs(d);
        for (size_t i = 0; i < runs.size(); i++)
            js += std::string(i ? ", " : "") + "{\"tokens\": \"" + range_text(runs[i]) + "\", \"kernel\": \"" + runs[i].kernel + "\"}";
        js += "]";
    }
    js += "}}";
    return emit_text(js, json, cap, needed);
    HB_GUARD_END
}

extern "C" int hb200_dispatch_banner(const int* dtypes, size_t n_dtypes, char* text, size_t cap, size_t* needed) {
    HB_GUARD_BEGIN
    if (!dtypes && n_dtypes) { set_error("null dtype list"); return HB200_ERR_NULL; }
    std::string b = "[kernel]";
    for (int d : distinct_formats(dtypes, n_dtypes)) {
        b += std::string(" ") + dtype_name(d) + "=";
        const std::vector<KernelRun> runs = kernel_runs(d);
        for (size_t i = 0; i < runs.size(); i++) b += std::string(i ? "," : "") + runs[i].kernel + "(" + range_text(runs[i]) + ")";
    }
    b += " . " + device_name() + " . " + (g_ctx.ready ? "sm_100 . " + std::to_string(g_ctx.sm_count) + " SMs" : "no device bound");
    return emit_text(b, text, cap, needed);
    HB_GUARD_END
}

// ----------------------------------------------------------------- weights --

static int weight_build(int dtype, size_t n_rows, size_t n_cols, const uint8_t* src, bool src_on_device, cudaStream_t st,
                        hb200_weight_t* out) {
    const int kind = kind_of(dtype);
    hb200_weight* w = new hb200_weight();
    w->slot = g_cur;
    w->dtype = dtype;
    w->kind = kind;
    w->n_rows = n_rows;
    w->n_cols = n_cols;
    w->row_bytes = hb200_byte_size(dtype, n_cols);
    const size_t bytes = n_rows * w->row_bytes;
    int rc = 0;
    uint8_t* d_raw = nullptr;
    uint8_t* d_recode = nullptr;
    bool own_raw = false;
    auto fail = [&](int code) {
        if (own_raw && d_raw) cudaFree(d_raw);
        if (d_recode) cudaFree(d_recode);
        if (w->bits) cudaFree(w->bits);
        if (w->scales) cudaFree(w->scales);
        if (w->kq) cudaFree(w->kq);
        if (w->d16) cudaFree(w->d16);
        delete w;
        return code;
    };
    if (bytes > 0) {
        if (src_on_device) {
            d_raw = const_cast<uint8_t*>(src);
        } else {
            cudaError_t e = cudaMalloc(&d_raw, bytes);
            if (e != cudaSuccess) { set_error("cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e)); return fail(HB200_ERR_CUDA); }
            own_raw = true;
            e = cudaMemcpyAsync(d_raw, src, bytes, src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, st);
            if (e != cudaSuccess) { set_error("weight copy failed: %s", cudaGetErrorString(e)); return fail(HB200_ERR_CUDA); }
        }
    }
    if (kind == KIND_Q4K || kind == KIND_Q6K) {
        w->nb = (int)(n_cols / 256);  // whole 256-column blocks only, as the reference's loops do
        w->n_panels = (int)((n_rows + 31) / 32);
        const size_t pieces = (size_t)w->n_panels * w->nb * kquant_pieces_per_block(kind) * 32;
        const size_t d_count = (kind == KIND_Q6K) ? (size_t)w->n_panels * w->nb * 32 : 0;
        if (pieces > 0) {
            cudaError_t e = cudaMalloc(&w->kq, pieces * sizeof(uint4));
            if (e == cudaSuccess && d_count) e = cudaMalloc(&w->d16, d_count * sizeof(unsigned short));
            if (e != cudaSuccess) { set_error("cudaMalloc for %zu weight bytes failed: %s", pieces * 16 + d_count * 2, cudaGetErrorString(e)); return fail(HB200_ERR_CUDA); }
            rc = launch_kquant_repack(kind, d_raw, w->row_bytes, (int)n_rows, w->nb, w->n_panels, w->kq, w->d16, st);
            if (rc) return fail(rc);
        }
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) { set_error("weight re-tiling failed: %s", cudaGetErrorString(e)); return fail(HB200_ERR_CUDA); }
        if (own_raw) { cudaFree(d_raw); own_raw = false; }
        w->resident_bytes = pieces * 16 + d_count * 2;
    } else {
        const int rpg = rows_per_group(kind);
        const size_t rp = 32 * (size_t)rpg;
        w->n_panels = (int)((n_rows + rp - 1) / rp);
        if (kind == KIND_Q8) {
            w->nb = (int)((n_cols + 127) / 128);
            w->n_sub = (int)(n_cols / 32);
        } else {
            w->nb = (int)(n_cols / 128);  // a tail shorter than a block is dropped, as in the reference
            w->n_sub = w->nb * 4;
        }
        const size_t tiles = (size_t)w->n_panels * w->nb * 32;
        const size_t bits_bytes = tiles * 128;
        const size_t scale_bytes = tiles * (size_t)scales_per_tile(kind) * 2;
        if (tiles > 0) {
            cudaError_t e = cudaMalloc(&w->bits, bits_bytes);
            if (e == cudaSuccess) e = cudaMalloc(&w->scales, scale_bytes);
            if (e != cudaSuccess) { set_error("cudaMalloc for %zu weight bytes failed: %s", bits_bytes + scale_bytes, cudaGetErrorString(e)); return fail(HB200_ERR_CUDA); }
            const int eff_cols = (kind == KIND_Q8) ? (int)n_cols : w->nb * 128;
            const uint8_t* rows = d_raw;
            size_t rows_stride = w->row_bytes;
            if (dtype == HB200_PTQ1_0) {  // base-3 digits -> 2-bit codes, then the Q2_0 panels
                rows_stride = (size_t)w->nb * 34;
                e = cudaMalloc(&d_recode, n_rows * rows_stride);
                if (e != cudaSuccess) { set_error("cudaMalloc(%zu) failed: %s", n_rows * rows_stride, cudaGetErrorString(e)); return fail(HB200_ERR_CUDA); }
                rc = launch_ptq1_to_q2(d_raw, w->row_bytes, (int)n_rows, w->nb, d_recode, rows_stride, st);
                if (rc) return fail(rc);
                rows = d_recode;
            }
            rc = launch_repack(kind, rows, rows_stride, (int)n_rows, eff_cols, w->nb, w->n_panels, w->bits, w->scales, st);
            if (rc) return fail(rc);
        }
        cudaError_t e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) { set_error("weight re-tiling failed: %s", cudaGetErrorString(e)); return fail(HB200_ERR_CUDA); }
        if (own_raw) { cudaFree(d_raw); own_raw = false; }
        if (d_recode) { cudaFree(d_recode); d_recode = nullptr; }
        w->resident_bytes = bits_bytes + scale_bytes;
    }
    *out = w;
    return HB200_OK;
}

static int weight_check(int dtype, size_t n_rows, size_t n_cols, const void* packed, size_t bytes, hb200_weight_t* out) {
    int rc = need_ctx();
    if (rc) return rc;
    if (!out) { set_error("null output handle"); return HB200_ERR_NULL; }
    if (kind_of(dtype) == KIND_NONE) { set_error("GGML type id %d is not on this path", dtype); return HB200_ERR_BAD_DTYPE; }
    if (n_cols == 0) { set_error("Matmul dim mismatch: weight has 0 columns"); return HB200_ERR_BAD_SHAPE; }
    const size_t want = n_rows * hb200_byte_size(dtype, n_cols);
    if (bytes != want) { set_error("weight byte count %zu != n_rows * byte_size = %zu", bytes, want); return HB200_ERR_BAD_SHAPE; }
    if (!packed && bytes) { set_error("null weight bytes"); return HB200_ERR_NULL; }
    if (n_rows > (1u << 30) || n_cols > (1u << 24)) { set_error("weight shape %zu x %zu too large", n_rows, n_cols); return HB200_ERR_TOO_LARGE; }
    return 0;
}

extern "C" int hb200_weight_upload(int dtype, size_t n_rows, size_t n_cols, const uint8_t* packed, size_t bytes,
                                   hb200_weight_t* out) {
    HB_GUARD_BEGIN
    int rc = weight_check(dtype, n_rows, n_cols, packed, bytes, out);
    if (rc) return rc;
    return weight_build(dtype, n_rows, n_cols, packed, false, g_ctx.stream, out);
    HB_GUARD_END
}

extern "C" int hb200_weight_upload_dev(int dtype, size_t n_rows, size_t n_cols, const uint8_t* packed_dev, size_t bytes,
                                       void* stream, hb200_weight_t* out) {
    HB_GUARD_BEGIN
    int rc = weight_check(dtype, n_rows, n_cols, packed_dev, bytes, out);
    if (rc) return rc;
    return weight_build(dtype, n_rows, n_cols, packed_dev, true, (cudaStream_t)stream, out);
    HB_GUARD_END
}

extern "C" int hb200_weight_upload_rows(int dtype, size_t n_rows, size_t n_cols, const uint8_t* packed, size_t bytes,
                                        size_t row_begin, size_t row_end, hb200_weight_t* out) {
    HB_GUARD_BEGIN
    int rc = weight_check(dtype, n_rows, n_cols, packed, bytes, out);
    if (rc) return rc;
    if (row_begin > row_end || row_end > n_rows) { set_error("row range [%zu, %zu) outside 0..%zu", row_begin, row_end, n_rows); return HB200_ERR_BAD_SHAPE; }
    const size_t rb = hb200_byte_size(dtype, n_cols);
    return weight_build(dtype, row_end - row_begin, n_cols, packed + row_begin * rb, false, g_ctx.stream, out);
    HB_GUARD_END
}

extern "C" int hb200_weight_free(hb200_weight_t w) {
    HB_GUARD_BEGIN
    HB_USE(w);
    if (!w) return HB200_OK;
    if (w->bits) cudaFree(w->bits);
    if (w->scales) cudaFree(w->scales);
    if (w->kq) cudaFree(w->kq);
    if (w->d16) cudaFree(w->d16);
    delete w;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_weight_info(hb200_weight_t w, int* dtype, size_t* n_rows, size_t* n_cols, size_t* resident_bytes) {
    if (!w) { set_error("null weight handle"); return HB200_ERR_NULL; }
    if (dtype) *dtype = w->dtype;
    if (n_rows) *n_rows = w->n_rows;
    if (n_cols) *n_cols = w->n_cols;
    if (resident_bytes) *resident_bytes = w->resident_bytes;
    return HB200_OK;
}

// ------------------------------------------------------------- activations --

extern "C" int hb200_act_create(size_t max_seq_len, size_t n_cols, hb200_act_t* out) {
    HB_GUARD_BEGIN
    if (!out) { set_error("null output handle"); return HB200_ERR_NULL; }
    if (n_cols == 0 || max_seq_len == 0) { set_error("activation of %zu x %zu", max_seq_len, n_cols); return HB200_ERR_BAD_SHAPE; }
    // the per-token kernels put the token index in gridDim.y
    if (n_cols > (1u << 24) || max_seq_len > HB200_MAX_SEQ_LEN) {
        set_error("activation %zu x %zu too large (at most %d tokens of %u columns)", max_seq_len, n_cols, HB200_MAX_SEQ_LEN, 1u << 24);
        return HB200_ERR_TOO_LARGE;
    }
    int rc = need_ctx();
    if (rc) return rc;
    hb200_act* a = new hb200_act();
    a->slot = g_cur;
    a->max_seq = max_seq_len;
    a->n_cols = n_cols;
    a->ld_q = (int)((n_cols + ACT_PAD - 1) / ACT_PAD * ACT_PAD);
    a->ld_b = a->ld_q / 32;
    cudaError_t e = cudaMalloc(&a->x, max_seq_len * n_cols * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&a->q, max_seq_len * (size_t)a->ld_q);
    if (e == cudaSuccess) e = cudaMalloc(&a->d, max_seq_len * (size_t)a->ld_b * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&a->sums, max_seq_len * (size_t)a->ld_b * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(a->q, 0, max_seq_len * (size_t)a->ld_q);
    if (e == cudaSuccess) e = cudaMemset(a->d, 0, max_seq_len * (size_t)a->ld_b * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(a->sums, 0, max_seq_len * (size_t)a->ld_b * sizeof(float));
    if (e != cudaSuccess) {
        set_error("activation allocation failed: %s", cudaGetErrorString(e));
        hb200_act_free(a);
        return HB200_ERR_CUDA;
    }
    if ((rc = encode_qmap(a))) { hb200_act_free(a); return rc; }
    *out = a;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_act_free(hb200_act_t a) {
    HB_GUARD_BEGIN
    HB_USE(a);
    if (!a) return HB200_OK;
    if (a->x) cudaFree(a->x);
    if (a->q) cudaFree(a->q);
    if (a->d) cudaFree(a->d);
    if (a->sums) cudaFree(a->sums);
    if (a->qmap_dev) cudaFree(a->qmap_dev);
    if (a->qmap32_dev) cudaFree(a->qmap32_dev);
    delete a;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_act_f32_ptr(hb200_act_t a, float** dev_ptr) {
    if (!a || !dev_ptr) { set_error("null handle"); return HB200_ERR_NULL; }
    *dev_ptr = a->x;
    return HB200_OK;
}

extern "C" int hb200_act_q8_planes(hb200_act_t a, int8_t** q, float** d, float** sums, size_t* ld_q, size_t* ld_b) {
    if (!a) { set_error("null handle"); return HB200_ERR_NULL; }
    if (q) *q = a->q;
    if (d) *d = a->d;
    if (sums) *sums = a->sums;
    if (ld_q) *ld_q = (size_t)a->ld_q;
    if (ld_b) *ld_b = (size_t)a->ld_b;
    return HB200_OK;
}

extern "C" int hb200_act_quantize_dev(hb200_act_t a, const float* x_dev, size_t seq_len, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(a);
    int rc = need_ctx();
    if (rc) return rc;
    if (!a) { set_error("null activation handle"); return HB200_ERR_NULL; }
    if (seq_len > a->max_seq) { set_error("seq_len %zu exceeds capacity %zu", seq_len, a->max_seq); return HB200_ERR_BAD_SHAPE; }
    return launch_quantize_q8_0(x_dev ? x_dev : a->x, (int)seq_len, (int)a->n_cols, a->q, a->d, a->sums, a->ld_q, a->ld_b,
                                nullptr, 0, (cudaStream_t)stream);
    HB_GUARD_END
}

extern "C" int hb200_act_load_q8_0_dev(hb200_act_t a, const uint8_t* q8_dev, size_t seq_len, size_t q8_stride, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(a);
    int rc = need_ctx();
    if (rc) return rc;
    if (!a || !q8_dev) { set_error("null handle or pointer"); return HB200_ERR_NULL; }
    if (seq_len > a->max_seq) { set_error("seq_len %zu exceeds capacity %zu", seq_len, a->max_seq); return HB200_ERR_BAD_SHAPE; }
    if (q8_stride < hb200_byte_size(HB200_Q8_0, a->n_cols)) { set_error("q8_stride %zu shorter than a Q8_0 row", q8_stride); return HB200_ERR_BAD_SHAPE; }
    return launch_load_q8_0(q8_dev, q8_stride, (int)seq_len, (int)a->n_cols, a->q, a->d, a->sums, a->ld_q, a->ld_b,
                            (cudaStream_t)stream);
    HB_GUARD_END
}

extern "C" int hb200_act_store_q8_0_dev(hb200_act_t a, uint8_t* q8_dev, size_t seq_len, size_t q8_stride, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(a);
    int rc = need_ctx();
    if (rc) return rc;
    if (!a || !q8_dev) { set_error("null handle or pointer"); return HB200_ERR_NULL; }
    if (seq_len > a->max_seq) { set_error("seq_len %zu exceeds capacity %zu", seq_len, a->max_seq); return HB200_ERR_BAD_SHAPE; }
    if (q8_stride < hb200_byte_size(HB200_Q8_0, a->n_cols)) { set_error("q8_stride %zu shorter than a Q8_0 row", q8_stride); return HB200_ERR_BAD_SHAPE; }
    return launch_store_q8_0(a->q, a->d, a->ld_q, a->ld_b, (int)seq_len, (int)a->n_cols, q8_dev, q8_stride, (cudaStream_t)stream);
    HB_GUARD_END
}

static int producer_check(hb200_act_t a, size_t seq_len) {
    if (!a) { set_error("null activation handle"); return HB200_ERR_NULL; }
    if (seq_len > a->max_seq) { set_error("seq_len %zu exceeds capacity %zu", seq_len, a->max_seq); return HB200_ERR_BAD_SHAPE; }
    return 0;
}

static int hadamard_check(size_t block_size) {
    if (block_size > 1024 || (block_size & (block_size - 1)) != 0) {
        set_error("rotation block of %zu columns: must be a power of two up to 1024", block_size);
        return HB200_ERR_BAD_SHAPE;
    }
    return 0;
}

extern "C" int hb200_act_rms_norm_q8_dev(hb200_act_t a, const float* x_dev, const float* weight_dev, float eps, size_t seq_len,
                                         void* stream) {
    HB_GUARD_BEGIN
    HB_USE(a);
    int rc = need_ctx();
    if (rc) return rc;
    if ((rc = producer_check(a, seq_len))) return rc;
    if (!x_dev || !weight_dev) { set_error("null pointer"); return HB200_ERR_NULL; }
    if (a->n_cols > (size_t)RMS_NORM_MAX_COLS) { set_error("rms_norm_q8 of %zu columns (limit %d)", a->n_cols, RMS_NORM_MAX_COLS); return HB200_ERR_TOO_LARGE; }
    return launch_rms_norm_q8(x_dev, weight_dev, eps, (int)seq_len, (int)a->n_cols, a->q, a->d, a->sums, a->ld_q, a->ld_b, nullptr, 0,
                              (cudaStream_t)stream);
    HB_GUARD_END
}

extern "C" int hb200_act_silu_mul_q8_dev(hb200_act_t a, const float* gate_dev, const float* up_dev, size_t seq_len, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(a);
    int rc = need_ctx();
    if (rc) return rc;
    if ((rc = producer_check(a, seq_len))) return rc;
    if (!gate_dev || !up_dev) { set_error("null pointer"); return HB200_ERR_NULL; }
    return launch_silu_mul_q8(gate_dev, up_dev, (int)seq_len, (int)a->n_cols, (int)(a->n_cols / 32 * 32), a->q, a->d, a->sums,
                              a->ld_q, a->ld_b, nullptr, 0, (cudaStream_t)stream);
    HB_GUARD_END
}

extern "C" int hb200_act_hadamard_quantize_dev(hb200_act_t a, const float* x_dev, const float* signs_dev, size_t block_size,
                                               size_t seq_len, float* rotated_dev, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(a);
    int rc = need_ctx();
    if (rc) return rc;
    if ((rc = producer_check(a, seq_len))) return rc;
    if ((rc = hadamard_check(block_size))) return rc;
    const float* x = x_dev ? x_dev : a->x;
    if (block_size == 0 && !signs_dev && !rotated_dev)
        return launch_quantize_q8_0(x, (int)seq_len, (int)a->n_cols, a->q, a->d, a->sums, a->ld_q, a->ld_b, nullptr, 0,
                                    (cudaStream_t)stream);
    return launch_hadamard_quantize(x, signs_dev, block_size ? (int)block_size : 1, (int)seq_len, (int)a->n_cols, rotated_dev, a->q,
                                    a->d, a->sums, a->ld_q, a->ld_b, nullptr, 0, (cudaStream_t)stream);
    HB_GUARD_END
}

// ------------------------------------------------------- device-buffer calls --

extern "C" int hb200_dot_rows_dev(hb200_weight_t w, hb200_act_t a, size_t seq_len, float* out_dev, size_t ld_out, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(w);
    int rc = need_ctx();
    if (rc) return rc;
    if ((rc = check_pair(w, a, seq_len, ld_out))) return rc;
    if (!out_dev) { set_error("null output"); return HB200_ERR_NULL; }
    if (seq_len == 0 || w->n_rows == 0) return HB200_OK;  // par_dot_rows returns early on n == 0 (pool.rs:520)
    return dot_rows_launch(w, a, seq_len, out_dev, ld_out, (cudaStream_t)stream);
    HB_GUARD_END
}

extern "C" int hb200_matmul_f32_dev(hb200_weight_t w, hb200_act_t a, size_t seq_len, float* out_dev, size_t ld_out, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(w);
    int rc = need_ctx();
    if (rc) return rc;
    if ((rc = check_pair(w, a, seq_len, ld_out))) return rc;
    if (!out_dev) { set_error("null output"); return HB200_ERR_NULL; }
    if (seq_len == 0 || w->n_rows == 0) return HB200_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (w->kind == KIND_Q4K || w->kind == KIND_Q6K)
        return launch_kquant_gemv(w->kind, w->kq, w->d16, (int)w->n_rows, (int)w->n_cols, w->nb, w->n_panels, a->x, (int)seq_len,
                                  out_dev, (int)ld_out, g_ctx.sm_count, st, g_ctx.d_status);
    rc = launch_quantize_q8_0(a->x, (int)seq_len, (int)a->n_cols, a->q, a->d, a->sums, a->ld_q, a->ld_b, nullptr, 0, st);
    if (rc) return rc;
    return dot_rows_launch(w, a, seq_len, out_dev, ld_out, st);
    HB_GUARD_END
}

// ------------------------------------------------- f32-activation matmul --

// One kernel when (panels x tokens) fills the GPU, otherwise terms and ordered sums in two kernels, so that a single
// decode matvec spreads over panels x rounds CTAs instead of panels.  The scratch grows on demand (a synchronising
// allocation the first time a larger product is asked for).
static int f32act_launch(hb200_weight_t w, const float* x_dev, size_t seq_len, float* out_dev, size_t ld_out, bool accumulate, cudaStream_t st) {
    const size_t pairs = (size_t)w->n_panels * seq_len;
    const int rounds = (w->nb + 7) / 8;
    if (pairs >= (size_t)g_ctx.sm_count || rounds < 2)
        return launch_f32act(w->kind, w->bits, w->scales, (int)w->n_rows, (int)w->n_cols, w->nb, w->n_panels, x_dev, (int)seq_len, out_dev,
                             (int)ld_out, accumulate, st);
    int rc = grow(&g_ctx.d_terms, &g_ctx.d_terms_bytes, f32act_terms_bytes(w->kind, w->nb, w->n_panels, (int)seq_len));
    if (rc) return rc;
    return launch_f32act_two_phase(w->kind, w->bits, w->scales, (int)w->n_rows, (int)w->n_cols, w->nb, w->n_panels, x_dev, (int)seq_len,
                                   out_dev, (int)ld_out, accumulate, reinterpret_cast<float*>(g_ctx.d_terms), st);
}

static int f32act_check(hb200_weight_t w, size_t seq_len, size_t ld_out) {
    if (!w) { set_error("null weight handle"); return HB200_ERR_NULL; }
    if (w->dtype == HB200_PTQ1_0 || (w->kind != KIND_Q1 && w->kind != KIND_Q2)) {
        set_error("f32-activation matmul: GGML type %d has no shader counterpart (Q1_0, Q1_0_G128 and Q2_0 do)", w->dtype);
        return HB200_ERR_UNSUPPORTED;
    }
    if (seq_len > 65535) { set_error("f32-activation matmul of %zu tokens (limit 65535)", seq_len); return HB200_ERR_TOO_LARGE; }
    if (ld_out < w->n_rows) { set_error("ld_out %zu smaller than n_rows %zu", ld_out, w->n_rows); return HB200_ERR_BAD_SHAPE; }
    return 0;
}

extern "C" int hb200_matmul_f32act_dev(hb200_weight_t w, const float* x_dev, size_t seq_len, float* out_dev, size_t ld_out,
                                       int accumulate, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(w);
    int rc = need_ctx();
    if (rc) return rc;
    if ((rc = f32act_check(w, seq_len, ld_out))) return rc;
    if (!x_dev || !out_dev) { set_error("null pointer"); return HB200_ERR_NULL; }
    if (seq_len == 0 || w->n_rows == 0) return HB200_OK;
    return f32act_launch(w, x_dev, seq_len, out_dev, ld_out, accumulate != 0, (cudaStream_t)stream);
    HB_GUARD_END
}

extern "C" int hb200_matmul_f32act(hb200_weight_t w, const float* x, size_t seq_len, float* out, int accumulate) {
    HB_GUARD_BEGIN
    HB_USE(w);
    int rc = need_ctx();
    if (rc) return rc;
    if ((rc = f32act_check(w, seq_len, w ? w->n_rows : 0))) return rc;
    if (seq_len == 0 || w->n_rows == 0) return HB200_OK;
    if (!x || !out) { set_error("null buffer"); return HB200_ERR_NULL; }
    const size_t in_bytes = seq_len * w->n_cols * sizeof(float), out_bytes = seq_len * w->n_rows * sizeof(float);
    if ((rc = grow(&g_ctx.d_in, &g_ctx.d_in_bytes, in_bytes))) return rc;
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, out_bytes))) return rc;
    cudaStream_t st = g_ctx.stream;
    HB_CUDA(cudaMemcpyAsync(g_ctx.d_in, x, in_bytes, cudaMemcpyHostToDevice, st));
    if (accumulate) HB_CUDA(cudaMemcpyAsync(g_ctx.d_out, out, out_bytes, cudaMemcpyHostToDevice, st));
    if ((rc = f32act_launch(w, (const float*)g_ctx.d_in, seq_len, (float*)g_ctx.d_out, w->n_rows, accumulate != 0, st))) return rc;
    HB_CUDA(cudaMemcpyAsync(out, g_ctx.d_out, out_bytes, cudaMemcpyDeviceToHost, st));
    HB_CUDA(cudaStreamSynchronize(st));
    return HB200_OK;
    HB_GUARD_END
}

// ------------------------------------------------------------------ argmax --

static int argmax_check(size_t n) {
    if (n == 0) { set_error("argmax of an empty row"); return HB200_ERR_BAD_SHAPE; }
    if (n > (size_t)ARGMAX_CHUNK * ARGMAX_MAX_CHUNKS) { set_error("argmax of %zu values (limit %zu)", n, (size_t)ARGMAX_CHUNK * ARGMAX_MAX_CHUNKS); return HB200_ERR_TOO_LARGE; }
    return 0;
}

extern "C" int hb200_argmax_f32_dev_async(const float* x_dev, size_t n, uint32_t* index_dev, void* stream) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (!x_dev || !index_dev) { set_error("null pointer"); return HB200_ERR_NULL; }
    if ((rc = argmax_check(n))) return rc;
    return launch_argmax(x_dev, n, g_ctx.d_argmax, index_dev, (cudaStream_t)stream);
    HB_GUARD_END
}

extern "C" int hb200_argmax_f32_dev(const float* x_dev, size_t n, uint32_t* index_out, void* stream) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (!x_dev || !index_out) { set_error("null pointer"); return HB200_ERR_NULL; }
    if ((rc = argmax_check(n))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* res = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(g_ctx.d_argmax) + argmax_scratch_bytes());
    if ((rc = launch_argmax(x_dev, n, g_ctx.d_argmax, res, st))) return rc;
    HB_CUDA(cudaMemcpyAsync(index_out, res, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    HB_CUDA(cudaStreamSynchronize(st));
    return HB200_OK;
    HB_GUARD_END
}

// --------------------------------------------------------- host-buffer calls --

extern "C" int hb200_quantize_q8_0(const float* x, size_t seq_len, size_t dim, uint8_t* q8_out) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (seq_len == 0) return HB200_OK;  // par_quantize returns early (pool.rs:468)
    if (!x || !q8_out) { set_error("null buffer"); return HB200_ERR_NULL; }
    if (dim == 0) return HB200_OK;
    if ((rc = ensure_ctx_act(seq_len, dim))) return rc;
    const size_t q8_size = hb200_byte_size(HB200_Q8_0, dim);
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, seq_len * q8_size))) return rc;
    hb200_act* a = g_ctx.act;
    cudaStream_t st = g_ctx.stream;
    HB_CUDA(cudaMemcpyAsync(a->x, x, seq_len * dim * sizeof(float), cudaMemcpyHostToDevice, st));
    if ((rc = launch_quantize_q8_0(a->x, (int)seq_len, (int)dim, a->q, a->d, a->sums, a->ld_q, a->ld_b, g_ctx.d_out, q8_size, st))) return rc;
    HB_CUDA(cudaMemcpyAsync(q8_out, g_ctx.d_out, seq_len * q8_size, cudaMemcpyDeviceToHost, st));
    HB_CUDA(cudaStreamSynchronize(st));
    return HB200_OK;
    HB_GUARD_END
}

// Host-buffer forms of the fused producers: inputs up, one kernel, Q8_0 rows (reference byte layout) back.
extern "C" int hb200_rms_norm_q8(const float* x, const float* weight, float eps, uint8_t* q8_out, size_t seq_len, size_t dim) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (seq_len == 0 || dim == 0) return HB200_OK;
    if (!x || !weight || !q8_out) { set_error("null buffer"); return HB200_ERR_NULL; }
    if (dim > (size_t)RMS_NORM_MAX_COLS) { set_error("rms_norm_q8 of %zu columns (limit %d)", dim, RMS_NORM_MAX_COLS); return HB200_ERR_TOO_LARGE; }
    if ((rc = ensure_ctx_act(seq_len, dim))) return rc;
    const size_t q8_size = hb200_byte_size(HB200_Q8_0, dim);
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, seq_len * q8_size))) return rc;
    if ((rc = grow(&g_ctx.d_in, &g_ctx.d_in_bytes, dim * sizeof(float)))) return rc;
    hb200_act* a = g_ctx.act;
    cudaStream_t st = g_ctx.stream;
    HB_CUDA(cudaMemcpyAsync(a->x, x, seq_len * dim * sizeof(float), cudaMemcpyHostToDevice, st));
    HB_CUDA(cudaMemcpyAsync(g_ctx.d_in, weight, dim * sizeof(float), cudaMemcpyHostToDevice, st));
    if ((rc = launch_rms_norm_q8(a->x, (const float*)g_ctx.d_in, eps, (int)seq_len, (int)dim, a->q, a->d, a->sums, a->ld_q, a->ld_b,
                                 g_ctx.d_out, q8_size, st))) return rc;
    HB_CUDA(cudaMemcpyAsync(q8_out, g_ctx.d_out, seq_len * q8_size, cudaMemcpyDeviceToHost, st));
    HB_CUDA(cudaStreamSynchronize(st));
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_silu_mul_q8(const float* gate, const float* up, uint8_t* q8_out, size_t seq_len, size_t dim) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    const size_t blocks = dim / 32;
    if (seq_len == 0 || blocks == 0) return HB200_OK;
    if (!gate || !up || !q8_out) { set_error("null buffer"); return HB200_ERR_NULL; }
    if ((rc = ensure_ctx_act(seq_len, dim))) return rc;
    const size_t q8_size = blocks * 34;
    const size_t in_bytes = seq_len * dim * sizeof(float);
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, seq_len * q8_size))) return rc;
    if ((rc = grow(&g_ctx.d_in, &g_ctx.d_in_bytes, in_bytes))) return rc;
    hb200_act* a = g_ctx.act;
    cudaStream_t st = g_ctx.stream;
    HB_CUDA(cudaMemcpyAsync(a->x, gate, in_bytes, cudaMemcpyHostToDevice, st));
    HB_CUDA(cudaMemcpyAsync(g_ctx.d_in, up, in_bytes, cudaMemcpyHostToDevice, st));
    if ((rc = launch_silu_mul_q8(a->x, (const float*)g_ctx.d_in, (int)seq_len, (int)dim, (int)(blocks * 32), a->q, a->d, a->sums,
                                 a->ld_q, a->ld_b, g_ctx.d_out, q8_size, st))) return rc;
    HB_CUDA(cudaMemcpyAsync(q8_out, g_ctx.d_out, seq_len * q8_size, cudaMemcpyDeviceToHost, st));
    HB_CUDA(cudaStreamSynchronize(st));
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_hadamard_quantize_q8_0(const float* x, const float* signs, size_t block_size, uint8_t* q8_out,
                                            float* rotated_out, size_t seq_len, size_t dim) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (seq_len == 0 || dim == 0) return HB200_OK;
    if (!x || !q8_out) { set_error("null buffer"); return HB200_ERR_NULL; }
    if ((rc = hadamard_check(block_size))) return rc;
    if ((rc = ensure_ctx_act(seq_len, dim))) return rc;
    const size_t q8_size = hb200_byte_size(HB200_Q8_0, dim);
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, seq_len * q8_size))) return rc;
    if (signs && (rc = grow(&g_ctx.d_in, &g_ctx.d_in_bytes, dim * sizeof(float)))) return rc;
    hb200_act* a = g_ctx.act;
    cudaStream_t st = g_ctx.stream;
    HB_CUDA(cudaMemcpyAsync(a->x, x, seq_len * dim * sizeof(float), cudaMemcpyHostToDevice, st));
    if (signs) HB_CUDA(cudaMemcpyAsync(g_ctx.d_in, signs, dim * sizeof(float), cudaMemcpyHostToDevice, st));
    if ((rc = launch_hadamard_quantize(a->x, signs ? (const float*)g_ctx.d_in : nullptr, block_size ? (int)block_size : 1,
                                       (int)seq_len, (int)dim, rotated_out ? a->x : nullptr, a->q, a->d, a->sums, a->ld_q, a->ld_b,
                                       g_ctx.d_out, q8_size, st))) return rc;
    HB_CUDA(cudaMemcpyAsync(q8_out, g_ctx.d_out, seq_len * q8_size, cudaMemcpyDeviceToHost, st));
    if (rotated_out) HB_CUDA(cudaMemcpyAsync(rotated_out, a->x, seq_len * dim * sizeof(float), cudaMemcpyDeviceToHost, st));
    HB_CUDA(cudaStreamSynchronize(st));
    return HB200_OK;
    HB_GUARD_END
}

static int host_q8_to_act(hb200_weight_t w, const uint8_t* a_q8, size_t seq_len, size_t q8_stride) {
    int rc;
    const size_t q8_size = hb200_byte_size(HB200_Q8_0, w->n_cols);
    if (q8_stride < q8_size) { set_error("q8_stride %zu shorter than a Q8_0 row of %zu bytes", q8_stride, q8_size); return HB200_ERR_BAD_SHAPE; }
    if ((rc = ensure_ctx_act(seq_len, w->n_cols))) return rc;
    const size_t span = (seq_len - 1) * q8_stride + q8_size;
    if ((rc = grow(&g_ctx.d_in, &g_ctx.d_in_bytes, span))) return rc;
    HB_CUDA(cudaMemcpyAsync(g_ctx.d_in, a_q8, span, cudaMemcpyHostToDevice, g_ctx.stream));
    hb200_act* a = g_ctx.act;
    return launch_load_q8_0(g_ctx.d_in, q8_stride, (int)seq_len, (int)w->n_cols, a->q, a->d, a->sums, a->ld_q, a->ld_b, g_ctx.stream);
}

extern "C" int hb200_dot_rows_batched(hb200_weight_t w, const uint8_t* a_q8, size_t seq_len, size_t q8_stride, float* out) {
    HB_GUARD_BEGIN
    HB_USE(w);
    int rc = need_ctx();
    if (rc) return rc;
    if (!w) { set_error("null weight handle"); return HB200_ERR_NULL; }
    if (w->n_rows == 0 || seq_len == 0) return HB200_OK;  // pool.rs:581
    if (!a_q8 || !out) { set_error("null buffer"); return HB200_ERR_NULL; }
    if (w->kind == KIND_Q4K || w->kind == KIND_Q6K) { set_error("K-quant weights have no Q8_0 dot in the reference; use hb200_matmul_f32"); return HB200_ERR_UNSUPPORTED; }
    if ((rc = host_q8_to_act(w, a_q8, seq_len, q8_stride))) return rc;
    const size_t out_bytes = seq_len * w->n_rows * sizeof(float);
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, out_bytes))) return rc;
    if ((rc = dot_rows_launch(w, g_ctx.act, seq_len, (float*)g_ctx.d_out, w->n_rows, g_ctx.stream))) return rc;
    HB_CUDA(cudaMemcpyAsync(out, g_ctx.d_out, out_bytes, cudaMemcpyDeviceToHost, g_ctx.stream));
    HB_CUDA(cudaStreamSynchronize(g_ctx.stream));
    if (seq_len >= (size_t)GEMM_TCR_MIN_TOKENS_Q1) return check_device_status();
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_dot_rows(hb200_weight_t w, const uint8_t* a_q8, float* out) {
    if (!w) { set_error("null weight handle"); return HB200_ERR_NULL; }
    return hb200_dot_rows_batched(w, a_q8, 1, hb200_byte_size(HB200_Q8_0, w->n_cols), out);
}

extern "C" int hb200_matmul_f32(hb200_weight_t w, const float* x, size_t seq_len, float* out) {
    HB_GUARD_BEGIN
    HB_USE(w);
    int rc = need_ctx();
    if (rc) return rc;
    if (!w) { set_error("null weight handle"); return HB200_ERR_NULL; }
    if (w->n_rows == 0 || seq_len == 0) return HB200_OK;
    if (!x || !out) { set_error("null buffer"); return HB200_ERR_NULL; }
    if ((rc = ensure_ctx_act(seq_len, w->n_cols))) return rc;
    const size_t out_bytes = seq_len * w->n_rows * sizeof(float);
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, out_bytes))) return rc;
    HB_CUDA(cudaMemcpyAsync(g_ctx.act->x, x, seq_len * w->n_cols * sizeof(float), cudaMemcpyHostToDevice, g_ctx.stream));
    if ((rc = hb200_matmul_f32_dev(w, g_ctx.act, seq_len, (float*)g_ctx.d_out, w->n_rows, g_ctx.stream))) return rc;
    HB_CUDA(cudaMemcpyAsync(out, g_ctx.d_out, out_bytes, cudaMemcpyDeviceToHost, g_ctx.stream));
    HB_CUDA(cudaStreamSynchronize(g_ctx.stream));
    if (seq_len >= (size_t)GEMM_TCR_MIN_TOKENS_Q1) return check_device_status();
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_matmul_f32_fused(const hb200_weight_t* ws, size_t n_weights, const float* x, size_t seq_len, float* const* outs) {
    HB_GUARD_BEGIN
    if (!ws || !outs) { set_error("null weight or output list"); return HB200_ERR_NULL; }
    if (n_weights == 0 || seq_len == 0) return HB200_OK;
    size_t total = 0;
    for (size_t i = 0; i < n_weights; i++) {
        if (!ws[i]) { set_error("null weight handle at position %zu", i); return HB200_ERR_NULL; }
        if (ws[i]->n_cols != ws[0]->n_cols || ws[i]->slot != ws[0]->slot) {
            // matmul_fused2 / matmul_fused_qkv require one input for all weights (hearth-llm/src/model/matmul.rs:383-567)
            set_error("Matmul dim mismatch: weight %zu has %zu columns, weight 0 has %zu", i, ws[i]->n_cols, ws[0]->n_cols);
            return HB200_ERR_BAD_SHAPE;
        }
        if (ws[i]->n_rows && !outs[i]) { set_error("null output at position %zu", i); return HB200_ERR_NULL; }
        total += (ws[i]->n_rows + 3) & ~(size_t)3;  // every weight's columns start 16-byte aligned
    }
    HB_USE(ws[0]);
    int rc = need_ctx();
    if (rc) return rc;
    if (!x) { set_error("null input"); return HB200_ERR_NULL; }
    if (total == 0) return HB200_OK;
    const size_t n_cols = ws[0]->n_cols;
    if ((rc = ensure_ctx_act(seq_len, n_cols))) return rc;
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, seq_len * total * sizeof(float)))) return rc;
    hb200_act* a = g_ctx.act;
    cudaStream_t st = g_ctx.stream;
    // one upload and one quantization of x for all weights, one buffer [seq_len][sum of rows] for all outputs
    HB_CUDA(cudaMemcpyAsync(a->x, x, seq_len * n_cols * sizeof(float), cudaMemcpyHostToDevice, st));
    bool quantized = false, tensor = false;
    size_t off = 0;
    for (size_t i = 0; i < n_weights; i++) {
        hb200_weight* w = ws[i];
        if (w->n_rows == 0) continue;
        float* out_dev = reinterpret_cast<float*>(g_ctx.d_out) + off;
        if (w->kind == KIND_Q4K || w->kind == KIND_Q6K) {
            if ((rc = launch_kquant_gemv(w->kind, w->kq, w->d16, (int)w->n_rows, (int)w->n_cols, w->nb, w->n_panels, a->x, (int)seq_len,
                                         out_dev, (int)total, g_ctx.sm_count, st, g_ctx.d_status))) return rc;
        } else {
            if (!quantized) {
                if ((rc = launch_quantize_q8_0(a->x, (int)seq_len, (int)n_cols, a->q, a->d, a->sums, a->ld_q, a->ld_b, nullptr, 0, st))) return rc;
                quantized = true;
            }
            tensor = tensor || dot_path(w, a, seq_len) != PATH_DP4A;
            if ((rc = dot_rows_launch(w, a, seq_len, out_dev, total, st))) return rc;
        }
        HB_CUDA(cudaMemcpy2DAsync(outs[i], w->n_rows * sizeof(float), out_dev, total * sizeof(float), w->n_rows * sizeof(float), seq_len,
                                  cudaMemcpyDeviceToHost, st));
        off += (w->n_rows + 3) & ~(size_t)3;
    }
    HB_CUDA(cudaStreamSynchronize(st));
    if (tensor) return check_device_status();
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_block_dots_i32(hb200_weight_t w, const uint8_t* a_q8, size_t seq_len, size_t q8_stride, int32_t* out) {
    HB_GUARD_BEGIN
    HB_USE(w);
    int rc = need_ctx();
    if (rc) return rc;
    if (!w) { set_error("null weight handle"); return HB200_ERR_NULL; }
    if (w->kind == KIND_Q4K || w->kind == KIND_Q6K) { set_error("K-quant dots have no integer form in the reference"); return HB200_ERR_UNSUPPORTED; }
    if (w->n_rows == 0 || seq_len == 0 || w->n_sub == 0) return HB200_OK;
    if (!a_q8 || !out) { set_error("null buffer"); return HB200_ERR_NULL; }
    if ((rc = host_q8_to_act(w, a_q8, seq_len, q8_stride))) return rc;
    const size_t per_tok = w->n_rows * (size_t)w->n_sub;
    const size_t out_bytes = seq_len * per_tok * sizeof(int32_t);
    if ((rc = grow(&g_ctx.d_out, &g_ctx.d_out_bytes, out_bytes))) return rc;
    for (size_t s = 0; s < seq_len; s++) {
        DotOp op;
        fill_op(op, w, g_ctx.act, s, nullptr, w->n_rows, (int32_t*)g_ctx.d_out + s * per_tok);
        int grid = g_ctx.sm_count * gemv_dp4a_ctas_per_sm(w->kind, 1);
        if (grid > w->n_panels) grid = w->n_panels;
        if ((rc = launch_gemv_dp4a(w->kind, 1, true, nullptr, grid, w->n_panels, &op, g_ctx.stream))) return rc;
    }
    HB_CUDA(cudaMemcpyAsync(out, g_ctx.d_out, out_bytes, cudaMemcpyDeviceToHost, g_ctx.stream));
    HB_CUDA(cudaStreamSynchronize(g_ctx.stream));
    return HB200_OK;
    HB_GUARD_END
}

// ------------------------------------------------------------------ batches --

extern "C" int hb200_batch_create(hb200_batch_t* out) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (!out) { set_error("null output handle"); return HB200_ERR_NULL; }
    *out = new hb200_batch();
    (*out)->slot = g_cur;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_batch_add(hb200_batch_t b, hb200_weight_t w, hb200_act_t a, size_t seq_len, float* out_dev, size_t ld_out) {
    HB_GUARD_BEGIN
    HB_USE(b);
    if (!b) { set_error("null batch"); return HB200_ERR_NULL; }
    if (b->sealed) { set_error("batch is sealed"); return HB200_ERR_BAD_SHAPE; }
    int rc = check_pair(w, a, seq_len, ld_out);
    if (rc) return rc;
    if (w->slot != b->slot) { set_error("the batch lives in device slot %d, the weight in slot %d", b->slot, w->slot); return HB200_ERR_BAD_SHAPE; }
    if (!out_dev) { set_error("null output"); return HB200_ERR_NULL; }
    if (seq_len == 0 || w->n_rows == 0) return HB200_OK;
    BatchEntry e{w, a, seq_len, out_dev, ld_out};
    if (w->kind == KIND_Q4K || w->kind == KIND_Q6K) { b->order.push_back({1, b->kquant.size()}); b->kquant.push_back(e); }
    else { b->order.push_back({0, b->entries.size()}); b->entries.push_back(e); }
    size_t ai = 0;
    for (; ai < b->acts.size(); ai++)
        if (b->acts[ai] == a) break;
    if (ai == b->acts.size()) { b->acts.push_back(a); b->act_seq.push_back(seq_len); }
    else if (seq_len > b->act_seq[ai]) b->act_seq[ai] = seq_len;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_batch_seal(hb200_batch_t b);
extern "C" int hb200_batch_free(hb200_batch_t b);

// Splits a sealed batch into sub-batches over contiguous runs of its ops (in the order they were added), balanced by
// weight bytes, for the pipelined host path: while the GPU works on one run the next one's inputs arrive and the
// previous one's outputs leave.  Only done when the runs write disjoint, ascending spans of the output buffer (one
// token per op, as in decode); otherwise the batch keeps the single-copy path.
static int build_segments(hb200_batch* b) {
    const size_t n_ops = b->order.size();
    if (n_ops < 32) return 0;
    auto entry_of = [&](size_t i) -> const BatchEntry& { return b->order[i].first ? b->kquant[b->order[i].second] : b->entries[b->order[i].second]; };
    for (size_t i = 0; i < n_ops; i++)
        if (entry_of(i).seq_len != 1) return 0;
    // Shares of the runs, in 1/32 of the weight bytes: a short first run lets the kernels start after a thirtieth of the
    // inputs has arrived, a short last one leaves a thirtieth of the outputs to read back after the last kernel.  Measured
    // on the 27B step (device time 0.96 ms on that GPU): eight equal runs 1.03 ms end to end, 1-7-8-8-7-1 0.988,
    // 1-6-9-9-6-1 0.977, 1-3-12-12-3-1 0.980, 1-10-10-10-1 1.013, 1-15-15-1 1.051; more than eight runs cost more than
    // their shorter ends save.
    std::vector<int> cum;
    int den = 0;
    for (int v : {1, 6, 9, 9, 6, 1}) { den += v; cum.push_back(den); }
    std::vector<size_t> bytes(n_ops);
    size_t total = 0;
    for (size_t i = 0; i < n_ops; i++) { bytes[i] = entry_of(i).w->resident_bytes; total += bytes[i]; }
    const int n_runs = (int)cum.size();
    std::vector<size_t> cut(n_runs + 1, n_ops);
    cut[0] = 0;
    size_t run = 0;
    int next = 1;
    for (size_t i = 0; i < n_ops && next < n_runs; i++) {
        run += bytes[i];
        while (next < n_runs && run * den >= total * (size_t)cum[next - 1]) cut[next++] = i + 1;
    }
    std::vector<hb200_batch::Segment> segs;
    size_t act_seen = 0;  // activations are listed in order of first use, so each run's new ones are a contiguous range
    const float* prev_hi = nullptr;
    for (int k = 0; k < n_runs; k++) {
        if (cut[k] >= cut[k + 1]) continue;
        hb200_batch::Segment sg;
        sg.ops = new hb200_batch();
        sg.ops->is_child = true;
        size_t act_max = act_seen;
        for (size_t i = cut[k]; i < cut[k + 1]; i++) {
            const BatchEntry& e = entry_of(i);
            (b->order[i].first ? sg.ops->kquant : sg.ops->entries).push_back(e);
            const float* lo = e.out;
            const float* hi = e.out + e.w->n_rows;
            if (!sg.out_lo || lo < sg.out_lo) sg.out_lo = lo;
            if (!sg.out_hi || hi > sg.out_hi) sg.out_hi = hi;
            for (size_t ai = 0; ai < b->acts.size(); ai++)
                if (b->acts[ai] == e.a && ai + 1 > act_max) act_max = ai + 1;
        }
        sg.act_lo = act_seen;
        sg.act_hi = act_max;
        act_seen = act_max;
        segs.push_back(sg);
    }
    bool ok = true;
    for (const auto& sg : segs) {
        if (prev_hi && sg.out_lo < prev_hi) ok = false;  // spans must not interleave
        prev_hi = sg.out_hi;
    }
    // descriptor ranges: qdescs_dev lists the activations that feed Q8_0 ops, in activation order
    {
        std::vector<int> qidx(b->acts.size() + 1, 0);
        int q = 0;
        for (size_t ai = 0; ai < b->acts.size(); ai++) {
            qidx[ai] = q;
            bool q8_user = false;
            for (const BatchEntry& e : b->entries) q8_user = q8_user || e.a == b->acts[ai];
            for (const BatchEntry& e : b->tensor) q8_user = q8_user || e.a == b->acts[ai];
            if (q8_user) q++;
        }
        qidx[b->acts.size()] = q;
        for (auto& sg : segs) { sg.q_lo = qidx[sg.act_lo]; sg.q_hi = qidx[sg.act_hi]; }
    }
    int rc = 0;
    if (ok)
        for (auto& sg : segs)
            if ((rc = hb200_batch_seal(sg.ops))) { ok = false; break; }
    if (!ok) {
        for (auto& sg : segs) hb200_batch_free(sg.ops);
        return rc;
    }
    b->segments = segs;
    b->seg_in.resize(segs.size());
    b->seg_done.resize(segs.size());
    for (size_t k = 0; k < segs.size(); k++) {
        HB_CUDA(cudaEventCreateWithFlags(&b->seg_in[k], cudaEventDisableTiming));
        HB_CUDA(cudaEventCreateWithFlags(&b->seg_done[k], cudaEventDisableTiming));
    }
    if (!g_ctx.copy_in) HB_CUDA(cudaStreamCreateWithFlags(&g_ctx.copy_in, cudaStreamNonBlocking));
    if (!g_ctx.copy_out) HB_CUDA(cudaStreamCreateWithFlags(&g_ctx.copy_out, cudaStreamNonBlocking));
    return 0;
}

// Boundaries of `grid` contiguous runs of items whose largest run cost is as small as contiguity allows (binary search
// on the capacity, greedy fill): chunks[c] .. chunks[c+1]-1 are CTA c's items.  A prefix rule (boundary c at c/grid of
// the total) leaves the largest run up to one item above the mean, 20 % on a 1.7B decode set.
static std::vector<int> balanced_chunks(const std::vector<int>& cost, int grid) {
    const int n = (int)cost.size();
    std::vector<int> chunks(grid + 1, n);
    chunks[0] = 0;
    if (n == 0 || grid <= 0) return chunks;
    long long lo = 0, hi = 0;
    for (int c : cost) { if (c > lo) lo = c; hi += c; }
    auto runs_needed = [&](long long cap) {
        int runs = 1;
        long long run = 0;
        for (int c : cost) {
            if (run + c > cap) { runs++; run = 0; }
            run += c;
        }
        return runs;
    };
    while (lo < hi) {
        const long long mid = (lo + hi) / 2;
        if (runs_needed(mid) <= grid) hi = mid; else lo = mid + 1;
    }
    long long run = 0;
    int next_c = 1;
    for (int i = 0; i < n; i++) {
        if (run + cost[i] > lo) { chunks[next_c++] = i; run = 0; }
        run += cost[i];
    }
    return chunks;
}

// Work plan of a list launch of the decode matvec.  Item i is panel panel[i] of op op[i] and takes rounds[i] rounds.
// With enough work (at least two of the longest items per CTA) and a balance that cuts between items cannot reach
// (largest share more than 3 % above the mean), the list of ALL rounds is cut into `grid` equal shares,
// and a cut inside an item splits it between two neighbouring CTAs (the earlier one hands its running sums over in
// carry slot c, c = index of the later CTA); otherwise the cuts fall between items (balanced_chunks).  Per CTA the
// segments come in the order [first rounds of the item cut at its end] [whole items, consecutive panels of one op
// merged] [last rounds of the item cut at its start], so that a CTA produces the carry its neighbour needs before
// anything else and consumes the carry it needs after everything else.
static void plan_flat(const int* op, const int* panel, const int* rounds, int n, int grid, std::vector<FlatSeg>& segs,
                      std::vector<int>& seg_begin) {
    segs.clear();
    seg_begin.assign(grid + 1, 0);
    if (n <= 0 || grid <= 0) return;
    std::vector<long long> pre(n + 1, 0);
    int maxr = 1;
    for (int i = 0; i < n; i++) {
        pre[i + 1] = pre[i] + rounds[i];
        if (rounds[i] > maxr) maxr = rounds[i];
    }
    const long long R = pre[n];
    std::vector<long long> cut(grid + 1, R);
    cut[0] = 0;
    // Cuts between items first; panels are cut only where that leaves the largest share more than 3 % above the mean (a
    // big model on one GPU balances to within 0.5 % without, and every cut panel costs its two CTAs a segment more).
    std::vector<int> cost(rounds, rounds + n);
    for (int& v : cost) v = v * 8 + 1;  // a small fixed share per panel, as measured for the item-granular plan
    const std::vector<int> chunks = balanced_chunks(cost, grid);
    long long largest = 0;
    for (int c = 0; c < grid; c++) largest = std::max(largest, pre[chunks[c + 1]] - pre[chunks[c]]);
    const bool cut_panels = R >= 2LL * grid * maxr && largest * grid * 100 > R * 103;
    if (cut_panels) {
        for (int c = 1; c < grid; c++) cut[c] = (R * c) / grid;
    } else {
        for (int c = 1; c < grid; c++) cut[c] = pre[chunks[c]];
    }
    int i = 0;
    for (int c = 0; c < grid; c++) {
        seg_begin[c] = (int)segs.size();
        const long long lo = cut[c], hi = cut[c + 1];
        if (lo >= hi) continue;
        while (pre[i + 1] <= lo) i++;
        std::vector<FlatSeg> whole;
        FlatSeg head{}, tail{};
        bool has_head = false, has_tail = false;
        for (int j = i; j < n && pre[j] < hi; j++) {
            const int a = (int)(std::max(lo, pre[j]) - pre[j]), b = (int)(std::min(hi, pre[j + 1]) - pre[j]);
            FlatSeg sg{};
            sg.op = op[j]; sg.p0 = panel[j]; sg.cnt = 1; sg.r0 = a; sg.r1 = b;
            sg.flags = (a > 0 ? 1 : 0) | (b < rounds[j] ? 2 : 0);
            sg.carry_in = a > 0 ? c : 0;
            sg.carry_out = b < rounds[j] ? c + 1 : 0;
            if (sg.flags & 2) { head = sg; has_head = true; }       // the item cut at this CTA's end (may also start from a carry)
            else if (sg.flags & 1) { tail = sg; has_tail = true; }  // the item cut at this CTA's start
            else if (!whole.empty() && whole.back().op == sg.op && whole.back().p0 + whole.back().cnt == sg.p0 && whole.back().r1 == sg.r1) whole.back().cnt++;
            else whole.push_back(sg);
        }
        if (has_head) segs.push_back(head);
        for (const FlatSeg& w : whole) segs.push_back(w);
        if (has_tail) segs.push_back(tail);
    }
    seg_begin[grid] = (int)segs.size();
}

extern "C" int hb200_plan_rounds(const int* op, const int* panel, const int* rounds, size_t n_items, int grid, int* seg_begin,
                                 int* segs, size_t seg_cap, size_t* n_segs) {
    HB_GUARD_BEGIN
    if ((n_items && (!op || !panel || !rounds)) || !seg_begin || !n_segs || (seg_cap && !segs)) { set_error("null buffer"); return HB200_ERR_NULL; }
    if (grid <= 0) { set_error("grid must be positive"); return HB200_ERR_BAD_SHAPE; }
    for (size_t i = 0; i < n_items; i++)
        if (rounds[i] <= 0) { set_error("an item takes at least one round"); return HB200_ERR_BAD_SHAPE; }
    std::vector<FlatSeg> out;
    std::vector<int> begin;
    plan_flat(op, panel, rounds, (int)n_items, grid, out, begin);
    *n_segs = out.size();
    if (out.size() > seg_cap) { set_error("%zu segments do not fit the %zu given", out.size(), seg_cap); return HB200_ERR_TOO_LARGE; }
    for (int c = 0; c <= grid; c++) seg_begin[c] = begin[c];
    static_assert(sizeof(FlatSeg) == 8 * sizeof(int), "a segment is eight ints");
    if (!out.empty()) memcpy(segs, out.data(), out.size() * sizeof(FlatSeg));
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_bounds_checked(void) {
#ifdef HB200_BOUNDS
    return 1;
#else
    return 0;
#endif
}

extern "C" int hb200_bounds_selftest(void) {
    HB_GUARD_BEGIN
#ifdef HB200_BOUNDS
    int rc = need_ctx();
    if (rc) return rc;
    // The quantizer on one token of 2048 columns with a block-value pitch that is too small on purpose (32 instead of
    // 64; the buffers themselves are large enough): the 32 stores of block values beyond the pitch must be counted and
    // skipped, and reported by the status check as site 23.
    float* x = nullptr; int8_t* q = nullptr; float* d = nullptr; float* sums = nullptr;
    HB_CUDA(cudaMalloc(&x, 2048 * sizeof(float)));
    HB_CUDA(cudaMalloc(&q, 2048));
    HB_CUDA(cudaMalloc(&d, 64 * sizeof(float)));
    HB_CUDA(cudaMalloc(&sums, 64 * sizeof(float)));
    HB_CUDA(cudaMemset(x, 0, 2048 * sizeof(float)));
    rc = launch_quantize_q8_0(x, 1, 2048, q, d, sums, 2048, 32, nullptr, 0, g_ctx.stream);
    if (!rc) { HB_CUDA(cudaStreamSynchronize(g_ctx.stream)); }
    cudaFree(x); cudaFree(q); cudaFree(d); cudaFree(sums);
    if (rc) return rc;
    int site = 0, count = 0;
    if ((rc = bounds_fetch_quantize(&site, &count))) return rc;
    if (site != 23 || count != 32) {
        set_error("bounds self-test: expected 32 skipped accesses at site 23, found %d at site %d", count, site);
        return HB200_ERR_CUDA;
    }
    return HB200_OK;
#else
    set_error("not the bounds-checked build");
    return HB200_ERR_UNSUPPORTED;
#endif
    HB_GUARD_END
}

extern "C" int hb200_plan_chunks(const int* cost, size_t n_items, int grid, int* chunks) {
    HB_GUARD_BEGIN
    if ((!cost && n_items) || !chunks) { set_error("null buffer"); return HB200_ERR_NULL; }
    if (grid <= 0) { set_error("grid must be positive"); return HB200_ERR_BAD_SHAPE; }
    for (size_t i = 0; i < n_items; i++)
        if (cost[i] < 0) { set_error("negative cost"); return HB200_ERR_BAD_SHAPE; }
    const std::vector<int> c = balanced_chunks(std::vector<int>(cost, cost + n_items), grid);
    for (int i = 0; i <= grid; i++) chunks[i] = c[i];
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_batch_seal(hb200_batch_t b) {
    HB_GUARD_BEGIN
    HB_USE(b);
    if (!b) { set_error("null batch"); return HB200_ERR_NULL; }
    if (b->sealed) return HB200_OK;
    if (b->peers.n > 1) {
        if (!b->kquant.empty()) { set_error("peer-store batches carry Q8_0-activation ops only"); return HB200_ERR_UNSUPPORTED; }
        for (const BatchEntry& e : b->entries)
            if (gemm_tc_wanted(e.w->kind, e.seq_len)) {
                set_error("peer-store batches take at most %d tokens per op", GEMM_TC_MIN_TOKENS - 1);
                return HB200_ERR_UNSUPPORTED;
            }
    }
    // One launch per (kind, tokens-per-op) combination.
    struct Acc { std::vector<DotOp> first; std::vector<DotItem> second; std::vector<int> cost; };
    std::map<std::pair<int, int>, Acc> acc;
    for (const BatchEntry& e : b->entries) {
        // tensor-core kernels: all such ops of one kind share a launch (a peer-store batch stays on the streaming kernel,
        // the only one with that epilogue)
        const DotPath path = b->peers.n > 1 ? PATH_DP4A : dot_path(e.w, e.a, e.seq_len);
        if (path == PATH_TC) { b->tensor.push_back(e); continue; }
        if (path == PATH_TC_ROWS) { b->tensor_rows.push_back(e); continue; }
        for (size_t tok0 = 0, m = 0; tok0 < e.seq_len; tok0 += m) {
            m = dp4a_pass_tokens(e.seq_len - tok0);
            auto& slot = acc[{e.w->kind, (int)m}];
            DotOp op;
            fill_op(op, e.w, e.a, tok0, e.out, e.ld_out, nullptr);
            const int idx = (int)slot.first.size();
            slot.first.push_back(op);
            for (int p = 0; p < e.w->n_panels; p++) {
                slot.second.push_back(make_int2(idx, p));
                slot.cost.push_back(e.w->nb > 8 ? (e.w->nb + 7) / 8 : 1);  // rounds of the panel
            }
        }
    }
    for (auto& kv : acc) {
        BatchGroup g;
        g.kind = kv.first.first;
        g.m = kv.first.second;
        g.n_items = (int)kv.second.second.size();
        if (g.n_items == 0) continue;
        // One wave of CTAs; each gets an equal share of the launch's rounds (see plan_flat).
        g.grid = g_ctx.sm_count * gemv_dp4a_ctas_per_sm(g.kind, g.m);
        {
            std::vector<int> iop(g.n_items), ipanel(g.n_items);
            long long total_rounds = 0;
            for (int i = 0; i < g.n_items; i++) {
                iop[i] = kv.second.second[i].x;
                ipanel[i] = kv.second.second[i].y;
                total_rounds += kv.second.cost[i];
            }
            int max_rounds = 1;
            for (int c : kv.second.cost) max_rounds = c > max_rounds ? c : max_rounds;
            // too little work to cut panels (plan_flat's rule): whole panels, and no more CTAs than panels
            if (total_rounds < 2LL * g.grid * max_rounds && g.grid > g.n_items) g.grid = g.n_items;
            std::vector<FlatSeg> segs;
            std::vector<int> seg_begin;
            plan_flat(iop.data(), ipanel.data(), kv.second.cost.data(), g.n_items, g.grid, segs, seg_begin);
            g.n_segs = (int)segs.size();
            std::vector<FlatRec> recs(segs.size());
            for (size_t i = 0; i < segs.size(); i++) {
                recs[i].seg = segs[i];
                recs[i].op = kv.second.first[segs[i].op];
            }
            HB_CUDA(cudaMalloc(&g.recs_dev, recs.size() * sizeof(FlatRec)));
            HB_CUDA(cudaMemcpy(g.recs_dev, recs.data(), recs.size() * sizeof(FlatRec), cudaMemcpyHostToDevice));
            HB_CUDA(cudaMalloc(&g.seg_begin_dev, seg_begin.size() * sizeof(int)));
            HB_CUDA(cudaMemcpy(g.seg_begin_dev, seg_begin.data(), seg_begin.size() * sizeof(int), cudaMemcpyHostToDevice));
            HB_CUDA(cudaMalloc(&g.carry_dev, (size_t)(g.grid + 1) * FLAT_CARRY_FLOATS * sizeof(float)));
            HB_CUDA(cudaMalloc(&g.cflags_dev, (size_t)(g.grid + 1) * sizeof(int)));
            HB_CUDA(cudaMemset(g.cflags_dev, 0, (size_t)(g.grid + 1) * sizeof(int)));
        }
        b->groups.push_back(g);
    }
    // Tensor-core ops: per weight kind one list of matrices whose 128 x 64 tiles are numbered consecutively, and
    // contiguous runs of tiles per CTA balanced by 128-column blocks (plus a fixed share per tile for its fill and drain).
    for (int rows = 0; rows < 2; rows++)
    for (int kind : {KIND_Q1, KIND_Q2}) {
        std::vector<TcMat> mats;
        std::vector<int> cost;
        int n_tiles = 0;
        for (const BatchEntry& e : (rows ? b->tensor_rows : b->tensor)) {
            if (e.w->kind != kind) continue;
            TcMat m;
            if (rows)
                gemm_tcr_fill(m, e.a->qmap32_dev, e.w->bits, e.w->scales, e.a->d, e.a->ld_b, (int)e.w->n_rows, e.w->nb, (int)e.seq_len,
                              e.out, (int)e.ld_out, n_tiles);
            else
                gemm_tc_fill(m, e.a->qmap_dev, e.w->bits, e.w->scales, e.a->d, e.a->ld_b, (int)e.w->n_rows, e.w->nb, (int)e.seq_len, e.out,
                             (int)e.ld_out, n_tiles);
            for (int t = m.tile_begin; t < m.tile_end; t++) cost.push_back(e.w->nb + 4);
            n_tiles = m.tile_end;
            mats.push_back(m);
        }
        if (n_tiles == 0) continue;
        hb200_batch::TcGroup g;
        g.kind = kind;
        g.rows = rows != 0;
        g.n_tiles = n_tiles;
        g.grid = n_tiles < g_ctx.sm_count ? n_tiles : g_ctx.sm_count;
        const std::vector<int> chunks = balanced_chunks(cost, g.grid);
        HB_CUDA(cudaMalloc(&g.mats_dev, mats.size() * sizeof(TcMat)));
        HB_CUDA(cudaMemcpy(g.mats_dev, mats.data(), mats.size() * sizeof(TcMat), cudaMemcpyHostToDevice));
        HB_CUDA(cudaMalloc(&g.chunks_dev, chunks.size() * sizeof(int)));
        HB_CUDA(cudaMemcpy(g.chunks_dev, chunks.data(), chunks.size() * sizeof(int), cudaMemcpyHostToDevice));
        b->tc_groups.push_back(g);
    }
    // K-quant ops: per (kind, tokens per pass) one list of matrices whose items (32-row panel x token tile) are numbered
    // consecutively, and contiguous runs of items per CTA balanced by rounds.
    for (int kind : {KIND_Q4K, KIND_Q6K})
        for (int mt : {1, 2, 4, 8, 16}) {
            std::vector<KqMat> mats;
            std::vector<int> cost;
            int n_items = 0;
            for (const BatchEntry& e : b->kquant) {
                if (e.w->kind != kind || kquant_tokens_per_pass(kind, (int)e.seq_len) != mt) continue;
                KqMat m;
                m.kq = e.w->kq; m.d16 = e.w->d16; m.x = e.a->x; m.out = e.out;
                m.n_rows = (int)e.w->n_rows; m.n_cols = (int)e.w->n_cols; m.nblk = e.w->nb; m.n_panels = e.w->n_panels;
                m.seq_len = (int)e.seq_len; m.ld_out = (int)e.ld_out;
                m.item_begin = n_items;
                m.item_end = n_items + kquant_items(kind, m.n_panels, m.seq_len);
                for (int t = m.item_begin; t < m.item_end; t++) cost.push_back(kquant_rounds(kind, m.nblk));
                n_items = m.item_end;
                mats.push_back(m);
            }
            if (n_items == 0) continue;
            hb200_batch::KqGroup g;
            g.kind = kind; g.mt = mt; g.n_items = n_items;
            g.grid = kquant_grid(kind, mt, g_ctx.sm_count, n_items);
            const std::vector<int> chunks = balanced_chunks(cost, g.grid);
            HB_CUDA(cudaMalloc(&g.mats_dev, mats.size() * sizeof(KqMat)));
            HB_CUDA(cudaMemcpy(g.mats_dev, mats.data(), mats.size() * sizeof(KqMat), cudaMemcpyHostToDevice));
            HB_CUDA(cudaMalloc(&g.chunks_dev, chunks.size() * sizeof(int)));
            HB_CUDA(cudaMemcpy(g.chunks_dev, chunks.data(), chunks.size() * sizeof(int), cudaMemcpyHostToDevice));
            b->kq_groups.push_back(g);
        }
    // Host-input path: one staging buffer for every distinct activation's f32 rows and one descriptor list for the
    // list quantizer.  K-quant ops read f32 from the activation's own area, so those rows are also copied there.
    {
        std::vector<QuantDesc> qd;
        size_t off = 0;
        for (size_t i = 0; i < b->acts.size(); i++) {
            hb200_act* a = b->acts[i];
            b->act_offset.push_back(off);
            off += b->act_seq[i] * a->n_cols;
            off = (off + 3) & ~(size_t)3;  // keep every activation 16-byte aligned in the staging buffer
        }
        b->input_floats = off;
        if (off) HB_CUDA(cudaMalloc(&b->x_stage, off * sizeof(float)));
        for (size_t i = 0; i < b->acts.size(); i++) {
            hb200_act* a = b->acts[i];
            bool q8_user = false;
            for (const BatchEntry& e : b->entries) q8_user = q8_user || e.a == a;
            for (const BatchEntry& e : b->tensor) q8_user = q8_user || e.a == a;
            for (const BatchEntry& e : b->kquant) b->has_kquant_inputs = b->has_kquant_inputs || e.a == a;
            if (!q8_user) continue;
            QuantDesc d;
            d.x = b->x_stage + b->act_offset[i];
            d.q = a->q; d.d = a->d; d.sums = a->sums;
            d.n_cols = (int)a->n_cols; d.seq_len = (int)b->act_seq[i]; d.ld_q = a->ld_q; d.ld_b = a->ld_b;
            qd.push_back(d);
            if (a->ld_q / 1024 > b->q_max_chunks) b->q_max_chunks = a->ld_q / 1024;
            if ((int)b->act_seq[i] > b->q_max_seq) b->q_max_seq = (int)b->act_seq[i];
        }
        b->n_qacts = (int)qd.size();
        if (!qd.empty()) {
            HB_CUDA(cudaMalloc(&b->qdescs_dev, qd.size() * sizeof(QuantDesc)));
            HB_CUDA(cudaMemcpy(b->qdescs_dev, qd.data(), qd.size() * sizeof(QuantDesc), cudaMemcpyHostToDevice));
        }
    }
    if (!b->is_child && b->peers.n <= 1) {
        int rc2 = build_segments(b);
        if (rc2) return rc2;
    }
    b->sealed = true;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_batch_launch(hb200_batch_t b, void* stream) {
    HB_GUARD_BEGIN
    HB_USE(b);
    int rc = need_ctx();
    if (rc) return rc;
    if (!b) { set_error("null batch"); return HB200_ERR_NULL; }
    if (!b->sealed) { set_error("batch is not sealed"); return HB200_ERR_BAD_SHAPE; }
    cudaStream_t st = (cudaStream_t)stream;
    // A peer launch is one epoch, however many kernels it takes: they run in stream order, each makes its peer stores
    // visible before it ends, and the last one alone runs the flag exchange.  A rank whose shard is empty still
    // publishes, so that the epochs of all ranks advance together.
    PeerTable pt = b->peers;
    if (pt.n > 1) {
        pt.epoch = ++b->epoch;
        pt.status = g_ctx.d_status;
        pt.area_off = b->peer_area_floats ? (long long)((pt.epoch - 1) & 1) * (long long)b->peer_area_floats : 0;
    }
    for (size_t gi = 0; gi < b->groups.size(); gi++) {
        BatchGroup& g = b->groups[gi];
        pt.publish = (gi + 1 == b->groups.size()) ? 1 : 0;
        FlatLaunch fl;
        fl.recs = g.recs_dev; fl.seg_begin = g.seg_begin_dev; fl.carry = g.carry_dev; fl.cflags = g.cflags_dev;
        fl.epoch = ++g.epoch;
        fl.status = g_ctx.d_status;
        if ((rc = launch_gemv_dp4a(g.kind, g.m, false, &fl, g.grid, g.n_segs, nullptr, st, pt.n > 1 ? &pt : nullptr))) return rc;
    }
    if (pt.n > 1 && b->groups.empty() && (rc = launch_peer_publish(pt, st))) return rc;
    for (const hb200_batch::TcGroup& g : b->tc_groups)
        if ((rc = (g.rows ? launch_gemm_tcr_list : launch_gemm_tc_list)(g.kind, g.mats_dev, g.chunks_dev, g.n_tiles, g.grid, g_ctx.d_status, st)))
            return rc;
    for (const hb200_batch::KqGroup& g : b->kq_groups)
        if ((rc = launch_kquant_gemv_list(g.kind, g.mt, g.mats_dev, g.chunks_dev, g.n_items, g.grid, st, g_ctx.d_status))) return rc;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_multi_batch_launch(hb200_batch_t const* batches, int n, void* const* streams) {
    HB_GUARD_BEGIN
    if (!batches) { set_error("null batch list"); return HB200_ERR_NULL; }
    for (int i = 0; i < n; i++) {
        const int rc = hb200_batch_launch(batches[i], streams ? streams[i] : nullptr);
        if (rc) return rc;
    }
    return HB200_OK;
    HB_GUARD_END
}

extern "C" size_t hb200_batch_input_floats(hb200_batch_t b) { return (b && b->sealed) ? b->input_floats : 0; }

// One recorded step: inputs from host memory (x_host) or, x_dev given, from a device buffer of the same layout that was
// filled on x_stream; outputs read back to out_host.
static int batch_run(hb200_batch_t b, const float* x_host, const float* x_dev, cudaStream_t x_stream, const float* out_dev_base,
                     size_t out_floats, float* out_host) {
    int rc = need_ctx();
    if (rc) return rc;
    if (!b) { set_error("null batch"); return HB200_ERR_NULL; }
    if (!b->sealed) { set_error("batch is not sealed"); return HB200_ERR_BAD_SHAPE; }
    if ((b->input_floats && !x_host && !x_dev) || (out_floats && (!out_dev_base || !out_host))) { set_error("null buffer"); return HB200_ERR_NULL; }
    cudaStream_t st = g_ctx.stream;
    if (x_dev) {
        // the inputs are on the device already: one device copy into the staging area the quantizer reads (8 MB take a few
        // microseconds), ordered behind the stream that produced them
        if (!g_ctx.ev_inputs) HB_CUDA(cudaEventCreateWithFlags(&g_ctx.ev_inputs, cudaEventDisableTiming));
        HB_CUDA(cudaEventRecord(g_ctx.ev_inputs, x_stream));
        HB_CUDA(cudaStreamWaitEvent(st, g_ctx.ev_inputs, 0));
        if (b->input_floats) HB_CUDA(cudaMemcpyAsync(b->x_stage, x_dev, b->input_floats * sizeof(float), cudaMemcpyDeviceToDevice, st));
    }
    if (!b->segments.empty() && out_floats) {
        // Pipelined: uploads on one stream, quantize + matvec on the compute stream, readbacks on a third; run k's
        // compute overlaps run k+1's upload and run k-1's readback.  Every stream is drained before returning.
        const float* base = out_dev_base;
        bool spans_ok = true;
        for (const auto& sg : b->segments) spans_ok = spans_ok && sg.out_lo >= base && sg.out_hi <= base + out_floats;
        if (spans_ok) {
            for (size_t k = 0; k < b->segments.size(); k++) {
                const auto& sg = b->segments[k];
                if (!x_dev) {
                    if (sg.act_hi > sg.act_lo) {
                        const size_t f_lo = b->act_offset[sg.act_lo];
                        const size_t f_hi = sg.act_hi < b->acts.size() ? b->act_offset[sg.act_hi] : b->input_floats;
                        HB_CUDA(cudaMemcpyAsync(b->x_stage + f_lo, x_host + f_lo, (f_hi - f_lo) * sizeof(float), cudaMemcpyHostToDevice, g_ctx.copy_in));
                    }
                    HB_CUDA(cudaEventRecord(b->seg_in[k], g_ctx.copy_in));
                    HB_CUDA(cudaStreamWaitEvent(st, b->seg_in[k], 0));
                }
                if (b->has_kquant_inputs)
                    for (size_t i = sg.act_lo; i < sg.act_hi; i++)
                        HB_CUDA(cudaMemcpyAsync(b->acts[i]->x, b->x_stage + b->act_offset[i], b->act_seq[i] * b->acts[i]->n_cols * sizeof(float),
                                                cudaMemcpyDeviceToDevice, st));
                if (sg.q_hi > sg.q_lo && (rc = launch_quantize_q8_0_list(b->qdescs_dev + sg.q_lo, sg.q_hi - sg.q_lo, b->q_max_chunks, b->q_max_seq, st))) return rc;
                if ((rc = hb200_batch_launch(sg.ops, st))) return rc;
                HB_CUDA(cudaEventRecord(b->seg_done[k], st));
                HB_CUDA(cudaStreamWaitEvent(g_ctx.copy_out, b->seg_done[k], 0));
                HB_CUDA(cudaMemcpyAsync(out_host + (sg.out_lo - base), sg.out_lo, (size_t)(sg.out_hi - sg.out_lo) * sizeof(float), cudaMemcpyDeviceToHost,
                                        g_ctx.copy_out));
            }
            HB_CUDA(cudaStreamSynchronize(g_ctx.copy_out));
            HB_CUDA(cudaStreamSynchronize(st));
            if (!b->tensor.empty() || !b->tensor_rows.empty()) return check_device_status();
            return HB200_OK;
        }
    }
    if (b->input_floats && !x_dev) HB_CUDA(cudaMemcpyAsync(b->x_stage, x_host, b->input_floats * sizeof(float), cudaMemcpyHostToDevice, st));
    if (b->has_kquant_inputs)
        for (size_t i = 0; i < b->acts.size(); i++)
            HB_CUDA(cudaMemcpyAsync(b->acts[i]->x, b->x_stage + b->act_offset[i], b->act_seq[i] * b->acts[i]->n_cols * sizeof(float),
                                    cudaMemcpyDeviceToDevice, st));
    if ((rc = launch_quantize_q8_0_list(b->qdescs_dev, b->n_qacts, b->q_max_chunks, b->q_max_seq, st))) return rc;
    if ((rc = hb200_batch_launch(b, st))) return rc;
    if (b->peers.n > 1 && b->peer_area_floats) out_dev_base += (size_t)((b->epoch - 1) & 1) * b->peer_area_floats;
    if (out_floats) HB_CUDA(cudaMemcpyAsync(out_host, out_dev_base, out_floats * sizeof(float), cudaMemcpyDeviceToHost, st));
    HB_CUDA(cudaStreamSynchronize(st));
    if (!b->tensor.empty() || !b->tensor_rows.empty()) return check_device_status();
    return HB200_OK;
}

extern "C" int hb200_batch_run_host(hb200_batch_t b, const float* x_host, const float* out_dev_base, size_t out_floats,
                                    float* out_host) {
    HB_GUARD_BEGIN
    HB_USE(b);
    return batch_run(b, x_host, nullptr, nullptr, out_dev_base, out_floats, out_host);
    HB_GUARD_END
}

extern "C" int hb200_batch_run_dev(hb200_batch_t b, const float* x_dev, void* x_stream, const float* out_dev_base, size_t out_floats,
                                   float* out_host) {
    HB_GUARD_BEGIN
    HB_USE(b);
    if (b && b->input_floats && !x_dev) { set_error("null input buffer"); return HB200_ERR_NULL; }
    return batch_run(b, nullptr, x_dev, (cudaStream_t)x_stream, out_dev_base, out_floats, out_host);
    HB_GUARD_END
}

extern "C" int hb200_batch_launch_count(hb200_batch_t b) {
    if (!b || !b->sealed) return 0;
    int n = (int)(b->groups.size() + b->kq_groups.size() + b->tc_groups.size());
    if (b->peers.n > 1 && b->groups.empty()) n += 1;                         // the flag exchange on its own
    return n;
}

extern "C" int hb200_batch_free(hb200_batch_t b) {
    HB_GUARD_BEGIN
    HB_USE(b);
    if (!b) return HB200_OK;
    for (BatchGroup& g : b->groups) {
        if (g.recs_dev) cudaFree(g.recs_dev);
        if (g.seg_begin_dev) cudaFree(g.seg_begin_dev);
        if (g.carry_dev) cudaFree(g.carry_dev);
        if (g.cflags_dev) cudaFree(g.cflags_dev);
    }
    for (hb200_batch::TcGroup& g : b->tc_groups) {
        if (g.mats_dev) cudaFree(g.mats_dev);
        if (g.chunks_dev) cudaFree(g.chunks_dev);
    }
    for (hb200_batch::KqGroup& g : b->kq_groups) {
        if (g.mats_dev) cudaFree(g.mats_dev);
        if (g.chunks_dev) cudaFree(g.chunks_dev);
    }
    for (auto& sg : b->segments) hb200_batch_free(sg.ops);
    for (cudaEvent_t e : b->seg_in) cudaEventDestroy(e);
    for (cudaEvent_t e : b->seg_done) cudaEventDestroy(e);
    if (b->x_stage) cudaFree(b->x_stage);
    if (b->qdescs_dev) cudaFree(b->qdescs_dev);
    delete b;
    return HB200_OK;
    HB_GUARD_END
}

// ------------------------------------------------------------ peer buffers --

extern "C" int hb200_peer_alloc(size_t bytes, void** data_dev, uint8_t handle[HB200_PEER_HANDLE_BYTES]) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (!data_dev || !handle) { set_error("null output"); return HB200_ERR_NULL; }
    static_assert(sizeof(cudaIpcMemHandle_t) == HB200_PEER_HANDLE_BYTES, "IPC handle size");
    char* base = nullptr;
    HB_CUDA(cudaMalloc(&base, bytes + PEER_CTRL_BYTES));
    HB_CUDA(cudaMemset(base, 0, bytes + PEER_CTRL_BYTES));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, base);
    if (e != cudaSuccess) { cudaFree(base); set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e)); return HB200_ERR_CUDA; }
    memcpy(handle, &h, sizeof(h));
    *data_dev = base + PEER_CTRL_BYTES;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_peer_free(void* data_dev) {
    HB_GUARD_BEGIN
    if (!data_dev) return HB200_OK;
    HB_CUDA(cudaFree(static_cast<char*>(data_dev) - PEER_CTRL_BYTES));
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_peer_open(const uint8_t handle[HB200_PEER_HANDLE_BYTES], void** data_dev) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    if (!data_dev || !handle) { set_error("null argument"); return HB200_ERR_NULL; }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    HB_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
    *data_dev = static_cast<char*>(base) + PEER_CTRL_BYTES;
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_peer_close(void* data_dev) {
    HB_GUARD_BEGIN
    if (!data_dev) return HB200_OK;
    HB_CUDA(cudaIpcCloseMemHandle(static_cast<char*>(data_dev) - PEER_CTRL_BYTES));
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_batch_set_peers(hb200_batch_t b, int n_ranks, int my_rank, void* const* data, size_t area_bytes, int wait) {
    HB_GUARD_BEGIN
    HB_USE(b);
    if (!b || !data) { set_error("null argument"); return HB200_ERR_NULL; }
    if (b->sealed) { set_error("set the peers before sealing the batch"); return HB200_ERR_BAD_SHAPE; }
    if (n_ranks < 1 || n_ranks > MAX_PEERS || my_rank < 0 || my_rank >= n_ranks) {
        set_error("rank %d of %d: at most %d ranks", my_rank, n_ranks, MAX_PEERS);
        return HB200_ERR_BAD_SHAPE;
    }
    PeerTable pt = {};
    for (int r = 0; r < n_ranks; r++) {
        if (!data[r]) { set_error("null buffer for rank %d", r); return HB200_ERR_NULL; }
        pt.data[r] = static_cast<float*>(data[r]);
    }
    if (area_bytes % 16) { set_error("area_bytes %zu is not a multiple of 16", area_bytes); return HB200_ERR_BAD_SHAPE; }
    pt.n = n_ranks; pt.me = my_rank; pt.wait = wait ? 1 : 0;
    b->peers = pt;
    b->peer_area_floats = area_bytes / sizeof(float);
    return HB200_OK;
    HB_GUARD_END
}

extern "C" int hb200_batch_peer_area(hb200_batch_t b) {
    if (!b || b->peers.n <= 1 || !b->peer_area_floats || b->epoch == 0) return 0;
    return (b->epoch - 1) & 1;
}

extern "C" int hb200_check_status(void) {
    HB_GUARD_BEGIN
    int rc = need_ctx();
    if (rc) return rc;
    HB_CUDA(cudaDeviceSynchronize());
    return check_device_status();
    HB_GUARD_END
}

extern "C" int hb200_stream_synchronize(void* stream) {
    HB_GUARD_BEGIN
    HB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return HB200_OK;
    HB_GUARD_END
}
