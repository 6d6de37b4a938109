// hb200_matmul_f32_noalloc: matmul for callers that must not allocate device memory.
//
// Who needs it.  Some hosts hand every byte of device memory to another owner before inference starts
// (a serving process that pre-sizes its KV cache, a framework with a caching allocator set to take the
// whole card), so a cudaMalloc inside a matmul call can fail there; and cudaMalloc / cudaFree synchronise
// the whole device, which a latency-bound decode loop with work in flight on other streams cannot afford.
// Those callers keep their own input and output buffers and want the library to bring its own scratch.
//
// What it does.  The regular device entry point (hb200_matmul_f32_dev) quantizes the f32 input into the Q8_0
// planes of an hb200_act object, which was cudaMalloc'ed.  Here the planes live in one fixed array in the
// library's own device image; every GPU that loads the library carries that array until the process exits.
// The size is modest and fixed: at most HB200_NOALLOC_MAX_TOKENS tokens of at most HB200_NOALLOC_MAX_COLS
// columns (4 x 32768: 128 KiB of int8 values plus 2 x 16 KiB of block scales and sums).
#include "../../include/hb200.h"
#include "objects.h"

using namespace hb200;

namespace {

constexpr size_t MAX_TOKENS = HB200_NOALLOC_MAX_TOKENS;
constexpr size_t MAX_COLS = HB200_NOALLOC_MAX_COLS;
constexpr size_t Q_BYTES = MAX_TOKENS * MAX_COLS;                   // int8 plane
constexpr size_t B_BYTES = MAX_TOKENS * (MAX_COLS / 32) * sizeof(float);  // one f32 plane of block values
constexpr size_t SCRATCH_BYTES = Q_BYTES + 2 * B_BYTES;

// The scratch itself.  In host code this name is only a stand-in for the symbol; the address a kernel can
// use comes from cudaGetSymbolAddress below, once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
unsigned char* g_scratch_ptr[MAX_DEVICES] = {};

// Looks up (first call on a device: resolves) the device address of the scratch on the device the library is bound
// to.  The weights, the SM count and the scratch must all belong to that one device, so a calling thread whose
// current device is another one is refused rather than paired with the wrong GPU's array.  The table below is
// filled without a lock: two host threads making the FIRST call on a device at the same moment both resolve the
// same address, which is harmless, but the library as a whole expects calls to be serialised per context anyway.
int scratch_for_bound_device(unsigned char** out) {
    int dev = -1;
    HB_CUDA(cudaGetDevice(&dev));
    if (dev != bound_device()) {
        set_error("the calling thread's current device is %d but the library is bound to device %d; "
                  "call cudaSetDevice(%d) on this thread first", dev, bound_device(), bound_device());
        return HB200_ERR_BAD_SHAPE;
    }
    if (dev < 0 || dev >= MAX_DEVICES) {
        set_error("device ordinal %d outside 0..%d", dev, MAX_DEVICES - 1);
        return HB200_ERR_TOO_LARGE;
    }
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        HB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        if (!p) {
            set_error("cudaGetSymbolAddress returned a null scratch address");
            return HB200_ERR_CUDA;
        }
        g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_scratch_ptr[dev];
    return 0;
}

}  // namespace

extern "C" int hb200_matmul_f32_noalloc(hb200_weight_t w, const float* x_dev, size_t seq_len, float* out_dev,
                                        size_t ld_out, void* stream) {
    try {
        if (hb200_sm_count() <= 0) {
            set_error("hb200_init has not succeeded in this process");
            return HB200_ERR_NOT_INITIALIZED;
        }
        if (!w) { set_error("null weight handle"); return HB200_ERR_NULL; }
        {
            const int rc = use_slot_of(w->slot);  // the weight's device slot becomes the current one
            if (rc) return rc;
        }
        if (seq_len == 0 || w->n_rows == 0) return HB200_OK;
        const int sms = hb200_sm_count();
        if (!x_dev || !out_dev) { set_error("null input or output"); return HB200_ERR_NULL; }
        if (ld_out < w->n_rows) { set_error("ld_out %zu is smaller than n_rows %zu", ld_out, w->n_rows); return HB200_ERR_BAD_SHAPE; }
        if (seq_len > MAX_TOKENS || w->n_cols > MAX_COLS) {
            set_error("hb200_matmul_f32_noalloc handles at most %zu tokens of %zu columns (got %zu x %zu); "
                      "use hb200_matmul_f32_dev for larger inputs",
                      MAX_TOKENS, MAX_COLS, seq_len, w->n_cols);
            return HB200_ERR_TOO_LARGE;
        }
        cudaStream_t st = (cudaStream_t)stream;
        if (w->kind == KIND_Q4K || w->kind == KIND_Q6K)  // f32-activation formats need no scratch at all
            return launch_kquant_gemv(w->kind, w->kq, w->d16, (int)w->n_rows, (int)w->n_cols, w->nb, w->n_panels, x_dev, (int)seq_len,
                                      out_dev, (int)ld_out, sms, st);

        unsigned char* base = nullptr;
        int rc = scratch_for_bound_device(&base);
        if (rc) return rc;
        // Planes carved from the fixed array: [int8 values][block scales][block sums], row pitch from this call's width.
        hb200_act view;
        view.max_seq = seq_len;
        view.n_cols = w->n_cols;
        view.ld_q = (int)((w->n_cols + ACT_PAD - 1) / ACT_PAD * ACT_PAD);
        view.ld_b = view.ld_q / 32;
        view.q = reinterpret_cast<int8_t*>(base);
        view.d = reinterpret_cast<float*>(base + Q_BYTES);
        view.sums = reinterpret_cast<float*>(base + Q_BYTES + B_BYTES);
        // The quantizer writes every byte of [0, ld_q) and every block value of [0, ld_b) of each token it is
        // given, zeros where a column is padding, so nothing the dot kernel reads is left over from an earlier call.
        rc = launch_quantize_q8_0(x_dev, (int)seq_len, (int)w->n_cols, view.q, view.d, view.sums, view.ld_q, view.ld_b,
                                  nullptr, 0, st);
        if (rc) return rc;
        DotOp op;
        op.bits = w->bits;
        op.scales = w->scales;
        op.aq = view.q;
        op.ad = view.d;
        op.asum = view.sums;
        op.out = out_dev;
        op.iout = nullptr;
        op.n_rows = (int)w->n_rows;
        op.nb = w->nb;
        op.n_sub = w->n_sub;
        op.ld_out = (int)ld_out;
        op.ld_q = view.ld_q;
        op.ld_b = view.ld_b;
        int grid = sms * gemv_dp4a_ctas_per_sm(w->kind, (int)seq_len);
        if (grid > w->n_panels) grid = w->n_panels;
        return launch_gemv_dp4a(w->kind, (int)seq_len, false, nullptr, grid, w->n_panels, &op, st);
    } catch (...) {
        set_error("unexpected C++ exception");
        return HB200_ERR_CUDA;
    }
}
