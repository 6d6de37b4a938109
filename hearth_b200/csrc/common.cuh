// Shared definitions for the sm_100a kernels and the C-ABI host layer.
//
// Device data layouts (all chosen once at upload; the resident byte count
// equals the reference's packed byte count up to row / column padding):
//
//  Weights, Q1_0 / Q2_0 / Q8_0 ("panel" layout).
//    A row group (rg) is RPG consecutive rows whose codes share one byte per
//    column: Q1_0 RPG=8 (bit r of the byte = sign bit of row 8*rg+r),
//    Q2_0 RPG=4 (bits 2r..2r+1 = code of row 4*rg+r), Q8_0 RPG=1 (the int8).
//    A tile is one row group x one 128-column block = 128 bytes = 32 words.
//    Word position q = t*8 + s*2 + e (t 0..3, s 0..3, e 0..1) holds columns
//    s*32 + (2t+e)*4 .. +3 of the block, one column per byte.  This order
//    puts, for every 32-column sub-block s, words {2t, 2t+1} in the 16-byte
//    pieces 2t and 2t+1, which is what one thread of an m16n8k32 MMA quad
//    needs, and is as good as any other order for the dp4a kernel.
//    A panel is 32 row groups.  Address of 16-byte piece p (0..7) of tile
//    (panel, blk) for lane l:  bits[((panel*nb + blk)*8 + p)*32 + l]  (uint4),
//    so a warp reads 512 contiguous bytes per piece and a panel is contiguous.
//    Scales are f16, per tile: Q1_0 8 (one per row) as uint4, Q2_0 4 as uint2,
//    Q8_0 4 (one per 32-column sub-block) as uint2, at [(panel*nb + blk)*32 + l].
//
//  Activations, Q8_0 ("planes").  Per token: int8 values q[ld_q] (ld_q = n_cols
//    rounded up to 1024, padding zero), block scales d[ld_b] (ld_b = ld_q/32; the
//    stored f16 widened to f32) and block sums sum[ld_b] (sum of the 32 int8 as f32).
//
//  Weights, Q4_K / Q6_K: re-tiled at upload into 32-row panels of interleaved 16-byte pieces (layout in kquant.cu).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hb200 {

enum Kind : int { KIND_Q1 = 0, KIND_Q2 = 1, KIND_Q8 = 2, KIND_Q4K = 3, KIND_Q6K = 4, KIND_NONE = -1 };

__host__ __device__ constexpr int rows_per_group(int kind) { return kind == KIND_Q1 ? 8 : (kind == KIND_Q2 ? 4 : 1); }
__host__ __device__ constexpr int scales_per_tile(int kind) { return kind == KIND_Q1 ? 8 : 4; }

constexpr int ACT_PAD = 1024;  // activation planes are padded to this many columns

// One dot-rows operation: every row of one weight against M consecutive tokens.
struct DotOp {
    const uint4* bits;     // panel layout
    const void* scales;    // uint4 (Q1_0) or uint2 (Q2_0, Q8_0) per (tile, lane)
    const int8_t* aq;      // first token's int8 plane
    const float* ad;       // first token's scale plane
    const float* asum;     // first token's sum plane
    float* out;            // out[m*ld_out + row], m relative to the first token
    int32_t* iout;         // optional: iout[(m*n_rows + row)*n_sub + sub]
    int n_rows;
    int nb;                // 128-column blocks per row used by the dot
    int n_sub;             // 32-column sub-blocks that carry data (Q8_0: n_cols/32)
    int ld_out;
    int ld_q;              // bytes between tokens in aq
    int ld_b;              // floats between tokens in ad / asum
};

// Peer buffers of a row-sharded launch.  Every rank owns one buffer of identical layout: a 512-byte control block
// (int flags[8] at byte 0: flags[r] = last epoch rank r finished writing here; int counter at byte 256) followed by
// one or two output areas.  A kernel stores each output value at the same offset in every rank's output area (plain
// peer stores).  One batch launch is one epoch, whatever the number of kernels it takes: only the launch's last kernel
// has `publish` set, and its last CTA writes `epoch` into every rank's flags[me] and, if `wait` is set, waits with a
// bound until all ranks have published theirs here.  With two areas, launch number e writes area (e - 1) & 1
// (`area_off` floats beyond the area-0 address), so a rank that is one launch ahead never overwrites what a slower
// rank's consumer is still reading.
constexpr int MAX_PEERS = 8;
constexpr int PEER_CTRL_BYTES = 512;
struct PeerTable {
    float* data[MAX_PEERS];  // output areas (area 0); data[me] is local
    long long area_off;      // floats added to every store address of this launch
    int n;                   // ranks (0 or 1: not sharded, plain local stores)
    int me;
    int epoch;
    int wait;
    int publish;             // this kernel closes the launch: flag exchange after its last CTA
    int* status;             // device word for an expired wait
};

// A 16-byte read of weight data that a launch uses once: no line is kept in L1 for it (measured on the decode matvec:
// 1.5 to 3 % faster than the allocating read-only load).
__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// One work item of a batched launch: panel `y` of op `x`.
typedef int2 DotItem;

// Error plumbing shared by the .cu files.
void set_error(const char* fmt, ...);
// Ordinal of the device hb200_init bound this process to; -1 before it succeeded.
int bound_device();
// Makes device slot `slot` (and its CUDA device) current; an error code if that slot is not initialised.
int use_slot_of(int slot);
#define HB_CUDA(expr)                                                                        \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess) {                                                             \
            hb200::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return -6; /* HB200_ERR_CUDA */                                                  \
        }                                                                                    \
    } while (0)

// ---- bounds-checked debug build (-DHB200_BOUNDS: libhearth_b200_bounds.so) ------------------------------------------
// In that build every global-memory index the streaming kernels compute (decode matvec, K-quant matvec, quantizer
// core and the producers built on it) is compared with the extent its buffer has by the op's own dimensions before
// the access is made.  A violation is counted, the first one's site number kept, and the access skipped, so nothing
// faults; hb200_check_status then returns an error naming the site.  The tensor-core kernels read global memory through
// TMA tensor maps, which the hardware bounds-checks.  In the normal build HB_IDX is the constant true.
#ifdef HB200_BOUNDS
struct BoundsWord { int site, count; };
static __device__ BoundsWord t_bounds_word;  // one per translation unit
__device__ __forceinline__ bool hb_idx_ok(bool ok, int site) {
    if (!ok) {
        atomicCAS(&t_bounds_word.site, 0, site);
        atomicAdd(&t_bounds_word.count, 1);
    }
    return ok;
}
#define HB_IDX(idx, extent, site) hb200::hb_idx_ok((unsigned long long)(idx) < (unsigned long long)(extent), (site))
// Host side of a translation unit: fetch and clear its word.
#define HB_BOUNDS_FETCH(fn)                                                                        \
    int fn(int* site, int* count) {                                                                \
        BoundsWord h = {0, 0};                                                                     \
        HB_CUDA(cudaMemcpyFromSymbol(&h, t_bounds_word, sizeof(h)));                                \
        if (h.count) {                                                                             \
            const BoundsWord z = {0, 0};                                                           \
            HB_CUDA(cudaMemcpyToSymbol(t_bounds_word, &z, sizeof(z)));                              \
        }                                                                                          \
        *site = h.site;                                                                            \
        *count = h.count;                                                                          \
        return 0;                                                                                  \
    }
#else
#define HB_IDX(idx, extent, site) (true)
#define HB_BOUNDS_FETCH(fn) \
    int fn(int* site, int* count) { *site = 0; *count = 0; return 0; }
#endif
int bounds_fetch_dp4a(int* site, int* count);      // sites 1..9
int bounds_fetch_kquant(int* site, int* count);    // sites 11..19
int bounds_fetch_quantize(int* site, int* count);  // sites 21..24 (quantize.cu)
int bounds_fetch_producers(int* site, int* count); // sites 21..24 (producers.cu)

// ---- launchers implemented in the kernel translation units ----------------

// One activation of a list quantization: f32 rows at x -> the Q8_0 planes q / d / sums.
struct QuantDesc {
    const float* x;
    int8_t* q;
    float* d;
    float* sums;
    int n_cols, seq_len, ld_q, ld_b;
};

// quantize.cu
int launch_quantize_q8_0_list(const QuantDesc* descs_dev, int n_acts, int max_chunks, int max_seq, cudaStream_t st);
int launch_quantize_q8_0(const float* x, int seq_len, int n_cols, int8_t* q, float* d, float* sums, int ld_q, int ld_b,
                         uint8_t* raw_out, size_t raw_stride, cudaStream_t st);
int launch_load_q8_0(const uint8_t* raw, size_t raw_stride, int seq_len, int n_cols, int8_t* q, float* d, float* sums,
                     int ld_q, int ld_b, cudaStream_t st);
int launch_store_q8_0(const int8_t* q, const float* d, int ld_q, int ld_b, int seq_len, int n_cols, uint8_t* raw,
                      size_t raw_stride, cudaStream_t st);

// producers.cu: f32 rows -> Q8_0 planes with the producing arithmetic fused in (norm, gated activation, rotation).
constexpr int RMS_NORM_MAX_COLS = 32768;  // one row is staged in shared memory
int producers_prepare();
int launch_rms_norm_q8(const float* x, const float* weight, float eps, int seq_len, int n_cols, int8_t* q, float* d, float* sums,
                       int ld_q, int ld_b, uint8_t* raw_out, size_t raw_stride, cudaStream_t st);
int launch_silu_mul_q8(const float* gate, const float* up, int seq_len, int ld_x, int n_cols, int8_t* q, float* d, float* sums,
                       int ld_q, int ld_b, uint8_t* raw_out, size_t raw_stride, cudaStream_t st);
// block_size: a power of two up to 1024.  `rotated` (may be null) also receives the rotated f32 rows.
int launch_hadamard_quantize(const float* x, const float* signs, int block_size, int seq_len, int n_cols, float* rotated,
                             int8_t* q, float* d, float* sums, int ld_q, int ld_b, uint8_t* raw_out, size_t raw_stride,
                             cudaStream_t st);

// repack.cu
int launch_repack(int kind, const uint8_t* raw, size_t row_bytes, int n_rows, int n_cols, int nb, int n_panels,
                  uint4* bits, void* scales, cudaStream_t st);

// PTQ1_0 rows (28 B per 128 columns) -> Q2_0 rows (34 B per 128), the same weights in 2-bit codes.
int launch_ptq1_to_q2(const uint8_t* raw, size_t row_bytes_in, int n_rows, int nb, uint8_t* out, size_t row_bytes_out,
                      cudaStream_t st);

// gemv_dp4a.cu
constexpr int GEMV_MAX_M = 4;  // tokens one dp4a launch handles per op
// Either an op list in device memory (ops_dev / items_dev, with chunks_dev[grid + 1] giving each CTA its contiguous,
// cost-balanced run of items; items of one op must be consecutive panels), or, with ops_dev == nullptr, the one op
// `single` (host memory, passed by value to the grid) whose n_items panels are split evenly over `grid` CTAs.
// `peers` (may be null) turns the output stores into stores to every rank's buffer plus the closing flag exchange.

int gemv_dp4a_ctas_per_sm(int kind, int m);  // resident CTAs per SM the kernel of this kind for m tokens is built for
// List launches of the decode matvec: per CTA a run of segments (consecutive whole panels of one op, or rounds
// [r0, r1) of ONE panel).  A panel cut between two CTAs is summed in order across them: the first part's CTA writes
// its running sums to carry slot `carry_out`, the second part's CTA starts from slot `carry_in` (flags bit 0: starts
// from a carry, bit 1: ends in a carry).  For whole panels r0 = 0 and r1 = rounds of the op.
struct FlatSeg {
    int op, p0, cnt, r0, r1, flags, carry_in, carry_out;
};
constexpr int FLAT_CARRY_FLOATS = GEMV_MAX_M * 256;  // one slot: running sums of a panel (up to 256 rows) for up to 4 tokens
struct FlatRec {  // what a CTA needs to start a segment, in one 112-byte record (copied ahead into shared memory)
    FlatSeg seg;
    DotOp op;
};
struct FlatLaunch {
    const FlatRec* recs;   // null: not a list launch
    const int* seg_begin;  // [grid + 1]
    float* carry;          // [slots][FLAT_CARRY_FLOATS]
    int* cflags;           // [slots]: warps that have written the slot so far (eight per launch)
    unsigned epoch;        // launches of this work list so far, this one included
    int* status;           // device word for an expired wait (may be null)
};
// `list` (a planned work list, n_items = its number of segments) or, when list is null, the one op `single` whose
// n_items panels are split evenly over the grid.
int launch_gemv_dp4a(int kind, int m, bool int_out, const FlatLaunch* list, int grid, int n_items, const DotOp* single,
                     cudaStream_t st, const PeerTable* peers = nullptr);
// The flag exchange alone (one thread): closes a peer launch of a rank whose shard is empty, so that every rank
// publishes every epoch.
int launch_peer_publish(const PeerTable& peers, cudaStream_t st);
int gemv_dp4a_prepare();  // sets the dynamic shared-memory attributes once

// gemm_tc.cu: tcgen05 kind::i8 path for prefill-sized token counts (Q1_0 / Q2_0), see gemm_tc_wanted.  `amap` points at a CUtensorMap over the
// activation's int8 plane ([max_seq][ld_q] bytes, box 128 x 128, SWIZZLE_128B).  `status` is a device word that
// receives a non-zero code if a bounded wait inside the kernel expires.
// Below these token counts, passes of the streaming dp4a kernel (four tokens each) are faster than 128-token
// tensor-core tiles that are mostly empty.  Measured on B200 on the 27B layer set: a tensor-core pass costs what six
// dp4a passes of Q2_0 cost (24 tokens), or four of Q1_0, whose dp4a kernel is slower.  (With the few-token kernel
// below taking everything up to 64 tokens, these two limits only matter where that kernel is not available.)
constexpr int GEMM_TC_MIN_TOKENS_Q2 = 25;
constexpr int GEMM_TC_MIN_TOKENS_Q1 = 17;
constexpr int GEMM_TC_MIN_TOKENS = GEMM_TC_MIN_TOKENS_Q1;  // no tensor-core launch below this, whatever the kind
inline bool gemm_tc_wanted(int kind, size_t seq_len) {
    return (kind == KIND_Q1 && seq_len >= (size_t)GEMM_TC_MIN_TOKENS_Q1) || (kind == KIND_Q2 && seq_len >= (size_t)GEMM_TC_MIN_TOKENS_Q2);
}
// One matrix of a tensor-core launch.  amap: a CUtensorMap in device memory.  Tiles (128 tokens x 64 rows) of the
// matrices of a launch are numbered consecutively, tile_begin .. tile_end - 1 belonging to this one.
struct TcMat {
    const uint4* bits;
    const void* scales;
    const float* ad;
    float* out;
    const void* amap;
    int n_rows, nb, seq_len, ld_out, ld_b;
    int tok_tiles, tile_begin, tile_end;
};
int gemm_tc_tiles(int n_rows, int seq_len);
void gemm_tc_fill(TcMat& m, const void* amap_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                  int nb, int seq_len, float* out, int ld_out, int tile_begin);
// One matrix: persistent CTAs (at most sm_count) take its tiles in turn.
int launch_gemm_tc(int kind, const void* amap_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                   int nb, int seq_len, float* out, int ld_out, int sm_count, int* status, cudaStream_t st);
// Many matrices of one kind in one launch: mats_dev[...] in device memory, chunks_dev[grid + 1] gives CTA c the tiles
// chunks[c] .. chunks[c+1]-1.
int launch_gemm_tc_list(int kind, const TcMat* mats_dev, const int* chunks_dev, int n_tiles, int grid, int* status, cudaStream_t st);
int gemm_tc_prepare();

// gemm_tc_rows.cu: the same arithmetic with the weight rows on the MMA's M side (tiles of 128 rows x 32 tokens), for
// token counts between the streaming kernel's and the prefill kernel's.  `amap32` points at a CUtensorMap over the
// activation's int8 plane with a box of 32 rows x 128 bytes.  Same TcMat, same status word.
constexpr int GEMM_TCR_TOK_TILE = 32;
constexpr int GEMM_TCR_ROW_TILE = 128;
// Measured on B200 on whole layer sets in one launch (8B Q1_0: two streaming passes, eight tokens, 1.45 ms against
// 1.90 ms here; 27B PQ2_0: 4.7 ms against 5.7 ms): up to two full passes of the streaming kernel and a partial one are
// cheaper than one pass of this kernel, whose time hardly depends on the token count; from 65 tokens on the
// 128-token tiles of the prefill kernel are ahead.
constexpr int GEMM_TCR_MIN_TOKENS_Q1 = 11;
constexpr int GEMM_TCR_MIN_TOKENS_Q2 = 12;
constexpr int GEMM_TCR_MAX_TOKENS = 64;
inline bool gemm_tcr_wanted(int kind, size_t seq_len) {
    return seq_len <= (size_t)GEMM_TCR_MAX_TOKENS &&
           ((kind == KIND_Q1 && seq_len >= (size_t)GEMM_TCR_MIN_TOKENS_Q1) || (kind == KIND_Q2 && seq_len >= (size_t)GEMM_TCR_MIN_TOKENS_Q2));
}
int gemm_tcr_tiles(int n_rows, int seq_len);
void gemm_tcr_fill(TcMat& m, const void* amap32_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                   int nb, int seq_len, float* out, int ld_out, int tile_begin);
int launch_gemm_tcr(int kind, const void* amap32_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                    int nb, int seq_len, float* out, int ld_out, int sm_count, int* status, cudaStream_t st);
int launch_gemm_tcr_list(int kind, const TcMat* mats_dev, const int* chunks_dev, int n_tiles, int grid, int* status, cudaStream_t st);
int gemm_tcr_prepare();

// argmax.cu: lowest index of the largest value (the reference's greedy-sampling reduction).  `scratch` is
// argmax_scratch_bytes() of zero-initialised device memory owned by the caller, reused by every call on one stream.
constexpr int ARGMAX_CHUNK = 2048;
constexpr int ARGMAX_MAX_CHUNKS = 1 << 15;  // up to 64 Mi values
size_t argmax_scratch_bytes();
int launch_argmax(const float* x, size_t n, void* scratch, uint32_t* out_dev, cudaStream_t st);

// f32act.cu: the shaders' f32-activation matmul on the panel layout (Q1_0 / Q2_0 kinds).  accumulate: out += result.
int launch_f32act(int kind, const uint4* bits, const void* scales, int n_rows, int n_cols, int nb, int n_panels, const float* x,
                  int seq_len, float* out, int ld_out, bool accumulate, cudaStream_t st);

// The same result in two kernels, for launches that would leave most SMs idle: per-block terms into `terms`
// (f32act_terms_bytes() of device memory), then the ordered sums.
size_t f32act_terms_bytes(int kind, int nb, int n_panels, int seq_len);
int launch_f32act_two_phase(int kind, const uint4* bits, const void* scales, int n_rows, int n_cols, int nb, int n_panels,
                            const float* x, int seq_len, float* out, int ld_out, bool accumulate, float* terms, cudaStream_t st);

// tc_peak.cu: dense kind::i8 tensor-core rate of this GPU, measured (TOP/s).
int measure_i8_peak(int sm_count, int* status, cudaStream_t st, double* tops);

// kquant.cu: Q4_K / Q6_K weights are re-tiled at upload into 32-row panels of interleaved 16-byte pieces
// (layout described in kquant.cu); d16 holds Q6_K's per-block f16 scale and is null for Q4_K.
size_t kquant_pieces_per_block(int kind);
int launch_kquant_repack(int kind, const uint8_t* raw, size_t row_bytes, int n_rows, int nblk, int n_panels, uint4* kq,
                         unsigned short* d16, cudaStream_t st);
// One matrix of a K-quant launch; items item_begin .. item_end - 1 of the launch belong to it
// (item = panel * token tiles + token tile).
struct KqMat {
    const uint4* kq;
    const unsigned short* d16;  // Q6_K only
    const float* x;             // [seq_len][n_cols]
    float* out;
    int n_rows, n_cols, nblk, n_panels, seq_len, ld_out;
    int item_begin, item_end;
};
int launch_kquant_gemv(int kind, const uint4* kq, const unsigned short* d16, int n_rows, int n_cols, int nblk, int n_panels,
                       const float* x, int seq_len, float* out, int ld_out, int sm_count, cudaStream_t st, int* status = nullptr);
// Many matrices of one kind and one tokens-per-pass class (1, 2, 4, 8; Q4_K also 16) in one launch.  `status`: device word that the
// eight-token Q4_K kernel sets (code 40) if its bounded wait for a bulk copy of x expires; may be null.
int kquant_tokens_per_pass(int kind, int seq_len);
int kquant_items(int kind, int n_panels, int seq_len);
int kquant_rounds(int kind, int nblk);
int kquant_grid(int kind, int mt, int sm_count, int n_items);
int launch_kquant_gemv_list(int kind, int mt, const KqMat* mats_dev, const int* chunks_dev, int n_items, int grid, cudaStream_t st,
                            int* status = nullptr);
int kquant_prepare();

}  // namespace hb200
