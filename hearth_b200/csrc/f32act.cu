// f32-activation matmul: the arithmetic of the reference's GPU shaders, for callers that keep activations in f32
// and expect exactly what GpuCompute::dequant_matmul_fused / _batch / _fused_add_inplace and the fused gate|up and
// q|k|v shaders return (hearth-compute/src/lib.rs:483-507, :1123-1173, :1237-1420;
// hearth-compute/src/shaders/q1_0_matmul.wgsl:38-97, q2_0_matmul.wgsl:48-106 and their _batch, _add_inplace and
// fused_* siblings, which repeat the same arithmetic).
//
// Per weight row and 128-column block the shader forms partial[i] = w_i * x_i with one invocation per column, reduces
// the 128 partials by a tree (partial[i] += partial[i + offset], offset = 64, 32, .. 1) and adds
// partial[0] * w_scale to the row sum, product and sum rounded separately.  The f16 scale is widened by the shader's
// own bit formula, which has no case for zero, subnormals, infinity or NaN.
//
// Here one lane owns one row group (8 rows of Q1_0, 4 of Q2_0, sharing a byte per column in the device layout) and
// evaluates the same tree depth-first for all its rows at once, so every activation value is read from shared memory
// once per row group and no partial ever leaves registers.  A warp takes one 128-column block per round, eight warps
// 1024 columns; the per-block terms go through shared memory to one thread per row, which adds them in block order.
// Instruction-bound by design of the arithmetic: about three instructions per weight (sign or code to float, multiply
// or sign flip, tree add).
#include "common.cuh"

namespace hb200 {

namespace {

constexpr int FA_THREADS = 256;
constexpr int FA_WARPS = 8;

__device__ __forceinline__ float shader_h2f(uint32_t h) {
    return __uint_as_float(((h >> 15) << 31) | ((((h >> 10) & 0x1Fu) + 112u) << 23) | ((h & 0x3FFu) << 13));
}

// Column c of a 128-column tile lives in word word_of(c) of the lane's 32 words, byte c & 3.
__host__ __device__ constexpr int word_of(int c) { return (((c & 31) >> 2) >> 1) * 8 + (c >> 5) * 2 + (((c & 31) >> 2) & 1); }

template <int KIND>
struct Leaf {
    static constexpr int RPG = rows_per_group(KIND);
    // products w * x of column C for the RPG rows of this lane
    template <int C>
    static __device__ __forceinline__ void eval(const uint32_t (&w)[32], const float* __restrict__ xs, float (&out)[RPG]) {
        const float x = xs[C];
        const uint32_t word = w[word_of(C)];
        constexpr int b = C & 3;
#pragma unroll
        for (int r = 0; r < RPG; r++) {
            if (KIND == KIND_Q1) {
                // bit 1 -> +1, bit 0 -> -1: flip the sign of x where the bit is clear (the product with +-1 is exact)
                const uint32_t t = word << (31 - (8 * b + r));
                out[r] = __uint_as_float(__float_as_uint(x) ^ (~t & 0x80000000u));
            } else {
                // code - 1 in {-1, 0, 1, 2} as a float: 0x4B400000 | code is 12582912 + code
                const uint32_t code = (word >> (8 * b + 2 * r)) & 3u;
                const float wf = __fadd_rn(__uint_as_float(0x4B400000u | code), -12582913.0f);
                out[r] = __fmul_rn(wf, x);
            }
        }
    }
};

// node(O, I) of the reduction tree: the value partial[I] holds after the step with offset O.
template <int KIND, int O, int I>
struct Node {
    static constexpr int RPG = rows_per_group(KIND);
    static __device__ __forceinline__ void eval(const uint32_t (&w)[32], const float* __restrict__ xs, float (&out)[RPG]) {
        float a[RPG], b[RPG];
        Node<KIND, O * 2, I>::eval(w, xs, a);
        Node<KIND, O * 2, I + O>::eval(w, xs, b);
#pragma unroll
        for (int r = 0; r < RPG; r++) out[r] = __fadd_rn(a[r], b[r]);
    }
};
template <int KIND, int I>
struct Node<KIND, 128, I> {
    static constexpr int RPG = rows_per_group(KIND);
    static __device__ __forceinline__ void eval(const uint32_t (&w)[32], const float* __restrict__ xs, float (&out)[RPG]) {
        Leaf<KIND>::template eval<I>(w, xs, out);
    }
};

struct FaArgs {
    const uint4* bits;
    const void* scales;
    const float* x;  // [seq_len][n_cols]
    float* out;
    int n_rows, n_cols, nb, n_panels, seq_len, ld_out, accumulate;
};

template <int KIND>
struct FaSmem {
    static constexpr int RPG = rows_per_group(KIND);
    alignas(16) float x[2][FA_WARPS * 128];
    float term[2][FA_WARPS][32 * RPG];
};

// grid (n_panels, seq_len), block 256.
template <int KIND>
__global__ void __launch_bounds__(FA_THREADS) f32act_kernel(const __grid_constant__ FaArgs a) {
    constexpr int RPG = rows_per_group(KIND);
    constexpr int SPT = scales_per_tile(KIND);
    __shared__ FaSmem<KIND> sm;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int panel = blockIdx.x, tok = blockIdx.y;
    const int nb = a.nb;
    const int rounds = (nb + FA_WARPS - 1) / FA_WARPS;
    const float* xr = a.x + (size_t)tok * a.n_cols;
    const bool vec_ok = ((a.n_cols & 3) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);

    auto stage = [&](int r, int buf) {  // 1024 columns of x, zero past the last whole block
        const int c = r * FA_WARPS * 128 + tid * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c + 3 < nb * 128) {
            if (vec_ok) v = *reinterpret_cast<const float4*>(xr + c);
            else v = make_float4(xr[c], xr[c + 1], xr[c + 2], xr[c + 3]);
        }
        *reinterpret_cast<float4*>(&sm.x[buf][tid * 4]) = v;
    };

    // rows of this panel: row = panel * 32 * RPG + lane * RPG + r; one thread per row owns its running sum
    constexpr int ROWS = 32 * RPG;
    float run = 0.0f;
    auto replay = [&](int r, int buf) {
        for (int row = tid; row < ROWS; row += FA_THREADS) {  // ROWS is 256 (Q1_0) or 128 (Q2_0): one pass
            float acc = run;
            const int nvalid = min(FA_WARPS, nb - r * FA_WARPS);
            for (int k = 0; k < nvalid; k++) acc = __fadd_rn(acc, sm.term[buf][k][row]);
            run = acc;
        }
    };

    stage(0, 0);
    for (int r = 0; r < rounds; r++) {
        __syncthreads();  // x of this round staged; terms of the previous round written
        if (r + 1 < rounds) stage(r + 1, (r + 1) & 1);
        if (r > 0) replay(r - 1, (r - 1) & 1);
        const int blk = r * FA_WARPS + warp;
        if (blk < nb) {
            const size_t tile = (size_t)panel * nb + blk;
            uint32_t w[32];
#pragma unroll
            for (int p = 0; p < 8; p++) {
                const uint4 v = __ldg(a.bits + (tile * 8 + p) * 32 + lane);
                w[4 * p] = v.x; w[4 * p + 1] = v.y; w[4 * p + 2] = v.z; w[4 * p + 3] = v.w;
            }
            float tree[RPG];
            Node<KIND, 1, 0>::eval(w, &sm.x[r & 1][warp * 128], tree);
            uint32_t sc[SPT / 2];
            if (KIND == KIND_Q1) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.scales) + tile * 32 + lane);
                sc[0] = v.x; sc[1] = v.y; sc[2] = v.z; sc[3] = v.w;
            } else {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(a.scales) + tile * 32 + lane);
                sc[0] = v.x; sc[1] = v.y;
            }
#pragma unroll
            for (int rr = 0; rr < RPG; rr++) {
                const float ws = shader_h2f((sc[rr >> 1] >> (16 * (rr & 1))) & 0xffffu);
                sm.term[r & 1][warp][lane * RPG + rr] = __fmul_rn(tree[rr], ws);
            }
        }
    }
    __syncthreads();
    if (rounds > 0) replay(rounds - 1, (rounds - 1) & 1);
    for (int row = tid; row < ROWS; row += FA_THREADS) {
        const int grow = panel * ROWS + row;
        if (grow < a.n_rows) {
            float* o = a.out + (size_t)tok * a.ld_out + grow;
            *o = a.accumulate ? __fadd_rn(*o, run) : run;
        }
    }
}

// Two-phase form for launches with too few (panel, token) pairs to fill the GPU (one decode matvec: 48 panels of a
// 12288-row matrix on 148 SMs).  The per-block terms are independent; only their addition is ordered.  Phase one takes
// one round of eight blocks of one panel per CTA, so the grid grows by the number of rounds, and leaves every term in
// a scratch array; phase two adds each row's terms in block order.  Same terms, same order, same bits.
// terms[((tok * n_panels + panel) * nb + blk) * ROWS + row]
template <int KIND>
__global__ void __launch_bounds__(FA_THREADS) f32act_terms_kernel(const __grid_constant__ FaArgs a, float* __restrict__ terms) {
    constexpr int RPG = rows_per_group(KIND);
    constexpr int SPT = scales_per_tile(KIND);
    constexpr int ROWS = 32 * RPG;
    __shared__ __align__(16) float xs[FA_WARPS * 128];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int panel = blockIdx.x, r = blockIdx.y, tok = blockIdx.z;
    const int nb = a.nb;
    const float* xr = a.x + (size_t)tok * a.n_cols;
    const bool vec_ok = ((a.n_cols & 3) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
    {
        const int c = r * FA_WARPS * 128 + tid * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c + 3 < nb * 128) {
            if (vec_ok) v = *reinterpret_cast<const float4*>(xr + c);
            else v = make_float4(xr[c], xr[c + 1], xr[c + 2], xr[c + 3]);
        }
        *reinterpret_cast<float4*>(&xs[tid * 4]) = v;
    }
    __syncthreads();
    const int blk = r * FA_WARPS + warp;
    if (blk >= nb) return;
    const size_t tile = (size_t)panel * nb + blk;
    uint32_t w[32];
#pragma unroll
    for (int p = 0; p < 8; p++) {
        const uint4 v = __ldg(a.bits + (tile * 8 + p) * 32 + lane);
        w[4 * p] = v.x; w[4 * p + 1] = v.y; w[4 * p + 2] = v.z; w[4 * p + 3] = v.w;
    }
    float tree[RPG];
    Node<KIND, 1, 0>::eval(w, &xs[warp * 128], tree);
    uint32_t sc[SPT / 2];
    if (KIND == KIND_Q1) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(a.scales) + tile * 32 + lane);
        sc[0] = v.x; sc[1] = v.y; sc[2] = v.z; sc[3] = v.w;
    } else {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(a.scales) + tile * 32 + lane);
        sc[0] = v.x; sc[1] = v.y;
    }
    float* dst = terms + (((size_t)tok * a.n_panels + panel) * nb + blk) * ROWS + lane * RPG;
#pragma unroll
    for (int rr = 0; rr < RPG; rr++) dst[rr] = __fmul_rn(tree[rr], shader_h2f((sc[rr >> 1] >> (16 * (rr & 1))) & 0xffffu));
}

// One thread per (token, row): the terms of its row in block order.
template <int KIND>
__global__ void __launch_bounds__(256) f32act_sum_kernel(const __grid_constant__ FaArgs a, const float* __restrict__ terms) {
    constexpr int ROWS = 32 * rows_per_group(KIND);
    const int grow = blockIdx.x * 256 + threadIdx.x, tok = blockIdx.y;
    if (grow >= a.n_rows) return;
    const int panel = grow / ROWS, row = grow % ROWS;
    const float* t = terms + ((size_t)tok * a.n_panels + panel) * a.nb * ROWS + row;
    float acc = 0.0f;
    for (int b = 0; b < a.nb; b++) acc = __fadd_rn(acc, t[(size_t)b * ROWS]);
    float* o = a.out + (size_t)tok * a.ld_out + grow;
    *o = a.accumulate ? __fadd_rn(*o, acc) : acc;
}

}  // namespace

size_t f32act_terms_bytes(int kind, int nb, int n_panels, int seq_len) {
    return (size_t)seq_len * n_panels * nb * 32 * rows_per_group(kind) * sizeof(float);
}

int launch_f32act_two_phase(int kind, const uint4* bits, const void* scales, int n_rows, int n_cols, int nb, int n_panels,
                            const float* x, int seq_len, float* out, int ld_out, bool accumulate, float* terms, cudaStream_t st) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    FaArgs a;
    a.bits = bits; a.scales = scales; a.x = x; a.out = out;
    a.n_rows = n_rows; a.n_cols = n_cols; a.nb = nb; a.n_panels = n_panels; a.seq_len = seq_len; a.ld_out = ld_out;
    a.accumulate = accumulate ? 1 : 0;
    const int rounds = (nb + FA_WARPS - 1) / FA_WARPS;
    if (rounds > 0) {
        const dim3 g1(n_panels, rounds, seq_len);
        if (kind == KIND_Q1) f32act_terms_kernel<KIND_Q1><<<g1, FA_THREADS, 0, st>>>(a, terms);
        else if (kind == KIND_Q2) f32act_terms_kernel<KIND_Q2><<<g1, FA_THREADS, 0, st>>>(a, terms);
        else { set_error("f32-activation matmul: kind %d has no shader counterpart", kind); return -7; }
        HB_CUDA(cudaGetLastError());
    }
    const dim3 g2((n_rows + 255) / 256, seq_len);
    if (kind == KIND_Q1) f32act_sum_kernel<KIND_Q1><<<g2, 256, 0, st>>>(a, terms);
    else f32act_sum_kernel<KIND_Q2><<<g2, 256, 0, st>>>(a, terms);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_f32act(int kind, const uint4* bits, const void* scales, int n_rows, int n_cols, int nb, int n_panels, const float* x,
                  int seq_len, float* out, int ld_out, bool accumulate, cudaStream_t st) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    FaArgs a;
    a.bits = bits; a.scales = scales; a.x = x; a.out = out;
    a.n_rows = n_rows; a.n_cols = n_cols; a.nb = nb; a.n_panels = n_panels; a.seq_len = seq_len; a.ld_out = ld_out;
    a.accumulate = accumulate ? 1 : 0;
    dim3 grid(n_panels, seq_len);
    if (kind == KIND_Q1) f32act_kernel<KIND_Q1><<<grid, FA_THREADS, 0, st>>>(a);
    else if (kind == KIND_Q2) f32act_kernel<KIND_Q2><<<grid, FA_THREADS, 0, st>>>(a);
    else { set_error("f32-activation matmul: kind %d has no shader counterpart", kind); return -7; }
    HB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace hb200
