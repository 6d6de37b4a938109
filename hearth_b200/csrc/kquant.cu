// Q4_K / Q6_K x f32 matvec (Hearth's own linear K-quant layouts).
//
// Replaces the per-row rayon loops over dot_q4_k_f32
// (hearth-quant/src/q4_k.rs:51-96; hearth-llm/src/model/matmul.rs:270-280) and
// dot_q6_k_f32 (hearth-quant/src/qk_quant.rs:141-176; matmul.rs:333-343).  The
// activation is f32; there is no integer dot on this path in the reference.
//
// fp32 order reproduced: values are dequantised with separately rounded
// multiply / subtract, eight lanes accumulate by fused multiply-add (lane j
// takes elements 8i+j), the lanes are reduced as ((l0+l4)+(l2+l6))+((l1+l5)+(l3+l7)),
// and the row sum adds one reduced term per 32 elements (Q4_K) or per 8
// elements (Q6_K), in order.  The lane-reduction order belongs to the `wide`
// crate, whose source is not part of the reference tree; it is an assumption
// shared with the CPU checker, so this path's parity is tolerance-level.
//
// Shape of the kernel: a CTA owns RT rows of one token; all threads produce
// the per-unit terms into shared memory, then one thread per row adds them in
// order.  Weights stream from HBM once per token (Q4_K 144 B, Q6_K 210 B per
// 256 columns); x is read through L1/L2.
#include "common.cuh"

namespace hb200 {

namespace {

constexpr int KQ_THREADS = 256;

__device__ __forceinline__ float h2f_bytes(const uint8_t* p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}
__device__ __forceinline__ float reduce8(const float* l) {
    const float q0 = __fadd_rn(l[0], l[4]), q1 = __fadd_rn(l[1], l[5]);
    const float q2 = __fadd_rn(l[2], l[6]), q3 = __fadd_rn(l[3], l[7]);
    return __fadd_rn(__fadd_rn(q0, q2), __fadd_rn(q1, q3));
}

// One 32-element sub-block of Q4_K: [f16 d][f16 dmin][12 B scales][128 B nibbles].
__device__ __forceinline__ float term_q4k(const uint8_t* __restrict__ row, const float* __restrict__ x, int unit) {
    const int b = unit >> 3, sb = unit & 7;
    const uint8_t* bp = row + (size_t)b * 144;
    const float d = h2f_bytes(bp), dmin = h2f_bytes(bp + 2);
    const int i = sb >> 1;
    const uint32_t s0 = bp[4 + 3 * i], s1 = bp[5 + 3 * i], s2 = bp[6 + 3 * i];
    uint32_t sc, mn;
    if ((sb & 1) == 0) {
        sc = s0 & 0x3F;
        mn = (s0 >> 6) | ((s1 & 0x0F) << 2);
    } else {
        sc = (s1 >> 4) | ((s2 & 0x03) << 4);
        mn = (s2 >> 2) & 0x3F;
    }
    const float scf = __fmul_rn((float)sc, d), mnf = __fmul_rn((float)mn, dmin);
    const uint4 qv = *reinterpret_cast<const uint4*>(bp + 16 + sb * 16);  // 144-byte blocks keep this 16-byte aligned
    const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
    const float* xv = x + (size_t)b * 256 + sb * 32;
    float lanes[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int t = 0; t < 4; t++) {  // elements 8t..8t+7 live in word t: byte k holds elements 2k (low) and 2k+1 (high)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t nib = (qw[t] >> (4 * j)) & 0xF;
            const float v = __fsub_rn(__fmul_rn((float)nib, scf), mnf);
            lanes[j] = fmaf(v, xv[8 * t + j], lanes[j]);
        }
    }
    return reduce8(lanes);
}

// Eight elements of Q6_K: [ql 128][qh 64][i8 scales 16][f16 d]; blocks are 210 B, so byte loads.
__device__ __forceinline__ float term_q6k(const uint8_t* __restrict__ row, const float* __restrict__ x, int unit) {
    const int b = unit >> 5, e0 = (unit & 31) * 8;
    const uint8_t* bp = row + (size_t)b * 210;
    const float d = h2f_bytes(bp + 208);
    const float sd = __fmul_rn((float)(int8_t)bp[192 + (e0 >> 4)], d);
    const float* xv = x + (size_t)b * 256 + e0;
    float lanes[8];
    const uint32_t qh2 = bp[128 + (e0 >> 2)] | ((uint32_t)bp[129 + (e0 >> 2)] << 8);  // 8 x 2 bits
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint32_t ql = bp[(e0 + j) >> 1];
        const uint32_t low4 = (j & 1) ? (ql >> 4) : (ql & 0x0F);
        const uint32_t high2 = (qh2 >> (2 * j)) & 3;
        const int quant = (int)(low4 | (high2 << 4)) - 32;
        const float q = __fmul_rn((float)quant, sd);
        lanes[j] = fmaf(q, xv[j], 0.0f);
    }
    return reduce8(lanes);
}

template <int KIND, int RT>
__global__ void __launch_bounds__(KQ_THREADS) kquant_gemv_kernel(const uint8_t* __restrict__ w, size_t row_bytes,
                                                                 int n_rows, int n_cols, const float* __restrict__ x,
                                                                 float* __restrict__ out, int ld_out) {
    extern __shared__ float terms[];  // RT rows x (units + 1)
    const int units = (n_cols / 256) * (KIND == KIND_Q4K ? 8 : 32);
    const int stride = units + 1;
    const int r0 = blockIdx.x * RT, m = blockIdx.y;
    const float* xr = x + (size_t)m * n_cols;
    for (int u = threadIdx.x; u < RT * units; u += KQ_THREADS) {
        const int row = u / units, unit = u - row * units;
        const int grow = r0 + row;
        if (grow < n_rows) {
            const uint8_t* rp = w + (size_t)grow * row_bytes;
            terms[row * stride + unit] = (KIND == KIND_Q4K) ? term_q4k(rp, xr, unit) : term_q6k(rp, xr, unit);
        }
    }
    __syncthreads();
    if (threadIdx.x < RT && r0 + threadIdx.x < n_rows) {
        const float* t = terms + threadIdx.x * stride;
        float sum = 0.0f;
        for (int i = 0; i < units; i++) sum = __fadd_rn(sum, t[i]);
        out[(size_t)m * ld_out + r0 + threadIdx.x] = sum;
    }
}

constexpr int RT_Q4K = 8, RT_Q6K = 4;
constexpr int KQ_MAX_SMEM = 200 * 1024;

}  // namespace

int kquant_prepare() {
    HB_CUDA(cudaFuncSetAttribute(kquant_gemv_kernel<KIND_Q4K, RT_Q4K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 KQ_MAX_SMEM));
    HB_CUDA(cudaFuncSetAttribute(kquant_gemv_kernel<KIND_Q6K, RT_Q6K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 KQ_MAX_SMEM));
    return 0;
}

int launch_kquant_gemv(int kind, const uint8_t* w, size_t row_bytes, int n_rows, int n_cols, const float* x, int seq_len, float* out,
                       int ld_out, cudaStream_t st) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    const int blocks = n_cols / 256;
    if (kind == KIND_Q4K) {
        const size_t smem = (size_t)RT_Q4K * (blocks * 8 + 1) * sizeof(float);
        if (smem > (size_t)KQ_MAX_SMEM) { set_error("Q4_K row of %d columns exceeds the shared-memory tile", n_cols); return -8; }
        dim3 grid((n_rows + RT_Q4K - 1) / RT_Q4K, seq_len);
        kquant_gemv_kernel<KIND_Q4K, RT_Q4K><<<grid, KQ_THREADS, smem, st>>>(w, row_bytes, n_rows, n_cols, x, out, ld_out);
    } else if (kind == KIND_Q6K) {
        const size_t smem = (size_t)RT_Q6K * (blocks * 32 + 1) * sizeof(float);
        if (smem > (size_t)KQ_MAX_SMEM) { set_error("Q6_K row of %d columns exceeds the shared-memory tile", n_cols); return -8; }
        dim3 grid((n_rows + RT_Q6K - 1) / RT_Q6K, seq_len);
        kquant_gemv_kernel<KIND_Q6K, RT_Q6K><<<grid, KQ_THREADS, smem, st>>>(w, row_bytes, n_rows, n_cols, x, out, ld_out);
    } else {
        set_error("kquant_gemv: kind %d", kind);
        return -7;
    }
    HB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace hb200
