// Fused producers of Q8_0 activation rows: the three places where the reference
// computes an f32 row and quantizes it in the same pass, so that the f32 row
// never goes back to memory between the two steps.
//
//   rms_norm_q8        ops::rms_norm_q8 / rms_norm_q8_batch (hearth-llm/src/ops.rs:442-504)
//   silu_mul_q8        ops::silu_mul_q8                      (hearth-llm/src/ops.rs:273-306)
//   hadamard_quantize  hadamard_rotate + quantize_q8_0       (hearth-llm/src/model/qwen35.rs:49-87, :924-943)
//
// All three end in the shared Q8_0 block arithmetic (quantize_core.cuh) and
// write the device planes, optionally also the reference's 34-byte blocks.
// HBM-bound: 4 B (norm, rotation) or 8 B (gated activation) read per element,
// ~1.06 B written.
//
// Exactness.  The norm and the rotation use only IEEE add / multiply / fma /
// divide / sqrt in the reference's order, so they are bit-exact with it (the
// norm's eight-lane reduction order is the one assumed for `wide`'s
// reduce_add).  The gated activation calls exp, which the reference takes from
// `wide`'s polynomial; this file uses CUDA's expf, so its values can differ in
// the last bits and a quantized value can move by one step at a rounding
// boundary.  Never compile this file with fast-math.
#include "common.cuh"
#include "quantize_core.cuh"

namespace hb200 {

namespace {

// ------------------------------------------------------------------ rms norm --
// One CTA per token.  The row is staged in shared memory; lanes 0..7 of warp 0
// run the eight fused-multiply-add chains (lane j takes elements 8i + j in
// order of i, a serial dependency the reference's f32x8 accumulator has too).
template <bool RAW_OUT>
__global__ void __launch_bounds__(256) rms_norm_q8_kernel(const float* __restrict__ x, const float* __restrict__ weight, float eps,
                                                          int n_cols, int8_t* __restrict__ q, float* __restrict__ d,
                                                          float* __restrict__ sums, int ld_q, int ld_b,
                                                          uint8_t* __restrict__ raw, size_t raw_stride) {
    extern __shared__ float row[];
    __shared__ float s_inv;
    const int m = blockIdx.x;
    const float* xr = x + (size_t)m * n_cols;
    const bool vec_ok = row_vec_ok(x, n_cols);
    for (int c0 = threadIdx.x * 4; c0 < n_cols; c0 += 1024) {
        float v[4];
        load4(xr, n_cols, c0, vec_ok, v);
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (c0 + i < n_cols) row[c0 + i] = v[i];
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int j = threadIdx.x & 7;
        const int chunks = n_cols >> 3;
        float acc = 0.0f;
        int i = 0;
        for (; i + 8 <= chunks; i += 8) {
            float t[8];
#pragma unroll
            for (int u = 0; u < 8; u++) t[u] = row[(i + u) * 8 + j];
#pragma unroll
            for (int u = 0; u < 8; u++) acc = fmaf(t[u], t[u], acc);
        }
        for (; i < chunks; i++) {
            const float t = row[i * 8 + j];
            acc = fmaf(t, t, acc);
        }
        // ((l0+l4)+(l2+l6)) + ((l1+l5)+(l3+l7))
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
        if (threadIdx.x == 0) {
            float sum_sq = __fadd_rn(0.0f, acc);
            for (int k = chunks * 8; k < n_cols; k++) sum_sq = __fadd_rn(sum_sq, __fmul_rn(row[k], row[k]));
            const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)n_cols), eps));
            s_inv = __fdiv_rn(1.0f, rms);
        }
    }
    __syncthreads();
    const float inv = s_inv;
    const bool wvec = row_vec_ok(weight, n_cols);
    for (int c0 = threadIdx.x * 4; c0 < ld_q; c0 += 1024) {
        float w[4], v[4];
        load4(weight, n_cols, c0, wvec, w);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float xv = (c0 + i < n_cols) ? row[c0 + i] : 0.0f;
            v[i] = __fmul_rn(__fmul_rn(w[i], xv), inv);
        }
        quantize_vals<RAW_OUT>(v, n_cols, m, c0, q, d, sums, ld_q, ld_b, raw, raw_stride);
    }
}

// -------------------------------------------------------------- silu * up --
// grid (ld_q/1024, seq_len), block 256.  Rows of gate / up are ld_x floats apart; only the n_cols = 32 * (dim / 32)
// columns of whole blocks are produced, as in the reference.
template <bool RAW_OUT>
__global__ void __launch_bounds__(256) silu_mul_q8_kernel(const float* __restrict__ gate, const float* __restrict__ up, int ld_x,
                                                          int n_cols, int8_t* __restrict__ q, float* __restrict__ d,
                                                          float* __restrict__ sums, int ld_q, int ld_b,
                                                          uint8_t* __restrict__ raw, size_t raw_stride) {
    const int m = blockIdx.y;
    const int c0 = blockIdx.x * 1024 + threadIdx.x * 4;
    float g[4], u[4], v[4];
    load4(gate + (size_t)m * ld_x, n_cols, c0, row_vec_ok(gate, ld_x), g);
    load4(up + (size_t)m * ld_x, n_cols, c0, row_vec_ok(up, ld_x), u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float s = __fdiv_rn(g[i], __fadd_rn(1.0f, expf(-g[i])));
        v[i] = __fmul_rn(s, u[i]);
    }
    quantize_vals<RAW_OUT>(v, n_cols, m, c0, q, d, sums, ld_q, ld_b, raw, raw_stride);
}

// ------------------------------------------------- sign, Walsh-Hadamard, quantize --
// grid (ld_q/1024, seq_len), block 256, four consecutive columns per thread.  block_size is a power of two that
// divides 1024, so a rotation block never leaves the CTA: stages h = 1, 2 run inside the thread, h = 4..64 by
// warp shuffle, h = 128..512 through shared memory.  Each stage is the reference's butterfly: the element without
// bit h becomes a + b, the one with it a - b, with a the lower element.  A tail shorter than block_size is not
// rotated (chunks_exact_mut), only sign-multiplied.
template <bool RAW_OUT>
__global__ void __launch_bounds__(256) hadamard_quantize_kernel(const float* x, const float* __restrict__ signs,
                                                                int n_cols, int block_size, float* rotated,
                                                                int8_t* __restrict__ q, float* __restrict__ d,
                                                                float* __restrict__ sums, int ld_q, int ld_b,
                                                                uint8_t* __restrict__ raw, size_t raw_stride) {
    __shared__ float4 xchg[256];
    const int m = blockIdx.y;
    const int c0 = blockIdx.x * 1024 + threadIdx.x * 4;
    float v[4];
    load4(x + (size_t)m * n_cols, n_cols, c0, row_vec_ok(x, n_cols), v);
    if (signs) {
        float sg[4];
        load4(signs, n_cols, c0, row_vec_ok(signs, n_cols), sg);
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = __fmul_rn(v[i], sg[i]);
    }
    const float s = __fdiv_rn(1.0f, __fsqrt_rn((float)block_size));
    float w[4] = {v[0], v[1], v[2], v[3]};
    if (block_size >= 2) {
        float a = w[0], b = w[1];
        w[0] = __fadd_rn(a, b); w[1] = __fsub_rn(a, b);
        a = w[2]; b = w[3];
        w[2] = __fadd_rn(a, b); w[3] = __fsub_rn(a, b);
    }
    if (block_size >= 4) {
        float a = w[0], b = w[2];
        w[0] = __fadd_rn(a, b); w[2] = __fsub_rn(a, b);
        a = w[1]; b = w[3];
        w[1] = __fadd_rn(a, b); w[3] = __fsub_rn(a, b);
    }
    const int quads = block_size >> 2;  // threads per rotation block
    for (int h4 = 1; h4 < quads && h4 < 32; h4 <<= 1) {
        const bool upper = (threadIdx.x & h4) != 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float o = __shfl_xor_sync(0xffffffffu, w[i], h4);
            w[i] = upper ? __fsub_rn(o, w[i]) : __fadd_rn(w[i], o);
        }
    }
    for (int h4 = 32; h4 < quads; h4 <<= 1) {  // uniform over the CTA
        xchg[threadIdx.x] = make_float4(w[0], w[1], w[2], w[3]);
        __syncthreads();
        const float4 o = xchg[threadIdx.x ^ h4];
        __syncthreads();
        if (threadIdx.x & h4) {
            w[0] = __fsub_rn(o.x, w[0]); w[1] = __fsub_rn(o.y, w[1]); w[2] = __fsub_rn(o.z, w[2]); w[3] = __fsub_rn(o.w, w[3]);
        } else {
            w[0] = __fadd_rn(w[0], o.x); w[1] = __fadd_rn(w[1], o.y); w[2] = __fadd_rn(w[2], o.z); w[3] = __fadd_rn(w[3], o.w);
        }
    }
    if (block_size >= 4) {
        const bool whole = (c0 / block_size + 1) * block_size <= n_cols;
        if (whole) {
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = __fmul_rn(w[i], s);
        }
    } else if (block_size == 2) {
        if (c0 + 2 <= n_cols) { v[0] = __fmul_rn(w[0], s); v[1] = __fmul_rn(w[1], s); }
        if (c0 + 4 <= n_cols) { v[2] = __fmul_rn(w[2], s); v[3] = __fmul_rn(w[3], s); }
    } else if (block_size == 1) {
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = __fmul_rn(v[i], s);  // n = 1: no stage, s = 1
    }
    if (rotated) {
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (c0 + i < n_cols) rotated[(size_t)m * n_cols + c0 + i] = v[i];
    }
    quantize_vals<RAW_OUT>(v, n_cols, m, c0, q, d, sums, ld_q, ld_b, raw, raw_stride);
}

}  // namespace

int producers_prepare() {
    HB_CUDA(cudaFuncSetAttribute(rms_norm_q8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, RMS_NORM_MAX_COLS * 4));
    HB_CUDA(cudaFuncSetAttribute(rms_norm_q8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, RMS_NORM_MAX_COLS * 4));
    return 0;
}

int launch_rms_norm_q8(const float* x, const float* weight, float eps, int seq_len, int n_cols, int8_t* q, float* d, float* sums,
                       int ld_q, int ld_b, uint8_t* raw_out, size_t raw_stride, cudaStream_t st) {
    if (seq_len <= 0) return 0;
    const size_t smem = (size_t)n_cols * sizeof(float);
    if (raw_out)
        rms_norm_q8_kernel<true><<<seq_len, 256, smem, st>>>(x, weight, eps, n_cols, q, d, sums, ld_q, ld_b, raw_out, raw_stride);
    else
        rms_norm_q8_kernel<false><<<seq_len, 256, smem, st>>>(x, weight, eps, n_cols, q, d, sums, ld_q, ld_b, nullptr, 0);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_silu_mul_q8(const float* gate, const float* up, int seq_len, int ld_x, int n_cols, int8_t* q, float* d, float* sums,
                       int ld_q, int ld_b, uint8_t* raw_out, size_t raw_stride, cudaStream_t st) {
    if (seq_len <= 0) return 0;
    dim3 grid(ld_q / 1024, seq_len);
    if (raw_out)
        silu_mul_q8_kernel<true><<<grid, 256, 0, st>>>(gate, up, ld_x, n_cols, q, d, sums, ld_q, ld_b, raw_out, raw_stride);
    else
        silu_mul_q8_kernel<false><<<grid, 256, 0, st>>>(gate, up, ld_x, n_cols, q, d, sums, ld_q, ld_b, nullptr, 0);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_hadamard_quantize(const float* x, const float* signs, int block_size, int seq_len, int n_cols, float* rotated,
                             int8_t* q, float* d, float* sums, int ld_q, int ld_b, uint8_t* raw_out, size_t raw_stride,
                             cudaStream_t st) {
    if (seq_len <= 0) return 0;
    dim3 grid(ld_q / 1024, seq_len);
    if (raw_out)
        hadamard_quantize_kernel<true><<<grid, 256, 0, st>>>(x, signs, n_cols, block_size, rotated, q, d, sums, ld_q, ld_b, raw_out,
                                                            raw_stride);
    else
        hadamard_quantize_kernel<false><<<grid, 256, 0, st>>>(x, signs, n_cols, block_size, rotated, q, d, sums, ld_q, ld_b, nullptr,
                                                             0);
    HB_CUDA(cudaGetLastError());
    return 0;
}

HB_BOUNDS_FETCH(bounds_fetch_producers)

}  // namespace hb200
