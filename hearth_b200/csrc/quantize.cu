// Q8_0 activation quantizer and the converters between the reference's Q8_0
// byte layout and the device planes.
//
// Arithmetic follows q8_0::quantize_into (hearth-quant/src/q8_0.rs:20-51) and
// must stay bit-exact with it: max |x| by strict '>' from 0 (NaN never wins),
// scale = max==0 ? 1 : max/127 as an IEEE divide, stored scale = RNE f16 of
// it, q = clamp(roundf(x / scale), -128, 127) with the divide by the unrounded
// f32 scale, round half away from zero, NaN -> 0.  Never compile this file
// with fast-math.
//
// HBM-bound: reads 4 B and writes ~1.06 B (+1.06 B for the byte-layout copy)
// per element; one CTA handles 1024 columns of one token, four per thread.
#include "common.cuh"

namespace hb200 {

namespace {

__device__ __forceinline__ int quant_one(float x, float scale) {
    float r = roundf(__fdiv_rn(x, scale));
    if (r != r) return 0;
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    return (int)r;
}

// One thread's share of the quantizer: columns c0..c0+3 of token m; eight consecutive threads share one
// 32-column block (all 32 lanes of the warp must call this together: it shuffles).
template <bool RAW_OUT>
__device__ __forceinline__ void quantize_thread(const float* __restrict__ x, int n_cols, int m, int c0, int8_t* __restrict__ q,
                                                float* __restrict__ d, float* __restrict__ sums, int ld_q, int ld_b,
                                                uint8_t* __restrict__ raw, size_t raw_stride) {
    const float* xr = x + (size_t)m * n_cols;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const bool vec_ok = ((n_cols & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (vec_ok && c0 + 3 < n_cols) {
        float4 f = *reinterpret_cast<const float4*>(xr + c0);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (c0 + i < n_cols) v[i] = xr[c0 + i];
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float a = fabsf(v[i]);
        if (a > amax) amax = a;  // NaN compares false, as in the reference
    }
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) {
        float o = __shfl_xor_sync(0xffffffffu, amax, off);
        if (o > amax) amax = o;
    }
    const float scale = (amax == 0.0f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const __half h = __float2half_rn(scale);
    int qi[4];
#pragma unroll
    for (int i = 0; i < 4; i++) qi[i] = (c0 + i < n_cols) ? quant_one(v[i], scale) : 0;
    const uint32_t word = (uint32_t)(qi[0] & 0xff) | ((uint32_t)(qi[1] & 0xff) << 8) | ((uint32_t)(qi[2] & 0xff) << 16) |
                          ((uint32_t)(qi[3] & 0xff) << 24);
    int s = qi[0] + qi[1] + qi[2] + qi[3];
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);

    const int blk = c0 >> 5;
    const bool live = (blk * 32) < n_cols;  // block holds at least one real column
    *reinterpret_cast<uint32_t*>(q + (size_t)m * ld_q + c0) = live ? word : 0u;
    if ((threadIdx.x & 7) == 0) {
        d[(size_t)m * ld_b + blk] = live ? __half2float(h) : 0.0f;
        sums[(size_t)m * ld_b + blk] = live ? (float)s : 0.0f;
    }
    if (RAW_OUT && live) {
        uint8_t* rb = raw + (size_t)m * raw_stride + (size_t)blk * 34;
        if ((threadIdx.x & 7) == 0) {
            const unsigned short hb = __half_as_ushort(h);
            rb[0] = (uint8_t)(hb & 0xff);
            rb[1] = (uint8_t)(hb >> 8);
        }
        const int i0 = (threadIdx.x & 7) * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) rb[2 + i0 + i] = (uint8_t)(qi[i] & 0xff);
    }
}

// grid (ld_q/1024, seq_len), block 256.
template <bool RAW_OUT>
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float* __restrict__ x, int n_cols,
                                                            int8_t* __restrict__ q, float* __restrict__ d,
                                                            float* __restrict__ sums, int ld_q, int ld_b,
                                                            uint8_t* __restrict__ raw, size_t raw_stride) {
    quantize_thread<RAW_OUT>(x, n_cols, blockIdx.y, blockIdx.x * 1024 + threadIdx.x * 4, q, d, sums, ld_q, ld_b, raw, raw_stride);
}

// Many activations in one launch: grid (max chunks, max seq_len, n_acts); CTAs outside an activation's extent exit.
__global__ void __launch_bounds__(256) quantize_q8_0_list_kernel(const QuantDesc* __restrict__ descs) {
    const QuantDesc qd = descs[blockIdx.z];
    if ((int)blockIdx.y >= qd.seq_len || (int)blockIdx.x * 1024 >= qd.ld_q) return;
    quantize_thread<false>(qd.x, qd.n_cols, blockIdx.y, blockIdx.x * 1024 + threadIdx.x * 4, qd.q, qd.d, qd.sums, qd.ld_q, qd.ld_b,
                           nullptr, 0);
}

// Reference byte layout -> planes.  Same grid shape as the quantizer.
__global__ void __launch_bounds__(256) load_q8_0_kernel(const uint8_t* __restrict__ raw, size_t raw_stride, int n_cols,
                                                        int8_t* __restrict__ q, float* __restrict__ d,
                                                        float* __restrict__ sums, int ld_q, int ld_b) {
    const int m = blockIdx.y;
    const int c0 = blockIdx.x * 1024 + threadIdx.x * 4;
    const int blk = c0 >> 5;
    const bool live = (blk * 32) < n_cols;  // a row carries ceil(n_cols/32) blocks
    uint32_t word = 0;
    float dv = 0.0f;
    int s = 0;
    if (live) {
        const uint8_t* rb = raw + (size_t)m * raw_stride + (size_t)blk * 34;
        const int i0 = (threadIdx.x & 7) * 4;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t b = rb[2 + i0 + i];
            word |= b << (8 * i);
            s += (int)(int8_t)b;
        }
        dv = __half2float(__ushort_as_half((unsigned short)(rb[0] | (rb[1] << 8))));
    }
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    *reinterpret_cast<uint32_t*>(q + (size_t)m * ld_q + c0) = word;
    if ((threadIdx.x & 7) == 0) {
        d[(size_t)m * ld_b + blk] = dv;
        sums[(size_t)m * ld_b + blk] = (float)s;
    }
}

// Planes -> reference byte layout (every block that has a real column).
__global__ void __launch_bounds__(256) store_q8_0_kernel(const int8_t* __restrict__ q, const float* __restrict__ d,
                                                         int ld_q, int ld_b, int n_cols, uint8_t* __restrict__ raw,
                                                         size_t raw_stride) {
    const int m = blockIdx.y;
    const int c0 = blockIdx.x * 1024 + threadIdx.x * 4;
    const int blk = c0 >> 5;
    if (blk * 32 >= n_cols) return;
    uint8_t* rb = raw + (size_t)m * raw_stride + (size_t)blk * 34;
    const uint32_t word = *reinterpret_cast<const uint32_t*>(q + (size_t)m * ld_q + c0);
    const uint32_t hbits = __half_as_ushort(__float2half_rn(d[(size_t)m * ld_b + blk]));
    if ((threadIdx.x & 7) == 0) {
        rb[0] = (uint8_t)(hbits & 0xffu);
        rb[1] = (uint8_t)((hbits >> 8) & 0xffu);
    }
    uint8_t* vals = rb + 2 + (threadIdx.x & 7) * 4;
    vals[0] = (uint8_t)(word & 0xffu);
    vals[1] = (uint8_t)((word >> 8) & 0xffu);
    vals[2] = (uint8_t)((word >> 16) & 0xffu);
    vals[3] = (uint8_t)(word >> 24);
}

}  // namespace

int launch_quantize_q8_0(const float* x, int seq_len, int n_cols, int8_t* q, float* d, float* sums, int ld_q, int ld_b,
                         uint8_t* raw_out, size_t raw_stride, cudaStream_t st) {
    if (seq_len <= 0) return 0;
    dim3 grid(ld_q / 1024, seq_len);
    if (raw_out)
        quantize_q8_0_kernel<true><<<grid, 256, 0, st>>>(x, n_cols, q, d, sums, ld_q, ld_b, raw_out, raw_stride);
    else
        quantize_q8_0_kernel<false><<<grid, 256, 0, st>>>(x, n_cols, q, d, sums, ld_q, ld_b, nullptr, 0);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_quantize_q8_0_list(const QuantDesc* descs_dev, int n_acts, int max_chunks, int max_seq, cudaStream_t st) {
    if (n_acts <= 0 || max_chunks <= 0 || max_seq <= 0) return 0;
    dim3 grid(max_chunks, max_seq, n_acts);
    quantize_q8_0_list_kernel<<<grid, 256, 0, st>>>(descs_dev);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_load_q8_0(const uint8_t* raw, size_t raw_stride, int seq_len, int n_cols, int8_t* q, float* d, float* sums,
                     int ld_q, int ld_b, cudaStream_t st) {
    if (seq_len <= 0) return 0;
    dim3 grid(ld_q / 1024, seq_len);
    load_q8_0_kernel<<<grid, 256, 0, st>>>(raw, raw_stride, n_cols, q, d, sums, ld_q, ld_b);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_store_q8_0(const int8_t* q, const float* d, int ld_q, int ld_b, int seq_len, int n_cols, uint8_t* raw,
                      size_t raw_stride, cudaStream_t st) {
    if (seq_len <= 0) return 0;
    dim3 grid(ld_q / 1024, seq_len);
    store_q8_0_kernel<<<grid, 256, 0, st>>>(q, d, ld_q, ld_b, n_cols, raw, raw_stride);
    HB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace hb200
