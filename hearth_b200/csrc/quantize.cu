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
#include "quantize_core.cuh"

namespace hb200 {

namespace {

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

HB_BOUNDS_FETCH(bounds_fetch_quantize)

}  // namespace hb200
