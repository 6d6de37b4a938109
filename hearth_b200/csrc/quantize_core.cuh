// Device-side core of the Q8_0 activation quantizer, shared by the plain
// quantizer and by the fused producers (norm, gated activation, rotation).
//
// Arithmetic follows q8_0::quantize_into (hearth-quant/src/q8_0.rs:20-51) and
// must stay bit-exact with it: max |x| by strict '>' from 0 (NaN never wins),
// scale = max==0 ? 1 : max/127 as an IEEE divide, stored scale = RNE f16 of
// it, q = clamp(roundf(x / scale), -128, 127) with the divide by the unrounded
// f32 scale, round half away from zero, NaN -> 0.  Never compile a file that
// includes this header with fast-math.
#pragma once
#include "common.cuh"

namespace hb200 {

__device__ __forceinline__ int quant_one(float x, float scale) {
    float r = roundf(__fdiv_rn(x, scale));
    if (r != r) return 0;
    r = fminf(fmaxf(r, -128.0f), 127.0f);
    return (int)r;
}

// The same integer as quant_one(x, scale), without the IEEE division for all but about one element in four thousand.
// t = x * inv with inv = 1/scale to within one ulp (rcp.approx) lies within 2^-14 of r = RN(x / scale) for every
// |x| <= 127.0001 * scale: |t - x/scale| <= |x/scale| (2^-23 + 2^-24) < 2^-15.3 and |r - x/scale| <= 2^-18.  So when t is
// at least 2^-13 away from every k + 0.5 the two are on the same side of every rounding boundary, there is no tie, and
// round-half-away(r) = nearest integer to t; the clamp to [-128, 127] cannot act (|r| < 127.5).  Otherwise (t near a
// boundary, or NaN) the exact sequence runs.  `fast` is false for blocks whose scale is not a comfortably normal
// number (zero, subnormal, huge, infinite, NaN): those take the exact sequence for every element.
__device__ __forceinline__ int quant_fast(float x, float scale, float inv, bool fast) {
    const float t = __fmul_rn(x, inv);
    const float y = fabsf(t) - 0.5f;
    const float dist = fabsf(y - rintf(y));  // distance of |t| from the nearest k + 0.5
    if (fast && dist >= 0.0001220703125f) return __float2int_rn(t);
    return quant_one(x, scale);
}
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Columns c0..c0+3 of a row of n_cols floats; columns past the end read as 0.
__device__ __forceinline__ void load4(const float* __restrict__ xr, int n_cols, int c0, bool vec_ok, float v[4]) {
    v[0] = v[1] = v[2] = v[3] = 0.f;
    if (vec_ok && c0 + 3 < n_cols) {
        float4 f = *reinterpret_cast<const float4*>(xr + c0);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (c0 + i < n_cols) v[i] = xr[c0 + i];
    }
}

__device__ __forceinline__ bool row_vec_ok(const float* base, int ld) {
    return ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(base) & 15) == 0);
}

// One thread's share of the Q8_0 block arithmetic: values v[0..3] of columns c0..c0+3 of token m; eight
// consecutive threads share one 32-column block (all 32 lanes of the warp must call this together: it shuffles).
template <bool RAW_OUT>
__device__ __forceinline__ void quantize_vals(const float v[4], int n_cols, int m, int c0, int8_t* __restrict__ q,
                                              float* __restrict__ d, float* __restrict__ sums, int ld_q, int ld_b,
                                              uint8_t* __restrict__ raw, size_t raw_stride) {
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
    const bool fast = scale >= 1e-30f && scale <= 1e30f;
    const float inv = rcp_approx(scale);
    int qi[4];
#pragma unroll
    for (int i = 0; i < 4; i++) qi[i] = (c0 + i < n_cols) ? quant_fast(v[i], scale, inv, fast) : 0;
    const uint32_t word = (uint32_t)(qi[0] & 0xff) | ((uint32_t)(qi[1] & 0xff) << 8) | ((uint32_t)(qi[2] & 0xff) << 16) |
                          ((uint32_t)(qi[3] & 0xff) << 24);
    int s = qi[0] + qi[1] + qi[2] + qi[3];
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);

    const int blk = c0 >> 5;
    const bool live = (blk * 32) < n_cols;  // block holds at least one real column
    if (HB_IDX(c0 + 3, ld_q, 22)) *reinterpret_cast<uint32_t*>(q + (size_t)m * ld_q + c0) = live ? word : 0u;
    if ((threadIdx.x & 7) == 0 && HB_IDX(blk, ld_b, 23)) {
        d[(size_t)m * ld_b + blk] = live ? __half2float(h) : 0.0f;
        sums[(size_t)m * ld_b + blk] = live ? (float)s : 0.0f;
    }
    if (RAW_OUT && live && HB_IDX((size_t)blk * 34 + 33, raw_stride, 24)) {
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

template <bool RAW_OUT>
__device__ __forceinline__ void quantize_thread(const float* __restrict__ x, int n_cols, int m, int c0, int8_t* __restrict__ q,
                                                float* __restrict__ d, float* __restrict__ sums, int ld_q, int ld_b,
                                                uint8_t* __restrict__ raw, size_t raw_stride) {
    float v[4];
    load4(x + (size_t)m * n_cols, n_cols, c0, row_vec_ok(x, n_cols), v);
    quantize_vals<RAW_OUT>(v, n_cols, m, c0, q, d, sums, ld_q, ld_b, raw, raw_stride);
}

}  // namespace hb200
