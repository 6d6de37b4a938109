/*
 * hearth_oracle.c -- CPU restatement of Hearth's scalar quantized matrix-product path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the product (hearth_b200/) may call, link or load it.
 *
 * Every function follows one function of the reference (Eric-Lautanen/hearth,
 * v0.2.0, Rust) and cites it.  The reference cannot be compiled where this
 * oracle is built (no Rust toolchain), so this is a restatement in plain C.
 *
 * Parity status.  Pinned against the reference's own known-answer tests
 * (code -> value mappings, q2_0.rs:738-766, q1_0g128.rs:1206-1220), its
 * deterministic paired-token fixtures (q1_0g128.rs:1504-1552,
 * q2_0.rs:939-986), the Q8_0 round-trip bound (q8_0.rs:177-194) and the
 * Q2_0-vs-f32 bound (q2_0.rs:787-818).  NOT pinned by any reference test, hence
 * "parity unpinned" beyond the restatement itself: exact Q8_0 output bytes, the
 * exact fp32 results of the scalar dots, and everything about Q4_K / Q6_K
 * (whose lane-reduction order lives in the un-vendored `wide` 1.4.0 crate).
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (see Makefile).  No FMA may
 * be formed by the compiler: every fp32 operation below rounds separately,
 * exactly as the Rust source does, except where fmaf() is written out.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define HO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ f16 -- */

/* IEEE binary16 -> binary32, exact (half 2.7.1 `f16::to_f32`). */
HO_API float ho_h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* IEEE binary32 -> binary16, round-to-nearest-even (half 2.7.1 `f16::from_f32`). */
HO_API uint16_t ho_f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFF) { /* inf / nan */
        if (man == 0) return (uint16_t)(sign | 0x7C00u);
        uint32_t m = man >> 13;
        return (uint16_t)(sign | 0x7C00u | m | (m == 0)); /* keep it a NaN */
    }
    int e = (int)exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u); /* overflow -> inf */
    if (e <= 0) {                                   /* subnormal or zero */
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        int shift = 14 - e; /* 14..24 */
        uint32_t half_m = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_m & 1))) half_m++;
        return (uint16_t)(sign | half_m);
    }
    uint32_t half_m = man >> 13;
    uint32_t rem = man & 0x1FFFu;
    uint16_t out = (uint16_t)(sign | ((uint32_t)e << 10) | half_m);
    if (rem > 0x1000u || (rem == 0x1000u && (half_m & 1))) out++; /* may carry into exp: correct */
    return out;
}

static inline float rd_h(const uint8_t *p) { return ho_h2f((uint16_t)(p[0] | (p[1] << 8))); }

/* ------------------------------------------------------- block geometry -- */

/* GGML type ids as the reference parses them (hearth-gguf/src/ggml.rs:49-101). */
enum {
    HO_Q8_0 = 8,
    HO_Q4_K = 12,
    HO_Q6_K = 14,
    HO_Q1_0_G128_LEGACY = 39,
    HO_Q1_0 = 41,
    HO_Q2_0 = 42,
    HO_Q1_0_G128 = 43,
    HO_PQ2_0 = 142,
    HO_PTQ1_0 = 143,
};

/* GgmlDType::block_size (hearth-gguf/src/ggml.rs:105-129); 0 = not on this path. */
HO_API size_t ho_block_size(int dtype) {
    switch (dtype) {
        case HO_Q8_0: return 32;
        case HO_Q4_K: case HO_Q6_K: return 256;
        case HO_Q1_0: case HO_Q1_0_G128: case HO_Q1_0_G128_LEGACY: return 128;
        case HO_Q2_0: case HO_PQ2_0: return 128;
        case HO_PTQ1_0: return 128;
        default: return 0;
    }
}

/* GgmlDType::block_bytes (hearth-gguf/src/ggml.rs:131-171). */
HO_API size_t ho_block_bytes(int dtype) {
    switch (dtype) {
        case HO_Q8_0: return 34;
        case HO_Q4_K: return 144;
        case HO_Q6_K: return 210;
        case HO_Q1_0: case HO_Q1_0_G128: case HO_Q1_0_G128_LEGACY: return 18;
        case HO_Q2_0: case HO_PQ2_0: return 34;
        case HO_PTQ1_0: return 28;
        default: return 0;
    }
}

/* GgmlDType::byte_size (hearth-gguf/src/ggml.rs:173-176): ceil(n/block)*block_bytes. */
HO_API size_t ho_byte_size(int dtype, size_t n) {
    size_t bs = ho_block_size(dtype);
    if (!bs) return 0;
    return ((n + bs - 1) / bs) * ho_block_bytes(dtype);
}

/* ------------------------------------------------- Q8_0 activation quant -- */

/* q8_0::quantize_into (hearth-quant/src/q8_0.rs:20-51).  dst holds
 * ceil(n/32) blocks of [f16 d][32 x i8].  The divide uses the unrounded f32
 * scale; rounding is half-away-from-zero (Rust f32::round == C roundf); the
 * `as i8` cast saturates and maps NaN to 0. */
HO_API void ho_quantize_q8_0_into(const float *src, size_t n, uint8_t *dst) {
    size_t blocks = (n + 31) / 32;
    for (size_t b = 0; b < blocks; b++) {
        size_t start = b * 32;
        float max_abs = 0.0f;
        for (size_t i = 0; i < 32; i++) {
            size_t idx = start + i;
            if (idx < n) {
                float v = fabsf(src[idx]);
                if (v > max_abs) max_abs = v;
            }
        }
        float scale = (max_abs == 0.0f) ? 1.0f : max_abs / 127.0f;
        uint16_t h = ho_f2h(scale);
        size_t off = b * 34;
        dst[off] = (uint8_t)(h & 0xFF);
        dst[off + 1] = (uint8_t)(h >> 8);
        for (size_t i = 0; i < 32; i++) {
            size_t idx = start + i;
            int8_t q = 0;
            if (idx < n) {
                float r = roundf(src[idx] / scale);
                if (r != r) {
                    q = 0; /* NaN as i8 == 0 */
                } else {
                    if (r < -128.0f) r = -128.0f;
                    if (r > 127.0f) r = 127.0f;
                    q = (int8_t)r;
                }
            }
            dst[off + 2 + i] = (uint8_t)q;
        }
    }
}

/* ThreadPool::par_quantize (hearth-llm/src/pool.rs:467-508, worker body
 * :328-343): token s of f32[seq_len x dim] -> q8 + s * ceil(dim/32)*34. */
HO_API void ho_par_quantize(size_t seq_len, size_t dim, const float *f32_base, uint8_t *q8_base) {
    size_t q8_size = ((dim + 31) / 32) * 34;
    for (size_t s = 0; s < seq_len; s++)
        ho_quantize_q8_0_into(f32_base + s * dim, dim, q8_base + s * q8_size);
}

/* q8_0::dequantize (hearth-quant/src/q8_0.rs:4-18). */
HO_API void ho_dequantize_q8_0(const uint8_t *data, size_t bytes, float *out, size_t n_out) {
    size_t blocks = bytes / 34;
    for (size_t b = 0; b < blocks; b++) {
        float scale = rd_h(data + b * 34);
        for (size_t i = 0; i < 32; i++) {
            size_t idx = b * 32 + i;
            if (idx < n_out) out[idx] = scale * (float)(int8_t)data[b * 34 + 2 + i];
        }
    }
}

/* --------------------------------------------------- element decoders ---- */

/* Q1V table entry (q1_0g128.rs:31-45): bit 1 -> +1, bit 0 -> -1, LSB first. */
static inline int q1_sign(const uint8_t *bits, size_t e) { return ((bits[e >> 3] >> (e & 7)) & 1) ? 1 : -1; }

/* Q2V table entry (q2_0.rs:9-23): 2-bit code minus one, LSB first -> {-1,0,1,2}. */
static inline int q2_val(const uint8_t *qs, size_t e) { return (int)((qs[e >> 2] >> (2 * (e & 3))) & 3) - 1; }

/* q1_0g128::dequantize (q1_0g128.rs:76-98): value = sign * scale. */
HO_API void ho_dequantize_q1_0g128(const uint8_t *data, size_t bytes, float *out, size_t n_out) {
    size_t blocks = bytes / 18;
    for (size_t b = 0; b < blocks; b++) {
        float scale = rd_h(data + b * 18);
        for (size_t e = 0; e < 128; e++) {
            size_t idx = b * 128 + e;
            if (idx < n_out) out[idx] = (float)q1_sign(data + b * 18 + 2, e) * scale;
        }
    }
}

/* q2_0::dequantize: value = (code-1) * scale (pinned by q2_0.rs:738-766). */
HO_API void ho_dequantize_q2_0(const uint8_t *data, size_t bytes, float *out, size_t n_out) {
    size_t blocks = bytes / 34;
    for (size_t b = 0; b < blocks; b++) {
        float scale = rd_h(data + b * 34);
        for (size_t e = 0; e < 128; e++) {
            size_t idx = b * 128 + e;
            if (idx < n_out) out[idx] = (float)q2_val(data + b * 34 + 2, e) * scale;
        }
    }
}

/* ------------------------------------------------ PTQ1_0 (dense trits) ---- */

/* Block of 128 weights in 28 bytes: qs[24] with five base-3 digits per byte,
 * qh[2] with four, f16 d at byte 26 (hearth-quant/src/ptq1_0.rs:1-13).
 * Digit n of byte b, already in weight space {-1, 0, +1}: the TRIT_N / QH_TRIT
 * tables (ptq1_0.rs:22-57) are this expression evaluated for every byte. */
static inline int ptq_trit(uint8_t b, int n) {
    static const uint16_t pow3[5] = {1, 3, 9, 27, 81};
    uint8_t prod = (uint8_t)(((uint16_t)b * pow3[n]) & 0xFF);
    return (int)(((uint16_t)prod * 3) >> 8) - 1;
}

/* The 128 weights of one block in element order (the wvals fill of
 * dot_ptq1_0_q8_0_ptr_scalar, ptq1_0.rs:563-585): a 16-byte stage emits
 * elements n*16 + m, an 8-byte stage 80 + n*8 + m, then qh 120 + n*2 + h. */
static void ptq_decode_block(const uint8_t *blk, int8_t wvals[128]) {
    static const size_t stages[3] = {32, 16, 8};
    size_t out_off = 0, j = 0;
    for (int si = 0; si < 3; si++) {
        size_t c = stages[si];
        while (j + c <= 24) {
            for (size_t m = 0; m < c; m++)
                for (int n = 0; n < 5; n++) wvals[out_off + (size_t)n * c + m] = (int8_t)ptq_trit(blk[j + m], n);
            out_off += 5 * c;
            j += c;
        }
    }
    for (int n = 0; n < 4; n++)
        for (int h = 0; h < 2; h++) wvals[out_off + (size_t)n * 2 + (size_t)h] = (int8_t)ptq_trit(blk[24 + h], n);
}

/* ptq1_0::dequantize (ptq1_0.rs:59-105). */
HO_API void ho_dequantize_ptq1_0(const uint8_t *data, size_t bytes, float *out, size_t n_out) {
    size_t blocks = bytes / 28;
    int8_t wv[128];
    for (size_t b = 0; b < blocks; b++) {
        float scale = rd_h(data + b * 28 + 26);
        ptq_decode_block(data + b * 28, wv);
        for (size_t e = 0; e < 128; e++) {
            size_t idx = b * 128 + e;
            if (idx < n_out) out[idx] = (float)wv[e] * scale;
        }
    }
}

/* ptq1_0::quantize (ptq1_0.rs:604-646), the reference's own packer; its
 * tests build their fixtures with it.  n / 128 whole blocks. */
HO_API void ho_quantize_ptq1_0(const float *src, size_t n, uint8_t *dst) {
    static const size_t stages[3] = {32, 16, 8};
    size_t blocks = n / 128;
    for (size_t b = 0; b < blocks; b++) {
        const float *x = src + b * 128;
        uint8_t *block = dst + b * 28;
        float amax = 0.0f;
        for (int i = 0; i < 128; i++) {
            float a = fabsf(x[i]);
            if (a > amax) amax = a; /* f32::max skips NaN */
        }
        float d = amax, id = (d != 0.0f) ? 1.0f / d : 0.0f;
        uint16_t h = ho_f2h(d);
        memset(block, 0, 28);
        block[26] = (uint8_t)(h & 0xFF);
        block[27] = (uint8_t)(h >> 8);
        size_t x_off = 0, j = 0;
        for (int si = 0; si < 3; si++) {
            size_t c = stages[si];
            while (j + c <= 24) {
                for (size_t m = 0; m < c; m++) {
                    uint8_t q = 0;
                    for (size_t k = 0; k < 5; k++) {
                        int xi = (int)roundf(x[x_off + m + k * c] * id) + 1;
                        q = (uint8_t)(q * 3 + (uint8_t)xi);
                    }
                    block[j + m] = (uint8_t)(((uint16_t)q * 256 + 242) / 243);
                }
                x_off += 5 * c;
                j += c;
            }
        }
        for (size_t hh = 0; hh < 2; hh++) {
            uint8_t q = 0;
            for (size_t m = 0; m < 4; m++) {
                int xi = (int)roundf(x[x_off + hh + m * 2] * id) + 1;
                q = (uint8_t)(q * 3 + (uint8_t)xi);
            }
            q = (uint8_t)(q * 3);
            block[24 + hh] = (uint8_t)(((uint16_t)q * 256 + 242) / 243);
        }
    }
}

/* dot_ptq1_0_f32 (ptq1_0.rs:107-142): slot-major accumulation order. */
HO_API float ho_dot_ptq1_0_f32(const uint8_t *w, const float *x, size_t n) {
    static const size_t stages[3] = {32, 16, 8};
    size_t blocks = n / 128;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *blk = w + b * 28;
        float scale = rd_h(blk + 26);
        size_t base = b * 128, out_off = 0, j = 0;
        float acc = 0.0f;
        for (int si = 0; si < 3; si++) {
            size_t c = stages[si];
            while (j + c <= 24) {
                for (int k = 0; k < 5; k++)
                    for (size_t m = 0; m < c; m++) acc += (float)ptq_trit(blk[j + m], k) * x[base + out_off + (size_t)k * c + m];
                out_off += 5 * c;
                j += c;
            }
        }
        for (int k = 0; k < 4; k++)
            for (size_t hh = 0; hh < 2; hh++) acc += (float)ptq_trit(blk[24 + hh], k) * x[base + out_off + (size_t)k * 2 + hh];
        sum += acc * scale;
    }
    return sum;
}

/* ---------------------------------------------- integer sub-block dots --- */

/* The exact int32 dot of one 32-element Q8_0 sub-block against the matching
 * 32 weights.  These are the `dot` variables of q1_0g128.rs:1033-1047 and
 * q2_0.rs:553-568 and `sumi` of q8_0.rs:164-168. */
static inline int32_t isub_q1(const uint8_t *w_bits /*16B*/, int sub, const int8_t *a) {
    int32_t d = 0;
    for (int i = 0; i < 32; i++) d += q1_sign(w_bits, (size_t)(sub * 32 + i)) * (int32_t)a[i];
    return d;
}
static inline int32_t isub_q2(const uint8_t *qs /*32B*/, int sub, const int8_t *a) {
    int32_t d = 0;
    for (int i = 0; i < 32; i++) d += q2_val(qs, (size_t)(sub * 32 + i)) * (int32_t)a[i];
    return d;
}
static inline int32_t isub_q8(const int8_t *w, const int8_t *a) {
    int32_t d = 0;
    for (int i = 0; i < 32; i++) d += (int32_t)w[i] * (int32_t)a[i];
    return d;
}

/* Per-(32-block) integer dots of one weight row against one Q8_0 activation:
 * out[n/32].  dtype selects the weight format. Returns 0, or -1 for a dtype
 * that has no integer path (Q4_K / Q6_K take f32 activations). */
HO_API int ho_block_dots_i32(int dtype, const uint8_t *w, const uint8_t *a, size_t n, int32_t *out) {
    switch (dtype) {
        case HO_Q1_0: case HO_Q1_0_G128: case HO_Q1_0_G128_LEGACY:
            for (size_t b = 0; b < n / 128; b++)
                for (int s = 0; s < 4; s++)
                    out[b * 4 + s] = isub_q1(w + b * 18 + 2, s, (const int8_t *)(a + (b * 4 + s) * 34 + 2));
            return 0;
        case HO_Q2_0: case HO_PQ2_0:
            for (size_t b = 0; b < n / 128; b++)
                for (int s = 0; s < 4; s++)
                    out[b * 4 + s] = isub_q2(w + b * 34 + 2, s, (const int8_t *)(a + (b * 4 + s) * 34 + 2));
            return 0;
        case HO_PTQ1_0: {
            int8_t wv[128];
            for (size_t b = 0; b < n / 128; b++) {
                ptq_decode_block(w + b * 28, wv);
                for (int s = 0; s < 4; s++) out[b * 4 + s] = isub_q8(wv + s * 32, (const int8_t *)(a + (b * 4 + s) * 34 + 2));
            }
            return 0;
        }
        case HO_Q8_0:
            for (size_t b = 0; b < n / 32; b++)
                out[b] = isub_q8((const int8_t *)(w + b * 34 + 2), (const int8_t *)(a + b * 34 + 2));
            return 0;
        default: return -1;
    }
}

/* ------------------------------------------------------- scalar row dots -- */

/* dot_q1_0g128_q8_0_ptr, scalar association (q1_0g128.rs:1019-1052; the SSE4.1
 * arm :794-827 that x86 falls back to has the same integer sums and the same
 * float order).  n/128 blocks, a tail is dropped. */
HO_API float ho_dot_q1_0g128_q8_0(const uint8_t *w, const uint8_t *a, size_t n) {
    size_t blocks = n / 128;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        float w_scale = rd_h(w + b * 18);
        float block_acc = 0.0f;
        for (int sub = 0; sub < 4; sub++) {
            const uint8_t *ab = a + (b * 4 + (size_t)sub) * 34;
            float a_scale = rd_h(ab);
            int32_t dot = isub_q1(w + b * 18 + 2, sub, (const int8_t *)(ab + 2));
            block_acc += (float)dot * a_scale;
        }
        sum += block_acc * w_scale;
    }
    return sum;
}

/* dot_q2_0_q8_0_ptr_scalar (q2_0.rs:537-574); also serves PQ2_0
 * (hearth-quant/src/lib.rs:414, hearth-llm/src/model/matmul.rs:153). */
HO_API float ho_dot_q2_0_q8_0(const uint8_t *w, const uint8_t *a, size_t n) {
    size_t blocks = n / 128;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        float w_scale = rd_h(w + b * 34);
        float block_acc = 0.0f;
        for (int sub = 0; sub < 4; sub++) {
            const uint8_t *ab = a + (b * 4 + (size_t)sub) * 34;
            float a_scale = rd_h(ab);
            int32_t dot = isub_q2(w + b * 34 + 2, sub, (const int8_t *)(ab + 2));
            block_acc += (float)dot * a_scale;
        }
        sum += block_acc * w_scale;
    }
    return sum;
}

/* dot_q8_0_q8_0_ptr (q8_0.rs:154-171): sumf += ((float)sumi * d0) * d1. */
HO_API float ho_dot_q8_0_q8_0(const uint8_t *w, const uint8_t *a, size_t n) {
    size_t blocks = n / 32;
    float sumf = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        float d0 = rd_h(w + b * 34);
        float d1 = rd_h(a + b * 34);
        int32_t sumi = isub_q8((const int8_t *)(w + b * 34 + 2), (const int8_t *)(a + b * 34 + 2));
        sumf += (float)sumi * d0 * d1;
    }
    return sumf;
}

/* dot_q2_0_f32 / dot_q1_0g128 f32-activation forms, used only to re-create the
 * reference's sanity test q2_0.rs:787-818 (Q8_0 path within 1% + 0.5 of it). */
HO_API float ho_dot_q2_0_f32(const uint8_t *w, const float *x, size_t n) {
    size_t blocks = n / 128;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        float scale = rd_h(w + b * 34);
        float acc = 0.0f;
        for (size_t e = 0; e < 128; e++) acc += (float)q2_val(w + b * 34 + 2, e) * x[b * 128 + e];
        sum += acc * scale;
    }
    return sum;
}

/* 8-lane horizontal add in the order of an AVX hadd ladder:
 * ((l0+l4)+(l2+l6)) + ((l1+l5)+(l3+l7)).  `wide` 1.4.0 (Cargo.lock:1306) owns
 * the real order of f32x8::reduce_add and is not vendored, so this order is an
 * assumption: K-quant fp32 parity is tolerance-only. */
static inline float reduce8(const float *l) {
    float q0 = l[0] + l[4], q1 = l[1] + l[5], q2 = l[2] + l[6], q3 = l[3] + l[7];
    float d0 = q0 + q2, d1 = q1 + q3;
    return d0 + d1;
}

/* dot_q4_k_f32 (q4_k.rs:51-96), Hearth's own linear Q4_K layout:
 * [f16 d][f16 dmin][12 B scales][128 B nibbles]. */
HO_API float ho_dot_q4_k_f32(const uint8_t *row, const float *x, size_t n) {
    size_t blocks = n / 256;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *bp = row + b * 144;
        float d = rd_h(bp), dmin = rd_h(bp + 2);
        const uint8_t *sd = bp + 4;
        uint8_t sc8[8], mn8[8];
        for (int i = 0; i < 4; i++) {
            uint8_t s0 = sd[i * 3], s1 = sd[i * 3 + 1], s2 = sd[i * 3 + 2];
            sc8[i * 2] = s0 & 0x3F;
            mn8[i * 2] = (uint8_t)((s0 >> 6) | ((s1 & 0x0F) << 2));
            sc8[i * 2 + 1] = (uint8_t)((s1 >> 4) | ((s2 & 0x03) << 4));
            mn8[i * 2 + 1] = (s2 >> 2) & 0x3F;
        }
        const uint8_t *qs = bp + 16;
        for (int sb = 0; sb < 8; sb++) {
            float sc = (float)sc8[sb] * d;
            float mn = (float)mn8[sb] * dmin;
            const float *xv = x + b * 256 + (size_t)sb * 32;
            float nibs[32];
            for (int i = 0; i < 32; i++) {
                int byte_idx = (sb * 32 + i) / 2;
                uint8_t nib = (i % 2 == 0) ? (qs[byte_idx] & 0x0F) : ((qs[byte_idx] >> 4) & 0x0F);
                nibs[i] = (float)nib * sc - mn; /* two roundings, as written in Rust */
            }
            float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int i = 0; i < 32; i += 8)
                for (int j = 0; j < 8; j++) lanes[j] = fmaf(nibs[i + j], xv[i + j], lanes[j]);
            sum += reduce8(lanes);
        }
    }
    return sum;
}

/* dot_q6_k_f32 (qk_quant.rs:141-176), Hearth's linear Q6_K layout:
 * [ql 128][qh 64][int8 scales 16][f16 d]. */
HO_API float ho_dot_q6_k_f32(const uint8_t *row, const float *x, size_t n) {
    size_t blocks = n / 256;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *bp = row + b * 210;
        float d = rd_h(bp + 208);
        for (int sb = 0; sb < 16; sb++) {
            float sc = (float)(int8_t)bp[192 + sb];
            float sd = sc * d;
            int elem_base = sb * 16;
            for (int i = 0; i < 16; i += 8) {
                float lanes[8];
                for (int j = 0; j < 8; j++) {
                    int elem = elem_base + i + j;
                    uint8_t ql = bp[elem >> 1];
                    uint8_t low4 = (elem & 1) ? (ql >> 4) : (ql & 0x0F);
                    uint8_t qh = bp[128 + (elem >> 2)];
                    uint8_t high2 = (qh >> ((elem & 3) << 1)) & 0x03;
                    int quant = (int)(low4 | (high2 << 4)) - 32;
                    float q = (float)quant * sd;
                    lanes[j] = fmaf(q, x[b * 256 + (size_t)elem], 0.0f);
                }
                sum += reduce8(lanes);
            }
        }
    }
    return sum;
}

/* q4_k::dequantize (q4_k.rs:9-49) and dequantize_q6_k (qk_quant.rs:108-137). */
HO_API void ho_dequantize_q4_k(const uint8_t *data, size_t bytes, float *out, size_t n_out) {
    size_t blocks = bytes / 144;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *bp = data + b * 144;
        float d = rd_h(bp), dmin = rd_h(bp + 2);
        const uint8_t *sd = bp + 4;
        for (int sb = 0; sb < 8; sb++) {
            int i = sb / 2;
            uint8_t s0 = sd[i * 3], s1 = sd[i * 3 + 1], s2 = sd[i * 3 + 2];
            uint8_t sc = (sb & 1) ? (uint8_t)((s1 >> 4) | ((s2 & 3) << 4)) : (uint8_t)(s0 & 0x3F);
            uint8_t mn = (sb & 1) ? (uint8_t)((s2 >> 2) & 0x3F) : (uint8_t)((s0 >> 6) | ((s1 & 0x0F) << 2));
            float scale = (float)sc * d, min = (float)mn * dmin;
            for (int e = 0; e < 32; e++) {
                int byte_idx = (sb * 32 + e) / 2;
                uint8_t nib = (e % 2 == 0) ? (bp[16 + byte_idx] & 0x0F) : (bp[16 + byte_idx] >> 4);
                size_t idx = b * 256 + (size_t)sb * 32 + (size_t)e;
                if (idx < n_out) out[idx] = (float)nib * scale - min;
            }
        }
    }
}
HO_API void ho_dequantize_q6_k(const uint8_t *data, size_t bytes, float *out, size_t n_out) {
    size_t blocks = bytes / 210;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *bp = data + b * 210;
        float d = rd_h(bp + 208);
        for (size_t i = 0; i < 256; i++) {
            size_t idx = b * 256 + i;
            if (idx >= n_out) break;
            uint8_t ql = bp[i / 2];
            uint8_t low4 = (i % 2 == 0) ? (ql & 0x0F) : (ql >> 4);
            uint8_t high2 = (bp[128 + i / 4] >> ((i % 4) * 2)) & 0x03;
            int q = (int)(low4 | (high2 << 4)) - 32;
            float scale = (float)(int8_t)bp[192 + i / 16];
            out[idx] = (float)q * scale * d;
        }
    }
}

/* dot_ptq1_0_q8_0_ptr_scalar (ptq1_0.rs:555-602): decode the block's 128
 * trits, then the same nesting as the other block dots. */
HO_API float ho_dot_ptq1_0_q8_0(const uint8_t *w, const uint8_t *a, size_t n) {
    size_t blocks = n / 128;
    int8_t wv[128];
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        float scale = rd_h(w + b * 28 + 26);
        ptq_decode_block(w + b * 28, wv);
        float block_acc = 0.0f;
        for (int sub = 0; sub < 4; sub++) {
            const uint8_t *ab = a + (b * 4 + (size_t)sub) * 34;
            float a_scale = rd_h(ab);
            int32_t dot = isub_q8(wv + sub * 32, (const int8_t *)(ab + 2));
            block_acc += (float)dot * a_scale;
        }
        sum += block_acc * scale;
    }
    return sum;
}

/* ------------------------------------------------------- row dispatch ----- */

/* The kernel the reference's table picks per dtype for Q8_0 activations
 * (hearth-llm/src/model/matmul.rs:152-269 decode, :606-633 prefill). */
typedef float (*ho_dot_fn)(const uint8_t *, const uint8_t *, size_t);
static ho_dot_fn dot_for(int dtype) {
    switch (dtype) {
        case HO_Q1_0: case HO_Q1_0_G128: case HO_Q1_0_G128_LEGACY: return ho_dot_q1_0g128_q8_0;
        case HO_Q2_0: case HO_PQ2_0: return ho_dot_q2_0_q8_0;
        case HO_PTQ1_0: return ho_dot_ptq1_0_q8_0;
        case HO_Q8_0: return ho_dot_q8_0_q8_0;
        default: return 0;
    }
}

/* ThreadPool::par_dot_rows_batched / batched_rows_chunk (pool.rs:40-80,
 * :568-618): every row against seq_len activations, output token-major
 * out[s*n + row].  Tiling, pairing and the worker split do not change any
 * result, so they are not restated.  seq_len == 1 is par_dot_rows
 * (pool.rs:510-566). */
HO_API int ho_par_dot_rows_batched(int dtype, size_t n, size_t seq_len, size_t q8_stride, const uint8_t *w_base,
                                   const uint8_t *a_ptr, float *out, size_t row_bytes, size_t n_cols) {
    ho_dot_fn f = dot_for(dtype);
    if (!f) return -1;
    for (size_t s = 0; s < seq_len; s++)
        for (size_t row = 0; row < n; row++) out[s * n + row] = f(w_base + row * row_bytes, a_ptr + s * q8_stride, n_cols);
    return 0;
}

/* The f32-activation row loop for K-quants (matmul.rs:270-280, :333-343) and
 * its per-token repetition in matmul_batch (:661-672). out token-major. */
HO_API int ho_matmul_kquant_f32(int dtype, size_t n, size_t seq_len, const uint8_t *w_base, const float *x, float *out,
                                size_t n_cols) {
    size_t row_bytes = ho_byte_size(dtype, n_cols);
    for (size_t s = 0; s < seq_len; s++)
        for (size_t row = 0; row < n; row++) {
            const uint8_t *w = w_base + row * row_bytes;
            const float *xv = x + s * n_cols;
            if (dtype == HO_Q4_K) out[s * n + row] = ho_dot_q4_k_f32(w, xv, n_cols);
            else if (dtype == HO_Q6_K) out[s * n + row] = ho_dot_q6_k_f32(w, xv, n_cols);
            else return -1;
        }
    return 0;
}

/* ------------------------------------------- fused producers of Q8_0 rows -- */

/* hadamard_rotate + walsh_hadamard_in_place (hearth-llm/src/model/qwen35.rs:49-87):
 * optional sign vector, then per block_size chunk the in-place butterfly
 * (stages h = 1, 2, 4, ...; x[i] = a + b, x[i|h] = a - b) and a final multiply
 * by s = 1 / sqrt(n) computed in f32.  A tail shorter than block_size is left
 * untouched (chunks_exact_mut).  Every operation is a plain f32 add / multiply. */
HO_API void ho_hadamard_rotate(float *x, size_t n, const float *signs, size_t block_size) {
    if (signs)
        for (size_t i = 0; i < n; i++) x[i] *= signs[i];
    if (block_size == 0) return;
    for (size_t c = 0; c + block_size <= n; c += block_size) {
        float *v = x + c;
        float s = 1.0f / sqrtf((float)block_size);
        for (size_t h = 1; h < block_size; h <<= 1)
            for (size_t i = 0; i < block_size; i++)
                if ((i & h) == 0) {
                    float a = v[i], b = v[i | h];
                    v[i] = a + b;
                    v[i | h] = a - b;
                }
        for (size_t i = 0; i < block_size; i++) v[i] *= s;
    }
}

/* The step in front of every PQ2_0 / PTQ1_0 matmul of the hybrid models:
 * rotate a copy of x, then quantize_q8_0 (qwen35.rs:924-943). */
HO_API void ho_hadamard_quantize_q8_0(const float *x, size_t n, const float *signs, size_t block_size, float *tmp,
                                      uint8_t *q8_out) {
    memcpy(tmp, x, n * sizeof(float));
    ho_hadamard_rotate(tmp, n, signs, block_size);
    ho_quantize_q8_0_into(tmp, n, q8_out);
}

/* ops::rms_norm_q8 (hearth-llm/src/ops.rs:442-487): sum of squares in eight
 * fused-multiply-add lanes (lane j takes elements 8i+j), lanes reduced (order
 * assumed, see reduce8), scalar remainder, rms = sqrt(sum/n + eps),
 * inv = 1/rms, normed = (weight * x) * inv, then the Q8_0 block arithmetic. */
HO_API void ho_rms_norm_q8(const float *x, const float *weight, float eps, uint8_t *q8_out, size_t dim) {
    size_t n = dim, chunks = n / 8, rem = n % 8;
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (size_t i = 0; i < chunks; i++)
        for (int j = 0; j < 8; j++) lanes[j] = fmaf(x[i * 8 + j], x[i * 8 + j], lanes[j]);
    float sum_sq = 0.0f;
    sum_sq += reduce8(lanes);
    for (size_t i = n - rem; i < n; i++) sum_sq += x[i] * x[i];
    float rms = sqrtf(sum_sq / (float)n + eps);
    float inv_rms = 1.0f / rms;
    size_t blocks = (n + 31) / 32;
    for (size_t b = 0; b < blocks; b++) {
        size_t start = b * 32, cnt = (n - start < 32) ? n - start : 32;
        float max_abs = 0.0f;
        for (size_t i = 0; i < cnt; i++) {
            float normed = weight[start + i] * x[start + i] * inv_rms;
            float a = fabsf(normed);
            if (a > max_abs) max_abs = a;
        }
        float scale = (max_abs == 0.0f) ? 1.0f : max_abs / 127.0f;
        uint16_t h = ho_f2h(scale);
        size_t off = b * 34;
        q8_out[off] = (uint8_t)(h & 0xFF);
        q8_out[off + 1] = (uint8_t)(h >> 8);
        for (size_t i = 0; i < 32; i++) {
            int8_t q = 0;
            if (i < cnt) {
                float normed = weight[start + i] * x[start + i] * inv_rms;
                float r = roundf(normed / scale);
                if (r != r) q = 0;
                else {
                    if (r < -128.0f) r = -128.0f;
                    if (r > 127.0f) r = 127.0f;
                    q = (int8_t)r;
                }
            }
            q8_out[off + 2 + i] = (uint8_t)q;
        }
    }
}

/* ops::silu_mul_q8 (hearth-llm/src/ops.rs:273-306): v = (g / (1 + exp(-g))) * u
 * per element, then the Q8_0 block arithmetic; dim / 32 whole blocks.  The
 * reference's exp is `wide`'s f32x8 polynomial, which is not available here;
 * expf from libm stands in, so this function is a tolerance-level restatement
 * (quantized values may differ by one step at a rounding boundary). */
HO_API void ho_silu_mul_q8(const float *gate, const float *up, uint8_t *q8_out, size_t dim) {
    size_t blocks = dim / 32;
    for (size_t b = 0; b < blocks; b++) {
        float tmp[32], max_abs = 0.0f;
        for (int i = 0; i < 32; i++) {
            float g = gate[b * 32 + i];
            float s = g / (1.0f + expf(-g));
            float v = s * up[b * 32 + i];
            tmp[i] = v;
            float a = fabsf(v);
            if (a > max_abs) max_abs = a;
        }
        float scale = (max_abs == 0.0f) ? 1.0f : max_abs / 127.0f;
        uint16_t h = ho_f2h(scale);
        size_t off = b * 34;
        q8_out[off] = (uint8_t)(h & 0xFF);
        q8_out[off + 1] = (uint8_t)(h >> 8);
        for (int i = 0; i < 32; i++) {
            float r = roundf(tmp[i] / scale);
            int8_t q;
            if (r != r) q = 0;
            else {
                if (r < -128.0f) r = -128.0f;
                if (r > 127.0f) r = 127.0f;
                q = (int8_t)r;
            }
            q8_out[off + 2 + i] = (uint8_t)q;
        }
    }
}

/* ------------------------------------------------------------------ argmax -- */

/* GpuCompute::argmax_f32 with its shader (hearth-compute/src/lib.rs:338-450,
 * hearth-compute/src/shaders/argmax.wgsl), executed literally: workgroups of
 * 128 threads x 16 consecutive elements, each thread scanning with strict '>'
 * from -3.4028235e38 (index 0 when nothing is larger), a tree over the 128
 * thread results (offsets 64..1, strict '>' takes the upper entry), then the
 * host loop over the workgroup results with strict '>' from -inf. */
HO_API uint32_t ho_argmax_f32(const float *data, size_t n) {
    const size_t ept = 16, wg = 128, per_wg = ept * wg;
    size_t num_wgs = (n + per_wg - 1) / per_wg;
    uint32_t best_idx = 0;
    float best_val = -INFINITY;
    for (size_t g = 0; g < num_wgs; g++) {
        float wmax[128];
        uint32_t widx[128];
        for (size_t t = 0; t < wg; t++) {
            size_t start = g * per_wg + t * ept, end = start + ept < n ? start + ept : n;
            float my_max = -3.4028235e+38f;
            uint32_t my_idx = 0;
            for (size_t i = start; i < end; i++)
                if (data[i] > my_max) {
                    my_max = data[i];
                    my_idx = (uint32_t)i;
                }
            wmax[t] = my_max;
            widx[t] = my_idx;
        }
        for (size_t off = 64; off > 0; off >>= 1)
            for (size_t t = 0; t < off; t++)
                if (wmax[t + off] > wmax[t]) {
                    wmax[t] = wmax[t + off];
                    widx[t] = widx[t + off];
                }
        if (wmax[0] > best_val) {
            best_val = wmax[0];
            best_idx = widx[0];
        }
    }
    return best_idx;
}

/* ----------------------------------- f32-activation mode (the GPU shaders) -- */

/* f16_to_f32 of the matmul shaders (hearth-compute/src/shaders/q1_0_matmul.wgsl:26-32):
 * sign | (exp + 112) << 23 | mant << 13 with no special cases, so zero and
 * subnormal halves come out as 2^-15 * (1 + mant/1024) and exp = 31 as a finite
 * number.  Equal to the IEEE value for every normal half. */
static inline float shader_h2f(const uint8_t *p) {
    uint32_t lo = p[0], hi = p[1];
    uint32_t sign = (hi >> 7) & 1u, exp = (hi >> 2) & 0x1Fu, mant = ((hi & 3u) << 8) | lo;
    uint32_t bits = (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* One weight row against one f32 activation row, as q1_0_matmul.wgsl:38-97 and
 * q2_0_matmul.wgsl:48-106 compute it (the batch, add-in-place and fused
 * gate/up and q/k/v shaders repeat the same arithmetic): per 128-column block
 * partial[i] = w_i * x_i, a tree over the 128 partials (offsets 64, 32, .. 1,
 * partial[i] += partial[i + offset]), then sum = sum + partial[0] * w_scale
 * with the product and the sum rounded separately. */
HO_API float ho_dot_f32act(int dtype, const uint8_t *w, const float *x, size_t n) {
    int q1 = (dtype == HO_Q1_0 || dtype == HO_Q1_0_G128 || dtype == HO_Q1_0_G128_LEGACY);
    size_t bb = q1 ? 18 : 34, blocks = n / 128;
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; b++) {
        const uint8_t *blk = w + b * bb;
        float w_scale = shader_h2f(blk);
        float partial[128];
        for (size_t i = 0; i < 128; i++) {
            float wv = q1 ? (float)q1_sign(blk + 2, i) : (float)q2_val(blk + 2, i);
            partial[i] = wv * x[b * 128 + i];
        }
        for (size_t off = 64; off > 0; off >>= 1)
            for (size_t i = 0; i < off; i++) partial[i] = partial[i] + partial[i + off];
        sum = sum + partial[0] * w_scale;
    }
    return sum;
}

/* dequant_matmul_fused (n = 1), dequant_matmul_batch ([batch x k] in, [batch x m]
 * out) and dequant_matmul_fused_add_inplace (out[row] = out[row] + sum)
 * (hearth-compute/src/lib.rs:483-507, :1153-1173, :1123-1151). */
HO_API int ho_matmul_f32act(int dtype, size_t m, size_t batch, const uint8_t *w_base, const float *x, float *out, size_t k,
                            int add_inplace) {
    size_t row_bytes = ho_byte_size(dtype, k);
    if (dtype != HO_Q1_0 && dtype != HO_Q1_0_G128 && dtype != HO_Q1_0_G128_LEGACY && dtype != HO_Q2_0 && dtype != HO_PQ2_0) return -1;
    for (size_t s = 0; s < batch; s++)
        for (size_t row = 0; row < m; row++) {
            float v = ho_dot_f32act(dtype, w_base + row * row_bytes, x + s * k, k);
            out[s * m + row] = add_inplace ? out[s * m + row] + v : v;
        }
    return 0;
}
