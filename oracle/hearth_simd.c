/*
 * hearth_simd.c -- CPU baseline: the x86 SIMD arms and row-splitting thread pool
 * of the reference's quantized matrix-product path, restated in C.
 *
 * TEST / MEASUREMENT INFRASTRUCTURE ONLY.  It is what the benchmark times as
 * "the reference's CPU path" on the GPU box's host cores; nothing in the
 * product may call it.  It is a restatement because the reference is Rust and
 * no Rust toolchain exists where this is built.
 *
 * What is restated (Eric-Lautanen/hearth v0.2.0):
 *   Q1_0_G128 x Q8_0   AVX-512 VNNI-256 arm   hearth-quant/src/q1_0g128.rs:530-591
 *                      AVX2 shuffle arm        q1_0g128.rs:255-377
 *                      paired-token AVX2 arm   q1_0g128.rs:396-479
 *                      dispatch order          q1_0g128.rs:1000-1015
 *   Q2_0/PQ2_0 x Q8_0  VNNI-512 two-sub arm    hearth-quant/src/q2_0.rs:219-297
 *                      AVX2 LUT arm            q2_0.rs:308-392
 *                      paired-token AVX2 LUT   q2_0.rs:408-469
 *                      VNNI-256 arm            q2_0.rs:155-205
 *                      dispatch order          q2_0.rs:628-676
 *   PTQ1_0 x Q8_0      AVX-512 arm             hearth-quant/src/ptq1_0.rs:241-308
 *                      AVX2 arm                ptq1_0.rs:323-404
 *                      dispatch order          ptq1_0.rs:157-167
 *   Q4_K / Q6_K x f32  eight-lane FMA loops    hearth-quant/src/q4_k.rs:51-96, qk_quant.rs:141-176
 *                      (the reference's `wide` f32x8 code; rows through rayon's par_iter,
 *                      hearth-llm/src/model/matmul.rs:270-280, :333-343; here the same static pool)
 *   width policy       avx512_full_width       hearth-quant/src/lib.rs:27-43, :113-143
 *   pool               static ceil(n/T) split, 1 MiB row tiles, token pairs
 *                      inside the tile          hearth-llm/src/pool.rs:40-80, :321-323, :510-618
 *   worker count       physical cores (dense rule)  pool.rs:150-152, :199-219
 *
 * The integer sub-block sums of every arm equal the scalar oracle's; the fp32
 * association differs (eight FMA lanes, one horizontal add per row), exactly as
 * in the reference, so fp32 results are compared to the scalar oracle only
 * loosely.  Like the reference's Q1_0 SIMD arms, a -128 activation byte under a
 * -1 weight wraps (the quantizer never emits -128).
 */
#define _GNU_SOURCE
#include <cpuid.h>
#include <immintrin.h>
#include <pthread.h>
#include <sched.h>
#include <stdatomic.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HS_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- cpuid -- */

static int g_has_avx2, g_has_fma, g_has_f16c, g_has_avx512f, g_has_avx512bw, g_has_avx512vl, g_has_avx512dq,
    g_has_avx512vnni, g_is_amd, g_family, g_probed;

static void probe(void) {
    if (g_probed) return;
    __builtin_cpu_init();
    g_has_avx2 = __builtin_cpu_supports("avx2");
    g_has_fma = __builtin_cpu_supports("fma");
    g_has_f16c = __builtin_cpu_supports("f16c");
    g_has_avx512f = __builtin_cpu_supports("avx512f");
    g_has_avx512bw = __builtin_cpu_supports("avx512bw");
    g_has_avx512vl = __builtin_cpu_supports("avx512vl");
    g_has_avx512dq = __builtin_cpu_supports("avx512dq");
    g_has_avx512vnni = __builtin_cpu_supports("avx512vnni");
    unsigned a, b, c, d;
    __cpuid(0, a, b, c, d);
    g_is_amd = (b == 0x68747541u && d == 0x69746e65u && c == 0x444d4163u); /* "AuthenticAMD" */
    __cpuid(1, a, b, c, d);
    unsigned base = (a >> 8) & 0xF, ext = (a >> 20) & 0xFF;
    g_family = (int)(base == 0xF ? base + ext : base);
    g_probed = 1;
}

static int vnni256_ok(void) { return g_has_avx512f && g_has_avx512vnni && g_has_avx512vl; }
static int avx2_ok(void) { return g_has_avx2 && g_has_fma && g_has_f16c; }
/* Full-width AVX-512 unless the part is AMD family 19h (split datapath). */
static int full_width(void) { return g_has_avx512f && g_has_avx512bw && !(g_is_amd && g_family == 0x19); }

/* ------------------------------------------------------------- helpers --- */

#define T_AVX2 __attribute__((target("avx2,fma,f16c")))
#define T_VNNI256 __attribute__((target("avx2,fma,f16c,avx512f,avx512vl,avx512vnni")))
#define T_VNNI512 __attribute__((target("avx2,fma,f16c,avx512f,avx512bw,avx512dq,avx512vnni")))

T_AVX2 static inline float h2f(const uint8_t *p) {
    uint16_t bits;
    memcpy(&bits, p, 2);
    return _mm_cvtss_f32(_mm_cvtph_ps(_mm_cvtsi32_si128(bits)));
}

/* (l0..3 + l4..7), then (x0+x2, x1+x3), then lane0 + lane1. */
T_AVX2 static inline float hsum8(__m256 v) {
    __m128 r = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    r = _mm_add_ps(r, _mm_movehl_ps(r, r));
    r = _mm_add_ss(r, _mm_movehdup_ps(r));
    return _mm_cvtss_f32(r);
}

/* Bytes 0/0xFF: 0xFF where the weight bit is 0 (weight -1), for one 32-bit group of sign bits. */
T_AVX2 static inline __m256i q1_neg_mask(uint32_t bits32) {
    const __m256i spread = _mm256_setr_epi8(0, 0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 1, 1, 1, 2, 2, 2, 2, 2, 2, 2, 2, 3, 3,
                                            3, 3, 3, 3, 3, 3);
    const __m256i bit = _mm256_setr_epi8(1, 2, 4, 8, 16, 32, 64, -128, 1, 2, 4, 8, 16, 32, 64, -128, 1, 2, 4, 8, 16, 32,
                                         64, -128, 1, 2, 4, 8, 16, 32, 64, -128);
    __m256i rep = _mm256_shuffle_epi8(_mm256_set1_epi32((int)bits32), spread);
    return _mm256_cmpeq_epi8(_mm256_and_si256(rep, bit), _mm256_setzero_si256());
}

/* ----------------------------------------------------------- Q1_0 arms --- */

T_VNNI256 static float q1_vnni256(const uint8_t *w, const uint8_t *a, size_t n) {
    const __m256i ones = _mm256_set1_epi8(1);
    __m256 acc = _mm256_setzero_ps();
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *wb = w + b * 18;
        __m256 blk = _mm256_setzero_ps();
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            uint32_t bits;
            memcpy(&bits, wb + 2 + 4 * s, 4);
            __m256i neg = q1_neg_mask(bits);
            __m256i act = _mm256_loadu_si256((const __m256i *)(ab + 2));
            __m256i signed_act = _mm256_sub_epi8(_mm256_xor_si256(act, neg), neg);
            __m256i s32 = _mm256_dpbusd_epi32(_mm256_setzero_si256(), ones, signed_act);
            blk = _mm256_fmadd_ps(_mm256_set1_ps(h2f(ab)), _mm256_cvtepi32_ps(s32), blk);
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(h2f(wb)), blk, acc);
    }
    return hsum8(acc);
}

T_AVX2 static inline __m256i q1_sub_sum_avx2(uint32_t bits, const uint8_t *act_vals) {
    __m256i neg = q1_neg_mask(bits);
    __m256i act = _mm256_loadu_si256((const __m256i *)act_vals);
    __m256i signed_act = _mm256_sub_epi8(_mm256_xor_si256(act, neg), neg);
    return _mm256_madd_epi16(_mm256_maddubs_epi16(_mm256_set1_epi8(1), signed_act), _mm256_set1_epi16(1));
}

T_AVX2 static float q1_avx2(const uint8_t *w, const uint8_t *a, size_t n) {
    __m256 acc = _mm256_setzero_ps();
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *wb = w + b * 18;
        __m256 blk = _mm256_setzero_ps();
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            uint32_t bits;
            memcpy(&bits, wb + 2 + 4 * s, 4);
            blk = _mm256_fmadd_ps(_mm256_set1_ps(h2f(ab)), _mm256_cvtepi32_ps(q1_sub_sum_avx2(bits, ab + 2)), blk);
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(h2f(wb)), blk, acc);
    }
    return hsum8(acc);
}

/* One weight row against two activations; sign expansion shared. */
T_AVX2 static void q1_avx2_x2(const uint8_t *w, const uint8_t *a0, const uint8_t *a1, size_t n, float *o0, float *o1) {
    const __m256i ones8 = _mm256_set1_epi8(1), ones16 = _mm256_set1_epi16(1);
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *wb = w + b * 18;
        __m256 blk0 = _mm256_setzero_ps(), blk1 = _mm256_setzero_ps();
        for (int s = 0; s < 4; s++) {
            size_t off = (b * 4 + (size_t)s) * 34;
            uint32_t bits;
            memcpy(&bits, wb + 2 + 4 * s, 4);
            __m256i neg = q1_neg_mask(bits);
            __m256i y0 = _mm256_loadu_si256((const __m256i *)(a0 + off + 2));
            __m256i y1 = _mm256_loadu_si256((const __m256i *)(a1 + off + 2));
            y0 = _mm256_sub_epi8(_mm256_xor_si256(y0, neg), neg);
            y1 = _mm256_sub_epi8(_mm256_xor_si256(y1, neg), neg);
            __m256i s0 = _mm256_madd_epi16(_mm256_maddubs_epi16(ones8, y0), ones16);
            __m256i s1 = _mm256_madd_epi16(_mm256_maddubs_epi16(ones8, y1), ones16);
            blk0 = _mm256_fmadd_ps(_mm256_set1_ps(h2f(a0 + off)), _mm256_cvtepi32_ps(s0), blk0);
            blk1 = _mm256_fmadd_ps(_mm256_set1_ps(h2f(a1 + off)), _mm256_cvtepi32_ps(s1), blk1);
        }
        __m256 ws = _mm256_set1_ps(h2f(wb));
        acc0 = _mm256_fmadd_ps(ws, blk0, acc0);
        acc1 = _mm256_fmadd_ps(ws, blk1, acc1);
    }
    *o0 = hsum8(acc0);
    *o1 = hsum8(acc1);
}

/* Widening scalar form (the non-SIMD fallback order, q1_0g128.rs:1019-1052). */
static float half_scalar(const uint8_t *p) {
    uint16_t h = (uint16_t)(p[0] | (p[1] << 8));
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
    if (exp == 0) {
        if (!man) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400));
            bits = sign | ((uint32_t)(112 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
static float q1_scalar(const uint8_t *w, const uint8_t *a, size_t n) {
    float sum = 0.0f;
    for (size_t b = 0; b < n / 128; b++) {
        float blk = 0.0f;
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            int32_t d = 0;
            for (int i = 0; i < 32; i++) {
                int e = s * 32 + i;
                int sg = ((w[b * 18 + 2 + (e >> 3)] >> (e & 7)) & 1) ? 1 : -1;
                d += sg * (int32_t)(int8_t)ab[2 + i];
            }
            blk += (float)d * half_scalar(ab);
        }
        sum += blk * half_scalar(w + b * 18);
    }
    return sum;
}

/* ----------------------------------------------------------- Q2_0 arms --- */

/* code bytes -> four u8 codes {0..3} and four i16 values {-1..2}; built once. */
static uint8_t g_q2_u8[256][4];
static int16_t g_q2_i16[256][4];
static void build_q2_tables(void) {
    for (int b = 0; b < 256; b++)
        for (int j = 0; j < 4; j++) {
            int q = (b >> (2 * j)) & 3;
            g_q2_u8[b][j] = (uint8_t)q;
            g_q2_i16[b][j] = (int16_t)(q - 1);
        }
}

T_VNNI256 static float q2_vnni256(const uint8_t *w, const uint8_t *a, size_t n) {
    const __m256i ones = _mm256_set1_epi8(1), zero = _mm256_setzero_si256();
    __m256 acc = _mm256_setzero_ps();
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *wb = w + b * 34;
        __m256 blk = _mm256_setzero_ps();
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            uint8_t codes[32];
            for (int j = 0; j < 8; j++) memcpy(codes + 4 * j, g_q2_u8[wb[2 + 8 * s + j]], 4);
            __m256i wv = _mm256_loadu_si256((const __m256i *)codes);
            __m256i av = _mm256_loadu_si256((const __m256i *)(ab + 2));
            __m256i diff = _mm256_sub_epi32(_mm256_dpbusd_epi32(zero, wv, av), _mm256_dpbusd_epi32(zero, ones, av));
            blk = _mm256_fmadd_ps(_mm256_set1_ps(h2f(ab)), _mm256_cvtepi32_ps(diff), blk);
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(h2f(wb)), blk, acc);
    }
    return hsum8(acc);
}

T_VNNI512 static float q2_vnni512x2(const uint8_t *w, const uint8_t *a, size_t n) {
    const __m512i ones = _mm512_set1_epi8(1), zero = _mm512_setzero_si512();
    __m256 acc = _mm256_setzero_ps();
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *wb = w + b * 34;
        __m256 lo = _mm256_setzero_ps(), hi = _mm256_setzero_ps();
        for (int pair = 0; pair < 2; pair++) {
            const uint8_t *ab0 = a + (b * 4 + (size_t)pair * 2) * 34;
            const uint8_t *ab1 = ab0 + 34;
            uint8_t codes[64], acts[64];
            for (int j = 0; j < 16; j++) memcpy(codes + 4 * j, g_q2_u8[wb[2 + 16 * pair + j]], 4);
            memcpy(acts, ab0 + 2, 32);
            memcpy(acts + 32, ab1 + 2, 32);
            __m512i wv = _mm512_loadu_si512(codes), av = _mm512_loadu_si512(acts);
            __m512i diff = _mm512_sub_epi32(_mm512_dpbusd_epi32(zero, wv, av), _mm512_dpbusd_epi32(zero, ones, av));
            lo = _mm256_fmadd_ps(_mm256_set1_ps(h2f(ab0)), _mm256_cvtepi32_ps(_mm512_castsi512_si256(diff)), lo);
            hi = _mm256_fmadd_ps(_mm256_set1_ps(h2f(ab1)), _mm256_cvtepi32_ps(_mm512_extracti64x4_epi64(diff, 1)), hi);
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(h2f(wb)), _mm256_add_ps(lo, hi), acc);
    }
    return hsum8(acc);
}

/* 16 weights (4 code bytes) as i16. */
T_AVX2 static inline __m256i q2_w16(const uint8_t *codes4) {
    int16_t buf[16];
    for (int j = 0; j < 4; j++) memcpy(buf + 4 * j, g_q2_i16[codes4[j]], 8);
    return _mm256_loadu_si256((const __m256i *)buf);
}

T_AVX2 static float q2_avx2_lut(const uint8_t *w, const uint8_t *a, size_t n) {
    __m256 acc = _mm256_setzero_ps();
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *wb = w + b * 34;
        __m256 blk = _mm256_setzero_ps();
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            const uint8_t *qs = wb + 2 + 8 * s;
            __m256i lo = _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i *)(ab + 2))), q2_w16(qs));
            __m256i hi =
                _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i *)(ab + 18))), q2_w16(qs + 4));
            blk = _mm256_fmadd_ps(_mm256_set1_ps(h2f(ab)), _mm256_cvtepi32_ps(_mm256_add_epi32(lo, hi)), blk);
        }
        acc = _mm256_fmadd_ps(_mm256_set1_ps(h2f(wb)), blk, acc);
    }
    return hsum8(acc);
}

T_AVX2 static void q2_avx2_lut_x2(const uint8_t *w, const uint8_t *a0, const uint8_t *a1, size_t n, float *o0, float *o1) {
    __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *wb = w + b * 34;
        __m256 blk0 = _mm256_setzero_ps(), blk1 = _mm256_setzero_ps();
        for (int s = 0; s < 4; s++) {
            size_t off = (b * 4 + (size_t)s) * 34;
            const uint8_t *qs = wb + 2 + 8 * s;
            __m256i wl = q2_w16(qs), wh = q2_w16(qs + 4); /* expanded once for both tokens */
            __m256i s0 = _mm256_add_epi32(
                _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i *)(a0 + off + 2))), wl),
                _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i *)(a0 + off + 18))), wh));
            __m256i s1 = _mm256_add_epi32(
                _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i *)(a1 + off + 2))), wl),
                _mm256_madd_epi16(_mm256_cvtepi8_epi16(_mm_loadu_si128((const __m128i *)(a1 + off + 18))), wh));
            blk0 = _mm256_fmadd_ps(_mm256_set1_ps(h2f(a0 + off)), _mm256_cvtepi32_ps(s0), blk0);
            blk1 = _mm256_fmadd_ps(_mm256_set1_ps(h2f(a1 + off)), _mm256_cvtepi32_ps(s1), blk1);
        }
        __m256 ws = _mm256_set1_ps(h2f(wb));
        acc0 = _mm256_fmadd_ps(ws, blk0, acc0);
        acc1 = _mm256_fmadd_ps(ws, blk1, acc1);
    }
    *o0 = hsum8(acc0);
    *o1 = hsum8(acc1);
}

static float q2_scalar(const uint8_t *w, const uint8_t *a, size_t n) {
    float sum = 0.0f;
    for (size_t b = 0; b < n / 128; b++) {
        float blk = 0.0f;
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            int32_t d = 0;
            for (int i = 0; i < 32; i++) {
                int e = s * 32 + i;
                d += ((int)((w[b * 34 + 2 + (e >> 2)] >> (2 * (e & 3))) & 3) - 1) * (int32_t)(int8_t)ab[2 + i];
            }
            blk += (float)d * half_scalar(ab);
        }
        sum += blk * half_scalar(w + b * 34);
    }
    return sum;
}

/* Q8_0 x Q8_0 has a scalar arm only (q8_0.rs:154-171). */
static float q8_scalar(const uint8_t *w, const uint8_t *a, size_t n) {
    float sumf = 0.0f;
    for (size_t b = 0; b < n / 32; b++) {
        int32_t s = 0;
        for (int i = 0; i < 32; i++) s += (int32_t)(int8_t)w[b * 34 + 2 + i] * (int32_t)(int8_t)a[b * 34 + 2 + i];
        sumf += (float)s * half_scalar(w + b * 34) * half_scalar(a + b * 34);
    }
    return sumf;
}

/* ------------------------------------------------------------- dispatch -- */


/* ------------------------------------------------------------- PTQ1_0 ---- */

static int8_t g_qh_trit[256][4];
static void build_ptq_tables(void) {
    static const unsigned pow3[4] = {1, 3, 9, 27};
    for (unsigned b = 0; b < 256; b++)
        for (int n = 0; n < 4; n++) g_qh_trit[b][n] = (int8_t)(((((b * pow3[n]) & 255u) * 3u) >> 8) - 1);
}
static int g_ptq_ready;

static inline void ptq_qh(const uint8_t *blk, int8_t *wv) {
    const int8_t *t0 = g_qh_trit[blk[24]], *t1 = g_qh_trit[blk[25]];
    for (int n = 0; n < 4; n++) {
        wv[120 + 2 * n] = t0[n];
        wv[121 + 2 * n] = t1[n];
    }
}

/* AVX2 arm (ptq1_0.rs:323-404): digits by multiply / mask / shift on u16 lanes, trits widened to i16 and
 * multiplied with vpmaddwd, eight fp32 lanes per block summed left to right. */
T_AVX2 static float ptq_avx2(const uint8_t *w, const uint8_t *a, size_t n) {
    static const int16_t pow3[5] = {1, 3, 9, 27, 81};
    const __m128i ff = _mm_set1_epi16(0xFF), three = _mm_set1_epi16(3), one = _mm_set1_epi16(1), z = _mm_setzero_si128();
    int8_t wv[128];
    float sum = 0.0f;
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *blk = w + b * 28;
        float scale = h2f(blk + 26);
        __m128i qs = _mm_loadu_si128((const __m128i *)blk), q8 = _mm_loadl_epi64((const __m128i *)(blk + 16));
        __m128i alo = _mm_unpacklo_epi8(qs, z), ahi = _mm_unpackhi_epi8(qs, z);
        __m128i blo = _mm_unpacklo_epi8(q8, z), bhi = _mm_unpackhi_epi8(q8, z);
        for (int k = 0; k < 5; k++) {
            __m128i p = _mm_set1_epi16(pow3[k]);
#define HS_DIGIT(v) _mm_sub_epi16(_mm_srli_epi16(_mm_mullo_epi16(_mm_and_si128(_mm_mullo_epi16(v, p), ff), three), 8), one)
            _mm_storeu_si128((__m128i *)(wv + k * 16), _mm_packs_epi16(HS_DIGIT(alo), HS_DIGIT(ahi)));
            _mm_storel_epi64((__m128i *)(wv + 80 + k * 8), _mm_packs_epi16(HS_DIGIT(blo), HS_DIGIT(bhi)));
#undef HS_DIGIT
        }
        ptq_qh(blk, wv);
        __m256 acc = _mm256_setzero_ps();
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            __m256i w32 = _mm256_loadu_si256((const __m256i *)(wv + s * 32)), a32 = _mm256_loadu_si256((const __m256i *)(ab + 2));
            __m256i wl = _mm256_cvtepi8_epi16(_mm256_castsi256_si128(w32)), wh = _mm256_cvtepi8_epi16(_mm256_extracti128_si256(w32, 1));
            __m256i al = _mm256_cvtepi8_epi16(_mm256_castsi256_si128(a32)), ah = _mm256_cvtepi8_epi16(_mm256_extracti128_si256(a32, 1));
            __m256i p = _mm256_add_epi32(_mm256_madd_epi16(wl, al), _mm256_madd_epi16(wh, ah));
            acc = _mm256_add_ps(acc, _mm256_mul_ps(_mm256_cvtepi32_ps(p), _mm256_set1_ps(h2f(ab))));
        }
        float lanes[8], blk_acc = 0.0f;
        _mm256_storeu_ps(lanes, acc);
        for (int i = 0; i < 8; i++) blk_acc += lanes[i];
        sum += blk_acc * scale;
    }
    return sum;
}

/* AVX-512 arm (ptq1_0.rs:241-308): all 24 qs bytes in one register per digit slot, one 32-element
 * sub-block per vpmaddwd, sixteen fp32 lanes per block summed left to right. */
__attribute__((target("avx2,fma,f16c,avx512f,avx512bw,avx512vl"))) static float ptq_avx512(const uint8_t *w, const uint8_t *a, size_t n) {
    static const int16_t pow3[5] = {1, 3, 9, 27, 81};
    const __m512i ff = _mm512_set1_epi16(0xFF), three = _mm512_set1_epi16(3), one = _mm512_set1_epi16(1);
    int8_t wv[128];
    float sum = 0.0f;
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *blk = w + b * 28;
        float scale = h2f(blk + 26);
        __m512i bytes16 = _mm512_cvtepu8_epi16(_mm256_maskz_loadu_epi8((__mmask32)0x00FFFFFFu, blk));
        for (int k = 0; k < 5; k++) {
            __m512i t = _mm512_and_si512(_mm512_mullo_epi16(bytes16, _mm512_set1_epi16(pow3[k])), ff);
            __m256i packed = _mm512_cvtepi16_epi8(_mm512_sub_epi16(_mm512_srli_epi16(_mm512_mullo_epi16(t, three), 8), one));
            _mm_storeu_si128((__m128i *)(wv + k * 16), _mm256_castsi256_si128(packed));
            _mm_storel_epi64((__m128i *)(wv + 80 + k * 8), _mm256_extracti128_si256(packed, 1));
        }
        ptq_qh(blk, wv);
        __m512 acc = _mm512_setzero_ps();
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            __m512i w16 = _mm512_cvtepi8_epi16(_mm256_loadu_si256((const __m256i *)(wv + s * 32)));
            __m512i a16 = _mm512_cvtepi8_epi16(_mm256_loadu_si256((const __m256i *)(ab + 2)));
            acc = _mm512_add_ps(acc, _mm512_mul_ps(_mm512_cvtepi32_ps(_mm512_madd_epi16(w16, a16)), _mm512_set1_ps(h2f(ab))));
        }
        float lanes[16], blk_acc = 0.0f;
        _mm512_storeu_ps(lanes, acc);
        for (int i = 0; i < 16; i++) blk_acc += lanes[i];
        sum += blk_acc * scale;
    }
    return sum;
}

static float ptq_scalar(const uint8_t *w, const uint8_t *a, size_t n) {
    static const unsigned pow3[5] = {1, 3, 9, 27, 81};
    int8_t wv[128];
    float sum = 0.0f;
    for (size_t b = 0; b < n / 128; b++) {
        const uint8_t *blk = w + b * 28;
        for (int k = 0; k < 5; k++) {
            for (int m = 0; m < 16; m++) wv[k * 16 + m] = (int8_t)(((((blk[m] * pow3[k]) & 255u) * 3u) >> 8) - 1);
            for (int m = 0; m < 8; m++) wv[80 + k * 8 + m] = (int8_t)(((((blk[16 + m] * pow3[k]) & 255u) * 3u) >> 8) - 1);
        }
        ptq_qh(blk, wv);
        float acc = 0.0f;
        for (int s = 0; s < 4; s++) {
            const uint8_t *ab = a + (b * 4 + (size_t)s) * 34;
            int32_t d = 0;
            for (int i = 0; i < 32; i++) d += (int32_t)wv[s * 32 + i] * (int32_t)(int8_t)ab[2 + i];
            acc += (float)d * half_scalar(ab);
        }
        sum += acc * half_scalar(blk + 26);
    }
    return sum;
}

/* -------------------------------------------------- K-quants x f32 ------- */

/* Eight lanes, lane j takes elements 8t + j with a fused multiply-add, lanes reduced
 * ((l0+l4)+(l2+l6))+((l1+l5)+(l3+l7)) -- the order the scalar oracle assumes for `wide`'s reduce_add. */
T_AVX2 static inline float reduce8_ps(__m256 v) {
    __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
    __m128 s = _mm_add_ps(lo, hi);                        /* l0+l4, l1+l5, l2+l6, l3+l7 */
    __m128 t = _mm_add_ps(s, _mm_movehl_ps(s, s));        /* (l0+l4)+(l2+l6), (l1+l5)+(l3+l7) */
    return _mm_cvtss_f32(_mm_add_ss(t, _mm_shuffle_ps(t, t, 1)));
}

/* dot_q4_k_f32 (q4_k.rs:51-96); `a` carries the f32 activation row. */
T_AVX2 static float q4k_f32(const uint8_t *w, const uint8_t *a, size_t n) {
    const float *x = (const float *)a;
    float sum = 0.0f;
    for (size_t b = 0; b < n / 256; b++) {
        const uint8_t *bp = w + b * 144;
        float d = h2f(bp), dmin = h2f(bp + 2);
        uint8_t sc[8], mn[8];
        for (int i = 0; i < 4; i++) {
            uint8_t s0 = bp[4 + 3 * i], s1 = bp[5 + 3 * i], s2 = bp[6 + 3 * i];
            sc[2 * i] = s0 & 63;
            mn[2 * i] = (uint8_t)((s0 >> 6) | ((s1 & 15) << 2));
            sc[2 * i + 1] = (uint8_t)((s1 >> 4) | ((s2 & 3) << 4));
            mn[2 * i + 1] = (s2 >> 2) & 63;
        }
        for (int sb = 0; sb < 8; sb++) {
            float scale = (float)sc[sb] * d, minv = (float)mn[sb] * dmin;
            __m256 vs = _mm256_set1_ps(scale), vm = _mm256_set1_ps(minv), acc = _mm256_setzero_ps();
            const uint8_t *qs = bp + 16 + sb * 16;
            const float *xs = x + b * 256 + (size_t)sb * 32;
            for (int t = 0; t < 4; t++) {
                float nib[8];
                for (int j = 0; j < 8; j++) {
                    int i = t * 8 + j;
                    uint8_t byte = qs[i >> 1];
                    nib[j] = (float)((i & 1) ? (byte >> 4) : (byte & 15));
                }
                __m256 val = _mm256_sub_ps(_mm256_mul_ps(_mm256_loadu_ps(nib), vs), vm);
                acc = _mm256_fmadd_ps(val, _mm256_loadu_ps(xs + t * 8), acc);
            }
            sum += reduce8_ps(acc);
        }
    }
    return sum;
}

/* dot_q6_k_f32 (qk_quant.rs:141-176). */
T_AVX2 static float q6k_f32(const uint8_t *w, const uint8_t *a, size_t n) {
    const float *x = (const float *)a;
    float sum = 0.0f;
    for (size_t b = 0; b < n / 256; b++) {
        const uint8_t *bp = w + b * 210;
        float d = h2f(bp + 208);
        for (int sb = 0; sb < 16; sb++) {
            float scale = (float)(int8_t)bp[192 + sb] * d;
            __m256 vs = _mm256_set1_ps(scale);
            for (int g = 0; g < 2; g++) {
                float q[8];
                for (int j = 0; j < 8; j++) {
                    int i = sb * 16 + g * 8 + j;
                    uint8_t ql = bp[i >> 1];
                    int low4 = (i & 1) ? (ql >> 4) : (ql & 15);
                    int high2 = (bp[128 + (i >> 2)] >> (2 * (i & 3))) & 3;
                    q[j] = (float)((low4 | (high2 << 4)) - 32);
                }
                __m256 val = _mm256_mul_ps(_mm256_loadu_ps(q), vs);
                __m256 prod = _mm256_fmadd_ps(val, _mm256_loadu_ps(x + b * 256 + (size_t)sb * 16 + g * 8), _mm256_setzero_ps());
                sum += reduce8_ps(prod);
            }
        }
    }
    return sum;
}

typedef float (*dot1_fn)(const uint8_t *, const uint8_t *, size_t);
typedef void (*dot2_fn)(const uint8_t *, const uint8_t *, const uint8_t *, size_t, float *, float *);

enum { K_Q1 = 0, K_Q2 = 1, K_Q8 = 2, K_PTQ = 3, K_Q4K = 4, K_Q6K = 5 };

static int kind_of(int dtype) {
    switch (dtype) {
        case 39: case 41: case 43: return K_Q1;
        case 42: case 142: return K_Q2;
        case 8: return K_Q8;
        case 143: return K_PTQ;
        case 12: return K_Q4K;
        case 14: return K_Q6K;
        default: return -1;
    }
}

static dot1_fn pick1(int kind, const char **name) {
    probe();
    if (kind == K_Q1) {
        if (vnni256_ok()) { *name = "vnni256"; return q1_vnni256; }
        if (avx2_ok()) { *name = "avx2_shuffle"; return q1_avx2; }
        *name = "scalar";
        return q1_scalar;
    }
    if (kind == K_Q2) {
        if (full_width() && vnni256_ok() && g_has_avx512dq) { *name = "vnni512x2"; return q2_vnni512x2; }
        if (avx2_ok()) { *name = "avx2_lut"; return q2_avx2_lut; }
        if (vnni256_ok()) { *name = "vnni256"; return q2_vnni256; }
        *name = "scalar";
        return q2_scalar;
    }
    if (kind == K_PTQ) {
        if (!g_ptq_ready) { build_ptq_tables(); g_ptq_ready = 1; }
        if (full_width() && g_has_avx512vl) { *name = "avx512"; return ptq_avx512; }
        if (avx2_ok()) { *name = "avx2"; return ptq_avx2; }
        *name = "scalar";
        return ptq_scalar;
    }
    if (kind == K_Q4K || kind == K_Q6K) {
        if (!avx2_ok()) { *name = "none"; return 0; }  /* the shipped baseline target has AVX2 + FMA */
        *name = "wide_f32x8_fma";
        return kind == K_Q4K ? q4k_f32 : q6k_f32;
    }
    *name = "scalar";
    return q8_scalar;
}

static dot2_fn pick2(int kind) {
    probe();
    if (!avx2_ok()) return 0;
    if (kind == K_Q1) return q1_avx2_x2;
    if (kind == K_Q2) return q2_avx2_lut_x2;
    return 0;
}

/* Name of the arm the dispatch selects for a weight dtype on this CPU
 * (hearth_quant::selected_kernel, hearth-quant/src/lib.rs:411-418). */
HS_API const char *hs_selected_kernel(int dtype) {
    int kind = kind_of(dtype);
    if (kind < 0) return "none";
    const char *nm = "";
    if (kind == K_Q2 && !g_q2_u8[255][0]) build_q2_tables();
    pick1(kind, &nm);
    return nm;
}

/* Single row, dispatched arm (the DotFn the kernel table installs). */
HS_API float hs_dot(int dtype, const uint8_t *w, const uint8_t *a, size_t n) {
    int kind = kind_of(dtype);
    if (kind < 0) return 0.0f;
    if (!g_q2_u8[255][0]) build_q2_tables();
    const char *nm;
    return pick1(kind, &nm)(w, a, n);
}

/* ----------------------------------------------------------------- pool -- */

/* Logical CPUs this process may run on, and the physical-core estimate
 * logical / threads-per-core from CPUID leaf 0x1F / 0x0B sub-leaf 0. */
HS_API int hs_logical_cores(void) {
    cpu_set_t set;
    if (sched_getaffinity(0, sizeof(set), &set) == 0) {
        int n = CPU_COUNT(&set);
        if (n > 0) return n;
    }
    return 4;
}
HS_API int hs_physical_cores(void) {
    int logical = hs_logical_cores();
    unsigned a, b, c, d;
    __cpuid(0, a, b, c, d);
    unsigned leaf = a >= 0x1f ? 0x1f : (a >= 0x0b ? 0x0b : 0);
    if (!leaf) return logical;
    __cpuid_count(leaf, 0, a, b, c, d);
    int tpc = (int)(b & 0xffff);
    if (tpc >= 2 && tpc <= logical) {
        int p = logical / tpc;
        return p > 0 ? p : 1;
    }
    return logical;
}

typedef struct {
    size_t n, seq_len, q8_stride, row_bytes, n_cols, tile;
    const uint8_t *w, *a;
    float *out;
    dot1_fn f1;
    dot2_fn f2;
} job_t;

static void rows_chunk(const job_t *j, size_t begin, size_t end) {
    size_t r = begin;
    while (r < end) {
        size_t tile_end = r + j->tile < end ? r + j->tile : end;
        size_t s = 0;
        if (j->f2)
            for (; s + 1 < j->seq_len; s += 2) {
                const uint8_t *a0 = j->a + s * j->q8_stride, *a1 = a0 + j->q8_stride;
                for (size_t row = r; row < tile_end; row++)
                    j->f2(j->w + row * j->row_bytes, a0, a1, j->n_cols, j->out + s * j->n + row,
                          j->out + (s + 1) * j->n + row);
            }
        for (; s < j->seq_len; s++) {
            const uint8_t *a = j->a + s * j->q8_stride;
            for (size_t row = r; row < tile_end; row++) j->out[s * j->n + row] = j->f1(j->w + row * j->row_bytes, a, j->n_cols);
        }
        r = tile_end;
    }
}

#define HS_MAX_THREADS 512
static struct {
    int nthreads;
    pthread_t th[HS_MAX_THREADS];
    _Atomic unsigned long gen;
    _Atomic int done[HS_MAX_THREADS];
    _Atomic int stop;
    job_t job;
} g_pool;

static void *worker(void *arg) {
    int id = (int)(intptr_t)arg;
    unsigned long seen = 0;
    for (;;) {
        unsigned long g;
        unsigned spins = 0;
        while ((g = atomic_load_explicit(&g_pool.gen, memory_order_acquire)) == seen) {
            if (++spins > 65536) sched_yield();
        }
        seen = g;
        if (atomic_load(&g_pool.stop)) return 0;
        const job_t *j = &g_pool.job;
        size_t T = (size_t)g_pool.nthreads, chunk = (j->n + T - 1) / T;
        size_t begin = (size_t)id * chunk, end = begin + chunk < j->n ? begin + chunk : j->n;
        if (begin < end) rows_chunk(j, begin, end);
        atomic_store_explicit(&g_pool.done[id], 1, memory_order_release);
    }
}

/* Start (or resize) the pool.  threads <= 0 selects the physical core count. */
HS_API int hs_pool_start(int threads) {
    probe();
    if (!g_q2_u8[255][0]) build_q2_tables();
    if (threads <= 0) threads = hs_physical_cores();
    if (threads > HS_MAX_THREADS) threads = HS_MAX_THREADS;
    if (g_pool.nthreads == threads) return threads;
    if (g_pool.nthreads) {
        atomic_store(&g_pool.stop, 1);
        atomic_fetch_add(&g_pool.gen, 1);
        for (int i = 0; i < g_pool.nthreads; i++) pthread_join(g_pool.th[i], 0);
        atomic_store(&g_pool.stop, 0);
    }
    g_pool.nthreads = threads;
    /* Workers start with seen = 0; publish the current generation as their baseline by resetting it. */
    atomic_store(&g_pool.gen, 0);
    for (int i = 0; i < threads; i++) pthread_create(&g_pool.th[i], 0, worker, (void *)(intptr_t)i);
    return threads;
}

HS_API void hs_pool_stop(void) {
    if (!g_pool.nthreads) return;
    atomic_store(&g_pool.stop, 1);
    atomic_fetch_add(&g_pool.gen, 1);
    for (int i = 0; i < g_pool.nthreads; i++) pthread_join(g_pool.th[i], 0);
    atomic_store(&g_pool.stop, 0);
    g_pool.nthreads = 0;
}

/* par_dot_rows_batched (seq_len == 1: par_dot_rows).  Returns 0, -1 for a dtype
 * without a dot here, -2 if the pool was not started.  For Q4_K / Q6_K (ids 12, 14) a_ptr holds f32 rows and
 * q8_stride is their stride in bytes (the per-row loop of matmul.rs:270-280 and its per-token repetition). */
HS_API int hs_par_dot_rows_batched(int dtype, size_t n, size_t seq_len, size_t q8_stride, const uint8_t *w_base,
                                   const uint8_t *a_ptr, float *out, size_t row_bytes, size_t n_cols) {
    int kind = kind_of(dtype);
    if (kind < 0) return -1;
    if (!g_pool.nthreads) return -2;
    if (n == 0 || seq_len == 0) return 0;
    const char *nm;
    job_t j = {n, seq_len, q8_stride, row_bytes, n_cols, 0, w_base, a_ptr, out, pick1(kind, &nm),
               seq_len > 1 ? pick2(kind) : 0};
    if (!j.f1) return -1;
    j.tile = 1048576 / row_bytes;
    if (j.tile < 1) j.tile = 1;
    if (g_pool.nthreads <= 1) {
        rows_chunk(&j, 0, n);
        return 0;
    }
    g_pool.job = j;
    for (int i = 0; i < g_pool.nthreads; i++) atomic_store_explicit(&g_pool.done[i], 0, memory_order_relaxed);
    atomic_fetch_add_explicit(&g_pool.gen, 1, memory_order_release);
    for (int i = 0; i < g_pool.nthreads; i++) {
        unsigned spins = 0;
        while (!atomic_load_explicit(&g_pool.done[i], memory_order_acquire))
            if (++spins > 65536) sched_yield();
    }
    return 0;
}
