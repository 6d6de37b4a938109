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
// Device layout (built once at upload, same bytes as the reference's):
//   panel = 32 consecutive rows; the 16-byte pieces of one 256-column block are interleaved over the rows,
//   piece p of (panel, blk) for lane l at kq[((panel*nblk + blk)*NP + p)*32 + l], so a warp reads 512
//   contiguous bytes per piece.  Q4_K: NP = 9 (header with d, dmin and the 12 scale bytes; one piece of
//   nibbles per 32-element sub-block).  Q6_K: NP = 13: the 256 six-bit values (low nibble from ql, high two bits
//   from qh) re-coded at upload into one 6-bit stream, element e at stream bits 6e..6e+5 (12 pieces, three per
//   64-element quarter), then 1 piece of int8 scales; the f16 d of every block in a separate array
//   d16[(panel*nblk + blk)*32 + l].  Same 210 bytes per block; the stream lets a field be turned into a float by
//   one logic operation (no nibble / bit-pair merge per weight).
//
// Kernel: lane = row, so all lanes of a warp use the same columns and x comes from shared memory as
// broadcasts; a warp takes one block (Q4_K) or a quarter block (Q6_K) per round, eight warps make 64 ordered
// terms per row and round; next round's pieces are loaded into the registers of the pieces just used up; one thread per (token, row)
// adds the terms in order, one round behind.  Up to four tokens share one pass over the weights in this kernel; from
// eight tokens on kq_wide_kernel (further down: two rows per lane, x by bulk copy, 8 or 16 tokens per expansion) runs.
// All multiply-adds, adds and multiplies are issued two elements at a time (fma / add / mul .rn.f32x2, each half rounded
// as the scalar instruction rounds it).
#include "common.cuh"

#include <type_traits>

namespace hb200 {

namespace {

constexpr int KQ_THREADS = 256;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ float h2f_bits(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
// Reduction of the eight accumulation lanes in the order ((l0+l4)+(l2+l6))+((l1+l5)+(l3+l7)), lanes held as the pairs
// (l0,l1) (l2,l3) (l4,l5) (l6,l7): three packed adds (add.rn.f32x2, two independently rounded fp32 sums per instruction
// on sm_100) and one scalar add.
__device__ __forceinline__ float reduce8(const float2* l) {
    const float2 q01 = __fadd2_rn(l[0], l[2]);  // (l0+l4, l1+l5)
    const float2 q23 = __fadd2_rn(l[1], l[3]);  // (l2+l6, l3+l7)
    const float2 h = __fadd2_rn(q01, q23);      // (q0+q2, q1+q3)
    return __fadd_rn(h.x, h.y);
}

template <int KIND, int MT = 1>
struct KqGeom {
    static constexpr int NP = (KIND == KIND_Q4K) ? 9 : 13;           // pieces per block
    // Q6_K: 64-element quarters a warp takes per round.  Two make a round long enough to carry its fixed cost (step
    // bookkeeping, barrier, ordered replay); with four tokens per pass the term buffer of two would not leave room
    // for two CTAs per SM.
    static constexpr int H = (MT <= 2) ? 2 : 1;
    static constexpr int BLK_PER_ROUND = (KIND == KIND_Q4K) ? 8 : 2 * H;  // blocks the eight warps cover per round
    static constexpr int CH = BLK_PER_ROUND * 256;                    // columns of x per round
    static constexpr int NW = (KIND == KIND_Q4K) ? 9 : 3 * H + 1;     // pieces a thread holds per round
    static constexpr int TERMS_PER_BLK = (KIND == KIND_Q4K) ? 8 : 32;
    static constexpr int TERMS = BLK_PER_ROUND * TERMS_PER_BLK;       // ordered terms per row and round
};

// Two term buffers, so that the ordered replay of a round runs under the arithmetic of the next one.
template <int KIND, int MT>
struct KqSmem {
    static_assert(MT <= 4, "eight and more tokens per pass run kq_wide_kernel");
    alignas(16) float x[2][MT][KqGeom<KIND, MT>::CH];
    alignas(16) float4 term[2][KqGeom<KIND, MT>::TERMS / 4][MT][32];  // four consecutive ordered terms of a row side by side
};

// What one launch works through: `mats` (device memory) or, when mats is null, the one matrix `single`.  Items are
// numbered across the matrices (item = panel * token tiles + token tile inside its matrix); with `chunks`
// ([gridDim.x + 1] item indices) CTA c owns items chunks[c] .. chunks[c+1]-1, a contiguous run balanced by rounds;
// without, the items are split evenly.
struct KqLaunch {
    const KqMat* mats;
    const int* chunks;
    int n_items;
    uint32_t magic;  // 0x4B000000 (2^23 as a float), kept a run-time value: as a literal it was re-materialised before every byte permute
    int* status;     // device word for an expired bounded wait (may be null)
    KqMat single;
};
using KqArgs = KqMat;

// ---- one-time re-tiling -------------------------------------------------------------------------------------------

template <int KIND>
__global__ void kq_repack_kernel(const uint8_t* __restrict__ raw, size_t row_bytes, int n_rows, int nblk, long long n_pieces,
                                 uint4* __restrict__ kq, unsigned short* __restrict__ d16) {
    constexpr int NP = KqGeom<KIND>::NP;
    constexpr int BB = (KIND == KIND_Q4K) ? 144 : 210;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pieces) return;
    const int lane = (int)(i & 31);
    const long long t = i >> 5;
    const int p = (int)(t % NP);
    const long long pb = t / NP;
    const int blk = (int)(pb % nblk);
    const int panel = (int)(pb / nblk);
    const int row = panel * 32 + lane;
    uint32_t w[4] = {0, 0, 0, 0};
    if (row < n_rows) {
        const uint8_t* blkp = raw + (size_t)row * row_bytes + (size_t)blk * BB;
        if (KIND == KIND_Q6K && p < 12) {
            // Words 4p..4p+3 of the block's 6-bit stream: element e (its low nibble from ql, its two high bits from qh,
            // qk_quant.rs:141-176) sits at stream bits 6e..6e+5.
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int bit0 = 32 * (4 * p + k);
                uint32_t word = 0;
                for (int e = bit0 / 6; e <= (bit0 + 31) / 6; e++) {
                    const uint32_t ql = blkp[e >> 1], qh = blkp[128 + (e >> 2)];
                    const uint32_t v = ((e & 1) ? (ql >> 4) : (ql & 0x0F)) | (((qh >> ((e & 3) << 1)) & 0x03) << 4);
                    const int pos = 6 * e - bit0;
                    word |= pos >= 0 ? (v << pos) : (v >> -pos);
                }
                w[k] = word;
            }
        } else {
            const uint8_t* src = blkp + (KIND == KIND_Q6K ? 192 : p * 16);  // 2-byte aligned at least
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const unsigned short lo = *reinterpret_cast<const unsigned short*>(src + 4 * k);
                const unsigned short hi = *reinterpret_cast<const unsigned short*>(src + 4 * k + 2);
                w[k] = (uint32_t)lo | ((uint32_t)hi << 16);
            }
        }
        if (KIND == KIND_Q6K && p == 0) d16[pb * 32 + lane] = *reinterpret_cast<const unsigned short*>(blkp + 208);
    } else if (KIND == KIND_Q6K && p == 0) {
        d16[pb * 32 + lane] = 0;
    }
    kq[i] = make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- the matvec ------------------------------------------------------------------------------------------------

// Items of a matrix: item = panel * token tiles + token tile, so the token tiles of one 32-row panel follow each other
// and re-read its weights while they are still in cache.
template <int MT>
__device__ __forceinline__ int kq_tiles(const KqMat& a) { return (a.seq_len + MT - 1) / MT; }

// One step of a CTA's work: round r of item `item` of matrix m.
struct KqStep {
    const KqMat* m;
    int r;        // round inside the item
    int rounds;   // rounds of an item of this matrix
    int panel;    // the item's 32-row panel and first token (one division per item, none per round)
    int tok0;
    int nblk;
};

// Resident CTAs per SM the register allocation of the Q6_K kernels is held to (0: none given).  The Q4_K kernels are
// left to the allocator: told any number it schedules more aggressively and spills.
template <int KIND, int MT>
constexpr int kq_min_ctas() { return KIND == KIND_Q6K ? (MT == 1 ? 3 : 2) : 0; }

template <int KIND, int MT>
__global__ void __launch_bounds__(KQ_THREADS, kq_min_ctas<KIND, MT>()) kq_gemv_kernel(const __grid_constant__ KqLaunch L) {
    using G = KqGeom<KIND, MT>;
    using S = KqSmem<KIND, MT>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    S& sm = *reinterpret_cast<S*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // This CTA's contiguous run of items.
    int it0, it1;
    if (L.chunks) {
        it0 = L.chunks[blockIdx.x];
        it1 = L.chunks[blockIdx.x + 1];
    } else {
        it0 = (int)(((long long)L.n_items * blockIdx.x) / gridDim.x);
        it1 = (int)(((long long)L.n_items * (blockIdx.x + 1)) / gridDim.x);
    }
    if (it0 >= it1) return;

    int mi = 0;  // matrix cursor of the step generator (items come in increasing order)
    auto first_step = [&](int gitem) {
        KqStep st;
        st.m = &L.single;
        if (L.mats) {
            while (gitem >= L.mats[mi].item_end) mi++;
            st.m = &L.mats[mi];
        }
        const int item = gitem - st.m->item_begin, tiles = kq_tiles<MT>(*st.m);
        st.panel = item / tiles;
        st.tok0 = (item - st.panel * tiles) * MT;
        st.nblk = st.m->nblk;
        st.r = 0;
        st.rounds = max(1, (st.nblk + G::BLK_PER_ROUND - 1) / G::BLK_PER_ROUND);
        return st;
    };
    // gnext: the global index of the item after the one `st` belongs to
    auto next_step = [&](const KqStep& st, int& gitem) {
        KqStep n = st;
        if (++n.r == st.rounds) {
            gitem++;
            if (gitem < it1) n = first_step(gitem);
        }
        return n;
    };

    auto stage = [&](const KqStep& st, int buf) {
        const KqMat& a = *st.m;
        const int tok0 = st.tok0;
        constexpr int PIECES = G::CH / 4;
        const bool vec_ok = ((a.n_cols & 3) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
        for (int idx = tid; idx < MT * PIECES; idx += KQ_THREADS) {
            const int m = idx / PIECES, p = idx % PIECES;
            const int col = st.r * G::CH + p * 4;
            float* dst = &sm.x[buf][m][p * 4];
            if (tok0 + m < a.seq_len && col + 3 < a.n_cols && vec_ok) {
                if (HB_IDX((size_t)(tok0 + m) * a.n_cols + col + 3, (size_t)a.seq_len * a.n_cols, 13))
                    cp_async16(dst, a.x + (size_t)(tok0 + m) * a.n_cols + col);
            } else {
#pragma unroll
                for (int k = 0; k < 4; k++)
                    dst[k] = (tok0 + m < a.seq_len && col + k < a.n_cols) ? a.x[(size_t)(tok0 + m) * a.n_cols + col + k] : 0.0f;
            }
        }
    };

    // Weight registers: w[] holds the pieces of the current round.  Q6_K refills it piece by piece, each piece as soon
    // as its last use in the current round is behind, with the piece the next round needs (one set of registers, no
    // copies; a load has most of a round to arrive).  Q4_K fetches the next round's nine pieces up front into a
    // second set and copies: refilled in place (one by one, or in two bursts) it executed 6 % fewer instructions but
    // issued at 63 % instead of 69 %, or spilled.  piece_ptr: this thread's first piece of a step; a step without a
    // block for this warp (the ragged last round, or no next step at all) points at the matrix's first block instead,
    // so that the refills need no branch: what they fetch then is never used.
    uint4 w[G::NW];
    uint32_t dcur = 0;
    const int uq0 = warp * G::H;  // Q6_K: the first of this warp's quarters among the round's 8 H
    auto block_of = [&](const KqStep& st) { return (KIND == KIND_Q4K) ? (st.r * 8 + warp) : (st.r * G::BLK_PER_ROUND + (uq0 >> 2)); };
    auto piece_ptr = [&](const KqStep& st) -> const uint4* {
        const int blk = block_of(st);
        size_t base = blk < st.nblk ? ((size_t)st.panel * st.nblk + blk) : 0;
        if (!HB_IDX(base, (size_t)st.m->n_panels * st.nblk, 11)) base = 0;
        return st.m->kq + (base * G::NP + (KIND == KIND_Q4K ? 0 : 3 * (uq0 & 3))) * 32 + lane;
    };
    // Q6_K: the scale piece is number 12 of the block (the pointer stands at piece 3q), d sits in its own array.
    auto q6_scales = [&](const uint4* p) { return __ldg(p + (12 - 3 * (uq0 & 3)) * 32); };
    auto q6_d = [&](const KqStep& st) -> uint32_t {
        const int blk = block_of(st);
        size_t base = blk < st.nblk ? ((size_t)st.panel * st.nblk + blk) : 0;
        if (!HB_IDX(base, (size_t)st.m->n_panels * st.nblk, 12)) base = 0;
        return __ldg(st.m->d16 + base * 32 + lane);
    };
    auto load_all = [&](const uint4* p, const KqStep& st) {
        if (KIND == KIND_Q4K) {
#pragma unroll
            for (int i = 0; i < 9; i++) w[i] = __ldg(p + i * 32);
        } else {
#pragma unroll
            for (int i = 0; i < 3 * G::H; i++) w[i] = __ldg(p + i * 32);
            w[3 * G::H] = q6_scales(p);
            dcur = q6_d(st);
        }
    };

    float run = 0.0f;  // thread tid < MT*32 owns the chain of (token tid/32, row tid%32)
    auto replay = [&](const KqStep& st, int buf) {
        if (tid < MT * 32) {
            const KqMat& a = *st.m;
            const int m = tid >> 5, row = tid & 31;
            const int nvalid = min(G::TERMS, G::TERMS_PER_BLK * (st.nblk - st.r * G::BLK_PER_ROUND));
            float acc = run;
            for (int k = 0; k < nvalid / 4; k++) {  // nvalid is a multiple of eight
                const float4 t = sm.term[buf][k][m][row];
                acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, t.x), t.y), t.z), t.w);
            }
            if (st.r == st.rounds - 1) {
                const int grow = st.panel * 32 + row;
                const int tok = st.tok0 + m;
                if (grow < a.n_rows && tok < a.seq_len && HB_IDX((size_t)tok * a.ld_out + grow, (size_t)(a.seq_len - 1) * a.ld_out + a.n_rows, 14))
                    a.out[(size_t)tok * a.ld_out + grow] = acc;
                acc = 0.0f;
            }
            run = acc;
        }
    };

    int gitem = it0;
    KqStep cur = first_step(gitem), prev = cur;
    stage(cur, 0);
    load_all(piece_ptr(cur), cur);
    for (int t = 0; gitem < it1; t++) {
        cp_async_commit_wait_all();
        __syncthreads();
        // The next step is worked out twice, here for the fetches and again at the end of the round to move on, so
        // that it does not occupy registers across the arithmetic in between.
        const uint4* pn;  // next round's pieces of this thread (after the last step it has no block: an idle fetch)
        uint32_t dnext = 0;
        {
            int gnext = gitem;
            const KqStep nxt = next_step(cur, gnext);
            if (gnext < it1) stage(nxt, (t + 1) & 1);
            pn = piece_ptr(nxt);
            if (KIND == KIND_Q6K) dnext = q6_d(nxt);
        }
        uint4 wn[KIND == KIND_Q4K ? 9 : 1];
        if (KIND == KIND_Q4K) {  // fetched up front into a second set of registers (see the note at w[])
#pragma unroll
            for (int i = 0; i < 9; i++) wn[i] = __ldg(pn + i * 32);
        }
        if (t > 0) replay(prev, (t - 1) & 1);  // one round behind, from the other term buffer

        const int buf = t & 1;
        const int tbuf = buf;
        const int nblk = cur.nblk, r = cur.r;
        if (KIND == KIND_Q4K) {
            const int blk = r * 8 + warp;
            if (blk < nblk) {
                const float d = h2f_bits(w[0].x & 0xffffu), dmin = h2f_bits(w[0].x >> 16);
                const uint32_t sw[3] = {w[0].y, w[0].z, w[0].w};  // the 12 scale bytes
                const uint32_t magic = L.magic;
                // FAST: nibble -> float without a shift, a mask and a convert per weight: a byte permute drops the nibble
                // into the mantissa of 2^23 (0x4B0000nn = 8388608 + n), and fma(2^23 + n, scf, -(2^23 * scf)) is the
                // correctly rounded n * scf, i.e. the same bits as the separate multiply (2^23 * scf is exact).  That
                // needs a finite scf = sc * d, i.e. a finite d; a block whose d is infinite or NaN takes the literal
                // multiply, so that inf and NaN come out where the reference has them.
                auto block_body = [&](auto fast_tag) {
                    constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
                    for (int sb = 0; sb < 8; sb++) {
                        const int i3 = (sb >> 1) * 3;
                        const uint32_t s0 = (sw[i3 >> 2] >> (8 * (i3 & 3))) & 0xff;
                        const uint32_t s1 = (sw[(i3 + 1) >> 2] >> (8 * ((i3 + 1) & 3))) & 0xff;
                        const uint32_t s2 = (sw[(i3 + 2) >> 2] >> (8 * ((i3 + 2) & 3))) & 0xff;
                        uint32_t sc, mn;
                        if ((sb & 1) == 0) { sc = s0 & 0x3F; mn = (s0 >> 6) | ((s1 & 0x0F) << 2); }
                        else { sc = (s1 >> 4) | ((s2 & 0x03) << 4); mn = (s2 >> 2) & 0x3F; }
                        const float scf = __fmul_rn((float)sc, d), mnf = __fmul_rn((float)mn, dmin);
                        const float c0 = __fmul_rn(-8388608.0f, scf);
                        const uint32_t qw[4] = {w[1 + sb].x, w[1 + sb].y, w[1 + sb].z, w[1 + sb].w};
                        // Every multiply-add, subtract and add below works on two neighbouring elements at once
                        // (fma.rn.f32x2 / add.rn.f32x2: each half rounded as the scalar instruction rounds it), which halves
                        // the issue slots of the arithmetic; a - b is computed as a + (-b), the same value and rounding.
                        const float2 scf2 = make_float2(scf, scf), c02 = make_float2(c0, c0), nmn2 = make_float2(-mnf, -mnf);
                        auto expand8 = [&](int tt, float2 (&v)[4]) {  // elements 8tt..8tt+7 of the sub-block live in word tt
                            if (FAST) {
                                const uint32_t ev = qw[tt] & 0x0F0F0F0Fu, od = (qw[tt] >> 4) & 0x0F0F0F0Fu;  // elements 0,2,4,6 / 1,3,5,7
#pragma unroll
                                for (int p = 0; p < 4; p++) {
                                    const float2 nf = make_float2(__uint_as_float(__byte_perm(ev, magic, 0x7540u + p)),
                                                                  __uint_as_float(__byte_perm(od, magic, 0x7540u + p)));
                                    v[p] = __fadd2_rn(__ffma2_rn(nf, scf2, c02), nmn2);
                                }
                            } else {
#pragma unroll
                                for (int p = 0; p < 4; p++)
                                    v[p] = make_float2(__fsub_rn(__fmul_rn((float)((qw[tt] >> (8 * p)) & 0xF), scf), mnf),
                                                       __fsub_rn(__fmul_rn((float)((qw[tt] >> (8 * p + 4)) & 0xF), scf), mnf));
                            }
                        };
                        const float2 zero2 = make_float2(0.0f, 0.0f);
                        float2 lanes[MT][4];
#pragma unroll
                        for (int tt = 0; tt < 4; tt++) {
                            float2 v[4];
                            expand8(tt, v);
#pragma unroll
                            for (int m = 0; m < MT; m++) {
                                const float4* xp = reinterpret_cast<const float4*>(&sm.x[buf][m][warp * 256 + sb * 32 + tt * 8]);
                                const float4 x0 = xp[0], x1 = xp[1];
                                const float2 xs[4] = {make_float2(x0.x, x0.y), make_float2(x0.z, x0.w), make_float2(x1.x, x1.y), make_float2(x1.z, x1.w)};
#pragma unroll
                                for (int p = 0; p < 4; p++) lanes[m][p] = __ffma2_rn(v[p], xs[p], tt == 0 ? zero2 : lanes[m][p]);
                            }
                        }
#pragma unroll
                        for (int m = 0; m < MT; m++)  // scalar stores into the float4 slots: no registers held across sub-blocks
                            reinterpret_cast<float*>(&sm.term[tbuf][warp * 2 + (sb >> 2)][m][lane])[sb & 3] = reduce8(lanes[m]);
                    }
                };
                if (fabsf(d) <= 65504.0f) block_body(std::true_type{});
                else block_body(std::false_type{});
            }
        } else {
            const int blk = r * G::BLK_PER_ROUND + (uq0 >> 2);
            if (blk < nblk) {
                const float d = h2f_bits(dcur);
                const uint32_t magic = L.magic;
                uint32_t scw[G::H];
#pragma unroll
                for (int h = 0; h < G::H; h++) {
                    const int q = (uq0 + h) & 3;
                    const uint4& sp = w[3 * G::H];
                    scw[h] = (q == 0) ? sp.x : (q == 1 ? sp.y : (q == 2 ? sp.z : sp.w));
                }
                w[3 * G::H] = q6_scales(pn);
                float tq[MT][4];
#pragma unroll
                for (int h = 0; h < G::H; h++) {
#pragma unroll
                    for (int g = 0; g < 4; g++) {  // 16 elements = 96 stream bits = words 3g..3g+2 of the quarter, one int8 scale
                        const int sci = (int)(int8_t)((scw[h] >> (8 * g)) & 0xff);
                        const float sd = __fmul_rn((float)sci, d);
                        // A field that sits s bits up in a word is used in place: (word & 0x3F << s) | 2^23 is the float
                        // 2^23 + quant * 2^s, minus (2^23 + 32 * 2^s) is (quant - 32) * 2^s exactly, and times sd / 2^s
                        // rounds as (quant - 32) * sd does (the factor is a power of two, sd / 4096 stays normal).
                        const float mul[3] = {sd, __fmul_rn(sd, 0.015625f), __fmul_rn(sd, 0.000244140625f)};
                        auto word = [&](int i) { const uint4& v = w[i >> 2]; return (i & 3) == 0 ? v.x : ((i & 3) == 1 ? v.y : ((i & 3) == 2 ? v.z : v.w)); };
                        const uint32_t A = word(12 * h + 3 * g), B = word(12 * h + 3 * g + 1), C = word(12 * h + 3 * g + 2);
                        // windows of three fields each, at stream bits 0, 18, 36, 54, 72 and (one field) 90
                        const uint32_t win[6] = {A, __funnelshift_r(A, B, 18), B >> 4, __funnelshift_r(B, C, 22), C >> 8, C >> 26};
                        // Two neighbouring elements per instruction (add / mul / fma .rn.f32x2, each half rounded as the scalar
                        // instruction rounds it).  Element i sits 6 (i % 3) bits up in its window, so the pair (2p, 2p+1) has the
                        // shifts (0,6), (12,0), (6,12) for p % 3 = 0, 1, 2.
                        const float2 mul2[3] = {make_float2(mul[0], mul[1]), make_float2(mul[2], mul[0]), make_float2(mul[1], mul[2])};
                        const float2 off2[3] = {make_float2(-(8388608.0f + 32.0f), -(8388608.0f + 2048.0f)),
                                                make_float2(-(8388608.0f + 131072.0f), -(8388608.0f + 32.0f)),
                                                make_float2(-(8388608.0f + 2048.0f), -(8388608.0f + 131072.0f))};
                        float2 qf[8];
#pragma unroll
                        for (int p = 0; p < 8; p++) {
                            const int i0 = 2 * p, i1 = 2 * p + 1;
                            const float2 f = make_float2(__uint_as_float((win[i0 / 3] & (0x3Fu << (6 * (i0 % 3)))) | magic),
                                                         __uint_as_float((win[i1 / 3] & (0x3Fu << (6 * (i1 % 3)))) | magic));
                            qf[p] = __fmul2_rn(__fadd2_rn(f, off2[p % 3]), mul2[p % 3]);
                        }
                        const float2 zero2 = make_float2(0.0f, 0.0f);
#pragma unroll
                        for (int hh = 0; hh < 2; hh++) {
                            const int u = 2 * g + hh;  // the quarter's u-th run of eight elements
#pragma unroll
                            for (int m = 0; m < MT; m++) {
                                const float4* xp = reinterpret_cast<const float4*>(&sm.x[buf][m][(uq0 + h) * 64 + u * 8]);
                                const float4 x0 = xp[0], x1 = xp[1];
                                float2 lanes[4];
                                lanes[0] = __ffma2_rn(qf[4 * hh + 0], make_float2(x0.x, x0.y), zero2);
                                lanes[1] = __ffma2_rn(qf[4 * hh + 1], make_float2(x0.z, x0.w), zero2);
                                lanes[2] = __ffma2_rn(qf[4 * hh + 2], make_float2(x1.x, x1.y), zero2);
                                lanes[3] = __ffma2_rn(qf[4 * hh + 3], make_float2(x1.z, x1.w), zero2);
                                tq[m][u & 3] = reduce8(lanes);
                                if ((u & 3) == 3) sm.term[tbuf][(uq0 + h) * 2 + (u >> 2)][m][lane] = make_float4(tq[m][0], tq[m][1], tq[m][2], tq[m][3]);
                            }
                        }
                        if (g >= 1) w[3 * h + g - 1] = __ldg(pn + (3 * h + g - 1) * 32);  // group g ends in the quarter's piece g - 1
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 3 * G::H; i++) w[i] = __ldg(pn + i * 32);
                w[3 * G::H] = q6_scales(pn);
            }
            dcur = dnext;
        }
        if (KIND == KIND_Q4K) {
#pragma unroll
            for (int i = 0; i < 9; i++) w[i] = wn[i];
        }
        prev = cur;
        cur = next_step(cur, gitem);
        if (gitem >= it1) {  // the last round's terms
            __syncthreads();
            replay(prev, t & 1);
        }
    }
}

// ---- eight tokens per pass -----------------------------------------------------------------------------------------
//
// With eight tokens per expanded weight the general kernel above is bound by shared memory, not by arithmetic: lane =
// row makes every read of x a broadcast, a broadcast 16-byte read costs two wavefronts of the one-per-cycle shared
// memory pipe, and it feeds only four multiply-adds per lane (measured on Q4_K: 56 % of that pipe, 35 % of the FMA
// pipe); the x of a round went through 16 cp.async instructions per thread, which cost a fifth of the time.  Here
//   * a lane owns TWO rows of the panel (li and li + 16), and the two halves of a warp work on different blocks of the
//     round (half 0 on the first half of the round's blocks, half 1 on the second), so one 16-byte read per lane - two
//     addresses per warp - feeds eight multiply-adds per lane;
//   * x sits in shared memory as two half rows per token (the columns of the first and of the second half of the
//     round's blocks), the second one 16 bytes further than a multiple of 128, so that the two halves of a warp hit
//     different banks;
//   * every half row is one bulk copy (cp.async.bulk, completion on an mbarrier) issued by one thread; an x that is
//     not 16-byte aligned goes through ordinary loads instead.
// A round is eight blocks of Q4_K (a warp: sub-blocks 0..3 or 4..7 of one block per half, 64 ordered terms per row) or
// four blocks of Q6_K (a warp: one 64-element quarter of one block per half, 128 ordered terms per row).  Each weight
// of a row is still expanded once per eight tokens, every multiply-add, add and reduction is the same operation on
// the same operands as in the general kernel, and the ordered replay is unchanged: same bits.  Weight pieces are
// refilled in place with the next round's as soon as they have been expanded.  The wait for a bulk copy is bounded:
// on expiry the CTA records status code 40 and stops.
template <int KIND, int MT>
struct KqWideGeom {
    // Q4_K: a (warp, half) unit takes SPU = 32 / MT sub-blocks of a block, so that its expanded weights serve MT tokens
    // and the x of a round (2 SPU blocks) and its terms fill the same shared memory for 8 and 16 (or 32) tokens per pass.
    static constexpr int SPU = (KIND == KIND_Q4K) ? 32 / MT : 0;
    static constexpr int BLK_PER_ROUND = (KIND == KIND_Q4K) ? 2 * SPU : 4;
    static constexpr int CH = BLK_PER_ROUND * 256;                   // columns of x per round
    static constexpr int HALF_COLS = CH / 2;
    static constexpr int HALF = HALF_COLS + 4;                       // floats per half row in shared memory
    static constexpr int TERMS_PER_BLK = (KIND == KIND_Q4K) ? 8 : 32;
    static constexpr int TERMS = BLK_PER_ROUND * TERMS_PER_BLK;      // ordered terms per row and round
    static constexpr int NP = (KIND == KIND_Q4K) ? 9 : 13;
    static_assert(KIND != KIND_Q4K || MT == 8 || MT == 16 || MT == 32, "Q4_K: 8, 16 or 32 tokens per pass");
    static_assert(KIND != KIND_Q6K || MT == 8, "Q6_K: 8 tokens per pass");
};

template <int KIND, int MT>
struct KqWideSmem {
    using W = KqWideGeom<KIND, MT>;
    alignas(16) float x[2][MT][2][W::HALF];
    // Ordered terms of a round, in groups of four consecutive terms (group k4, member c) per (token, row):
    //   Q4_K  term[half][k4 % (K4/2)][m][c][row] as floats, the second half's terms (written by lanes 16..31 of every warp)
    //         64 bytes further than a multiple of 128, so that one 4-byte store per lane has no bank conflict;
    //   Q6_K  term[k4][m][c / 2][row][c % 2]: an 8-byte store per lane, rows next to each other.
    static constexpr int K4 = W::TERMS / 4;
    static constexpr int TERM_HALF = (K4 / 2) * MT * 4 * 32 + (KIND == KIND_Q4K ? 16 : 0);  // floats per half
    alignas(16) float term[2 * TERM_HALF];
    alignas(8) unsigned long long bar[2];
    // float index of term (k4, m, c) of row `row`
    __device__ __forceinline__ static int term_at(int k4, int m, int c, int row) {
        const int hh = k4 >= K4 / 2 ? 1 : 0, kk = k4 - hh * (K4 / 2);
        if (KIND == KIND_Q4K) return hh * TERM_HALF + ((kk * MT + m) * 4 + c) * 32 + row;
        return hh * TERM_HALF + (((kk * MT + m) * 2 + (c >> 1)) * 32 + row) * 2 + (c & 1);
    }
};

__device__ __forceinline__ uint32_t kq_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool kq_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool kq_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 22); i++)
        if (kq_mbar_try(bar, parity)) return true;
    return false;
}

template <int KIND, int MT>
__global__ void __launch_bounds__(KQ_THREADS, 1) kq_wide_kernel(const __grid_constant__ KqLaunch L) {
    using W = KqWideGeom<KIND, MT>;
    using S = KqWideSmem<KIND, MT>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    S& sm = *reinterpret_cast<S*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int half = lane >> 4, li = lane & 15;  // rows li and li + 16
    // Q4_K: sub-blocks SPU part + u (u = 0..SPU-1) of block rb of the round.  Q6_K: quarter `part` of block rb.
    constexpr int SPU = (KIND == KIND_Q4K) ? W::SPU : 1;
    constexpr int UPB = (KIND == KIND_Q4K) ? 8 / SPU : 4;  // units (warps) per block
    const int part = warp % UPB;
    const int bih = warp / UPB;  // block inside this half of the round
    const int rb = half * (W::BLK_PER_ROUND / 2) + bih;

    int it0, it1;
    if (L.chunks) {
        it0 = L.chunks[blockIdx.x];
        it1 = L.chunks[blockIdx.x + 1];
    } else {
        it0 = (int)(((long long)L.n_items * blockIdx.x) / gridDim.x);
        it1 = (int)(((long long)L.n_items * (blockIdx.x + 1)) / gridDim.x);
    }
    if (it0 >= it1) return;

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(kq_smem_u32(&sm.bar[0])), "r"(1) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(kq_smem_u32(&sm.bar[1])), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    int mi = 0;
    auto first_step = [&](int gitem) {
        KqStep st;
        st.m = &L.single;
        if (L.mats) {
            while (gitem >= L.mats[mi].item_end) mi++;
            st.m = &L.mats[mi];
        }
        const int item = gitem - st.m->item_begin, tiles = kq_tiles<MT>(*st.m);
        st.panel = item / tiles;
        st.tok0 = (item - st.panel * tiles) * MT;
        st.nblk = st.m->nblk;
        st.r = 0;
        st.rounds = max(1, (st.nblk + W::BLK_PER_ROUND - 1) / W::BLK_PER_ROUND);
        return st;
    };
    auto next_step = [&](const KqStep& st, int& gitem) {
        KqStep n = st;
        if (++n.r == st.rounds) {
            gitem++;
            if (gitem < it1) n = first_step(gitem);
        }
        return n;
    };

    // x of round st.r into buffer buf.  Returns true when the data comes by bulk copy (completion on bar[buf]).
    auto stage = [&](const KqStep& st, int buf) -> bool {
        const KqMat& a = *st.m;
        const int tok0 = st.tok0;
        const int col0 = st.r * W::CH;
        const bool bulk_ok = ((a.n_cols & 3) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
        if (bulk_ok) {
            if (warp == 0) {  // one copy per lane and turn: issued by one thread they would make its warp the round's straggler
                const int ntok = min(MT, a.seq_len - tok0);
                // valid columns of each half (multiples of 256)
                const int c0 = min(W::HALF_COLS, a.n_cols - col0), c1 = max(0, min(W::HALF_COLS, a.n_cols - col0 - W::HALF_COLS));
                const uint32_t bar = kq_smem_u32(&sm.bar[buf]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                if (lane == 0)
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)(ntok * (c0 + c1) * 4)) : "memory");
                __syncwarp();
                for (int c = lane; c < 2 * ntok; c += 32) {
                    const int m = c >> 1, hh = c & 1;
                    const int cols = hh ? c1 : c0;
                    if (cols > 0 && HB_IDX((size_t)(tok0 + m) * a.n_cols + col0 + hh * W::HALF_COLS + cols - 1, (size_t)a.seq_len * a.n_cols, 17)) {
                        const float* src = a.x + (size_t)(tok0 + m) * a.n_cols + col0 + hh * W::HALF_COLS;
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                         kq_smem_u32(&sm.x[buf][m][hh][0])),
                                     "l"(src), "r"((uint32_t)(cols * 4)), "r"(bar)
                                     : "memory");
                    }
                }
            }
            return true;
        }
        for (int idx = tid; idx < MT * W::CH; idx += KQ_THREADS) {
            const int m = idx / W::CH, c = idx % W::CH;
            const int col = col0 + c;
            sm.x[buf][m][c / W::HALF_COLS][c % W::HALF_COLS] =
                (tok0 + m < a.seq_len && col < a.n_cols) ? a.x[(size_t)(tok0 + m) * a.n_cols + col] : 0.0f;
        }
        return false;
    };

    // Index of this lane's block in a step (panel * nblk + blk); a step without that block (the ragged last round, or
    // no next step) gives the matrix's first block: what is fetched from it is never used.
    auto block_index = [&](const KqStep& st) -> size_t {
        const int blk = st.r * W::BLK_PER_ROUND + rb;
        const size_t base = blk < st.nblk ? ((size_t)st.panel * st.nblk + blk) : 0;
        return HB_IDX(base, (size_t)st.m->n_panels * st.nblk, 16) ? base : 0;
    };
    // Q4_K: headers hd[row] and the four sub-block pieces pc[u][row].  Q6_K: the quarter's three stream pieces pc[i][row],
    // its four int8 scales sq[row] and the block's d dq[row].
    uint4 hd[2], pc[4][2];
    uint32_t sq[2], dq[2];
    auto piece0 = [&](const KqStep& st) -> const uint4* {
        return st.m->kq + (block_index(st) * W::NP + (KIND == KIND_Q4K ? 0 : 3 * part)) * 32 + li;
    };
    auto q6_scale_word = [&](const KqStep& st, int rr) -> uint32_t {
        return __ldg(reinterpret_cast<const uint32_t*>(st.m->kq + (block_index(st) * 13 + 12) * 32 + li + rr * 16) + part);
    };
    auto q6_d = [&](const KqStep& st, int rr) -> uint32_t { return __ldg(st.m->d16 + block_index(st) * 32 + li + rr * 16); };
    auto load_all = [&](const KqStep& st) {
        const uint4* p = piece0(st);
#pragma unroll
        for (int rr = 0; rr < 2; rr++) {
            if (KIND == KIND_Q4K) {
                hd[rr] = __ldg(p + rr * 16);
#pragma unroll
                for (int u = 0; u < SPU; u++) pc[u][rr] = __ldg(p + (1 + SPU * part + u) * 32 + rr * 16);
            } else {
#pragma unroll
                for (int i = 0; i < 3; i++) pc[i][rr] = __ldg(p + i * 32 + rr * 16);
                sq[rr] = q6_scale_word(st, rr);
                dq[rr] = q6_d(st, rr);
            }
        }
    };

    float run[(MT * 32 + KQ_THREADS - 1) / KQ_THREADS];  // thread tid owns the chain of (token tid / 32, row tid % 32)
#pragma unroll
    for (int c = 0; c < (MT * 32 + KQ_THREADS - 1) / KQ_THREADS; c++) run[c] = 0.0f;
    auto replay = [&](const KqStep& st) {
        const KqMat& a = *st.m;
        const int nvalid = min(W::TERMS, W::TERMS_PER_BLK * (st.nblk - st.r * W::BLK_PER_ROUND));
#pragma unroll
        for (int c = 0; c < (MT * 32 + KQ_THREADS - 1) / KQ_THREADS; c++) {
            const int chain = tid + c * KQ_THREADS;
            if (chain < MT * 32) {
                const int m = chain >> 5, row = chain & 31;
                float acc = run[c];
                for (int k = 0; k < nvalid / 4; k++) {
                    float t0, t1, t2, t3;
                    if (KIND == KIND_Q4K) {
                        const float* tp = &sm.term[S::term_at(k, m, 0, row)];
                        t0 = tp[0]; t1 = tp[32]; t2 = tp[64]; t3 = tp[96];
                    } else {
                        const float2 ta = *reinterpret_cast<const float2*>(&sm.term[S::term_at(k, m, 0, row)]);
                        const float2 tb = *reinterpret_cast<const float2*>(&sm.term[S::term_at(k, m, 2, row)]);
                        t0 = ta.x; t1 = ta.y; t2 = tb.x; t3 = tb.y;
                    }
                    acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, t0), t1), t2), t3);
                }
                if (st.r == st.rounds - 1) {
                    const int grow = st.panel * 32 + row;
                    const int tok = st.tok0 + m;
                    if (grow < a.n_rows && tok < a.seq_len && HB_IDX((size_t)tok * a.ld_out + grow, (size_t)(a.seq_len - 1) * a.ld_out + a.n_rows, 18))
                        a.out[(size_t)tok * a.ld_out + grow] = acc;
                    acc = 0.0f;
                }
                run[c] = acc;
            }
        }
    };

    int gitem = it0;
    KqStep cur = first_step(gitem), prev = cur;
    uint32_t bulk = 0;   // bit b: buffer b is being filled by a bulk copy whose completion has not been waited for yet
    uint32_t phase = 0;  // bit b: parity of the next completion of bar[b]
    bulk = stage(cur, 0) ? 1u : 0u;
    load_all(cur);
    const uint32_t magic = L.magic;
    const float2 zero2 = make_float2(0.0f, 0.0f);
    for (int t = 0; gitem < it1; t++) {
        const int buf = t & 1;
        if ((bulk >> buf) & 1u) {
            if (!kq_mbar_wait(kq_smem_u32(&sm.bar[buf]), (phase >> buf) & 1u)) {
                if (L.status) atomicCAS(L.status, 0, 40);
                return;  // the copy engine did not deliver within the bound: nothing sensible can follow
            }
            phase ^= 1u << buf;
        }
        __syncthreads();
        int gnext = gitem;
        const KqStep nxt = next_step(cur, gnext);
        {
            const bool nb_bulk = (gnext < it1) ? stage(nxt, buf ^ 1) : false;
            bulk = (bulk & ~(1u << (buf ^ 1))) | ((nb_bulk ? 1u : 0u) << (buf ^ 1));
        }
        const uint4* pn = piece0(nxt);
        if (cur.r * W::BLK_PER_ROUND + rb < cur.nblk) {
            if constexpr (KIND == KIND_Q4K) {
                float d[2], dmin[2];
                uint32_t sw[2][3];  // the 12 scale bytes of the block (q4_k.rs:51-96)
#pragma unroll
                for (int rr = 0; rr < 2; rr++) {
                    d[rr] = h2f_bits(hd[rr].x & 0xffffu);
                    dmin[rr] = h2f_bits(hd[rr].x >> 16);
                    sw[rr][0] = hd[rr].y; sw[rr][1] = hd[rr].z; sw[rr][2] = hd[rr].w;
                    hd[rr] = __ldg(pn + rr * 16);
                }
#pragma unroll
                for (int u = 0; u < SPU; u++) {
                    const int sb = SPU * part + u;  // sub-block of the block; its pair sb >> 1 owns scale bytes 3 (sb >> 1) .. + 2
                    float2 vv[2][4][4];
#pragma unroll
                    for (int rr = 0; rr < 2; rr++) {
                        // the pair's three bytes as one window: bytes o .. o + 2 of the 12, o = 3 (sb >> 1)
                        const int o = 3 * (sb >> 1), wi = o >> 2;
                        const uint32_t lo = wi == 0 ? sw[rr][0] : (wi == 1 ? sw[rr][1] : sw[rr][2]);
                        const uint32_t hi = wi == 0 ? sw[rr][1] : (wi == 1 ? sw[rr][2] : 0u);
                        const uint32_t win = __funnelshift_r(lo, hi, 8 * (o & 3));
                        const uint32_t s0 = win & 0xffu, s1 = (win >> 8) & 0xffu, s2 = (win >> 16) & 0xffu;
                        const bool odd = sb & 1;
                        const uint32_t sc = odd ? ((s1 >> 4) | ((s2 & 0x03) << 4)) : (s0 & 0x3F);
                        const uint32_t mn = odd ? ((s2 >> 2) & 0x3F) : ((s0 >> 6) | ((s1 & 0x0F) << 2));
                        const float scf = __fmul_rn((float)sc, d[rr]), mnf = __fmul_rn((float)mn, dmin[rr]);
                        const uint32_t qw[4] = {pc[u][rr].x, pc[u][rr].y, pc[u][rr].z, pc[u][rr].w};
                        if (fabsf(d[rr]) <= 65504.0f) {
                            // nibble -> float by a byte permute into the mantissa of 2^23, then fma(2^23 + n, scf, -(2^23 scf)):
                            // the correctly rounded n * scf (see the general kernel), two elements per instruction
                            const float c0 = __fmul_rn(-8388608.0f, scf);
                            const float2 scf2 = make_float2(scf, scf), c02 = make_float2(c0, c0), nmn2 = make_float2(-mnf, -mnf);
#pragma unroll
                            for (int tt = 0; tt < 4; tt++) {
                                const uint32_t ev = qw[tt] & 0x0F0F0F0Fu, od = (qw[tt] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                                for (int p = 0; p < 4; p++) {
                                    const float2 nf = make_float2(__uint_as_float(__byte_perm(ev, magic, 0x7540u + p)),
                                                                  __uint_as_float(__byte_perm(od, magic, 0x7540u + p)));
                                    vv[rr][tt][p] = __fadd2_rn(__ffma2_rn(nf, scf2, c02), nmn2);
                                }
                            }
                        } else {  // an infinite or NaN d: the literal multiply and subtract, so that inf and NaN come out as in the reference
#pragma unroll
                            for (int tt = 0; tt < 4; tt++)
#pragma unroll
                                for (int p = 0; p < 4; p++)
                                    vv[rr][tt][p] = make_float2(__fsub_rn(__fmul_rn((float)((qw[tt] >> (8 * p)) & 0xF), scf), mnf),
                                                                __fsub_rn(__fmul_rn((float)((qw[tt] >> (8 * p + 4)) & 0xF), scf), mnf));
                        }
                        pc[u][rr] = __ldg(pn + (1 + SPU * part + u) * 32 + rr * 16);
                    }
                    const float* xsub = &sm.x[buf][0][half][bih * 256 + sb * 32];
                    float* tdst = &sm.term[S::term_at(rb * 2 + (sb >> 2), 0, sb & 3, li)];  // token m, row li + 16 rr: + m * 128 + rr * 16
                    // The terms of eight tokens at a time are kept in registers and stored after their loop: with a store
                    // between two tokens the compiler cannot move the next token's reads of x (same shared memory) ahead of
                    // it, and every token would wait out its own load, multiply-add and reduction latencies alone.
#pragma unroll
                    for (int m0 = 0; m0 < MT; m0 += 8) {
                        float tv[8][2];
#pragma unroll
                        for (int mm = 0; mm < 8; mm++) {
                            const int m = m0 + mm;
                            float2 l0[4], l1[4];
#pragma unroll
                            for (int tt = 0; tt < 4; tt++) {
                                const float4* xp = reinterpret_cast<const float4*>(xsub + m * (2 * W::HALF) + tt * 8);
                                const float4 x0 = xp[0], x1 = xp[1];
                                const float2 xs[4] = {make_float2(x0.x, x0.y), make_float2(x0.z, x0.w), make_float2(x1.x, x1.y), make_float2(x1.z, x1.w)};
#pragma unroll
                                for (int p = 0; p < 4; p++) {
                                    l0[p] = __ffma2_rn(vv[0][tt][p], xs[p], tt == 0 ? zero2 : l0[p]);
                                    l1[p] = __ffma2_rn(vv[1][tt][p], xs[p], tt == 0 ? zero2 : l1[p]);
                                }
                            }
                            tv[mm][0] = reduce8(l0);
                            tv[mm][1] = reduce8(l1);
                        }
#pragma unroll
                        for (int mm = 0; mm < 8; mm++) {
                            tdst[(m0 + mm) * 128] = tv[mm][0];
                            tdst[(m0 + mm) * 128 + 16] = tv[mm][1];
                        }
                    }
                }
            } else {
                float d[2];
                uint32_t scw[2];
#pragma unroll
                for (int rr = 0; rr < 2; rr++) {
                    d[rr] = h2f_bits(dq[rr]);
                    scw[rr] = sq[rr];
                    sq[rr] = q6_scale_word(nxt, rr);
                    dq[rr] = q6_d(nxt, rr);
                }
#pragma unroll
                for (int g = 0; g < 4; g++) {  // 16 elements = 96 stream bits = words 3g..3g+2 of the quarter, one int8 scale
                    float2 qf[2][8];
#pragma unroll
                    for (int rr = 0; rr < 2; rr++) {
                        const int sci = (int)(int8_t)((scw[rr] >> (8 * g)) & 0xff);
                        const float sd = __fmul_rn((float)sci, d[rr]);
                        // (word & 0x3F << s) | 2^23 is the float 2^23 + quant * 2^s, minus (2^23 + 32 * 2^s) is
                        // (quant - 32) * 2^s exactly, and times sd / 2^s rounds as (quant - 32) * sd does (see the general kernel)
                        const float mul[3] = {sd, __fmul_rn(sd, 0.015625f), __fmul_rn(sd, 0.000244140625f)};
                        auto word = [&](int i) { const uint4& v = pc[i >> 2][rr]; return (i & 3) == 0 ? v.x : ((i & 3) == 1 ? v.y : ((i & 3) == 2 ? v.z : v.w)); };
                        const uint32_t A = word(3 * g), B = word(3 * g + 1), C = word(3 * g + 2);
                        const uint32_t win[6] = {A, __funnelshift_r(A, B, 18), B >> 4, __funnelshift_r(B, C, 22), C >> 8, C >> 26};
                        const float2 mul2[3] = {make_float2(mul[0], mul[1]), make_float2(mul[2], mul[0]), make_float2(mul[1], mul[2])};
                        const float2 off2[3] = {make_float2(-(8388608.0f + 32.0f), -(8388608.0f + 2048.0f)),
                                                make_float2(-(8388608.0f + 131072.0f), -(8388608.0f + 32.0f)),
                                                make_float2(-(8388608.0f + 2048.0f), -(8388608.0f + 131072.0f))};
#pragma unroll
                        for (int p = 0; p < 8; p++) {
                            const int i0 = 2 * p, i1 = 2 * p + 1;
                            const float2 f = make_float2(__uint_as_float((win[i0 / 3] & (0x3Fu << (6 * (i0 % 3)))) | magic),
                                                         __uint_as_float((win[i1 / 3] & (0x3Fu << (6 * (i1 % 3)))) | magic));
                            qf[rr][p] = __fmul2_rn(__fadd2_rn(f, off2[p % 3]), mul2[p % 3]);
                        }
                        if (g >= 1) pc[g - 1][rr] = __ldg(pn + (g - 1) * 32 + rr * 16);  // group g ends in the quarter's piece g - 1
                    }
                    const float* xsub = &sm.x[buf][0][half][bih * 256 + part * 64 + g * 16];
                    // the two terms of the group are components 2 (g & 1), 2 (g & 1) + 1 of the row's float4 number (g >> 1) of the quarter
                    float* tdst = &sm.term[S::term_at((rb * 4 + part) * 2 + (g >> 1), 0, 2 * (g & 1), li)];  // token m, row li + 16 rr: + m * 128 + rr * 32
                    float2 tv[MT][2];  // stored after the loop, see the Q4_K branch
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const float4* xp = reinterpret_cast<const float4*>(xsub + m * (2 * W::HALF));
                        const float4 xa = xp[0], xb = xp[1], xc = xp[2], xd = xp[3];
                        const float2 xs[8] = {make_float2(xa.x, xa.y), make_float2(xa.z, xa.w), make_float2(xb.x, xb.y), make_float2(xb.z, xb.w),
                                              make_float2(xc.x, xc.y), make_float2(xc.z, xc.w), make_float2(xd.x, xd.y), make_float2(xd.z, xd.w)};
#pragma unroll
                        for (int rr = 0; rr < 2; rr++) {
                            float2 la[4], lb[4];
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                la[k] = __ffma2_rn(qf[rr][k], xs[k], zero2);
                                lb[k] = __ffma2_rn(qf[rr][4 + k], xs[4 + k], zero2);
                            }
                            tv[m][rr] = make_float2(reduce8(la), reduce8(lb));
                        }
                    }
#pragma unroll
                    for (int m = 0; m < MT; m++)
#pragma unroll
                        for (int rr = 0; rr < 2; rr++) *reinterpret_cast<float2*>(tdst + m * 128 + rr * 32) = tv[m][rr];
                }
                pc[2][0] = __ldg(pn + 2 * 32);
                pc[2][1] = __ldg(pn + 2 * 32 + 16);
            }
        } else {
            load_all(nxt);
        }
        prev = cur;
        cur = nxt;
        gitem = gnext;
        __syncthreads();  // the round's terms are complete; the next round's barrier protects them again
        replay(prev);
    }
}

// Resident CTAs per SM of each instantiation, measured by the occupancy API at prepare time: the grid of the
// persistent kernel is sized to exactly one wave.
int g_kq_ctas[2][17] = {};

template <int KIND, int MT>
int launch_mt(const KqLaunch& L, int grid, cudaStream_t st) {
    if (L.n_items <= 0 || grid <= 0) return 0;
    if constexpr (MT >= 8) kq_wide_kernel<KIND, MT><<<grid, KQ_THREADS, sizeof(KqWideSmem<KIND, MT>), st>>>(L);
    else kq_gemv_kernel<KIND, MT><<<grid, KQ_THREADS, sizeof(KqSmem<KIND, MT>), st>>>(L);
    HB_CUDA(cudaGetLastError());
    return 0;
}

template <int KIND>
int launch_kind(const KqLaunch& L, int mt, int grid, cudaStream_t st) {
    if (mt == 1) return launch_mt<KIND, 1>(L, grid, st);
    if (mt == 2) return launch_mt<KIND, 2>(L, grid, st);
    if (mt == 8) return launch_mt<KIND, 8>(L, grid, st);
    if constexpr (KIND == KIND_Q4K) {
        if (mt == 16) return launch_mt<KIND, 16>(L, grid, st);
    }
    return launch_mt<KIND, 4>(L, grid, st);
}

template <int KIND, int MT>
int prepare_one() {
    int n = 0;
    if constexpr (MT >= 8) {
        HB_CUDA(cudaFuncSetAttribute(kq_wide_kernel<KIND, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(KqWideSmem<KIND, MT>)));
        HB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kq_wide_kernel<KIND, MT>, KQ_THREADS, sizeof(KqWideSmem<KIND, MT>)));
    } else {
        HB_CUDA(cudaFuncSetAttribute(kq_gemv_kernel<KIND, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(KqSmem<KIND, MT>)));
        HB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kq_gemv_kernel<KIND, MT>, KQ_THREADS, sizeof(KqSmem<KIND, MT>)));
    }
    g_kq_ctas[KIND == KIND_Q4K ? 0 : 1][MT] = n > 0 ? n : 1;
    return 0;
}

}  // namespace

int kquant_prepare() {
    int rc;
    if ((rc = prepare_one<KIND_Q4K, 1>())) return rc;
    if ((rc = prepare_one<KIND_Q4K, 2>())) return rc;
    if ((rc = prepare_one<KIND_Q4K, 4>())) return rc;
    if ((rc = prepare_one<KIND_Q4K, 8>())) return rc;
    if ((rc = prepare_one<KIND_Q4K, 16>())) return rc;
    if ((rc = prepare_one<KIND_Q6K, 1>())) return rc;
    if ((rc = prepare_one<KIND_Q6K, 2>())) return rc;
    if ((rc = prepare_one<KIND_Q6K, 4>())) return rc;
    if ((rc = prepare_one<KIND_Q6K, 8>())) return rc;
    return 0;
}

size_t kquant_pieces_per_block(int kind) { return kind == KIND_Q4K ? 9 : 13; }

HB_BOUNDS_FETCH(bounds_fetch_kquant)

int launch_kquant_repack(int kind, const uint8_t* raw, size_t row_bytes, int n_rows, int nblk, int n_panels, uint4* kq,
                         unsigned short* d16, cudaStream_t st) {
    const long long n_pieces = (long long)n_panels * nblk * (long long)kquant_pieces_per_block(kind) * 32;
    if (n_pieces <= 0) return 0;
    const unsigned grid = (unsigned)((n_pieces + 255) / 256);
    if (kind == KIND_Q4K) kq_repack_kernel<KIND_Q4K><<<grid, 256, 0, st>>>(raw, row_bytes, n_rows, nblk, n_pieces, kq, d16);
    else if (kind == KIND_Q6K) kq_repack_kernel<KIND_Q6K><<<grid, 256, 0, st>>>(raw, row_bytes, n_rows, nblk, n_pieces, kq, d16);
    else { set_error("kquant repack: kind %d", kind); return -7; }
    HB_CUDA(cudaGetLastError());
    return 0;
}

// One pass over the weights serves 1, 2, 4 or 8 tokens: from eight tokens on the weights are expanded once per eight.
// One pass over the weights serves 1, 2, 4 or 8 tokens, Q4_K also 16.  From eight tokens on, the cheaper tiling: a pass
// costs its tokens (padding included) plus a fixed share worth 1.7 tokens (measured on the 14336 x 4096 set: 0.615 ms for
// a pass of eight, 1.123 ms for a pass of sixteen).  Thirty-two tokens per pass (rounds of two blocks) measured slower
// than two passes of sixteen: 2.49 against 2.25 ms, the fixed cost of four times as many rounds outweighs the expansion saved.
int kquant_tokens_per_pass(int kind, int seq_len) {
    if (seq_len < 8) return seq_len == 1 ? 1 : (seq_len == 2 ? 2 : 4);
    if (kind != KIND_Q4K) return 8;
    const double c8 = (double)((seq_len + 7) / 8) * (8 + 1.7), c16 = (double)((seq_len + 15) / 16) * (16 + 1.7);
    return c16 < c8 ? 16 : 8;
}

int kquant_items(int kind, int n_panels, int seq_len) {
    const int mt = kquant_tokens_per_pass(kind, seq_len);
    return ((seq_len + mt - 1) / mt) * n_panels;
}

int kquant_rounds(int kind, int nblk) {
    const int per = (kind == KIND_Q4K) ? 8 : 2;
    const int r = (nblk + per - 1) / per;
    return r > 0 ? r : 1;
}

int kquant_grid(int kind, int mt, int sm_count, int n_items) {
    const int per_sm = g_kq_ctas[kind == KIND_Q4K ? 0 : 1][mt] > 0 ? g_kq_ctas[kind == KIND_Q4K ? 0 : 1][mt] : 1;
    const int grid = sm_count * per_sm;
    return grid > n_items ? n_items : grid;
}

int launch_kquant_gemv(int kind, const uint4* kq, const unsigned short* d16, int n_rows, int n_cols, int nblk, int n_panels,
                       const float* x, int seq_len, float* out, int ld_out, int sm_count, cudaStream_t st, int* status) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    KqLaunch L;
    L.mats = nullptr; L.chunks = nullptr; L.magic = 0x4B000000u; L.status = status;
    KqMat& a = L.single;
    a.kq = kq; a.d16 = d16; a.x = x; a.out = out;
    a.n_rows = n_rows; a.n_cols = n_cols; a.nblk = nblk; a.n_panels = n_panels; a.seq_len = seq_len; a.ld_out = ld_out;
    const int mt = kquant_tokens_per_pass(kind, seq_len);
    a.item_begin = 0;
    a.item_end = L.n_items = kquant_items(kind, n_panels, seq_len);
    const int grid = kquant_grid(kind, mt, sm_count, L.n_items);
    if (kind == KIND_Q4K) return launch_kind<KIND_Q4K>(L, mt, grid, st);
    if (kind == KIND_Q6K) return launch_kind<KIND_Q6K>(L, mt, grid, st);
    set_error("kquant_gemv: kind %d", kind);
    return -7;
}

int launch_kquant_gemv_list(int kind, int mt, const KqMat* mats_dev, const int* chunks_dev, int n_items, int grid, cudaStream_t st,
                            int* status) {
    KqLaunch L;
    L.mats = mats_dev; L.chunks = chunks_dev; L.n_items = n_items; L.magic = 0x4B000000u; L.status = status;
    L.single = KqMat{};
    if (kind == KIND_Q4K) return launch_kind<KIND_Q4K>(L, mt, grid, st);
    if (kind == KIND_Q6K) return launch_kind<KIND_Q6K>(L, mt, grid, st);
    set_error("kquant_gemv: kind %d", kind);
    return -7;
}

}  // namespace hb200
