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
//   nibbles per 32-element sub-block).  Q6_K: NP = 13 (8 of ql, 4 of qh, 1 of int8 scales) and the f16 d of
//   every block in a separate array d16[(panel*nblk + blk)*32 + l].
//
// Kernel: lane = row, so all lanes of a warp use the same columns and x comes from shared memory as
// broadcasts; a warp takes one block (Q4_K) or a quarter block (Q6_K) per round, eight warps make 64 ordered
// terms per row and round; next round's pieces are prefetched into registers; one thread per (token, row)
// adds the terms in order, one round behind.  Up to four tokens share one pass over the weights.
#include "common.cuh"

#include <type_traits>

namespace hb200 {

namespace {

constexpr int KQ_THREADS = 256;
constexpr int TERMS = 64;  // ordered terms per row and round

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ float h2f_bits(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
__device__ __forceinline__ float reduce8(const float* l) {
    const float q0 = __fadd_rn(l[0], l[4]), q1 = __fadd_rn(l[1], l[5]);
    const float q2 = __fadd_rn(l[2], l[6]), q3 = __fadd_rn(l[3], l[7]);
    return __fadd_rn(__fadd_rn(q0, q2), __fadd_rn(q1, q3));
}

template <int KIND>
struct KqGeom {
    static constexpr int NP = (KIND == KIND_Q4K) ? 9 : 13;           // pieces per block
    static constexpr int BLK_PER_ROUND = (KIND == KIND_Q4K) ? 8 : 2;  // blocks the eight warps cover per round
    static constexpr int CH = BLK_PER_ROUND * 256;                    // columns of x per round
    static constexpr int NW = (KIND == KIND_Q4K) ? 9 : 4;             // pieces a thread holds per round
    static constexpr int TERMS_PER_BLK = (KIND == KIND_Q4K) ? 8 : 32;
};

template <int KIND, int MT>
struct KqSmem {
    alignas(16) float x[2][MT][KqGeom<KIND>::CH];
    alignas(16) float term[2][TERMS][MT][32];
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
        const uint8_t* src = raw + (size_t)row * row_bytes + (size_t)blk * BB + p * 16;  // 2-byte aligned at least
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const unsigned short lo = *reinterpret_cast<const unsigned short*>(src + 4 * k);
            const unsigned short hi = *reinterpret_cast<const unsigned short*>(src + 4 * k + 2);
            w[k] = (uint32_t)lo | ((uint32_t)hi << 16);
        }
        if (KIND == KIND_Q6K && p == 0)
            d16[pb * 32 + lane] = *reinterpret_cast<const unsigned short*>(raw + (size_t)row * row_bytes + (size_t)blk * BB + 208);
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
    int item;     // item index inside its matrix
    int r;        // round inside the item
    int rounds;   // rounds of an item of this matrix
};

template <int KIND, int MT>
__global__ void __launch_bounds__(KQ_THREADS) kq_gemv_kernel(const __grid_constant__ KqLaunch L) {
    using G = KqGeom<KIND>;
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
    auto rounds_of = [&](const KqMat* m) { return max(1, (m->nblk + G::BLK_PER_ROUND - 1) / G::BLK_PER_ROUND); };
    auto first_step = [&](int gitem) {
        KqStep st;
        st.m = &L.single;
        if (L.mats) {
            while (gitem >= L.mats[mi].item_end) mi++;
            st.m = &L.mats[mi];
        }
        st.item = gitem - st.m->item_begin;
        st.r = 0;
        st.rounds = rounds_of(st.m);
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
        const int tok0 = (st.item % kq_tiles<MT>(a)) * MT;
        constexpr int PIECES = G::CH / 4;
        const bool vec_ok = ((a.n_cols & 3) == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0);
        for (int idx = tid; idx < MT * PIECES; idx += KQ_THREADS) {
            const int m = idx / PIECES, p = idx % PIECES;
            const int col = st.r * G::CH + p * 4;
            float* dst = &sm.x[buf][m][p * 4];
            if (tok0 + m < a.seq_len && col + 3 < a.n_cols && vec_ok) {
                cp_async16(dst, a.x + (size_t)(tok0 + m) * a.n_cols + col);
            } else {
#pragma unroll
                for (int k = 0; k < 4; k++)
                    dst[k] = (tok0 + m < a.seq_len && col + k < a.n_cols) ? a.x[(size_t)(tok0 + m) * a.n_cols + col + k] : 0.0f;
            }
        }
    };

    uint4 wn[G::NW];
    uint32_t dn = 0;
    auto load_w = [&](const KqStep& st) {
        const KqMat& a = *st.m;
        const int panel = st.item / kq_tiles<MT>(a);
        const int blk = (KIND == KIND_Q4K) ? (st.r * 8 + warp) : (st.r * 2 + (warp >> 2));
        if (blk < a.nblk) {
            const size_t base = ((size_t)panel * a.nblk + blk);
            const uint4* p = a.kq + base * G::NP * 32 + lane;
            if (KIND == KIND_Q4K) {
#pragma unroll
                for (int i = 0; i < 9; i++) wn[i] = __ldg(p + i * 32);
            } else {
                const int q = warp & 3;
                wn[0] = __ldg(p + (2 * q) * 32);
                wn[1] = __ldg(p + (2 * q + 1) * 32);
                wn[2] = __ldg(p + (8 + q) * 32);
                wn[3] = __ldg(p + 12 * 32);
                dn = __ldg(a.d16 + base * 32 + lane);
            }
        }
    };

    float run = 0.0f;  // thread tid < MT*32 owns the chain of (token tid/32, row tid%32)
    auto replay = [&](const KqStep& st, int buf) {
        if (tid < MT * 32) {
            const KqMat& a = *st.m;
            const int m = tid >> 5, row = tid & 31;
            const int nvalid = min(TERMS, G::TERMS_PER_BLK * (a.nblk - st.r * G::BLK_PER_ROUND));
            float acc = run;
            int k = 0;
            for (; k + 4 <= nvalid; k += 4) {  // loads first, then the ordered adds
                const float t0 = sm.term[buf][k][m][row], t1 = sm.term[buf][k + 1][m][row];
                const float t2 = sm.term[buf][k + 2][m][row], t3 = sm.term[buf][k + 3][m][row];
                acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, t0), t1), t2), t3);
            }
            for (; k < nvalid; k++) acc = __fadd_rn(acc, sm.term[buf][k][m][row]);
            if (st.r == st.rounds - 1) {
                const int grow = (st.item / kq_tiles<MT>(a)) * 32 + row;
                const int tok = (st.item % kq_tiles<MT>(a)) * MT + m;
                if (grow < a.n_rows && tok < a.seq_len) a.out[(size_t)tok * a.ld_out + grow] = acc;
                acc = 0.0f;
            }
            run = acc;
        }
    };

    int gitem = it0;
    KqStep cur = first_step(gitem), prev = cur;
    stage(cur, 0);
    load_w(cur);
    for (int t = 0; gitem < it1; t++) {
        cp_async_commit_wait_all();
        __syncthreads();
        uint4 w[G::NW];
#pragma unroll
        for (int i = 0; i < G::NW; i++) w[i] = wn[i];
        const uint32_t dcur = dn;
        int gnext = gitem;
        const KqStep nxt = next_step(cur, gnext);
        if (gnext < it1) {
            stage(nxt, (t + 1) & 1);
            load_w(nxt);
        }
        if (t > 0) replay(prev, (t - 1) & 1);

        const int buf = t & 1;
        const int nblk = cur.m->nblk, r = cur.r;
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
                        const uint4 qv = w[1 + sb];
                        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
                        float lanes[MT][8];
#pragma unroll
                        for (int tt = 0; tt < 4; tt++) {  // elements 8tt..8tt+7 of the sub-block live in word tt
                            float v[8];
                            if (FAST) {
                                const uint32_t ev = qw[tt] & 0x0F0F0F0Fu, od = (qw[tt] >> 4) & 0x0F0F0F0Fu;  // elements 0,2,4,6 / 1,3,5,7
#pragma unroll
                                for (int j = 0; j < 8; j++) {
                                    const float nf = __uint_as_float(__byte_perm((j & 1) ? od : ev, magic, 0x7540u + (j >> 1)));
                                    v[j] = __fsub_rn(fmaf(nf, scf, c0), mnf);
                                }
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; j++) v[j] = __fsub_rn(__fmul_rn((float)((qw[tt] >> (4 * j)) & 0xF), scf), mnf);
                            }
#pragma unroll
                            for (int m = 0; m < MT; m++) {
                                const float4* xp = reinterpret_cast<const float4*>(&sm.x[buf][m][warp * 256 + sb * 32 + tt * 8]);
                                const float4 x0 = xp[0], x1 = xp[1];
                                const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                                for (int j = 0; j < 8; j++) lanes[m][j] = fmaf(v[j], xs[j], tt == 0 ? 0.0f : lanes[m][j]);
                            }
                        }
#pragma unroll
                        for (int m = 0; m < MT; m++) sm.term[buf][warp * 8 + sb][m][lane] = reduce8(lanes[m]);
                    }
                };
                if (fabsf(d) <= 65504.0f) block_body(std::true_type{});
                else block_body(std::false_type{});
            }
        } else {
            const int blk = r * 2 + (warp >> 2), q = warp & 3;
            if (blk < nblk) {
                const float d = h2f_bits(dcur);
                const uint32_t qlw[8] = {w[0].x, w[0].y, w[0].z, w[0].w, w[1].x, w[1].y, w[1].z, w[1].w};
                const uint32_t qhw[4] = {w[2].x, w[2].y, w[2].z, w[2].w};
                const uint32_t scw = (q == 0) ? w[3].x : (q == 1 ? w[3].y : (q == 2 ? w[3].z : w[3].w));
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int sci = (int)(int8_t)((scw >> (8 * (u >> 1))) & 0xff);
                    const float sd = __fmul_rn((float)sci, d);
                    const uint32_t qh16 = (qhw[u >> 1] >> (16 * (u & 1))) & 0xffffu;
                    float qf[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int quant = (int)(((qlw[u] >> (4 * j)) & 0xF) | (((qh16 >> (2 * j)) & 3) << 4)) - 32;
                        qf[j] = __fmul_rn((float)quant, sd);
                    }
#pragma unroll
                    for (int m = 0; m < MT; m++) {
                        const float4* xp = reinterpret_cast<const float4*>(&sm.x[buf][m][(warp >> 2) * 256 + q * 64 + u * 8]);
                        const float4 x0 = xp[0], x1 = xp[1];
                        float lanes[8];
                        lanes[0] = fmaf(qf[0], x0.x, 0.0f); lanes[1] = fmaf(qf[1], x0.y, 0.0f);
                        lanes[2] = fmaf(qf[2], x0.z, 0.0f); lanes[3] = fmaf(qf[3], x0.w, 0.0f);
                        lanes[4] = fmaf(qf[4], x1.x, 0.0f); lanes[5] = fmaf(qf[5], x1.y, 0.0f);
                        lanes[6] = fmaf(qf[6], x1.z, 0.0f); lanes[7] = fmaf(qf[7], x1.w, 0.0f);
                        sm.term[buf][warp * 8 + u][m][lane] = reduce8(lanes);
                    }
                }
            }
        }
        prev = cur;
        cur = nxt;
        gitem = gnext;
        if (gitem >= it1) {
            __syncthreads();
            replay(prev, t & 1);
        }
    }
}

// Resident CTAs per SM of each instantiation, measured by the occupancy API at prepare time: the grid of the
// persistent kernel is sized to exactly one wave.
int g_kq_ctas[2][5] = {};

int kq_items(const KqMat& m, int mt) { return ((m.seq_len + mt - 1) / mt) * m.n_panels; }

template <int KIND, int MT>
int launch_mt(const KqLaunch& L, int grid, cudaStream_t st) {
    if (L.n_items <= 0 || grid <= 0) return 0;
    kq_gemv_kernel<KIND, MT><<<grid, KQ_THREADS, sizeof(KqSmem<KIND, MT>), st>>>(L);
    HB_CUDA(cudaGetLastError());
    return 0;
}

template <int KIND>
int launch_kind(const KqLaunch& L, int mt, int grid, cudaStream_t st) {
    if (mt == 1) return launch_mt<KIND, 1>(L, grid, st);
    if (mt == 2) return launch_mt<KIND, 2>(L, grid, st);
    return launch_mt<KIND, 4>(L, grid, st);
}

template <int KIND, int MT>
int prepare_one() {
    HB_CUDA(cudaFuncSetAttribute(kq_gemv_kernel<KIND, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(KqSmem<KIND, MT>)));
    int n = 0;
    HB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kq_gemv_kernel<KIND, MT>, KQ_THREADS, sizeof(KqSmem<KIND, MT>)));
    g_kq_ctas[KIND == KIND_Q4K ? 0 : 1][MT] = n > 0 ? n : 1;
    return 0;
}

}  // namespace

int kquant_prepare() {
    int rc;
    if ((rc = prepare_one<KIND_Q4K, 1>())) return rc;
    if ((rc = prepare_one<KIND_Q4K, 2>())) return rc;
    if ((rc = prepare_one<KIND_Q4K, 4>())) return rc;
    if ((rc = prepare_one<KIND_Q6K, 1>())) return rc;
    if ((rc = prepare_one<KIND_Q6K, 2>())) return rc;
    if ((rc = prepare_one<KIND_Q6K, 4>())) return rc;
    return 0;
}

size_t kquant_pieces_per_block(int kind) { return kind == KIND_Q4K ? 9 : 13; }

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

int kquant_tokens_per_pass(int seq_len) { return seq_len == 1 ? 1 : (seq_len == 2 ? 2 : 4); }

int kquant_items(int n_panels, int seq_len) {
    const int mt = kquant_tokens_per_pass(seq_len);
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
                       const float* x, int seq_len, float* out, int ld_out, int sm_count, cudaStream_t st) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    KqLaunch L;
    L.mats = nullptr; L.chunks = nullptr; L.magic = 0x4B000000u;
    KqMat& a = L.single;
    a.kq = kq; a.d16 = d16; a.x = x; a.out = out;
    a.n_rows = n_rows; a.n_cols = n_cols; a.nblk = nblk; a.n_panels = n_panels; a.seq_len = seq_len; a.ld_out = ld_out;
    const int mt = kquant_tokens_per_pass(seq_len);
    a.item_begin = 0;
    a.item_end = L.n_items = kquant_items(n_panels, seq_len);
    const int grid = kquant_grid(kind, mt, sm_count, L.n_items);
    if (kind == KIND_Q4K) return launch_kind<KIND_Q4K>(L, mt, grid, st);
    if (kind == KIND_Q6K) return launch_kind<KIND_Q6K>(L, mt, grid, st);
    set_error("kquant_gemv: kind %d", kind);
    return -7;
}

int launch_kquant_gemv_list(int kind, int mt, const KqMat* mats_dev, const int* chunks_dev, int n_items, int grid, cudaStream_t st) {
    KqLaunch L;
    L.mats = mats_dev; L.chunks = chunks_dev; L.n_items = n_items; L.magic = 0x4B000000u;
    L.single = KqMat{};
    if (kind == KIND_Q4K) return launch_kind<KIND_Q4K>(L, mt, grid, st);
    if (kind == KIND_Q6K) return launch_kind<KIND_Q6K>(L, mt, grid, st);
    set_error("kquant_gemv: kind %d", kind);
    return -7;
}

}  // namespace hb200
