// Few-token matmul (batched decode, about 11 .. 64 tokens) on the tensor cores with the WEIGHT ROWS on the MMA's M side:
// tcgen05.mma kind::i8, 128 weight rows = TMEM lanes, 32 tokens = TMEM columns, for Q1_0 and Q2_0 / PQ2_0 / PTQ1_0
// weights against Q8_0 activations.
//
// Replaces ThreadPool::par_dot_rows_batched over the paired-token kernels
// (hearth-llm/src/pool.rs:40-80, :568-618; hearth-quant/src/q1_0g128.rs:396-502, q2_0.rs:408-492) for token counts
// where the streaming dp4a kernel needs several passes and 128-token tiles would be mostly padding.  With tokens on
// the M side (gemm_tc.cu) all real tokens of a small batch sit in one TMEM lane quarter, i.e. on one of the four
// schedulers, and a warp instruction costs the same whether 8 or 32 of its lanes carry a token; with rows on the M
// side every lane always carries a row, the promotion work is proportional to the real token count and spreads over
// all four schedulers.  The arithmetic is the scalar path's, bit for bit: each 32-column sub-block is ONE int8 MMA of
// depth K=32 whose int32 result is exact; then
//   block_acc = fma(I0,a0,0); block_acc = fma(I_s,a_s,block_acc) (s=1..3);  sum = sum + block_acc * w_scale.
//
// Persistent kernel: one CTA per SM walks a run of tiles (128 rows x up to 32 tokens, all of K), possibly of many
// matrices; the rings keep turning across tiles.
//   warp 0      TMA producer: int8 activation tile 32 tokens x 128 B per block (SWIZZLE_128B, K-major)
//   warps 1-2   TMEM allocation (warp 1) + MMA issue, one thread each: warp 1 the even blocks, warp 2 the odd ones;
//               4 MMAs (128 x 32 x 32) per block into 4 x 32 columns of that issuer's accumulator set
//   warps 3-6   unpack, each warp every fourth block (its own stage of the ring): 128 rows x 128 columns of 1-/2-bit
//               codes -> int8 in the swizzled K-major layout
//   warps 7-14  promotion: thread = weight row, warp = 16 tokens of one lane quarter; 16 running sums per thread
// Every wait on an mbarrier is bounded; on expiry the CTA records a status code, stops issuing, drains its
// outstanding bulk copies, frees its TMEM and returns.
#include "tc_common.cuh"

namespace hb200 {

namespace {

constexpr int UNPACK_WARPS = 4;
constexpr int EPI_WARPS = 8;      // two per TMEM lane quarter, sixteen tokens each
constexpr int TC_THREADS = 32 * (3 + UNPACK_WARPS + EPI_WARPS);
constexpr int TOK_TILE = GEMM_TCR_TOK_TILE;  // 32 tokens: the MMA's N
constexpr int ROW_TILE = GEMM_TCR_ROW_TILE;  // 128 rows: the MMA's M
constexpr int STAGES = 4;
constexpr int W_BYTES = ROW_TILE * 128;  // 16 KiB of expanded weights
constexpr int X_BYTES = TOK_TILE * 128;  // 4 KiB of activations
constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
constexpr int SET_COLS = 4 * TOK_TILE;   // TMEM columns of one accumulator set: four sub-blocks x 32 tokens
// Four accumulator sets: from the commit of a block's MMAs to the moment its set can be written again (arrival of the
// commit, wake-up of the promotion warps, their TMEM loads, their release, wake-up of the issuer) about two
// microseconds pass, whatever the tile's shape; with two sets that round trip bounded the kernel at a block per
// microsecond.
constexpr int NSETS = 4;
constexpr uint32_t TMEM_COLS = NSETS * SET_COLS;
static_assert(TMEM_COLS == 512, "a power of two of TMEM columns");
// kind::i8, D = S32, A (weights) and B (activations) signed int8, both K-major, M = 128, N = 32.
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TOK_TILE >> 3) << 17) | ((uint32_t)(ROW_TILE >> 4) << 24);

constexpr int SCALE_SLOTS = 8;
constexpr int PSLOTS = 8;
static_assert(UNPACK_WARPS == STAGES, "every stage needs exactly one producer warp (a parity wait cannot tell a phase from the one two before it)");
static_assert(PSLOTS == 2 * UNPACK_WARPS, "two packed-byte slots per unpack warp");

struct TcrLaunch {
    const TcMat* mats;
    const int* chunks;
    int* status;
    int n_tiles;
    TcMat single;
};

struct Barriers {
    uint64_t full[STAGES], empty[STAGES];
    uint64_t tmem_full[NSETS], tmem_empty[NSETS];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float wscale[SCALE_SLOTS][ROW_TILE];
    alignas(16) unsigned char packed[PSLOTS][4096];  // 128 rows x 128 columns of codes: 2 KiB (Q1_0) or 4 KiB (Q2_0)
    alignas(16) unsigned char pscale[PSLOTS][256];   // their f16 scales
    alignas(16) float4 pxs[PSLOTS][TOK_TILE];        // the four sub-block activation scales of the tile's 32 tokens (cp.async)
    alignas(16) float4 xscale[SCALE_SLOTS][TOK_TILE];  // the same, kept for the promotion warps like wscale
};

struct TileRef {
    const TcMat* m;
    int tok0, row0;
};

// Tile t of the launch; tiles of a matrix are numbered with the token tile fastest, so the second token tile of a
// row tile finds the weights in cache.
struct TileWalk {
    const TcrLaunch* L;
    int i, mi;
    __device__ __forceinline__ void init(const TcrLaunch* l) { L = l; i = 0; mi = 0; }
    __device__ __forceinline__ bool next(TileRef& r) {
        int t;
        if (L->chunks) {
            t = L->chunks[blockIdx.x] + i;
            if (t >= L->chunks[blockIdx.x + 1]) return false;
        } else {
            t = (int)blockIdx.x + i * (int)gridDim.x;
            if (t >= L->n_tiles) return false;
        }
        i++;
        const TcMat* m = &L->single;
        if (L->mats) {
            while (t >= L->mats[mi].tile_end) mi++;
            m = &L->mats[mi];
        }
        const int lt = t - m->tile_begin;
        r.m = m;
        r.tok0 = (lt % m->tok_tiles) * TOK_TILE;
        r.row0 = (lt / m->tok_tiles) * ROW_TILE;
        return true;
    }
};

template <int KIND>
struct UnpackCursor {
    TileWalk walk;
    bool valid;
    int g, blk, nb;
    const uint4* tp0;
    const unsigned char* sp0;
    const float* xs0;  // activation scales of this lane's token of the tile (a token past the end reads the last one: unused)
    __device__ __forceinline__ void load_tile() {
        constexpr int RPG = rows_per_group(KIND);
        constexpr int SPT = scales_per_tile(KIND);
        TileRef r;
        valid = walk.next(r);
        if (!valid) return;
        nb = r.m->nb;
        const int rg0 = r.row0 / RPG;  // first row group of the tile; 128 rows never straddle a 32-row-group panel
        const size_t tile0 = (size_t)(rg0 >> 5) * nb;
        const int lane0 = rg0 & 31;
        tp0 = r.m->bits + tile0 * 256 + lane0;
        sp0 = reinterpret_cast<const unsigned char*>(r.m->scales) + (tile0 * 32 + lane0) * SPT * 2;
        const int tok = min(r.tok0 + (int)(threadIdx.x & 31), r.m->seq_len - 1);
        xs0 = r.m->ad + (size_t)tok * r.m->ld_b;
    }
    __device__ __forceinline__ void init(const TcrLaunch* l, int first) {
        walk.init(l);
        g = 0;
        blk = 0;
        load_tile();
        advance(first);
    }
    __device__ __forceinline__ void advance(int n) {
        g += n;
        blk += n;
        while (valid && blk >= nb) {
            blk -= nb;
            load_tile();
        }
    }
};

template <int KIND>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tcr_kernel(const __grid_constant__ TcrLaunch L) {
    constexpr int RPG = rows_per_group(KIND);
    constexpr int SPT = scales_per_tile(KIND);
    constexpr int RGS = ROW_TILE / RPG;  // row groups per tile: 16 (Q1_0) or 32 (Q2_0)
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(tiles + STAGES * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(smem_u32(&bars->full[i]), 2);  // the TMA's expect_tx arrival + the unpack warp that filled the stage
            mbar_init(smem_u32(&bars->empty[i]), 1);
        }
        for (int i = 0; i < NSETS; i++) {
            mbar_init(smem_u32(&bars->tmem_full[i]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[i]), EPI_WARPS);
        }
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    // Every role walks the same sequence of tiles and, inside a tile, of 128-column blocks; g numbers the blocks of
    // the CTA across tiles and selects every ring slot and barrier phase.
    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (one lane)
        if (lane == 0) {
            TileWalk walk;
            walk.init(&L);
            TileRef tr;
            int g = 0;
            bool ok = true;
            while (ok && walk.next(tr)) {
                const int nb = tr.m->nb;
                const CUtensorMap* amap = static_cast<const CUtensorMap*>(tr.m->amap);
                for (int blk = 0; blk < nb; blk++, g++) {
                    const int st = g % STAGES;
                    if (g >= STAGES && !mbar_wait<200>(smem_u32(&bars->empty[st]), ((g / STAGES) - 1) & 1, abort_flag, L.status, 1)) {
                        ok = false;
                        break;
                    }
                    const uint32_t bar = smem_u32(&bars->full[st]);
                    mbar_expect_tx(bar, X_BYTES);
                    tma_load_2d(smem_u32(tiles + st * STAGE_BYTES + W_BYTES), amap, blk * 128, tr.tok0, bar);
                }
            }
            if (*abort_flag) {
                // Do not leave the CTA with bulk copies in flight: wait (bounded) for the ones already issued.
                const int first = g > STAGES ? g - STAGES : 0;
                for (int q = first; q < g; q++) {
                    const uint32_t bar = smem_u32(&bars->full[q % STAGES]);
                    for (uint32_t i = 0; i < (SPIN_LIMIT >> 8) && !mbar_try(bar, (q / STAGES) & 1); i++) {
                    }
                }
            }
        }
    } else if (warp <= 2) {
        // ---------------------------------------------------------------- MMA issue: warp 1 even blocks, warp 2 odd blocks
        if (lane == 0) {
            const int par = warp - 1;
            TileWalk walk;
            walk.init(&L);
            TileRef tr;
            int g = 0;
            bool ok = true;
            while (ok && walk.next(tr)) {
                const int nb = tr.m->nb;
                for (int blk = 0; blk < nb; blk++, g++) {
                    if ((g & 1) != par) continue;
                    const int st = g % STAGES, buf = g % NSETS;
                    const uint32_t w_addr = smem_u32(tiles + st * STAGE_BYTES);
                    const uint64_t wd0 = make_desc(w_addr), xd0 = make_desc(w_addr + W_BYTES);
                    const uint32_t d0 = tmem_base + buf * SET_COLS;
                    const uint32_t bar_full = smem_u32(&bars->tmem_full[buf]), bar_empty = smem_u32(&bars->empty[st]);
                    if (!mbar_wait<100>(smem_u32(&bars->full[st]), (g / STAGES) & 1, abort_flag, L.status, 2)) { ok = false; break; }
                    if (g >= NSETS && !mbar_wait<50>(smem_u32(&bars->tmem_empty[buf]), ((g / NSETS) - 1) & 1, abort_flag, L.status, 4)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int s = 0; s < 4; s++)  // one K=32 MMA per sub-block; +32 B inside the 128 B swizzle row = +2 in the address field
                        tc_mma_i8(d0 + s * TOK_TILE, wd0 + 2 * s, xd0 + 2 * s, IDESC);
                    tc_commit(bar_full);
                    tc_commit(bar_empty);
                }
            }
        }
    } else if (warp < 3 + UNPACK_WARPS) {
        // ---------------------------------------------------------------- unpack (one warp per stage, one block each in turn)
        const int uw = warp - 3;
        UnpackCursor<KIND> cur, pf;
        cur.init(&L, uw);
        pf = cur;
        auto issue = [&](const UnpackCursor<KIND>& c) {
            if (c.valid) {
                const int slot = c.g % PSLOTS;
                const uint4* tp = c.tp0 + (size_t)c.blk * 256;
#pragma unroll
                for (int k = 0; k < RGS * 8 / 32; k++) {
                    const int pi = lane + k * 32;  // piece: row group pi >> 3, piece pi & 7 of its tile
                    cp_async16(&bars->packed[slot][pi * 16], tp + (pi & 7) * 32 + (pi >> 3));
                }
                if (lane < 16)  // RGS * SPT f16 = 256 bytes
                    cp_async16(&bars->pscale[slot][lane * 16], c.sp0 + (size_t)c.blk * 32 * SPT * 2 + lane * 16);
                cp_async16(&bars->pxs[slot][lane], c.xs0 + 4 * c.blk);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        issue(pf);
        pf.advance(UNPACK_WARPS);
        issue(pf);
        pf.advance(UNPACK_WARPS);
        for (; cur.valid; cur.advance(UNPACK_WARPS)) {
            const int g = cur.g;
            const int st = g % STAGES, slot = g % PSLOTS;
            asm volatile("cp.async.wait_group 1;" ::: "memory");
            __syncwarp();
            bool ok = true;
            if (g >= STAGES) {
                if (lane == 0) ok = mbar_wait<200>(smem_u32(&bars->empty[st]), ((g / STAGES) - 1) & 1, abort_flag, L.status, 5);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (!ok) break;
            unsigned char* bt = tiles + st * STAGE_BYTES;
#pragma unroll 2
            for (int uu = 0; uu < ROW_TILE * 4 / 32; uu++) {
                const int u = lane + uu * 32;  // unit = (row of the tile, sub-block)
                const int ri = u >> 2, s = u & 3;
                const int rgl = ri / RPG, r = ri % RPG;
                const int sh = (KIND == KIND_Q1) ? r : 2 * r;
                const unsigned char* tsrc = &bars->packed[slot][rgl * 128];
                uint32_t vals[8];
#pragma unroll
                for (int jp = 0; jp < 4; jp++) {
                    // words 2jp, 2jp+1 of sub-block s live in piece 2jp + (s>>1), components (s&1)*2, +1
                    const uint2 w2 = *reinterpret_cast<const uint2*>(tsrc + (2 * jp + (s >> 1)) * 16 + (s & 1) * 8);
                    const uint32_t ww[2] = {w2.x, w2.y};
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        uint32_t v;
                        if (KIND == KIND_Q1) {
                            const uint32_t m = (ww[e] >> sh) & 0x01010101u;  // bit -> 0/1
                            v = (m * 0xFEu) ^ 0xFFFFFFFFu;                    // 1 -> 0x01 (+1), 0 -> 0xFF (-1)
                        } else {
                            const uint32_t c = ((ww[e] >> sh) & 0x03030303u) | 0x80808080u;
                            v = (c - 0x01010101u) ^ 0x80808080u;              // code - 1 per byte, no borrow across bytes
                        }
                        vals[2 * jp + e] = v;
                    }
                }
                unsigned char* rowp = bt + ri * 128;
                const int sw = ri & 7;
                *reinterpret_cast<uint4*>(rowp + (((2 * s) ^ sw) << 4)) = make_uint4(vals[0], vals[1], vals[2], vals[3]);
                *reinterpret_cast<uint4*>(rowp + (((2 * s + 1) ^ sw) << 4)) = make_uint4(vals[4], vals[5], vals[6], vals[7]);
            }
#pragma unroll
            for (int k = 0; k < ROW_TILE / 32; k++) {
                const int row = lane + 32 * k;
                const int rgl = row / RPG, r = row % RPG;
                const unsigned short h = *reinterpret_cast<const unsigned short*>(&bars->pscale[slot][(rgl * SPT + r) * 2]);
                bars->wscale[g % SCALE_SLOTS][row] = __half2float(__ushort_as_half(h));
            }
            bars->xscale[g % SCALE_SLOTS][lane] = bars->pxs[slot][lane];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // make the generic-proxy writes visible to the MMA
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->full[st]));
            issue(pf);  // refills the slot just consumed
            pf.advance(UNPACK_WARPS);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        // ---------------------------------------------------------------- promotion (8 warps; thread = weight row)
        const int e = warp - (3 + UNPACK_WARPS);
        const int quarter = warp & 3;   // TMEM lanes this warp may read: 32*(warp % 4) ..
        const int th = e >> 2;          // which 16 of the 32 token columns; the two warps of a quarter differ in th
        TileWalk walk;
        walk.init(&L);
        TileRef tr;
        int g = 0;
        bool ok = true;
        while (ok && walk.next(tr)) {
            const TcMat* M = tr.m;
            const int nb = M->nb;
            const int row = tr.row0 + quarter * 32 + lane;
            const int tokb = tr.tok0 + th * 16;                         // first token of this warp's columns
            const int ntok = min(16, max(0, M->seq_len - tokb));        // how many of them exist (the same for the whole warp)
            float sum[16];
#pragma unroll
            for (int t = 0; t < 16; t++) sum[t] = 0.0f;

            // Software pipeline over the halves (eight tokens each) of the blocks: the TMEM loads of the next half are in
            // flight while the current half is scaled, also across the boundary between two blocks, and the accumulator
            // set goes back to the MMA issuer as soon as its last needed half sits in registers.  Without it one block
            // costs the sum of a barrier wake-up, two TMEM round trips and the arithmetic, and that chain bounds the kernel.
            const bool need1 = ntok > 8;  // the same for the whole warp
            const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16) + th * 16;
            uint32_t v0[4][8], v1[4][8];
            auto wait_full = [&](int gg) {
                if (lane == 0) ok = mbar_wait<20>(smem_u32(&bars->tmem_full[gg % NSETS]), (gg / NSETS) & 1, abort_flag, L.status, 6);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                tc_fence_after();
            };
            auto release = [&](int gg) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[gg % NSETS]));
            };
            auto scale_half = [&](const uint32_t (&v)[4][8], int gg, int hf) {
                // block_acc = fma(I0,a0,0), fma(I1,a1,.), fma(I2,a2,.), fma(I3,a3,.); then sum += block_acc * w_scale,
                // rounded separately (q2_0.rs:545-573, q1_0g128.rs:1026-1051)
                const float wd = bars->wscale[gg % SCALE_SLOTS][quarter * 32 + lane];
                const float4* xsp = &bars->xscale[gg % SCALE_SLOTS][th * 16 + hf * 8];
#pragma unroll
                for (int t = 0; t < 8; t++) {
                    if (hf * 8 + t < ntok) {
                        const float4 a4 = xsp[t];  // the four sub-block scales of the token (a broadcast read)
                        float acc = fmaf((float)(int)v[0][t], a4.x, 0.0f);
                        acc = fmaf((float)(int)v[1][t], a4.y, acc);
                        acc = fmaf((float)(int)v[2][t], a4.z, acc);
                        acc = fmaf((float)(int)v[3][t], a4.w, acc);
                        sum[hf * 8 + t] = __fadd_rn(sum[hf * 8 + t], __fmul_rn(acc, wd));
                    }
                }
            };
            auto load_half = [&](uint32_t (&v)[4][8], int gg, int hf) {
#pragma unroll
                for (int s4 = 0; s4 < 4; s4++) tc_ld8(tlane + (gg % NSETS) * SET_COLS + s4 * TOK_TILE + hf * 8, v[s4]);
            };
            auto landed = [&](uint32_t (&v)[4][8]) {
                tc_wait_ld8(v[0]);
                tc_pin8(v[1]);
                tc_pin8(v[2]);
                tc_pin8(v[3]);
            };
            // The sums of a half are complete before the next volatile statement, so that no more than two halves of
            // loaded registers are ever alive together.
            auto pin_lo = [&]() { asm volatile("" : "+f"(sum[0]), "+f"(sum[1]), "+f"(sum[2]), "+f"(sum[3]), "+f"(sum[4]), "+f"(sum[5]), "+f"(sum[6]), "+f"(sum[7])); };
            auto pin_hi = [&]() { asm volatile("" : "+f"(sum[8]), "+f"(sum[9]), "+f"(sum[10]), "+f"(sum[11]), "+f"(sum[12]), "+f"(sum[13]), "+f"(sum[14]), "+f"(sum[15])); };
            const int g_end = g + nb;
            if (ntok == 0) {
                // none of this warp's tokens exist: it only keeps the barrier protocol going
                for (; ok && g < g_end; g++) {
                    wait_full(g);
                    if (ok) release(g);
                }
            } else if (need1) {
                // v0: first halves, v1: second halves
                wait_full(g);
                if (ok) load_half(v0, g, 0);
                for (; ok && g < g_end; g++) {
                    landed(v0);
                    load_half(v1, g, 1);
                    scale_half(v0, g, 0);
                    pin_lo();
                    landed(v1);
                    release(g);
                    if (g + 1 < g_end) {
                        wait_full(g + 1);
                        if (!ok) break;
                        load_half(v0, g + 1, 0);
                    }
                    scale_half(v1, g, 1);
                    pin_hi();
                }
            } else {
                // one half per block: v0 and v1 take the blocks in turn
                wait_full(g);
                if (ok) load_half(v0, g, 0);
                while (ok && g < g_end) {
                    landed(v0);
                    release(g);
                    if (g + 1 < g_end) {
                        wait_full(g + 1);
                        if (!ok) break;
                        load_half(v1, g + 1, 0);
                    }
                    scale_half(v0, g, 0);
                    pin_lo();
                    g++;
                    if (g >= g_end) break;
                    landed(v1);
                    release(g);
                    if (g + 1 < g_end) {
                        wait_full(g + 1);
                        if (!ok) break;
                        load_half(v0, g + 1, 0);
                    }
                    scale_half(v1, g, 0);
                    pin_lo();
                    g++;
                }
            }
            if (!ok) break;
            if (ok && row < M->n_rows && !*abort_flag) {
#pragma unroll
                for (int t = 0; t < 16; t++)
                    if (t < ntok) M->out[(size_t)(tokb + t) * M->ld_out + row] = sum[t];  // a warp writes 32 consecutive rows of one token
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

constexpr int TCR_SMEM = STAGES * STAGE_BYTES + (int)sizeof(Barriers) + 1024;

}  // namespace

int gemm_tcr_prepare() {
    HB_CUDA(cudaFuncSetAttribute(gemm_tcr_kernel<KIND_Q1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TCR_SMEM));
    HB_CUDA(cudaFuncSetAttribute(gemm_tcr_kernel<KIND_Q2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TCR_SMEM));
    return 0;
}

int gemm_tcr_tiles(int n_rows, int seq_len) {
    return ((seq_len + TOK_TILE - 1) / TOK_TILE) * ((n_rows + ROW_TILE - 1) / ROW_TILE);
}

void gemm_tcr_fill(TcMat& m, const void* amap_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                   int nb, int seq_len, float* out, int ld_out, int tile_begin) {
    m.bits = bits; m.scales = scales; m.ad = ad; m.out = out; m.amap = amap_dev;
    m.n_rows = n_rows; m.nb = nb; m.seq_len = seq_len; m.ld_out = ld_out; m.ld_b = ld_b;
    m.tok_tiles = (seq_len + TOK_TILE - 1) / TOK_TILE;
    m.tile_begin = tile_begin;
    m.tile_end = tile_begin + gemm_tcr_tiles(n_rows, seq_len);
}

static int run_tcr(int kind, const TcrLaunch& L, int grid, cudaStream_t st) {
    if (kind == KIND_Q1) gemm_tcr_kernel<KIND_Q1><<<grid, TC_THREADS, TCR_SMEM, st>>>(L);
    else if (kind == KIND_Q2) gemm_tcr_kernel<KIND_Q2><<<grid, TC_THREADS, TCR_SMEM, st>>>(L);
    else { set_error("gemm_tc_rows: kind %d has no tensor-core kernel", kind); return -7; }
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_gemm_tcr(int kind, const void* amap_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                    int nb, int seq_len, float* out, int ld_out, int sm_count, int* status, cudaStream_t st) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    TcrLaunch L;
    L.mats = nullptr; L.chunks = nullptr; L.status = status;
    gemm_tcr_fill(L.single, amap_dev, bits, scales, ad, ld_b, n_rows, nb, seq_len, out, ld_out, 0);
    L.n_tiles = L.single.tile_end;
    return run_tcr(kind, L, L.n_tiles < sm_count ? L.n_tiles : sm_count, st);
}

int launch_gemm_tcr_list(int kind, const TcMat* mats_dev, const int* chunks_dev, int n_tiles, int grid, int* status, cudaStream_t st) {
    if (n_tiles <= 0 || grid <= 0) return 0;
    TcrLaunch L;
    L.mats = mats_dev; L.chunks = chunks_dev; L.status = status; L.n_tiles = n_tiles;
    L.single = TcMat{};
    return run_tcr(kind, L, grid, st);
}

}  // namespace hb200
