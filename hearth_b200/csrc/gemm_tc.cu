// Prefill / multi-token matmul on the 5th-generation tensor cores: tcgen05.mma kind::i8 with TMEM
// accumulators, for Q1_0 (17 tokens or more) and Q2_0 / PQ2_0 (25 or more) weights against Q8_0 activations (prefill).
//
// Replaces ThreadPool::par_dot_rows_batched over the paired-token kernels
// (hearth-llm/src/pool.rs:40-80, :568-618; hearth-quant/src/q1_0g128.rs:396-502, q2_0.rs:408-492) and keeps
// the scalar path's arithmetic bit for bit: each 32-column sub-block is ONE int8 MMA of depth K=32 whose
// int32 result is exact; the fp32 scaling then runs in the reference's order
//   block_acc = fma(I0,a0,0); block_acc = fma(I_s,a_s,block_acc) (s=1..3)   [I*a is exact, so fma == mul+add]
//   sum       = sum + block_acc * w_scale                                    [separately rounded]
// Because every sub-block carries its own activation scale the accumulator can never run deeper than K=32:
// the tensor pipe is waiting on this fp32 promotion, not the other way round.
//
// Persistent kernel: one CTA per SM walks a run of tiles (128 tokens = TMEM lanes, 64 weight rows = TMEM columns),
// possibly of many matrices; every tile's K is walked in 128-column blocks and the rings keep turning across tiles.
//   warp 0      TMA producer: int8 activation tile 128 tokens x 128 B per block (SWIZZLE_128B, K-major); the tensor
//               map of the tile's activation is read from device memory
//   warps 1-2   TMEM allocation (warp 1) + MMA issue, one thread each: warp 1 the even blocks, warp 2 the odd ones;
//               4 MMAs (128x64x32) per block into 4 x 64 columns of that issuer's accumulator set
//   warps 3-6   unpack, each warp every fourth block: packed codes arrive through a cp.async ring; 64 rows x 128 columns
//               of 1-/2-bit codes -> int8 {-1,+1} / {-1,0,+1,+2} in the same swizzled K-major layout, 128-bit stores
//   warps 7-22  promotion: tcgen05.ld 16 columns x 4 sub-blocks at a time, thread = token, 16 running sums per thread,
//               64 contiguous output bytes per thread at the end of a tile
// Two accumulator sets (2 x 256 TMEM columns) let the MMAs of block b+1 run under the promotion of block b;
// a 4-stage shared-memory ring decouples TMA / unpack from the MMA issue.
// Every wait on an mbarrier is bounded; on expiry the CTA records a status code, stops issuing, drains its
// outstanding bulk copies, frees its TMEM and returns.
#include "tc_common.cuh"

namespace hb200 {

namespace {

constexpr int UNPACK_WARPS = 4;   // each warp expands every fourth block on its own (eight units per thread)
constexpr int EPI_WARPS = 16;     // four per TMEM lane quarter, 16 accumulator columns per thread
constexpr int TC_THREADS = 32 * (3 + UNPACK_WARPS + EPI_WARPS);  // 736: TMA, two MMA issuers, unpack, promotion
constexpr int TOK_TILE = 128;
constexpr int ROW_TILE = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = TOK_TILE * 128;  // 16 KiB
constexpr int B_BYTES = ROW_TILE * 128;  // 8 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t TMEM_COLS = 512;

// What one launch works through: `mats` (device memory, n_tiles tiles in all) or, when mats is null, the one matrix
// `single`.  With `chunks` ([gridDim.x + 1] tile indices) CTA c owns tiles chunks[c] .. chunks[c+1]-1, a contiguous
// run balanced by block count; without, CTA c takes tiles c, c + gridDim.x, ...
struct TcLaunch {
    const TcMat* mats;
    const int* chunks;
    int* status;  // device word: 0 ok, otherwise the code of the first wait that expired
    int n_tiles;
    TcMat single;
};


// Pairs of fp32 lanes, written as two scalar IEEE operations each.  The packed sm_100 forms are not used: ptxas 12.9
// contracts mul.rn.f32x2 followed by add.rn.f32x2 into a fused multiply-add (the scalar forms with .rn are kept apart),
// which changes the bits of the running sum; and the packed forms issue over two cycles, so they save little.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) { return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y)); }
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) { return make_float2(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y)); }
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) { return make_float2(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y)); }

constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ROW_TILE >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

constexpr int SCALE_SLOTS = 8;  // ring of per-block weight scales (f32); deeper than the tile ring, see the unpack loop
constexpr int PSLOTS = 8;       // ring of packed weight bytes (cp.async): two slots per unpack warp
// One unpack warp per stage: a stage's blocks g, g + STAGES, ... are then produced by one warp, in order.  With two
// producers on a stage the later one could find the stage's `empty` barrier two phases behind the one it waits for,
// and a parity wait cannot tell a phase from the one two before it: it would pass at once and overwrite a tile in use.
// (Five stages with five unpack warps were measured too: the same times as four, so the smaller kernel stays.)
static_assert(UNPACK_WARPS == STAGES, "every stage needs exactly one producer warp");
static_assert(PSLOTS == 2 * UNPACK_WARPS, "two packed-byte slots per unpack warp");
struct Barriers {
    uint64_t full[STAGES], empty[STAGES];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float wscale[SCALE_SLOTS][ROW_TILE];
    alignas(16) unsigned char packed[PSLOTS][2048];  // 64 rows x 128 columns of codes: 1 KiB (Q1_0) or 2 KiB (Q2_0)
    alignas(16) unsigned char pscale[PSLOTS][128];   // their f16 scales
};

// Tile t of the launch: which matrix, which 128 tokens, which 64 rows.  Tiles of a matrix are numbered with the
// token tile fastest, so CTAs working side by side read different activation tiles and the same weights.
struct TileRef {
    const TcMat* m;
    int tok0, row0;
};

struct TileWalk {
    const TcLaunch* L;
    int i;     // how many tiles of this CTA have been handed out
    int mi;    // matrix cursor (tiles come in increasing order)
    __device__ __forceinline__ void init(const TcLaunch* l) { L = l; i = 0; mi = 0; }
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

// Position of an unpack warp in the stream of blocks of this CTA (all tiles, in order): g counts blocks from the
// CTA's first one and selects every ring slot and barrier phase.
template <int KIND>
struct UnpackCursor {
    TileWalk walk;
    bool valid;
    int g, blk, nb;
    const uint4* tp0;                // packed pieces of block 0 of the tile's row groups
    const unsigned char* sp0;        // f16 scales of block 0
    __device__ __forceinline__ void load_tile() {
        constexpr int RPG = rows_per_group(KIND);
        constexpr int SPT = scales_per_tile(KIND);
        TileRef r;
        valid = walk.next(r);
        if (!valid) return;
        nb = r.m->nb;
        const int rg0 = r.row0 / RPG;  // first row group of the tile; a tile never straddles a 32-row-group panel
        const size_t tile0 = (size_t)(rg0 >> 5) * nb;
        const int lane0 = rg0 & 31;
        tp0 = r.m->bits + tile0 * 256 + lane0;
        sp0 = reinterpret_cast<const unsigned char*>(r.m->scales) + (tile0 * 32 + lane0) * SPT * 2;
    }
    __device__ __forceinline__ void init(const TcLaunch* l, int first) {
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
gemm_tc_kernel(const __grid_constant__ TcLaunch L) {
    constexpr int RPG = rows_per_group(KIND);
    constexpr int SPT = scales_per_tile(KIND);
    constexpr int RGS = ROW_TILE / RPG;  // row groups per tile: 8 (Q1_0) or 16 (Q2_0)
    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte alignment for the swizzled tiles
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(tiles + STAGES * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(smem_u32(&bars->full[i]), 2);  // the TMA's expect_tx arrival + the unpack warp that filled the stage
            mbar_init(smem_u32(&bars->empty[i]), 1);
        }
        for (int i = 0; i < 2; i++) {
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
    // the CTA across tiles, so the rings and their barrier phases simply keep turning from one tile into the next
    // and the producers start on the next tile while the promotion warps are still finishing the previous one.
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
                    mbar_expect_tx(bar, A_BYTES);
                    tma_load_2d(smem_u32(tiles + st * STAGE_BYTES), amap, blk * 128, tr.tok0, bar);
                }
            }
            if (*abort_flag) {
                // Do not leave the CTA with bulk copies in flight: wait (bounded) for the ones already issued.  If the
                // unpack warps have stopped arriving the phase cannot complete, so this loop simply runs out.
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
        // Two issuing threads halve the serial cost of the waits and commits per block; each owns one accumulator set.
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
                    const int st = g % STAGES, buf = par;
                    // Everything the issue needs is computed before the waits: between the moment the promotion warps
                    // hand the accumulator set back and the commit only four MMA and two commit instructions remain
                    // (this thread shares its scheduler with busy warps, so every extra instruction here costs many cycles).
                    const uint32_t a_addr = smem_u32(tiles + st * STAGE_BYTES);
                    const uint64_t ad0 = make_desc(a_addr), bd0 = make_desc(a_addr + A_BYTES);
                    const uint32_t d0 = tmem_base + buf * 256;
                    const uint32_t bar_full = smem_u32(&bars->tmem_full[buf]), bar_empty = smem_u32(&bars->empty[st]);
                    if (!mbar_wait<100>(smem_u32(&bars->full[st]), (g / STAGES) & 1, abort_flag, L.status, 2)) { ok = false; break; }
                    if (g >= 2 && !mbar_wait<50>(smem_u32(&bars->tmem_empty[buf]), ((g >> 1) - 1) & 1, abort_flag, L.status, 4)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int s = 0; s < 4; s++)  // one K=32 MMA per sub-block; +32 B inside the 128 B swizzle row = +2 in the address field
                        tc_mma_i8(d0 + s * ROW_TILE, ad0 + 2 * s, bd0 + 2 * s, IDESC);
                    tc_commit(bar_full);   // the accumulators are complete (first: the promotion warps wait on this one)
                    tc_commit(bar_empty);  // the stage may be refilled once these MMAs have read it
                }
            }
        }
    } else if (warp < 3 + UNPACK_WARPS) {
        // ---------------------------------------------------------------- unpack (4 warps, one block each in turn)
        // The expansion of one block is a long serial chain (ring wait, stage wait, expand, proxy fence, arrive), so
        // four warps run four such chains side by side: warp w owns blocks w, w+4, ... of the CTA's block stream.
        // Packed codes and scales of a warp's next two blocks stream into its two ring slots with cp.async while it
        // expands the current one.
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
                if (lane < 8)  // RGS * SPT f16 = 128 bytes
                    cp_async16(&bars->pscale[slot][lane * 16], c.sp0 + (size_t)c.blk * 32 * SPT * 2 + lane * 16);
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
            asm volatile("cp.async.wait_group 1;" ::: "memory");  // this block's group has landed (the next one may be in flight)
            __syncwarp();
            bool ok = true;
            if (g >= STAGES) {
                if (lane == 0) ok = mbar_wait<200>(smem_u32(&bars->empty[st]), ((g / STAGES) - 1) & 1, abort_flag, L.status, 5);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (!ok) break;
            unsigned char* bt = tiles + st * STAGE_BYTES + A_BYTES;
#pragma unroll
            for (int uu = 0; uu < 8; uu++) {
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
            // The scale ring is read by the promotion warps up to two blocks after the MMA released the tile stage;
            // SCALE_SLOTS = 8 keeps a slot untouched for that long (producers run at most STAGES + 2 blocks ahead).
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int row = lane + 32 * k;
                const int rgl = row / RPG, r = row % RPG;
                const unsigned short h = *reinterpret_cast<const unsigned short*>(&bars->pscale[slot][(rgl * SPT + r) * 2]);
                bars->wscale[g % SCALE_SLOTS][row] = __half2float(__ushort_as_half(h));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // make the generic-proxy writes visible to the MMA
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->full[st]));
            issue(pf);  // refills the slot just consumed (the cursor is two of this warp's blocks ahead: same slot modulo PSLOTS = 8)
            pf.advance(UNPACK_WARPS);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        // ---------------------------------------------------------------- promotion (16 warps; thread = token)
        const int e = warp - (3 + UNPACK_WARPS);
        const int quarter = warp & 3;   // TMEM lanes this warp may read: 32*(warp % 4) ..
        const int cg = e >> 2;          // which 16 of the 64 columns (weight rows); the four warps of a quarter differ in cg
        TileWalk walk;
        walk.init(&L);
        TileRef tr;
        int g = 0;
        bool ok = true;
        while (ok && walk.next(tr)) {
            const TcMat* M = tr.m;
            const int nb = M->nb, n_rows = M->n_rows;
            const int tok = tr.tok0 + quarter * 32 + lane;
            const bool tok_ok = tok < M->seq_len;
            const float* adp = M->ad + (size_t)(tok_ok ? tok : 0) * M->ld_b;
            const int rbase = tr.row0 + cg * 16;  // first weight row of this thread's columns
            // A warp none of whose 32 tokens exist only keeps the barrier protocol going.
            const bool warp_has_tokens = (tr.tok0 + quarter * 32) < M->seq_len;
            float2 sum[8];
#pragma unroll
            for (int c = 0; c < 8; c++) sum[c] = make_float2(0.0f, 0.0f);
            float4 as_next = (nb > 0) ? *reinterpret_cast<const float4*>(adp) : make_float4(0.f, 0.f, 0.f, 0.f);

            for (int blk = 0; blk < nb; blk++, g++) {
                const int buf = g & 1;
                const float4 as4 = as_next;
                if (blk + 1 < nb) as_next = *reinterpret_cast<const float4*>(adp + 4 * (blk + 1));
                if (lane == 0) ok = mbar_wait(smem_u32(&bars->tmem_full[buf]), (g >> 1) & 1, abort_flag, L.status, 6);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                tc_fence_after();
                if (warp_has_tokens) {
                    const float asv[4] = {as4.x, as4.y, as4.z, as4.w};
                    const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256 + cg * 16;
                    const float4* wsp = reinterpret_cast<const float4*>(&bars->wscale[g % SCALE_SLOTS][cg * 16]);
                    // Two halves of eight columns: the four sub-block sums of a half are fetched together, the accumulator
                    // set is handed back to the MMA issuer as soon as the second half sits in registers.
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        uint32_t v[4][8];
#pragma unroll
                        for (int s4 = 0; s4 < 4; s4++) tc_ld8(tbase + s4 * ROW_TILE + hf * 8, v[s4]);
                        tc_wait_ld8(v[0]);
                        tc_pin8(v[1]);
                        tc_pin8(v[2]);
                        tc_pin8(v[3]);
                        if (hf == 1) {
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[buf]));
                        }
                        // block_acc = fma(I0,a0,0), fma(I1,a1,.), fma(I2,a2,.), fma(I3,a3,.); then sum += block_acc * w_scale,
                        // rounded separately (q2_0.rs:545-573, q1_0g128.rs:1026-1051)
#pragma unroll
                        for (int c4 = 0; c4 < 2; c4++) {
                            const float4 wd = wsp[hf * 2 + c4];
#pragma unroll
                            for (int hh = 0; hh < 2; hh++) {
                                const int c = 4 * c4 + 2 * hh;
                                float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
                                for (int s4 = 0; s4 < 4; s4++)
                                    acc = ffma2(make_float2((float)(int)v[s4][c], (float)(int)v[s4][c + 1]), make_float2(asv[s4], asv[s4]), acc);
                                const float2 w2 = hh ? make_float2(wd.z, wd.w) : make_float2(wd.x, wd.y);
                                sum[hf * 4 + (c >> 1)] = fadd2(sum[hf * 4 + (c >> 1)], fmul2(acc, w2));
                            }
                        }
                    }
                } else {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[buf]));
                }
            }
            if (ok && tok_ok && !*abort_flag) {
                float* op = M->out + (size_t)tok * M->ld_out + rbase;
                if (rbase + 16 <= n_rows && (reinterpret_cast<uintptr_t>(op) & 15) == 0) {
                    // 64 contiguous bytes per thread: four 16-byte stores instead of sixteen 4-byte ones
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        reinterpret_cast<float4*>(op)[c] = make_float4(sum[2 * c].x, sum[2 * c].y, sum[2 * c + 1].x, sum[2 * c + 1].y);
                } else {
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        if (rbase + 2 * c < n_rows) op[2 * c] = sum[c].x;
                        if (rbase + 2 * c + 1 < n_rows) op[2 * c + 1] = sum[c].y;
                    }
                }
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

constexpr int TC_SMEM = STAGES * STAGE_BYTES + (int)sizeof(Barriers) + 1024;

}  // namespace

int gemm_tc_prepare() {
    HB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<KIND_Q1>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
    HB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<KIND_Q2>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
    return 0;
}

int gemm_tc_tiles(int n_rows, int seq_len) {
    return ((seq_len + TOK_TILE - 1) / TOK_TILE) * ((n_rows + ROW_TILE - 1) / ROW_TILE);
}

void gemm_tc_fill(TcMat& m, const void* amap_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                  int nb, int seq_len, float* out, int ld_out, int tile_begin) {
    m.bits = bits; m.scales = scales; m.ad = ad; m.out = out; m.amap = amap_dev;
    m.n_rows = n_rows; m.nb = nb; m.seq_len = seq_len; m.ld_out = ld_out; m.ld_b = ld_b;
    m.tok_tiles = (seq_len + TOK_TILE - 1) / TOK_TILE;
    m.tile_begin = tile_begin;
    m.tile_end = tile_begin + gemm_tc_tiles(n_rows, seq_len);
}

static int run_tc(int kind, const TcLaunch& L, int grid, cudaStream_t st) {
    if (kind == KIND_Q1) gemm_tc_kernel<KIND_Q1><<<grid, TC_THREADS, TC_SMEM, st>>>(L);
    else if (kind == KIND_Q2) gemm_tc_kernel<KIND_Q2><<<grid, TC_THREADS, TC_SMEM, st>>>(L);
    else { set_error("gemm_tc: kind %d has no tensor-core kernel", kind); return -7; }
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_gemm_tc(int kind, const void* amap_dev, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                   int nb, int seq_len, float* out, int ld_out, int sm_count, int* status, cudaStream_t st) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    TcLaunch L;
    L.mats = nullptr; L.chunks = nullptr; L.status = status;
    gemm_tc_fill(L.single, amap_dev, bits, scales, ad, ld_b, n_rows, nb, seq_len, out, ld_out, 0);
    L.n_tiles = L.single.tile_end;
    return run_tc(kind, L, L.n_tiles < sm_count ? L.n_tiles : sm_count, st);
}

int launch_gemm_tc_list(int kind, const TcMat* mats_dev, const int* chunks_dev, int n_tiles, int grid, int* status, cudaStream_t st) {
    if (n_tiles <= 0 || grid <= 0) return 0;
    TcLaunch L;
    L.mats = mats_dev; L.chunks = chunks_dev; L.status = status; L.n_tiles = n_tiles;
    L.single = TcMat{};
    return run_tc(kind, L, grid, st);
}

}  // namespace hb200
