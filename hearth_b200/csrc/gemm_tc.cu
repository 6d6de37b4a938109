// Prefill / multi-token matmul on the 5th-generation tensor cores: tcgen05.mma kind::i8 with TMEM
// accumulators, for Q1_0 and Q2_0 / PQ2_0 weights against 5 or more Q8_0 activations.
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
// Tile: 128 tokens (TMEM lanes) x 64 weight rows (TMEM columns) per CTA, K walked in 128-column blocks.
//   warp 0      TMA producer: int8 activation tile 128 tokens x 128 B per block (SWIZZLE_128B, K-major)
//   warp 1      TMEM allocation + single-thread MMA issue: 4 MMAs (128x64x32) per block into 4 x 64 columns
//   warps 2-5   unpack: 64 rows x 128 columns of 1-/2-bit codes -> int8 {-1,+1} / {-1,0,+1,+2} in the same
//               swizzled K-major layout, written with 128-bit shared stores
//   warps 6-13  promotion: tcgen05.ld 32 columns at a time, thread = token, 32 running sums per thread
// Two accumulator sets (2 x 256 TMEM columns) let the MMAs of block b+1 run under the promotion of block b;
// a 4-stage shared-memory ring decouples TMA / unpack from the MMA issue.
// Every wait on an mbarrier is bounded; on expiry the CTA records a status code, stops issuing, drains its
// outstanding bulk copies, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

namespace hb200 {

namespace {

constexpr int TC_THREADS = 448;
constexpr int TOK_TILE = 128;
constexpr int ROW_TILE = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = TOK_TILE * 128;  // 16 KiB
constexpr int B_BYTES = ROW_TILE * 128;  // 8 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t SPIN_LIMIT = 1u << 22;

struct TcArgs {
    const uint4* bits;
    const void* scales;
    const float* ad;   // activation block scales, ld_b floats per token
    float* out;
    int* status;       // device word: 0 ok, otherwise the code of the first wait that expired
    int n_rows, nb, seq_len, ld_out, ld_b;
};

// ---- PTX wrappers -----------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
// Bounded wait.  Returns false (after recording `code`) if the phase did not complete or the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 63) == 63 && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(0u)  // p = false: D = A*B, no accumulation
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
#define HB_R32(v)                                                                                                    \
    "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]), "+r"(v[9]),  \
        "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]), "+r"(v[16]), "+r"(v[17]), "+r"(v[18]),  \
        "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]),  \
        "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
// Waits for every outstanding tcgen05.ld of this thread.  The loaded registers are listed as read-write operands so
// that the compiler cannot schedule a use of them ahead of the wait.
__device__ __forceinline__ void tc_wait_ld(uint32_t (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : HB_R32(v)::"memory");
}
// Same ordering guarantee for a second register array covered by the same wait.
__device__ __forceinline__ void tc_pin(uint32_t (&v)[32]) { asm volatile("" : HB_R32(v)::"memory"); }

// K-major, SWIZZLE_128B shared-memory matrix descriptor: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);  // start address
    d |= (uint64_t)1 << 16;                  // leading byte offset (unused for swizzled K-major; canonical value 1)
    d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                  // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
    return d;
}
// kind::i8, D = S32, A and B signed int8, both K-major, M = 128, N = 64.
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ROW_TILE >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

constexpr int SCALE_SLOTS = 8;  // ring of per-block weight scales (f32); deeper than the tile ring, see the unpack loop
struct Barriers {
    uint64_t full_a[STAGES], full_b[STAGES], empty[STAGES];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    alignas(16) float wscale[SCALE_SLOTS][ROW_TILE];
};

template <int KIND>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap amap, const TcArgs args) {
    constexpr int RPG = rows_per_group(KIND);
    extern __shared__ unsigned char smem_dyn[];
    // 1024-byte alignment for the swizzled tiles
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    Barriers* bars = reinterpret_cast<Barriers*>(tiles + STAGES * STAGE_BYTES);
    volatile int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * ROW_TILE;
    const int tok0 = blockIdx.y * TOK_TILE;
    const int nb = args.nb;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(smem_u32(&bars->full_a[i]), 1);
            mbar_init(smem_u32(&bars->full_b[i]), 4);
            mbar_init(smem_u32(&bars->empty[i]), 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(smem_u32(&bars->tmem_full[i]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[i]), 8);
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

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (one lane)
        if (lane == 0) {
            int issued = 0;
            for (int blk = 0; blk < nb; blk++) {
                const int st = blk % STAGES;
                if (blk >= STAGES &&
                    !mbar_wait(smem_u32(&bars->empty[st]), ((blk / STAGES) - 1) & 1, abort_flag, args.status, 1))
                    break;
                const uint32_t bar = smem_u32(&bars->full_a[st]);
                mbar_expect_tx(bar, A_BYTES);
                tma_load_2d(smem_u32(tiles + st * STAGE_BYTES), &amap, blk * 128, tok0, bar);
                issued = blk + 1;
            }
            if (*abort_flag) {
                // Do not leave the CTA with bulk copies in flight: wait (bounded) for the ones already issued.
                const int first = issued > STAGES ? issued - STAGES : 0;
                for (int blk = first; blk < issued; blk++) {
                    const uint32_t bar = smem_u32(&bars->full_a[blk % STAGES]);
                    for (uint32_t i = 0; i < SPIN_LIMIT && !mbar_try(bar, (blk / STAGES) & 1); i++) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue (one lane)
        if (lane == 0) {
            for (int blk = 0; blk < nb; blk++) {
                const int st = blk % STAGES, buf = blk & 1;
                const uint32_t ph = (blk / STAGES) & 1;
                if (!mbar_wait(smem_u32(&bars->full_a[st]), ph, abort_flag, args.status, 2)) break;
                if (!mbar_wait(smem_u32(&bars->full_b[st]), ph, abort_flag, args.status, 3)) break;
                if (blk >= 2 && !mbar_wait(smem_u32(&bars->tmem_empty[buf]), ((blk >> 1) - 1) & 1, abort_flag, args.status, 4)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(tiles + st * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int s = 0; s < 4; s++)  // one K=32 MMA per sub-block; +32 B inside the 128 B swizzle row
                    tc_mma_i8(tmem_base + buf * 256 + s * ROW_TILE, make_desc(a_addr + s * 32), make_desc(b_addr + s * 32), IDESC);
                tc_commit(smem_u32(&bars->empty[st]));       // the stage may be refilled once these MMAs have read it
                tc_commit(smem_u32(&bars->tmem_full[buf]));  // the accumulators are complete
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------- unpack (128 threads)
        // Each thread owns two units (row of the tile, sub-block); the packed words of the next block are
        // fetched before the current block is expanded, so the global-load latency hides behind the ring.
        const int ut = threadIdx.x - 64;
        const uint2* src[2][4];
        int rsh[2], ris[2], ss[2];
#pragma unroll
        for (int uu = 0; uu < 2; uu++) {
            const int u = ut + uu * 128;
            const int ri = u >> 2, s = u & 3;
            const int grow = row0 + ri;
            const int rg = grow / RPG, r = grow % RPG;
            ris[uu] = ri; ss[uu] = s;
            rsh[uu] = (KIND == KIND_Q1) ? r : 2 * r;
            const uint4* tp = args.bits + (size_t)(rg >> 5) * nb * 256 + (rg & 31);
#pragma unroll
            for (int jp = 0; jp < 4; jp++)  // words 2jp, 2jp+1 of sub-block s: piece 2jp + (s>>1), components (s&1)*2, +1
                src[uu][jp] = reinterpret_cast<const uint2*>(tp + (2 * jp + (s >> 1)) * 32) + (s & 1);
        }
        // weight scale of row (ut & 63) of the tile, block 0 (only threads 0..63 stage scales)
        const int srow = row0 + (ut & 63);
        const int srg = srow / RPG, sr = srow % RPG;
        const unsigned short* sc16 = reinterpret_cast<const unsigned short*>(args.scales) +
                                     ((size_t)(srg >> 5) * nb * 32 + (srg & 31)) * scales_per_tile(KIND) + sr;
        uint2 cur[2][4], nxt[2][4];
        unsigned short sc_cur = 0, sc_nxt = 0;
        auto fetch = [&](int blk, uint2 (&dst)[2][4], unsigned short& sc) {
            const size_t off = (size_t)blk * 256 * 2;  // uint2 units per tile: 256 uint4
#pragma unroll
            for (int uu = 0; uu < 2; uu++)
#pragma unroll
                for (int jp = 0; jp < 4; jp++) dst[uu][jp] = __ldg(src[uu][jp] + off);
            if (ut < 64) sc = __ldg(sc16 + (size_t)blk * 32 * scales_per_tile(KIND));
        };
        if (nb > 0) fetch(0, cur, sc_cur);
        for (int blk = 0; blk < nb; blk++) {
            const int st = blk % STAGES;
            if (blk + 1 < nb) fetch(blk + 1, nxt, sc_nxt);
            bool ok = true;
            if (blk >= STAGES) {
                if (lane == 0) ok = mbar_wait(smem_u32(&bars->empty[st]), ((blk / STAGES) - 1) & 1, abort_flag, args.status, 5);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
            if (!ok) break;
            unsigned char* bt = tiles + st * STAGE_BYTES + A_BYTES;
#pragma unroll
            for (int uu = 0; uu < 2; uu++) {
                uint32_t vals[8];
#pragma unroll
                for (int jp = 0; jp < 4; jp++) {
                    const uint32_t ww[2] = {cur[uu][jp].x, cur[uu][jp].y};
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        uint32_t v;
                        if (KIND == KIND_Q1) {
                            const uint32_t m = (ww[e] >> rsh[uu]) & 0x01010101u;  // bit -> 0/1
                            v = (m * 0xFEu) ^ 0xFFFFFFFFu;                         // 1 -> 0x01 (+1), 0 -> 0xFF (-1)
                        } else {
                            const uint32_t c = ((ww[e] >> rsh[uu]) & 0x03030303u) | 0x80808080u;
                            v = (c - 0x01010101u) ^ 0x80808080u;                   // code - 1 per byte, no borrow across bytes
                        }
                        vals[2 * jp + e] = v;
                    }
                }
                unsigned char* rowp = bt + ris[uu] * 128;
                const int sw = ris[uu] & 7;
                *reinterpret_cast<uint4*>(rowp + (((2 * ss[uu]) ^ sw) << 4)) = make_uint4(vals[0], vals[1], vals[2], vals[3]);
                *reinterpret_cast<uint4*>(rowp + (((2 * ss[uu] + 1) ^ sw) << 4)) = make_uint4(vals[4], vals[5], vals[6], vals[7]);
            }
            // The scale ring is read by the promotion warps up to two blocks after the MMA released the tile
            // stage; SCALE_SLOTS = 8 keeps a slot untouched for that long (the producers run at most
            // STAGES + 2 blocks ahead of the slowest reader).
            if (ut < 64) bars->wscale[blk % SCALE_SLOTS][ut] = __half2float(__ushort_as_half(sc_cur));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // make the generic-proxy writes visible to the MMA
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->full_b[st]));
#pragma unroll
            for (int uu = 0; uu < 2; uu++)
#pragma unroll
                for (int jp = 0; jp < 4; jp++) cur[uu][jp] = nxt[uu][jp];
            sc_cur = sc_nxt;
        }
    } else {
        // ---------------------------------------------------------------- promotion (8 warps; thread = token)
        const int e = warp - 6;
        const int quarter = warp & 3;   // TMEM lanes this warp may read: 32*(warp % 4) ..
        const int half = e >> 2;        // which 32 of the 64 columns (weight rows)
        const int tok = tok0 + quarter * 32 + lane;
        const bool tok_ok = tok < args.seq_len;
        const float* adp = args.ad + (size_t)(tok_ok ? tok : 0) * args.ld_b;
        const int rbase = row0 + half * 32;  // first weight row of this thread's columns
        // A warp none of whose 32 tokens exist only keeps the barrier protocol going.
        const bool warp_has_tokens = (tok0 + quarter * 32) < args.seq_len;
        float sum[32];
#pragma unroll
        for (int c = 0; c < 32; c++) sum[c] = 0.0f;
        float4 as_next = (nb > 0) ? *reinterpret_cast<const float4*>(adp) : make_float4(0.f, 0.f, 0.f, 0.f);

        for (int blk = 0; blk < nb; blk++) {
            const int buf = blk & 1;
            const float4 as4 = as_next;
            if (blk + 1 < nb) as_next = *reinterpret_cast<const float4*>(adp + 4 * (blk + 1));
            bool ok = true;
            if (lane == 0) ok = mbar_wait(smem_u32(&bars->tmem_full[buf]), (blk >> 1) & 1, abort_flag, args.status, 6);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            tc_fence_after();
            if (warp_has_tokens) {
                const float asv[4] = {as4.x, as4.y, as4.z, as4.w};
                float bacc[32];
                const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256 + half * 32;
                uint32_t v0[32], v1[32];
                tc_ld32(tbase, v0);
                tc_ld32(tbase + ROW_TILE, v1);
                tc_wait_ld(v0);
                tc_pin(v1);
#pragma unroll
                for (int c = 0; c < 32; c++) bacc[c] = fmaf((float)(int)v0[c], asv[0], 0.0f);
                tc_ld32(tbase + 2 * ROW_TILE, v0);
#pragma unroll
                for (int c = 0; c < 32; c++) bacc[c] = fmaf((float)(int)v1[c], asv[1], bacc[c]);
                tc_ld32(tbase + 3 * ROW_TILE, v1);
                tc_wait_ld(v0);
                tc_pin(v1);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[buf]));
#pragma unroll
                for (int c = 0; c < 32; c++) bacc[c] = fmaf((float)(int)v0[c], asv[2], bacc[c]);
#pragma unroll
                for (int c = 0; c < 32; c++) bacc[c] = fmaf((float)(int)v1[c], asv[3], bacc[c]);
                // sum += block_acc * w_scale, rounded separately (q2_0.rs:572, q1_0g128.rs:1050)
                const float4* wsp = reinterpret_cast<const float4*>(&bars->wscale[blk % SCALE_SLOTS][half * 32]);
#pragma unroll
                for (int c4 = 0; c4 < 8; c4++) {
                    const float4 wd = wsp[c4];
                    sum[4 * c4 + 0] = __fadd_rn(sum[4 * c4 + 0], __fmul_rn(bacc[4 * c4 + 0], wd.x));
                    sum[4 * c4 + 1] = __fadd_rn(sum[4 * c4 + 1], __fmul_rn(bacc[4 * c4 + 1], wd.y));
                    sum[4 * c4 + 2] = __fadd_rn(sum[4 * c4 + 2], __fmul_rn(bacc[4 * c4 + 2], wd.z));
                    sum[4 * c4 + 3] = __fadd_rn(sum[4 * c4 + 3], __fmul_rn(bacc[4 * c4 + 3], wd.w));
                }
            } else {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[buf]));
            }
        }
        if (tok_ok && !*abort_flag) {
            float* op = args.out + (size_t)tok * args.ld_out + rbase;
#pragma unroll
            for (int c = 0; c < 32; c++)
                if (rbase + c < args.n_rows) op[c] = sum[c];
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

int launch_gemm_tc(int kind, const void* amap, const uint4* bits, const void* scales, const float* ad, int ld_b, int n_rows,
                   int nb, int seq_len, float* out, int ld_out, int* status, cudaStream_t st) {
    if (n_rows <= 0 || seq_len <= 0) return 0;
    TcArgs a;
    a.bits = bits; a.scales = scales; a.ad = ad; a.out = out; a.status = status;
    a.n_rows = n_rows; a.nb = nb; a.seq_len = seq_len; a.ld_out = ld_out; a.ld_b = ld_b;
    dim3 grid((n_rows + ROW_TILE - 1) / ROW_TILE, (seq_len + TOK_TILE - 1) / TOK_TILE);
    const CUtensorMap& map = *static_cast<const CUtensorMap*>(amap);
    if (kind == KIND_Q1) gemm_tc_kernel<KIND_Q1><<<grid, TC_THREADS, TC_SMEM, st>>>(map, a);
    else if (kind == KIND_Q2) gemm_tc_kernel<KIND_Q2><<<grid, TC_THREADS, TC_SMEM, st>>>(map, a);
    else { set_error("gemm_tc: kind %d has no tensor-core kernel", kind); return -7; }
    HB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace hb200
