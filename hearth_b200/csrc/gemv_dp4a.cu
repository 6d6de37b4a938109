// Decode matvec: every row of a Q1_0 / Q2_0 / Q8_0 weight against M <= 4 Q8_0
// activations, for a whole list of independent (weight, activation, output)
// operations in one launch.
//
// Replaces the per-row DotFn loop that ThreadPool::par_dot_rows{,_batched}
// (hearth-llm/src/pool.rs:40-80, :510-618) runs over
//   dot_q1_0g128_q8_0_ptr  hearth-quant/src/q1_0g128.rs:1000-1053
//   dot_q2_0_q8_0_ptr      hearth-quant/src/q2_0.rs:537-574, :628-676
//   dot_q8_0_q8_0_ptr      hearth-quant/src/q8_0.rs:154-171
// and reproduces their scalar arithmetic bit for bit:
//   * the int32 dot of every 32-column sub-block is exact;
//   * block_acc = (((0 + I0*a0) + I1*a1) + I2*a2) + I3*a3, sum += block_acc * w_scale,
//     blocks in order, every step separately rounded.  I*a is exact in fp32
//     (|I| <= 2^13, an f16 scale has 11 significant bits), so fmaf(I, a, acc)
//     rounds exactly as the reference's separate multiply and add do; the
//     `* w_scale` and the running sum use __fmul_rn / __fadd_rn.
//
// Work decomposition (HBM-bound streaming; grid = resident CTAs x SM count).
//   item  = one panel (32 row groups) of one op.  A list launch follows a plan made on the host (FlatRec records): per
//           CTA a run of segments, each consecutive whole panels of one op or the first / last rounds of one panel that
//           the plan cut between two neighbouring CTAs - the earlier CTA hands the panel's running sums over in global
//           memory and the later one continues the same ordered sum.  The next segment's record and its first round are
//           fetched while the current segment runs.
//   lane  = one row group of the panel; all lanes of a warp read the same
//           128-column block, so activation reads from shared memory are broadcasts.
//   warp  = one block per round; 8 warps cover 8 consecutive blocks (1024
//           columns) per round.  Weight pieces for the next round are loaded
//           into registers (8 x 128-bit, 512 contiguous bytes per warp per
//           piece) before the current round is computed.
//   unpack: the byte of a tile word holds RPG rows of one column, so
//           `word & (mask << r)` isolates row r's code for four columns and a
//           u8 x s8 dp4a accumulates (code << shift) * a: one LOP3 per dp4a, no
//           shifts.  The 2^shift factor and the "-sum(a)" term that turn codes
//           into {-1,+1} / {-1,0,+1,+2} weights are removed exactly when the
//           sub-block sum is widened to fp32.
//   order: per-block terms go to shared memory; one thread per (token, row)
//          adds them in block order, one round behind the producers.
#include "common.cuh"

namespace hb200 {

namespace {

constexpr int THREADS = 256;
constexpr int WARPS = 8;

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_s8s8(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_wait_all() {
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ uint32_t comp(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }
__device__ __forceinline__ int compi(const int4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

// Resident CTAs per SM the kernel of (kind, tokens) is compiled for: two, i.e. at most 128 registers, except Q8_0 at
// four tokens.  Q2_0 fits without spilling up to four tokens (three and four tokens: 12 % faster than one CTA per SM),
// Q8_0 up to three; Q1_0 - eight rows per lane - spills 58 bytes at three tokens and 218 at four and is still 2.5 and
// 5 % faster with two CTAs.
__host__ __device__ constexpr int dp4a_ctas_per_sm(int kind, int m) { return (kind == KIND_Q8 && m > 3) ? 1 : 2; }

template <int KIND, int M>
struct Smem {
    static constexpr int RPG = rows_per_group(KIND);
    static constexpr int RP = 32 * RPG;                               // rows per panel
    static constexpr int TPB = (KIND == KIND_Q8) ? 4 * 32 : RP;      // per-block terms per token
    // one round: 8 blocks
    alignas(16) int8_t aq[2][M][1024];
    alignas(16) float ad[2][M][32];
    alignas(16) float asum[2][M][32];
    alignas(16) float term[2][WARPS][M][TPB];
};

// as_float(MAGIC_I + x) == MAGIC_F + x exactly for |x| < 2^22: starting the dp4a accumulators at MAGIC_I turns the
// int -> float conversion of a sub-block sum into one FADD, off the ALU pipe that the LOP3 unpack saturates.
constexpr int MAGIC_I = 0x4B400000;
constexpr float MAGIC_F = 12582912.0f;

// Raises this rank's flag in every rank's control block, then (optionally) waits, with a bound, for the other ranks'
// flags here.  One thread.
__device__ __forceinline__ void peer_flag_exchange(const PeerTable& peers) {
    int* ctrl_me = reinterpret_cast<int*>(reinterpret_cast<char*>(peers.data[peers.me]) - PEER_CTRL_BYTES);
    __threadfence_system();
    for (int p = 0; p < peers.n; p++) {
        volatile int* f = reinterpret_cast<volatile int*>(reinterpret_cast<char*>(peers.data[p]) - PEER_CTRL_BYTES);
        f[peers.me] = peers.epoch;
    }
    if (peers.wait) {
        volatile int* mine = reinterpret_cast<volatile int*>(ctrl_me);
        for (int r = 0; r < peers.n; r++) {
            unsigned spins = 0;
            while (mine[r] - peers.epoch < 0) {  // epochs only grow; the difference also survives wrap-around
                if (++spins > (1u << 21)) {      // about a second and a half
                    atomicCAS(peers.status, 0, 100 + r);
                    break;
                }
                __nanosleep(64);
            }
        }
        __threadfence_system();
    }
}

// The arithmetic of one round for one warp: block `blk` of `panel` (weight pieces w, scales ws) against the staged
// activation columns in buffer `buf`; leaves the per-block terms in shared memory (or, INT_OUT, stores the int32
// sub-block dots).
template <int KIND, int M, bool INT_OUT>
__device__ __forceinline__ void round_terms(Smem<KIND, M>& sm, const uint4 (&w)[8], const uint4& ws, int buf, int warp, int lane, int blk,
                                            int panel, const DotOp* op) {  // op: read for INT_OUT only
    using S = Smem<KIND, M>;
    constexpr int RPG = S::RPG;
    constexpr int RP = S::RP;
    (void)RP; (void)blk; (void)panel;
    // Q2_0, one token: the last row of a lane's group needs no mask.  The dot of the whole word is sum_g 4^g S_g, so
    // that row's accumulator takes the unmasked word and the other three accumulators are subtracted from it once per
    // sub-block: three subtractions instead of eight LOP3, on the pipe the unpack saturates.  Started at
    // RPG * MAGIC_I (mod 2^32) it ends, like the others, at MAGIC_I + its own sum.  (The masks are shared by all
    // tokens, the subtractions are not: at two and three tokens it measured 1.5 and 0.7 % slower; for Q1_0 the chain of
    // seven subtractions measured slower than the eight LOP3.)
    constexpr bool TOTAL = (KIND == KIND_Q2 && M == 1);
    float bacc[M][RPG];
#pragma unroll
    for (int m = 0; m < M; m++)
#pragma unroll
        for (int g = 0; g < RPG; g++) bacc[m][g] = 0.0f;

#pragma unroll
    for (int s = 0; s < 4; s++) {
        int acc[M][RPG];
#pragma unroll
        for (int m = 0; m < M; m++)
#pragma unroll
            for (int g = 0; g < RPG; g++)
                acc[m][g] = INT_OUT ? 0 : ((TOTAL && g == RPG - 1) ? (int)((unsigned)MAGIC_I * (unsigned)RPG) : MAGIC_I);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            int4 a4[M];
#pragma unroll
            for (int m = 0; m < M; m++)
                a4[m] = *reinterpret_cast<const int4*>(&sm.aq[buf][m][warp * 128 + s * 32 + h * 16]);
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const int j = 4 * h + jj;                      // word of the sub-block: columns 4j..4j+3
                const int q = (j >> 1) * 8 + s * 2 + (j & 1);  // its position in the tile
                const uint32_t word = comp(w[q >> 2], q & 3);
#pragma unroll
                for (int g = 0; g < RPG; g++) {
                    uint32_t msk;
                    if (TOTAL && g == RPG - 1) msk = word;
                    else if (KIND == KIND_Q1) msk = word & (0x01010101u << g);
                    else if (KIND == KIND_Q2) msk = word & (0x03030303u << (2 * g));
                    else msk = word;
#pragma unroll
                    for (int m = 0; m < M; m++) {
                        if (KIND == KIND_Q8) acc[m][g] = dp4a_s8s8(msk, compi(a4[m], jj), acc[m][g]);
                        else acc[m][g] = dp4a_u8s8(msk, compi(a4[m], jj), acc[m][g]);
                    }
                }
            }
        }
        if (TOTAL) {
#pragma unroll
            for (int m = 0; m < M; m++) {
                unsigned t = (unsigned)acc[m][RPG - 1];
#pragma unroll
                for (int g = 0; g < RPG - 1; g++) t -= (unsigned)acc[m][g];
                acc[m][RPG - 1] = (int)t;
            }
        }
        // Widen the sub-block sums.
#pragma unroll
        for (int m = 0; m < M; m++) {
            const float a_d = sm.ad[buf][m][warp * 4 + s];
            const float a_sum = sm.asum[buf][m][warp * 4 + s];
#pragma unroll
            for (int g = 0; g < RPG; g++) {
                if (INT_OUT) {
                    int iv;
                    if (KIND == KIND_Q1) iv = ((acc[m][g] << 1) >> g) - (int)a_sum;       // 2*S1 - sum(a)
                    else if (KIND == KIND_Q2) iv = (acc[m][g] >> (2 * g)) - (int)a_sum;  // S_code - sum(a)
                    else iv = acc[m][g];
                    const int row = panel * RP + lane * RPG + g;
                    if (row < op->n_rows && blk * 4 + s < op->n_sub &&
                        HB_IDX(((size_t)m * op->n_rows + row) * op->n_sub + blk * 4 + s, (size_t)M * op->n_rows * op->n_sub, 6))
                        op->iout[((size_t)m * op->n_rows + row) * op->n_sub + blk * 4 + s] = iv;
                } else {
                    const float accf = __fadd_rn(__int_as_float(acc[m][g]), -MAGIC_F);  // exact (float)sum
                    if (KIND == KIND_Q8) {
                        const float wd = __half2float(__ushort_as_half(
                            (unsigned short)((s < 2 ? ws.x : ws.y) >> (16 * (s & 1)))));
                        // ((float)sumi * d_w) * d_a, each product rounded (q8_0.rs:169)
                        sm.term[buf][warp][m][s * 32 + lane] = __fmul_rn(__fmul_rn(accf, wd), a_d);
                    } else {
                        // exact integer I as fp32, then block_acc += I * a_scale (exact product, one rounding)
                        const float c = (KIND == KIND_Q1) ? (2.0f / (float)(1 << g)) : (1.0f / (float)(1 << (2 * g)));
                        const float i_f = fmaf(accf, c, -a_sum);
                        bacc[m][g] = fmaf(i_f, a_d, bacc[m][g]);
                    }
                }
            }
        }
    }
    if (!INT_OUT && KIND != KIND_Q8) {
        float wd[RPG];
#pragma unroll
        for (int g = 0; g < RPG; g++) {
            const uint32_t pair = (g < 2) ? ws.x : (g < 4 ? ws.y : (g < 6 ? ws.z : ws.w));
            wd[g] = __half2float(__ushort_as_half((unsigned short)(pair >> (16 * (g & 1)))));
        }
#pragma unroll
        for (int m = 0; m < M; m++) {
            float4* tp = reinterpret_cast<float4*>(&sm.term[buf][warp][m][lane * RPG]);
#pragma unroll
            for (int g4 = 0; g4 < RPG / 4; g4++)
                tp[g4] = make_float4(__fmul_rn(bacc[m][4 * g4], wd[4 * g4]), __fmul_rn(bacc[m][4 * g4 + 1], wd[4 * g4 + 1]),
                                     __fmul_rn(bacc[m][4 * g4 + 2], wd[4 * g4 + 2]), __fmul_rn(bacc[m][4 * g4 + 3], wd[4 * g4 + 3]));
        }
    }
}

template <int KIND, int M, bool INT_OUT>
__global__ void __launch_bounds__(THREADS, dp4a_ctas_per_sm(KIND, M))
gemv_dp4a_kernel(const __grid_constant__ FlatLaunch A, int n_items, const __grid_constant__ DotOp single,
                 const __grid_constant__ PeerTable peers) {
    const FlatRec* __restrict__ recs = A.recs;  // null: the one op `single`, its panels split evenly over the CTAs
    __shared__ __align__(16) FlatRec srec[2];   // this segment's record and, copied in while it runs, the next one's
    using S = Smem<KIND, M>;
    constexpr int RP = S::RP;
    constexpr int NRUN = (M * RP + THREADS - 1) / THREADS;  // running sums per thread
    extern __shared__ __align__(16) unsigned char smem_raw[];
    S& sm = *reinterpret_cast<S*>(smem_raw);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // This CTA's work.  A list launch reads its run of segments from the plan (FlatSeg: consecutive whole panels of one
    // op, or rounds [r0, r1) of ONE panel that the plan cut between two neighbouring CTAs); a single-op launch splits the
    // panels of `single` evenly.  Of a cut panel, the CTA before the cut computes the first rounds and hands the running
    // sums of the panel's rows over in a carry slot in global memory; the CTA after the cut starts its ordered sum from
    // them: the same additions in the same order, the same bits.  The plan puts the part a CTA hands over first in its
    // run and the part it receives a carry for last, so the carry was written long before it is read; the wait for it
    // is bounded all the same (status code 50).  A slot's flag counts the warps that have written it, eight per launch.
    int it = recs ? A.seg_begin[blockIdx.x] : (int)(((long long)n_items * blockIdx.x) / gridDim.x);
    const int it_end = recs ? A.seg_begin[blockIdx.x + 1] : (int)(((long long)n_items * (blockIdx.x + 1)) / gridDim.x);
    constexpr int REC_PIECES = (int)(sizeof(FlatRec) / 16);
    static_assert(sizeof(FlatRec) % 16 == 0, "a record is copied in 16-byte pieces");
    // The record of segment i into slot i & 1, asynchronously: it lands under the rounds of the segment before it (every
    // round waits for the thread's outstanding copies), so a change of segment costs no dependent global reads.
    auto fetch_rec = [&](int i) {
        if (tid < REC_PIECES && HB_IDX(i, n_items, 8))
            cp_async16(reinterpret_cast<char*>(&srec[i & 1]) + tid * 16, reinterpret_cast<const char*>(recs + i) + tid * 16);
    };
    if (recs && it < it_end) {
        fetch_rec(it);
        cp_async_commit_wait_all();
    }

    uint4 wn[8];   // weight pieces of the next round
    uint4 wsn;     // its scales (Q1_0: 8 f16; Q2_0 / Q8_0: 4 f16 in .x .y)
    int b0 = 0;        // shared-memory buffer of the segment's first round (rounds alternate from there)
    bool pre = false;  // the segment's first round was fetched under the last round of the segment before it

    while (it < it_end) {
        // One segment.  Rounds run back to back across its panels, so the weight prefetch never drains inside it; the
        // first round of the NEXT segment of a list is fetched under this segment's last round.
        FlatSeg sg;
        DotOp op;
        if (recs) {
            __syncthreads();  // the record is in place (copied during the previous segment, or just now)
            sg = srec[it & 1].seg;
            op = srec[it & 1].op;
            it++;
            if (it < it_end) fetch_rec(it);  // overwrites the slot of the segment before this one: nobody reads it any more
        } else {
            sg.op = 0; sg.p0 = it; sg.cnt = it_end - it; sg.r0 = 0; sg.r1 = 0; sg.flags = 0; sg.carry_in = 0; sg.carry_out = 0;
            it = it_end;
            op = single;
        }
        const int p0 = sg.p0;
        const int nb = op.nb;
        const int rounds = max(1, (nb + WARPS - 1) / WARPS);
        const int r_begin = sg.flags ? sg.r0 : 0;
        const int total = sg.flags ? (sg.r1 - sg.r0) : sg.cnt * rounds;
        const bool carry_in = sg.flags & 1, carry_out = sg.flags & 2;

        // Stage the activation columns of round r into buffer `buf` (cp.async, 16 B each).
        auto stage_of = [&](const DotOp& o, int r, int buf) {
            for (int idx = tid; idx < 80 * M; idx += THREADS) {
                const int m = idx / 80, p = idx % 80;
                if (p < 64) {
                    if (HB_IDX((size_t)r * 1024 + p * 16 + 15, o.ld_q, 3))
                        cp_async16(&sm.aq[buf][m][p * 16], o.aq + (size_t)m * o.ld_q + (size_t)r * 1024 + p * 16);
                } else if (p < 72) {
                    if (HB_IDX(r * 32 + (p - 64) * 4 + 3, o.ld_b, 4))
                        cp_async16(&sm.ad[buf][m][(p - 64) * 4], o.ad + (size_t)m * o.ld_b + r * 32 + (p - 64) * 4);
                } else {
                    if (HB_IDX(r * 32 + (p - 72) * 4 + 3, o.ld_b, 4))
                        cp_async16(&sm.asum[buf][m][(p - 72) * 4], o.asum + (size_t)m * o.ld_b + r * 32 + (p - 72) * 4);
                }
            }
        };
        auto stage = [&](int r, int buf) { stage_of(op, r, buf); };

        auto load_w_of = [&](const DotOp& o, int panel, int r) {
            const int blk = r * WARPS + warp;
            if (blk < o.nb && HB_IDX((size_t)panel * o.nb + blk, (size_t)((o.n_rows + RP - 1) / RP) * o.nb, 1)) {
                const size_t tile = (size_t)panel * o.nb + blk;
                const uint4* p = o.bits + tile * 256 + lane;
#pragma unroll
                for (int i = 0; i < 8; i++) wn[i] = ldg_stream(p + i * 32);
                if (KIND == KIND_Q1) {
                    wsn = __ldg(reinterpret_cast<const uint4*>(o.scales) + tile * 32 + lane);
                } else {
                    const uint2 s2 = __ldg(reinterpret_cast<const uint2*>(o.scales) + tile * 32 + lane);
                    wsn = make_uint4(s2.x, s2.y, 0u, 0u);
                }
            }
        };
        auto load_w = [&](int panel, int r) { load_w_of(op, panel, r); };

        float run[NRUN];
#pragma unroll
        for (int k = 0; k < NRUN; k++) run[k] = 0.0f;
        if (carry_in) {  // every thread polls for itself (no CTA barrier); normally the flag has long been raised
            volatile int* f = A.cflags + sg.carry_in;
            const unsigned target = A.epoch * (unsigned)WARPS;  // counts wrap around together: only their difference is looked at
            unsigned spins = 0;
            while ((int)((unsigned)*f - target) < 0) {
                if (++spins > (1u << 20)) {
                    if (A.status) atomicCAS(A.status, 0, 50);
                    break;
                }
                __nanosleep(64);
            }
            __threadfence();
#pragma unroll
            for (int k = 0; k < NRUN; k++) {
                const int idx = tid + k * THREADS;
                if (idx < M * RP && HB_IDX(sg.carry_in, gridDim.x + 1, 7) && HB_IDX(idx, FLAT_CARRY_FLOATS, 7))
                    run[k] = __ldcg(A.carry + (size_t)sg.carry_in * FLAT_CARRY_FLOATS + idx);
            }
        }

        // Adds the terms of round r of `panel` (buffer `buf`) to the running sums, in block order; after the last
        // round of a panel the sums are the outputs of that panel.
        auto replay = [&](int panel, int r, int buf) {
            const int nvalid = min(WARPS, nb - r * WARPS);
            const bool last = (r == rounds - 1);
#pragma unroll
            for (int k = 0; k < NRUN; k++) {
                const int idx = tid + k * THREADS;
                if (idx < M * RP) {
                    const int m = idx / RP, row = idx % RP;
                    float acc = run[k];
                    if (KIND == KIND_Q8) {
                        const int nsub = min(4 * nvalid, op.n_sub - r * WARPS * 4);
                        for (int sb = 0; sb < nsub; sb++)
                            acc = __fadd_rn(acc, sm.term[buf][sb >> 2][m][(sb & 3) * 32 + row]);
                    } else {
                        for (int b = 0; b < nvalid; b++) acc = __fadd_rn(acc, sm.term[buf][b][m][row]);
                    }
                    if (last) {
                        const int grow = panel * RP + row;
                        if (grow < op.n_rows && HB_IDX((size_t)m * op.ld_out + grow, (size_t)(M - 1) * op.ld_out + op.n_rows, 5)) {
                            float* dst = op.out + (size_t)m * op.ld_out + grow;
                            if (peers.n > 1) {
                                // the same offset inside every rank's output area: one local and n-1 peer stores
                                const ptrdiff_t off = (dst - peers.data[peers.me]) + peers.area_off;
#pragma unroll
                                for (int p = 0; p < MAX_PEERS; p++)
                                    if (p < peers.n) peers.data[p][off] = acc;
                            } else {
                                *dst = acc;
                            }
                        }
                        acc = 0.0f;
                    }
                    run[k] = acc;
                }
            }
        };

        if (!pre) {
            __syncthreads();  // the previous segment's shared memory is no longer read
            stage(r_begin, b0);
            load_w(p0, r_begin);
        }
        pre = false;
        const bool more_segs = recs && it < it_end;  // `it` is the next segment by now, its record is in srec[it & 1] after this segment's first barrier

        int panel = p0, r = r_begin;            // position of round t
        int ppanel = p0, pr = r_begin;          // position of round t - 1
        for (int t = 0; t < total; t++) {
            cp_async_commit_wait_all();
            __syncthreads();  // activations of round t landed; terms of round t-1 visible
            uint4 w[8];
#pragma unroll
            for (int i = 0; i < 8; i++) w[i] = wn[i];
            const uint4 ws = wsn;
            int npanel = panel, nr = r + 1;
            if (nr == rounds) { nr = 0; npanel = panel + 1; }
            if (t + 1 < total) {
                stage(nr, (t + 1 + b0) & 1);
                load_w(npanel, nr);
            } else if (more_segs) {  // the last round: fetch the first round of the next segment
                const FlatRec& nx = srec[it & 1];
                const int nr0 = nx.seg.flags ? nx.seg.r0 : 0;
                stage_of(nx.op, nr0, (t + 1 + b0) & 1);
                load_w_of(nx.op, nx.seg.p0, nr0);
                pre = true;
            }
            if (!INT_OUT && t > 0) replay(ppanel, pr, (t - 1 + b0) & 1);

            const int buf = (t + b0) & 1;
            const int blk = r * WARPS + warp;
            if (blk < nb) round_terms<KIND, M, INT_OUT>(sm, w, ws, buf, warp, lane, blk, panel, &op);
            ppanel = panel; pr = r;
            panel = npanel; r = nr;
        }
        if (!INT_OUT) {
            __syncthreads();
            replay(ppanel, pr, (total - 1 + b0) & 1);
            if (carry_out) {  // the part ended before the panel's last round: the sums go to the CTA that continues it
#pragma unroll
                for (int k = 0; k < NRUN; k++) {
                    const int idx = tid + k * THREADS;
                    if (idx < M * RP && HB_IDX(sg.carry_out, gridDim.x + 1, 7) && HB_IDX(idx, FLAT_CARRY_FLOATS, 7))
                        __stcg(A.carry + (size_t)sg.carry_out * FLAT_CARRY_FLOATS + idx, run[k]);
                }
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(A.cflags + sg.carry_out, 1);
            }
        }
        b0 = (b0 + total) & 1;
    }

    if (!INT_OUT && peers.n > 1) {
        // Every CTA makes its peer stores visible system-wide; in the kernel that closes the launch the last CTA to
        // finish then runs the flag exchange.
        __threadfence_system();
        __syncthreads();
        if (peers.publish && tid == 0) {
            int* counter = reinterpret_cast<int*>(reinterpret_cast<char*>(peers.data[peers.me]) - PEER_CTRL_BYTES) + 64;
            const int prev = atomicAdd(counter, 1);
            if (prev == (int)gridDim.x - 1) {
                *counter = 0;
                peer_flag_exchange(peers);
            }
        }
    }
}

__global__ void peer_publish_kernel(const __grid_constant__ PeerTable peers) { peer_flag_exchange(peers); }

template <int KIND, int M, bool INT_OUT>
int launch_one(const FlatLaunch& A, int grid, int n_items, const DotOp& single, const PeerTable& peers, cudaStream_t st) {
    using S = Smem<KIND, M>;
    if (grid <= 0 || n_items <= 0) return 0;
    gemv_dp4a_kernel<KIND, M, INT_OUT><<<grid, THREADS, sizeof(S), st>>>(A, n_items, single, peers);
    HB_CUDA(cudaGetLastError());
    return 0;
}

template <int KIND, int M, bool INT_OUT>
int prepare_one() {
    using S = Smem<KIND, M>;
    HB_CUDA(cudaFuncSetAttribute(gemv_dp4a_kernel<KIND, M, INT_OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)sizeof(S)));
    return 0;
}

template <int KIND>
int launch_kind(int m, bool int_out, const FlatLaunch& A, int grid, int n_items, const DotOp& single, const PeerTable& peers,
                cudaStream_t st) {
    if (int_out) {
        if (m != 1) { set_error("integer block-dot output runs one token per launch"); return -4; }
        return launch_one<KIND, 1, true>(A, grid, n_items, single, peers, st);
    }
    switch (m) {
        case 1: return launch_one<KIND, 1, false>(A, grid, n_items, single, peers, st);
        case 2: return launch_one<KIND, 2, false>(A, grid, n_items, single, peers, st);
        case 3: return launch_one<KIND, 3, false>(A, grid, n_items, single, peers, st);
        case 4: return launch_one<KIND, 4, false>(A, grid, n_items, single, peers, st);
        default: set_error("gemv_dp4a: m=%d outside 1..%d", m, GEMV_MAX_M); return -4;
    }
}

template <int KIND>
int prepare_kind() {
    int rc;
    if ((rc = prepare_one<KIND, 1, true>())) return rc;
    if ((rc = prepare_one<KIND, 1, false>())) return rc;
    if ((rc = prepare_one<KIND, 2, false>())) return rc;
    if ((rc = prepare_one<KIND, 3, false>())) return rc;
    if ((rc = prepare_one<KIND, 4, false>())) return rc;
    return 0;
}

}  // namespace

int gemv_dp4a_prepare() {
    int rc;
    if ((rc = prepare_kind<KIND_Q1>())) return rc;
    if ((rc = prepare_kind<KIND_Q2>())) return rc;
    if ((rc = prepare_kind<KIND_Q8>())) return rc;
    return 0;
}

int gemv_dp4a_ctas_per_sm(int kind, int m) { return dp4a_ctas_per_sm(kind, m); }

HB_BOUNDS_FETCH(bounds_fetch_dp4a)

int launch_peer_publish(const PeerTable& peers, cudaStream_t st) {
    if (peers.n <= 1) return 0;
    peer_publish_kernel<<<1, 1, 0, st>>>(peers);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_gemv_dp4a(int kind, int m, bool int_out, const FlatLaunch* list, int grid, int n_items, const DotOp* single,
                     cudaStream_t st, const PeerTable* peers) {
    static const DotOp none = {};
    static const PeerTable no_peers = {};
    static const FlatLaunch no_list = {};
    const DotOp& one = single ? *single : none;
    const PeerTable& pt = peers ? *peers : no_peers;
    const FlatLaunch& A = list ? *list : no_list;
    if (!list && !single) { set_error("gemv_dp4a: neither a work list nor a single op"); return -5; }
    if (list && (!list->recs || !list->seg_begin)) { set_error("gemv_dp4a: a list launch needs segment records and their boundaries"); return -5; }
    switch (kind) {
        case KIND_Q1: return launch_kind<KIND_Q1>(m, int_out, A, grid, n_items, one, pt, st);
        case KIND_Q2: return launch_kind<KIND_Q2>(m, int_out, A, grid, n_items, one, pt, st);
        case KIND_Q8: return launch_kind<KIND_Q8>(m, int_out, A, grid, n_items, one, pt, st);
        default: set_error("gemv_dp4a: kind %d has no Q8_0 dot", kind); return -7;
    }
}

}  // namespace hb200
