// Measures the dense int8 rate of the 5th-generation tensor cores on the device in use: the denominator the
// prefill kernel's roofline fraction is quoted against.  One CTA per SM issues a long run of
// tcgen05.mma kind::i8 (128 x 256 x 32, operands resident in shared memory, accumulators in TMEM) with nothing else
// in the way: no loads, no epilogue.  The figure is an upper bound for any kind::i8 kernel on this GPU at the
// clocks it runs at while measured.
#include "common.cuh"

namespace hb200 {

namespace {

constexpr int PK_M = 128, PK_N = 256, PK_K = 32;
constexpr int PK_A_BYTES = PK_M * 128, PK_B_BYTES = PK_N * 128;
constexpr int PK_SMEM = PK_A_BYTES + PK_B_BYTES + 1024;
constexpr uint32_t PK_SPIN = 1u << 24;

__device__ __forceinline__ uint32_t pk_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major, SWIZZLE_128B shared-memory matrix descriptor: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t pk_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::i8, D = S32, A and B signed int8, both K-major, M = 128, N = 256.
constexpr uint32_t PK_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PK_N >> 3) << 17) | ((uint32_t)(PK_M >> 4) << 24);

__global__ void __launch_bounds__(128, 1) tc_i8_peak_kernel(int n_mma, int* status) {
    extern __shared__ unsigned char pk_smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pk_smem) + 1023) & ~uintptr_t(1023));
    for (int i = threadIdx.x; i < (PK_A_BYTES + PK_B_BYTES) / 16; i += blockDim.x) reinterpret_cast<uint4*>(tiles)[i] = make_uint4(0x01010101u, 0xFF01FF01u, 0x02FE02FEu, 0u);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pk_smem_u32(&bar)), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pk_smem_u32(&tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    if (threadIdx.x == 0) {
        const uint64_t ad = pk_desc(pk_smem_u32(tiles)), bd = pk_desc(pk_smem_u32(tiles + PK_A_BYTES));
        for (int i = 0; i < n_mma; i++) {
            const uint32_t acc = (i >= 2) ? 1u : 0u;  // two accumulator sets of 256 columns, used alternately
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "setp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem + (i & 1) * 256),
                "l"(ad + 2 * (i & 3)), "l"(bd + 2 * (i & 3)), "r"(PK_IDESC), "r"(acc)
                : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pk_smem_u32(&bar)) : "memory");
        // Bounded wait for the last MMA; an expiry is reported, never spun on.
        bool done = false;
        for (uint32_t i = 0; i < PK_SPIN && !done; i++) {
            uint32_t ok;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(ok)
                : "r"(pk_smem_u32(&bar)), "r"(0)
                : "memory");
            done = ok != 0;
        }
        if (!done) atomicCAS(status, 0, 9);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace

// Returns the measured rate in TOP/s (2 ops per multiply-accumulate) through *tops; `status` is the device status word.
int measure_i8_peak(int sm_count, int* status, cudaStream_t st, double* tops) {
    HB_CUDA(cudaFuncSetAttribute(tc_i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM));
    const int n_mma = 16384;
    cudaEvent_t e0, e1;
    HB_CUDA(cudaEventCreate(&e0));
    HB_CUDA(cudaEventCreate(&e1));
    float best_ms = 0.0f;
    for (int rep = 0; rep < 4; rep++) {  // first pass warms up
        HB_CUDA(cudaEventRecord(e0, st));
        tc_i8_peak_kernel<<<sm_count, 128, PK_SMEM, st>>>(n_mma, status);
        HB_CUDA(cudaEventRecord(e1, st));
        HB_CUDA(cudaEventSynchronize(e1));
        HB_CUDA(cudaGetLastError());
        float ms = 0.0f;
        HB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        if (rep > 0 && (best_ms == 0.0f || ms < best_ms)) best_ms = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    const double ops = 2.0 * PK_M * PK_N * PK_K * (double)n_mma * sm_count;
    *tops = ops / (best_ms * 1e-3) / 1e12;
    return 0;
}

}  // namespace hb200
