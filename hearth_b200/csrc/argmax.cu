// Greedy-sampling argmax over the logits, so that only four bytes come back to the host instead of the whole
// vocabulary row.  Replaces GpuCompute::argmax_f32 and its shader
// (hearth-compute/src/lib.rs:338-450, hearth-compute/src/shaders/argmax.wgsl): chunks of 2048 values reduced by
// strict '>' comparisons starting from -3.4028235e38, ties and chunk order resolved towards the lower index, the
// chunk results reduced again by strict '>' from -inf.  The net effect, reproduced here in one launch: the lowest
// index among the largest values that exceed -FLT_MAX; NaN never wins; index 0 if nothing qualifies.
// HBM-bound: 4 bytes read per value.
#include <cfloat>

#include "common.cuh"

namespace hb200 {

namespace {

struct Best {
    float v;
    uint32_t i;
};
// `a` stays unless b is strictly larger, or equal with a lower index (what the reference's fixed scan order gives).
__device__ __forceinline__ Best better(Best a, Best b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// grid = chunks of ARGMAX_CHUNK values, block 256.  partial[] and *ticket live in library-owned device memory;
// the CTA that takes the last ticket reduces the partials, writes *out and resets the ticket for the next call.
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ x, size_t n, Best* __restrict__ partial,
                                                     unsigned int* __restrict__ ticket, uint32_t* __restrict__ out) {
    __shared__ Best sh[8];
    __shared__ bool last;
    const size_t base = (size_t)blockIdx.x * ARGMAX_CHUNK;
    Best b = {-FLT_MAX, 0u};
    for (int k = 0; k < ARGMAX_CHUNK / 256; k++) {
        const size_t i = base + (size_t)k * 256 + threadIdx.x;
        if (i < n) {
            const float v = x[i];
            if (v > b.v) b = {v, (uint32_t)i};  // increasing i per thread: the first of equal values stays
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        Best o = {__shfl_xor_sync(0xffffffffu, b.v, off), __shfl_xor_sync(0xffffffffu, b.i, off)};
        b = better(b, o);
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) b = better(b, sh[w]);
        partial[blockIdx.x] = b;
        __threadfence();
        last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    Best r = {-FLT_MAX, 0u};
    for (unsigned int c = threadIdx.x; c < gridDim.x; c += 256) r = better(r, partial[c]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        Best o = {__shfl_xor_sync(0xffffffffu, r.v, off), __shfl_xor_sync(0xffffffffu, r.i, off)};
        r = better(r, o);
    }
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = r;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) r = better(r, sh[w]);
        *out = r.i;
        *ticket = 0u;
    }
}

}  // namespace

size_t argmax_scratch_bytes() { return (size_t)ARGMAX_MAX_CHUNKS * sizeof(Best) + 256; }

int launch_argmax(const float* x, size_t n, void* scratch, uint32_t* out_dev, cudaStream_t st) {
    const size_t chunks = (n + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
    Best* partial = reinterpret_cast<Best*>(reinterpret_cast<unsigned char*>(scratch) + 256);
    unsigned int* ticket = reinterpret_cast<unsigned int*>(scratch);
    argmax_kernel<<<(unsigned)chunks, 256, 0, st>>>(x, n, partial, ticket, out_dev);
    HB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace hb200
