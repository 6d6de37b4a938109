// One-time re-tiling of the reference's packed weight bytes into the panel
// layout the dot kernels stream (layout: common.cuh).  Runs once per upload,
// like the reference's upload_tensors_to_gpu (hearth-llm/src/model/gpu.rs:8-49);
// speed is irrelevant, clarity is not.
//
// Source formats (hearth-gguf/src/ggml.rs:105-176 for the geometry):
//   Q1_0 / Q1_0_G128  18 B per 128: [f16 d][16 B sign bits, LSB first, 1 -> +1]
//                     (hearth-quant/src/q1_0g128.rs:31-45)
//   Q2_0 / PQ2_0      34 B per 128: [f16 d][32 B, four 2-bit codes per byte, LSB first]
//                     (hearth-quant/src/q2_0.rs:9-23)
//   Q8_0              34 B per 32:  [f16 d][32 x i8]            (hearth-quant/src/q8_0.rs:4-18)
#include "common.cuh"

namespace hb200 {

namespace {

// One thread per output word of the bit / code planes.
template <int KIND>
__global__ void repack_bits_kernel(const uint8_t* __restrict__ raw, size_t row_bytes, int n_rows, int n_cols, int nb,
                                   long long n_words, uint32_t* __restrict__ out) {
    constexpr int RPG = rows_per_group(KIND);
    const long long wi = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= n_words) return;
    // wi = (((panel*nb + blk)*8 + piece)*32 + lane)*4 + comp
    const int comp = (int)(wi & 3);
    const int lane = (int)((wi >> 2) & 31);
    const int piece = (int)((wi >> 7) & 7);
    const long long pb = wi >> 10;
    const int blk = (int)(pb % nb);
    const int panel = (int)(pb / nb);
    const int q = piece * 4 + comp;  // word position inside the tile
    const int t = q >> 3, s = (q >> 1) & 3, e = q & 1;
    const int col0 = blk * 128 + s * 32 + (2 * t + e) * 4;
    const int row0 = (panel * 32 + lane) * RPG;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int col = col0 + i;
        uint32_t byte = 0;
        if (col < n_cols) {
#pragma unroll
            for (int r = 0; r < RPG; r++) {
                const int row = row0 + r;
                if (row >= n_rows) continue;
                const uint8_t* rp = raw + (size_t)row * row_bytes;
                if (KIND == KIND_Q1) {
                    const uint8_t b = rp[(size_t)(col >> 7) * 18 + 2 + ((col & 127) >> 3)];
                    byte |= (uint32_t)((b >> (col & 7)) & 1) << r;
                } else if (KIND == KIND_Q2) {
                    const uint8_t b = rp[(size_t)(col >> 7) * 34 + 2 + ((col & 127) >> 2)];
                    byte |= (uint32_t)((b >> (2 * (col & 3))) & 3) << (2 * r);
                } else {
                    byte = rp[(size_t)(col >> 5) * 34 + 2 + (col & 31)];
                }
            }
        }
        word |= byte << (8 * i);
    }
    out[wi] = word;
}

// One thread per (tile, lane): gathers the tile's f16 scales.
template <int KIND>
__global__ void repack_scales_kernel(const uint8_t* __restrict__ raw, size_t row_bytes, int n_rows, int n_cols, int nb,
                                     long long n_tiles_lanes, unsigned short* __restrict__ out) {
    constexpr int RPG = rows_per_group(KIND);
    constexpr int SPT = scales_per_tile(KIND);
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tiles_lanes) return;
    const int lane = (int)(i & 31);
    const long long pb = i >> 5;
    const int blk = (int)(pb % nb);
    const int panel = (int)(pb / nb);
    const int row0 = (panel * 32 + lane) * RPG;
#pragma unroll
    for (int k = 0; k < SPT; k++) {
        unsigned short h = 0;
        if (KIND == KIND_Q8) {
            const int sub = blk * 4 + k;  // 32-column block index
            if (row0 < n_rows && sub * 32 < n_cols) {
                const uint8_t* p = raw + (size_t)row0 * row_bytes + (size_t)sub * 34;
                h = (unsigned short)(p[0] | (p[1] << 8));
            }
        } else {
            const int row = row0 + k;
            if (row < n_rows) {
                const uint8_t* p = raw + (size_t)row * row_bytes + (size_t)blk * (KIND == KIND_Q1 ? 18 : 34);
                h = (unsigned short)(p[0] | (p[1] << 8));
            }
        }
        out[i * SPT + k] = h;
    }
}

template <int KIND>
int run(const uint8_t* raw, size_t row_bytes, int n_rows, int n_cols, int nb, int n_panels, uint4* bits, void* scales,
        cudaStream_t st) {
    const long long n_words = (long long)n_panels * nb * 8 * 32 * 4;
    const long long n_tl = (long long)n_panels * nb * 32;
    if (n_words == 0) return 0;
    repack_bits_kernel<KIND><<<(unsigned)((n_words + 255) / 256), 256, 0, st>>>(raw, row_bytes, n_rows, n_cols, nb,
                                                                                 n_words, (uint32_t*)bits);
    HB_CUDA(cudaGetLastError());
    repack_scales_kernel<KIND><<<(unsigned)((n_tl + 255) / 256), 256, 0, st>>>(raw, row_bytes, n_rows, n_cols, nb, n_tl,
                                                                                (unsigned short*)scales);
    HB_CUDA(cudaGetLastError());
    return 0;
}

// PTQ1_0 (28 B per 128: qs[24] five base-3 digits per byte, qh[2] four, f16 d at byte 26;
// hearth-quant/src/ptq1_0.rs:1-57) -> the Q2_0 byte layout, digit + 1 being exactly Q2_0's code for the same
// weight (-1 -> 0, 0 -> 1, +1 -> 2).  Element e of a block (ptq1_0.rs:563-585): e < 80 is digit e / 16 of
// qs[e % 16], e < 120 digit (e - 80) / 8 of qs[16 + (e - 80) % 8], else digit (e - 120) / 2 of qh[(e - 120) % 2].
// One thread per output byte (four elements); thread 0 of a block also moves the scale.
__device__ __forceinline__ uint32_t ptq_digit(uint32_t byte, int n) {
    const uint32_t pow3 = (n == 0) ? 1u : (n == 1) ? 3u : (n == 2) ? 9u : (n == 3) ? 27u : 81u;
    return (((byte * pow3) & 255u) * 3u) >> 8;  // 0..2
}

__global__ void __launch_bounds__(256) ptq1_to_q2_kernel(const uint8_t* __restrict__ raw, size_t row_bytes_in, int n_rows, int nb,
                                                         uint8_t* __restrict__ out, size_t row_bytes_out) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)n_rows * nb * 32;
    if (idx >= total) return;
    const int j = (int)(idx & 31);
    const size_t blk = idx >> 5;
    const size_t row = blk / nb;
    const int b = (int)(blk % nb);
    const uint8_t* src = raw + row * row_bytes_in + (size_t)b * 28;
    uint8_t* dst = out + row * row_bytes_out + (size_t)b * 34;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int e = j * 4 + i;
        uint32_t digit;
        if (e < 80) digit = ptq_digit(src[e & 15], e >> 4);
        else if (e < 120) digit = ptq_digit(src[16 + ((e - 80) & 7)], (e - 80) >> 3);
        else digit = ptq_digit(src[24 + ((e - 120) & 1)], (e - 120) >> 1);
        packed |= digit << (2 * i);
    }
    dst[2 + j] = (uint8_t)packed;
    if (j == 0) { dst[0] = src[26]; dst[1] = src[27]; }
}

}  // namespace

int launch_ptq1_to_q2(const uint8_t* raw, size_t row_bytes_in, int n_rows, int nb, uint8_t* out, size_t row_bytes_out,
                      cudaStream_t st) {
    const size_t total = (size_t)n_rows * nb * 32;
    if (total == 0) return 0;
    ptq1_to_q2_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(raw, row_bytes_in, n_rows, nb, out, row_bytes_out);
    HB_CUDA(cudaGetLastError());
    return 0;
}

int launch_repack(int kind, const uint8_t* raw, size_t row_bytes, int n_rows, int n_cols, int nb, int n_panels,
                  uint4* bits, void* scales, cudaStream_t st) {
    switch (kind) {
        case KIND_Q1: return run<KIND_Q1>(raw, row_bytes, n_rows, n_cols, nb, n_panels, bits, scales, st);
        case KIND_Q2: return run<KIND_Q2>(raw, row_bytes, n_rows, n_cols, nb, n_panels, bits, scales, st);
        case KIND_Q8: return run<KIND_Q8>(raw, row_bytes, n_rows, n_cols, nb, n_panels, bits, scales, st);
        default: set_error("repack: kind %d has no panel layout", kind); return -7;
    }
}

}  // namespace hb200
