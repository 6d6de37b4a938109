// Definitions of the opaque handles of include/hb200.h, shared by the host-layer translation units.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

struct hb200_weight {
    int slot = 0;  // device slot of the context it was uploaded in
    int dtype = 0, kind = hb200::KIND_NONE;
    size_t n_rows = 0, n_cols = 0;
    size_t row_bytes = 0;  // of the reference layout
    int nb = 0, n_panels = 0, n_sub = 0;
    uint4* bits = nullptr;   // panel layout (Q1_0 / Q2_0 / Q8_0)
    void* scales = nullptr;
    uint4* kq = nullptr;             // Q4_K / Q6_K: 32-row panels of interleaved 16-byte pieces
    unsigned short* d16 = nullptr;   // Q6_K: per-block f16 scale
    size_t resident_bytes = 0;
};

struct hb200_act {
    int slot = 0;  // device slot of the context it was created in
    size_t max_seq = 0, n_cols = 0;
    int ld_q = 0, ld_b = 0;
    float* x = nullptr;
    int8_t* q = nullptr;
    float* d = nullptr;
    float* sums = nullptr;
    alignas(64) unsigned char qmap[128] = {};  // CUtensorMap over the int8 plane (tcgen05 path), host copy
    void* qmap_dev = nullptr;                  // the same 128 bytes in device memory, where the kernel reads them
    alignas(64) unsigned char qmap32[128] = {};  // the same plane with a box of 32 rows (few-token tensor-core kernel)
    void* qmap32_dev = nullptr;
    bool has_qmap = false;
};

