/*
 * hb200.h -- C ABI of the B200 (sm_100a) quantized matrix-product path for Hearth.
 *
 * Drop-in boundary for one path of Eric-Lautanen/hearth v0.2.0: the Q8_0
 * activation quantizer, the Q1_0 / Q2_0 / PQ2_0 / Q8_0 x Q8_0 block-dot
 * matvec / matmul, the Q4_K / Q6_K x f32 matvec, and the row dispatch around
 * them.  Every entry point names the reference interface it replaces
 * (path:line inside the reference repository).
 *
 * Conventions
 *   - Plain C types only.  Every function returns HB200_OK (0) or a negative
 *     hb200_status; hb200_last_error() gives the message of the calling
 *     thread's last failure.  Nothing throws or aborts across this boundary.
 *   - Calls are synchronous unless the name ends in _dev / _launch (those
 *     enqueue on the given CUDA stream and return).  Like the reference's
 *     ThreadPool (one shared WorkParams slot, hearth-llm/src/pool.rs:230-231)
 *     a context is not re-entrant: serialise calls per context.
 *   - Weights are uploaded once and stay resident, the residency model of
 *     hearth_compute::GpuCompute (hearth-compute/src/lib.rs:104, :239;
 *     hearth-llm/src/model/gpu.rs:8-49).  The caller keeps ownership of every
 *     host buffer; the library only reads / writes it during the call.
 *   - There is no CPU fallback: without a usable sm_100 device hb200_init
 *     fails and every other call returns HB200_ERR_NOT_INITIALIZED.
 *   - Activation layout is the reference's: f32 row-major [seq_len][n_cols];
 *     Q8_0 rows of ceil(n_cols/32) blocks [f16 d][32 x i8] at a byte stride
 *     (q8_stride); outputs token-major out[s * n_rows + row]
 *     (hearth-llm/src/pool.rs:36, :63-64, :73).
 */
#ifndef HB200_H
#define HB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define HB200_API __attribute__((visibility("default")))
#else
#define HB200_API
#endif

typedef enum hb200_status {
    HB200_OK = 0,
    HB200_ERR_NOT_INITIALIZED = -1,
    HB200_ERR_NO_DEVICE = -2,      /* no CUDA device, or not compute capability 10.x */
    HB200_ERR_BAD_DTYPE = -3,      /* GGML type id outside this path */
    HB200_ERR_BAD_SHAPE = -4,      /* size / stride / byte-count mismatch */
    HB200_ERR_NULL = -5,           /* null pointer or handle */
    HB200_ERR_CUDA = -6,           /* a CUDA runtime call failed; see hb200_last_error */
    HB200_ERR_UNSUPPORTED = -7,    /* valid request this build has no kernel for */
    HB200_ERR_TOO_LARGE = -8,      /* exceeds a stated fixed capacity */
    HB200_ERR_TIMEOUT = -9,        /* a bounded device-side wait ran out */
    HB200_ERR_IO = -10,            /* a file could not be opened or mapped */
    HB200_ERR_BAD_FORMAT = -11,    /* not a GGUF file this reader understands, or truncated */
    HB200_ERR_NOT_FOUND = -12      /* no tensor / metadata key of that name */
} hb200_status;

/* GGML type ids accepted, as the reference parses them
 * (hearth-gguf/src/ggml.rs:49-101). */
enum {
    HB200_Q8_0 = 8,
    HB200_Q4_K = 12,
    HB200_Q6_K = 14,
    HB200_Q1_0_G128_LEGACY = 39,
    HB200_Q1_0 = 41,
    HB200_Q2_0 = 42,
    HB200_Q1_0_G128 = 43,
    HB200_PQ2_0 = 142,
    HB200_PTQ1_0 = 143 /* dense base-3 ternary, 28 B per 128 (hearth-quant/src/ptq1_0.rs) */
};

typedef struct hb200_weight *hb200_weight_t; /* resident weight matrix */
typedef struct hb200_act *hb200_act_t;       /* resident activation (f32 and Q8_0 forms) */
typedef struct hb200_batch *hb200_batch_t;   /* recorded list of dot-row ops, one launch */
typedef struct hb200_gguf *hb200_gguf_t;     /* a mapped GGUF model file */

/* ---- lifecycle ---------------------------------------------------------- */

/* Replaces GpuCompute::new() (hearth-compute/src/lib.rs:127-184): binds the
 * calling process to CUDA device `device`.  Idempotent for the same device. */
HB200_API int hb200_init(int device);
/* Single-process use of several GPUs.  The reference is one process with one dispatching thread
 * (hearth-llm/src/pool.rs:398-425; LlamaModel serialises on one mutex, model/mod.rs:2781-2783), so one host thread
 * must be able to reach every GPU of the box.  hb200_init_multi binds device slots 0 .. n_devices-1 to CUDA devices
 * 0 .. n_devices-1 and enables peer access between all of them; hb200_init_slots does the same for an explicit device
 * list (a device may appear twice: two slots on one GPU emulate two shards where only one GPU is present).  Slots
 * already bound to the same devices are kept, so the calls are idempotent and may follow hb200_init(0).
 * Every weight, activation and batch belongs to the slot that was current when it was created (hb200_set_slot
 * selects it) and every call on such an object switches to its slot and device by itself; a batch takes weights and
 * activations of its own slot only.  Row-sharded matmuls over the slots: upload the row range of every weight to each
 * slot (hb200_weight_upload_rows), one batch per slot with hb200_batch_set_peers given the hb200_peer_alloc buffers of
 * all slots as they are (same process: no handle exchange), then hb200_multi_batch_launch, which launches the batches
 * one after the other from the calling thread; the kernels run concurrently on their GPUs and exchange flags. */
HB200_API int hb200_init_multi(int n_devices);
HB200_API int hb200_init_slots(const int *devices, int n_slots);
HB200_API int hb200_set_slot(int slot);
HB200_API int hb200_slot_count(void);
/* Shuts every slot down. */
HB200_API int hb200_shutdown(void);
HB200_API const char *hb200_last_error(void);
/* Number of streaming multiprocessors of the bound device (sizing of grids). */
HB200_API int hb200_sm_count(void);
/* Measures the dense int8 tensor-core rate of the device in use (a run of
 * tcgen05.mma kind::i8 with resident operands on every SM) and returns it in
 * TOP/s: the denominator for the prefill kernel's roofline fraction.  No
 * reference counterpart; takes about ten milliseconds. */
HB200_API int hb200_measure_i8_peak(double *tops);
/* 1 if this library is the bounds-checked debug build (compiled with
 * -DHB200_BOUNDS as libhearth_b200_bounds.so), 0 otherwise.  In that build the
 * streaming kernels compare every global-memory index they compute with the
 * extent the op's own dimensions give its buffer, skip an access that falls
 * outside and count it; hb200_check_status then returns HB200_ERR_CUDA with
 * the number of such accesses and the site of the first.  It stands in for
 * compute-sanitizer's memcheck where that tool is not available. */
HB200_API int hb200_bounds_checked(void);
/* Bounds-checked build only (HB200_ERR_UNSUPPORTED otherwise): runs the
 * quantizer with a block-value pitch that is too small on purpose, over buffers
 * that are large enough, and returns HB200_OK if exactly the stores beyond the
 * pitch were counted and skipped.  Nothing faults. */
HB200_API int hb200_bounds_selftest(void);

/* The split of a work list over persistent CTAs that hb200_batch_seal uses:
 * n_items items with the given costs, in order, become `grid` contiguous
 * runs whose largest total cost is as small as contiguity allows;
 * chunks[c] .. chunks[c+1]-1 are the items of CTA c (chunks has grid + 1
 * entries, trailing runs may be empty).  Needs no device.  The reference
 * splits rows evenly over its threads (hearth-llm/src/pool.rs:321-323); here
 * an item is a whole panel of rows whose cost depends on its matrix. */
HB200_API int hb200_plan_chunks(const int *cost, size_t n_items, int grid, int *chunks);

/* The work plan of a list launch of the decode matvec, exported for tests.
 * Item i is panel panel[i] of op op[i] and takes rounds[i] rounds (one round =
 * eight 128-column blocks).  With at least two of the longest items per CTA,
 * and when cuts between items would leave the largest share more than 3 %
 * above the mean, the list of all rounds is cut into `grid` equal shares, and an item that a
 * cut falls into is split between the two neighbouring CTAs: the earlier one
 * computes its first rounds and hands the running fp32 sums over, the later
 * one continues the same ordered sum (same bits as an unsplit panel).  With
 * less work the cuts fall between items.  seg_begin gets grid + 1 entries;
 * CTA c owns segments seg_begin[c] .. seg_begin[c+1]-1.  A segment is eight
 * ints {op, first panel, panel count, r0, r1, flags, carry_in, carry_out}:
 * rounds [r0, r1) of `count` consecutive panels (r0 = 0 and r1 = rounds for
 * whole panels; count = 1 for a part); flags bit 0: starts from the carry
 * slot carry_in, bit 1: ends by writing carry slot carry_out.  *n_segs
 * receives the number of segments; HB200_ERR_TOO_LARGE if seg_cap (segments
 * that fit in segs) is too small.  Needs no device.  Reference: rows are split
 * evenly over threads (hearth-llm/src/pool.rs:321-323). */
HB200_API int hb200_plan_rounds(const int *op, const int *panel, const int *rounds, size_t n_items, int grid,
                                int *seg_begin, int *segs, size_t seg_cap, size_t *n_segs);

/* ---- block geometry ----------------------------------------------------- */

/* GgmlDType::block_size / block_bytes / byte_size
 * (hearth-gguf/src/ggml.rs:105-176).  0 for a dtype outside this path. */
HB200_API size_t hb200_block_size(int dtype);
HB200_API size_t hb200_block_bytes(int dtype);
HB200_API size_t hb200_byte_size(int dtype, size_t n_cols);

/* hearth_quant::selected_kernel (hearth-quant/src/lib.rs:411-418): name of the
 * CUDA kernel variant that serves (dtype, seq_len); "none" if unsupported.
 * Q1_0 / Q2_0 family: "gemv_dp4a_*" (streaming, even passes of at most four tokens) up to 10 /
 * 11 tokens, "gemm_tcgen05_i8_rows_*" (weight rows on the MMA's M side) up to
 * 64 tokens, "gemm_tcgen05_i8_*" (tokens on the M side) above. */
HB200_API const char *hb200_selected_kernel(int dtype, size_t seq_len);

/* hearth_quant::dispatch_report / DispatchReport::banner (hearth-quant/src/lib.rs:426-473): which kernel serves
 * which token range of each weight format, for a load banner or a service endpoint.  `dtypes` lists the GGML type
 * ids a model uses; repeats collapse to the first occurrence and ids outside this path are skipped, as in the
 * reference.  hb200_dispatch_report writes JSON:
 *   {"device": "...", "sm": "10.0", "sm_count": 148, "kernels": {"q1_0": [{"tokens": "1-10", "kernel": "..."}, ...]}}
 * (keys are the lowercase format names, as DispatchReport::kernels has them); hb200_dispatch_banner writes the
 * one-liner "[kernel] Q1_0=gemv_dp4a_q1_0(1-10),...(65+) . NVIDIA B200 . sm_100 . 148 SMs".  Both write at most
 * `cap` bytes including the terminating zero and store the length needed (without the zero) in *needed (may be
 * null); a `cap` too small gives HB200_ERR_TOO_LARGE with *needed set.  Without hb200_init the device fields read
 * "none" / 0 and the table is still reported (it does not depend on the device). */
HB200_API int hb200_dispatch_report(const int *dtypes, size_t n_dtypes, char *json, size_t cap, size_t *needed);
HB200_API int hb200_dispatch_banner(const int *dtypes, size_t n_dtypes, char *text, size_t cap, size_t *needed);

/* ---- weights ------------------------------------------------------------ */

/* Replaces GpuCompute::upload_bytes (hearth-compute/src/lib.rs:239) for a
 * weight tensor: `packed` is the reference's row-major block stream,
 * n_rows * byte_size(dtype, n_cols) bytes (TensorEntry::data,
 * hearth-llm/src/model/tensor.rs:11-55).  The bytes are re-tiled once on the
 * device; the same number of bytes stays resident.  `packed` is host memory. */
HB200_API int hb200_weight_upload(int dtype, size_t n_rows, size_t n_cols, const uint8_t *packed, size_t bytes,
                                  hb200_weight_t *out);
/* Same, with `packed_dev` already in device memory (read on `stream`). */
HB200_API int hb200_weight_upload_dev(int dtype, size_t n_rows, size_t n_cols, const uint8_t *packed_dev, size_t bytes,
                                      void *stream, hb200_weight_t *out);
/* Rows [row_begin, row_end) only: the row split of pool.rs:321-323 applied
 * across GPUs instead of worker threads.  `packed` is the whole tensor. */
HB200_API int hb200_weight_upload_rows(int dtype, size_t n_rows, size_t n_cols, const uint8_t *packed, size_t bytes,
                                       size_t row_begin, size_t row_end, hb200_weight_t *out);
HB200_API int hb200_weight_free(hb200_weight_t w);
HB200_API int hb200_weight_info(hb200_weight_t w, int *dtype, size_t *n_rows, size_t *n_cols, size_t *resident_bytes);

/* ---- activations -------------------------------------------------------- */

/* A resident activation: up to max_seq_len rows of n_cols values.  At most HB200_MAX_SEQ_LEN tokens (the per-token
 * kernels index tokens with a grid dimension); more gives HB200_ERR_TOO_LARGE, from here and from every host-buffer
 * call that takes a seq_len. */
#define HB200_MAX_SEQ_LEN 65535
HB200_API int hb200_act_create(size_t max_seq_len, size_t n_cols, hb200_act_t *out);
HB200_API int hb200_act_free(hb200_act_t a);
/* Device address of the f32 [max_seq_len][n_cols] staging area of `a`. */
HB200_API int hb200_act_f32_ptr(hb200_act_t a, float **dev_ptr);
/* Device addresses of the Q8_0 planes of `a`: int8 values [seq][ld_q],
 * f32 block scales [seq][ld_b] (each an f16 value widened), f32 block sums. */
HB200_API int hb200_act_q8_planes(hb200_act_t a, int8_t **q, float **d, float **sums, size_t *ld_q, size_t *ld_b);

/* ThreadPool::par_quantize (hearth-llm/src/pool.rs:467-508) /
 * quantize_q8_0_into (hearth-quant/src/q8_0.rs:20-51) on the device: reads
 * f32 [seq_len][n_cols] at x_dev (or the act's own f32 area if x_dev is null)
 * and fills the Q8_0 planes of `a`. */
HB200_API int hb200_act_quantize_dev(hb200_act_t a, const float *x_dev, size_t seq_len, void *stream);
/* Loads caller-made Q8_0 rows (reference byte layout, device memory) into `a`. */
HB200_API int hb200_act_load_q8_0_dev(hb200_act_t a, const uint8_t *q8_dev, size_t seq_len, size_t q8_stride,
                                      void *stream);
/* Writes the Q8_0 planes of `a` back out in the reference byte layout. */
HB200_API int hb200_act_store_q8_0_dev(hb200_act_t a, uint8_t *q8_dev, size_t seq_len, size_t q8_stride, void *stream);

/* Fused producers: the f32 row is computed and quantized in one kernel, as the
 * reference does on the CPU, and lands in the Q8_0 planes of `a`.
 *
 * ops::rms_norm_q8_batch (hearth-llm/src/ops.rs:442-504): x_dev is
 * f32 [seq_len][n_cols], weight_dev f32 [n_cols]; n_cols <= 32768.  Bit-exact
 * with the reference given the eight-lane reduction order
 * ((l0+l4)+(l2+l6))+((l1+l5)+(l3+l7)) assumed for `wide`'s reduce_add. */
HB200_API int hb200_act_rms_norm_q8_dev(hb200_act_t a, const float *x_dev, const float *weight_dev, float eps,
                                        size_t seq_len, void *stream);
/* ops::silu_mul_q8 (hearth-llm/src/ops.rs:273-306) per token: gate_dev and
 * up_dev are f32 [seq_len][n_cols]; only the n_cols / 32 whole blocks are
 * produced, as in the reference.  exp is CUDA's expf, not `wide`'s polynomial:
 * equal to the reference within one quantization step, not bit for bit. */
HB200_API int hb200_act_silu_mul_q8_dev(hb200_act_t a, const float *gate_dev, const float *up_dev, size_t seq_len,
                                        void *stream);
/* hadamard_rotate then quantize_q8_0, the step in front of every folded
 * matmul (hearth-llm/src/model/qwen35.rs:49-87, :924-943): multiplies by
 * signs_dev[n_cols] (may be null), applies the normalized Walsh-Hadamard
 * transform to every whole block of block_size columns (a power of two, at
 * most 1024; 0 = no rotation) and quantizes.  x_dev null = the act's own f32
 * area.  rotated_dev (may be null) also receives the rotated f32 rows, which
 * may alias x_dev.  Bit-exact with the reference. */
HB200_API int hb200_act_hadamard_quantize_dev(hb200_act_t a, const float *x_dev, const float *signs_dev,
                                              size_t block_size, size_t seq_len, float *rotated_dev, void *stream);

/* f32-activation matmul with the arithmetic of the reference's GPU shaders:
 * GpuCompute::dequant_matmul_fused (seq_len = 1), dequant_matmul_batch
 * ([seq_len][n_cols] in, [seq_len][n_rows] out) and, with accumulate != 0,
 * dequant_matmul_fused_add_inplace (out += result)
 * (hearth-compute/src/lib.rs:483-507, :1153-1173, :1123-1151; shaders
 * q1_0_matmul.wgsl, q2_0_matmul.wgsl and their _batch / _add_inplace forms).
 * fused_gate_up / fused_qkv (lib.rs:1237, :1364) are two or three such calls
 * on one x with ld_out letting them share an output buffer.  Q1_0, Q1_0_G128
 * and Q2_0 / PQ2_0 weights only, as QuantKind has them (lib.rs:25-49); other
 * types return HB200_ERR_UNSUPPORTED, the analogue of the reference's None.
 * The activation is NOT quantized on this path, so results differ from
 * hb200_matmul_f32 (which follows the CPU path). */
HB200_API int hb200_matmul_f32act_dev(hb200_weight_t w, const float *x_dev, size_t seq_len, float *out_dev, size_t ld_out,
                                      int accumulate, void *stream);
/* The same with host buffers; with accumulate != 0 `out` is read, too. */
HB200_API int hb200_matmul_f32act(hb200_weight_t w, const float *x, size_t seq_len, float *out, int accumulate);

/* GpuCompute::argmax_f32 (hearth-compute/src/lib.rs:338-450, shader
 * hearth-compute/src/shaders/argmax.wgsl): index of the largest of n f32 values
 * in device memory, lowest index on ties, NaN never wins, 0 if no value
 * exceeds -FLT_MAX.  Synchronises `stream` and returns the index on the host,
 * as the reference's call does; four bytes cross the bus. */
HB200_API int hb200_argmax_f32_dev(const float *x_dev, size_t n, uint32_t *index_out, void *stream);
/* The same, without synchronising: the index lands in device memory.  Calls
 * on different streams must not overlap (one scratch area per context). */
HB200_API int hb200_argmax_f32_dev_async(const float *x_dev, size_t n, uint32_t *index_dev, void *stream);

/* ---- host-buffer calls (the reference's own call shapes) ---------------- */

/* quantize_q8_0_into / par_quantize with host buffers
 * (hearth-quant/src/lib.rs:381-387, hearth-llm/src/pool.rs:467).  q8_out gets
 * seq_len rows of ceil(dim/32)*34 bytes. */
HB200_API int hb200_quantize_q8_0(const float *x, size_t seq_len, size_t dim, uint8_t *q8_out);

/* ops::rms_norm_q8_batch with host buffers (hearth-llm/src/ops.rs:489-504):
 * q8_out gets seq_len rows of ceil(dim/32)*34 bytes. */
HB200_API int hb200_rms_norm_q8(const float *x, const float *weight, float eps, uint8_t *q8_out, size_t seq_len,
                                size_t dim);
/* ops::silu_mul_q8 per token with host buffers (hearth-llm/src/ops.rs:273):
 * rows of gate / up are dim floats apart, q8_out rows (dim/32)*34 bytes. */
HB200_API int hb200_silu_mul_q8(const float *gate, const float *up, uint8_t *q8_out, size_t seq_len, size_t dim);
/* hadamard_rotate + quantize_q8_0 with host buffers (qwen35.rs:924-943);
 * signs may be null; rotated_out (may be null) receives the rotated rows. */
HB200_API int hb200_hadamard_quantize_q8_0(const float *x, const float *signs, size_t block_size, uint8_t *q8_out,
                                           float *rotated_out, size_t seq_len, size_t dim);

/* ThreadPool::par_dot_rows(DotRowsParams) (pool.rs:246-257, :510-566): every
 * row of `w` against one Q8_0 activation; out[n_rows]. */
HB200_API int hb200_dot_rows(hb200_weight_t w, const uint8_t *a_q8, float *out);

/* ThreadPool::par_dot_rows_batched(BatchedDotRowsParams) (pool.rs:259-272,
 * :568-618): seq_len activations at byte stride q8_stride; out token-major
 * [seq_len][n_rows]. */
HB200_API int hb200_dot_rows_batched(hb200_weight_t w, const uint8_t *a_q8, size_t seq_len, size_t q8_stride,
                                     float *out);

/* LlamaModel::matmul / matmul_batch with x_q8 = None
 * (hearth-llm/src/model/matmul.rs:50-378, :580-674): quantizes x when the
 * weight's kernel wants Q8_0 (quantize_act :569-573), uses f32 x for
 * Q4_K / Q6_K (:270-280, :333-343).  x is [seq_len][n_cols]; out token-major. */
HB200_API int hb200_matmul_f32(hb200_weight_t w, const float *x, size_t seq_len, float *out);

/* LlamaModel::matmul_fused2 / matmul_fused_qkv (hearth-llm/src/model/matmul.rs:383-464, :469-567): several weights
 * that read the same input (q|k|v, gate|up).  x is uploaded and quantized once, every weight runs against it, and
 * outs[i] receives weight i's token-major [seq_len][n_rows_i] result.  All weights must have the same n_cols and live
 * in the same device slot; unlike the reference's fused calls any mix of formats is accepted. */
HB200_API int hb200_matmul_f32_fused(const hb200_weight_t *ws, size_t n_weights, const float *x, size_t seq_len,
                                     float *const *outs);

/* Per-(row, token, 32-block) int32 dots, out[seq_len][n_rows][n_cols/32]:
 * the `dot` / `sumi` integers of q1_0g128.rs:1033-1047, q2_0.rs:553-568,
 * q8_0.rs:164-168, exposed so the integer path can be checked bit for bit. */
HB200_API int hb200_block_dots_i32(hb200_weight_t w, const uint8_t *a_q8, size_t seq_len, size_t q8_stride,
                                   int32_t *out);

/* ---- device-buffer calls ------------------------------------------------ */

/* par_dot_rows / par_dot_rows_batched with everything resident: `a` holds
 * seq_len quantized rows, out_dev is f32 [seq_len][ld_out] with
 * ld_out >= n_rows (ld_out > n_rows lets several matrices that share an input
 * write one buffer, as matmul_fused_qkv / matmul_fused2 do,
 * hearth-llm/src/model/matmul.rs:383-567). */
HB200_API int hb200_dot_rows_dev(hb200_weight_t w, hb200_act_t a, size_t seq_len, float *out_dev, size_t ld_out,
                                 void *stream);
/* matmul / matmul_batch for f32 input resident in `a`'s f32 area. */
HB200_API int hb200_matmul_f32_dev(hb200_weight_t w, hb200_act_t a, size_t seq_len, float *out_dev, size_t ld_out,
                                   void *stream);

/* matmul for callers that cannot allocate device memory.  No counterpart in the
 * reference: it exists for hosts that have given all device memory to another
 * owner (a pre-sized KV cache, a caching allocator holding the whole card) or
 * that cannot take the device-wide synchronisation of cudaMalloc / cudaFree in
 * the middle of a decode loop.  Same result as hb200_matmul_f32_dev, but x_dev
 * is the caller's own f32 [seq_len][n_cols] device buffer and the quantized
 * activation lives in a fixed array inside the library's device image
 * (160 KiB, held by every GPU that loads the library until the process ends).
 * Limits: seq_len <= HB200_NOALLOC_MAX_TOKENS and n_cols <=
 * HB200_NOALLOC_MAX_COLS, otherwise HB200_ERR_TOO_LARGE.  The call itself
 * allocates and frees nothing.  The first call on a device resolves the
 * array's device address (cudaGetSymbolAddress); make that first call before
 * starting any stream capture.  All calls share the one array and it keeps the
 * previous call's contents: every call rewrites the part it reads, but two
 * calls whose kernels overlap on the GPU (different streams, no ordering)
 * race on it.  Serialise them.  The calling thread's current CUDA device must
 * be the one hb200_init bound (HB200_ERR_BAD_SHAPE otherwise).  Not thread-safe:
 * like every call on a context, calls from several host threads must be
 * serialised by the caller (two threads racing on the very first call of a
 * device would only resolve the same address twice). */
#define HB200_NOALLOC_MAX_TOKENS 4
#define HB200_NOALLOC_MAX_COLS 32768
HB200_API int hb200_matmul_f32_noalloc(hb200_weight_t w, const float *x_dev, size_t seq_len, float *out_dev,
                                       size_t ld_out, void *stream);

/* ---- recorded batches --------------------------------------------------- */

/* GpuCompute::begin_batch / end_batch (hearth-compute/src/lib.rs:206-224)
 * record many ops and submit them together.  Here: add independent dot-row
 * ops, seal once, then launch the whole list as one grid per launch call. */
HB200_API int hb200_batch_create(hb200_batch_t *out);
HB200_API int hb200_batch_add(hb200_batch_t b, hb200_weight_t w, hb200_act_t a, size_t seq_len, float *out_dev,
                              size_t ld_out);
HB200_API int hb200_batch_seal(hb200_batch_t b);
HB200_API int hb200_batch_launch(hb200_batch_t b, void *stream);
HB200_API int hb200_batch_free(hb200_batch_t b);
/* hb200_batch_launch of n batches (normally one per device slot), one after the other, on streams[i] (null: the
 * default stream of each device). */
HB200_API int hb200_multi_batch_launch(hb200_batch_t const *batches, int n, void *const *streams);
/* Number of kernel launches one hb200_batch_launch performs. */
HB200_API int hb200_batch_launch_count(hb200_batch_t b);
/* A whole recorded step from host memory, the shape of GpuCompute's
 * upload_f32 -> begin_batch .. end_batch -> one readback_f32
 * (hearth-compute/src/lib.rs:206-251): x_host holds, for every distinct
 * activation of the batch in order of first use, its f32 rows
 * [seq_len][n_cols] back to back (hb200_batch_input_floats() floats in all).
 * They are copied to the device in one transfer, quantized in one launch, the
 * batch runs, and out_floats floats starting at out_dev_base (the caller's
 * device buffer that the batch's ops write into) are copied to out_host.
 * Synchronous.  Ops on Q4_K / Q6_K weights read the f32 rows directly. */
HB200_API int hb200_batch_run_host(hb200_batch_t b, const float *x_host, const float *out_dev_base, size_t out_floats,
                                   float *out_host);
HB200_API size_t hb200_batch_input_floats(hb200_batch_t b);
/* The same step with the inputs already on the device: x_dev holds what x_host
 * would (same layout, hb200_batch_input_floats() floats), written on x_stream
 * (the step is ordered behind what that stream holds at the time of the call):
 * the step of a caller whose activations are produced on the device (the
 * reference's GPU path keeps them resident between ops,
 * hearth-compute/src/lib.rs:104-251).  The outputs are read back as above. */
HB200_API int hb200_batch_run_dev(hb200_batch_t b, const float *x_dev, void *x_stream, const float *out_dev_base,
                                  size_t out_floats, float *out_host);

/* ---- row-sharded multi-GPU outputs --------------------------------------- */

/* The reference has no multi-device path; its row split over worker threads
 * (hearth-llm/src/pool.rs:321-323) is applied here across GPUs, one process
 * per GPU.  Instead of gathering output slices with a collective after the
 * kernel, a sharded batch can store every output value straight into the
 * same place of every rank's output buffer over NVLink (ordinary peer stores
 * only) and close with a flag exchange.
 *
 * hb200_peer_alloc: device buffer of `bytes` for the assembled outputs plus a
 *   small control block; `handle` (64 bytes) identifies it to other processes.
 * hb200_peer_open / hb200_peer_close: map / unmap another rank's buffer.
 * hb200_batch_set_peers: before hb200_batch_seal.  data[r] is rank r's
 *   buffer as seen from this process (data[my_rank] the local one); every op
 *   of the batch must write inside data[my_rank].  One buffer serves one batch.
 *   With wait != 0 each launch returns only after all ranks' outputs have
 *   landed here (bounded wait, HB200_ERR_TIMEOUT is reported by the next
 *   synchronising call); with wait == 0 the kernel only publishes.  All ranks
 *   must launch the batch the same number of times: one launch is one epoch on
 *   every rank, whatever the number of kernels it takes there, and a rank whose
 *   row shards are all empty still takes part in the flag exchange.
 *
 * Consuming the outputs.  The flag exchange tells a rank that every writer has
 * finished; it does not tell a writer that every reader has.  With
 * area_bytes == 0 there is one output area, and no rank may launch step t + 1
 * before every rank has finished reading step t (synchronise the ranks on the
 * host).  With area_bytes > 0 every buffer holds two output areas, area_bytes
 * apart (allocate 2 * area_bytes; a multiple of 16): the ops are recorded
 * against area 0 and launch number e (counting from 1) stores into area
 * (e - 1) & 1, hb200_batch_peer_area gives the index of the area the latest
 * launch wrote, hb200_batch_run_host reads back from it.  A rank can then run
 * one launch ahead of the slowest one: with wait != 0, launch e + 2 - the next
 * to write the area of launch e - starts only after this rank's launch e + 1
 * has seen every rank finish its own launch e + 1, so each rank only has to
 * order its own reads of launch e before its own launch e + 1 (the same
 * stream, or an event), which a decode loop does anyway.  With wait == 0
 * nothing bounds how far ranks drift apart; synchronise on the host. */
#define HB200_PEER_HANDLE_BYTES 64
#define HB200_MAX_PEERS 8
HB200_API int hb200_peer_alloc(size_t bytes, void **data_dev, uint8_t handle[HB200_PEER_HANDLE_BYTES]);
HB200_API int hb200_peer_free(void *data_dev);
HB200_API int hb200_peer_open(const uint8_t handle[HB200_PEER_HANDLE_BYTES], void **data_dev);
HB200_API int hb200_peer_close(void *data_dev);
HB200_API int hb200_batch_set_peers(hb200_batch_t b, int n_ranks, int my_rank, void *const *data, size_t area_bytes,
                                    int wait);
HB200_API int hb200_batch_peer_area(hb200_batch_t b);
/* Reads and clears the device status word: HB200_OK, or HB200_ERR_TIMEOUT if a
 * bounded device-side wait expired since the last check.  Synchronises. */
HB200_API int hb200_check_status(void);

/* ---- stream helper ------------------------------------------------------ */
HB200_API int hb200_stream_synchronize(void *stream);

/* ---- GGUF reader (host only; needs no device) ---------------------------- */

/* hearth_gguf::GgufFile::open (hearth-gguf/src/gguf.rs:137-224): maps the file
 * read-only and parses header, metadata and tensor infos (GGUF version 2 or
 * 3).  Errors: HB200_ERR_IO, HB200_ERR_BAD_FORMAT (magic, version, truncation),
 * HB200_ERR_BAD_DTYPE (a tensor type id the reference's GgmlDType::from_id
 * rejects, hearth-gguf/src/ggml.rs:58-103). */
HB200_API int hb200_gguf_open(const char *path, hb200_gguf_t *out);
HB200_API int hb200_gguf_close(hb200_gguf_t g);
HB200_API uint32_t hb200_gguf_version(hb200_gguf_t g);
HB200_API uint64_t hb200_gguf_data_offset(hb200_gguf_t g);
HB200_API size_t hb200_gguf_tensor_count(hb200_gguf_t g);
/* TensorInfo (hearth-gguf/src/tensor.rs): any output may be null.  shape has
 * the innermost dimension first; bytes = byte_size of the tensor, 0 for a type
 * outside this path (F32, F16 and BF16 are sized too). */
HB200_API int hb200_gguf_tensor_info(hb200_gguf_t g, size_t index, const char **name, int *dtype_id, size_t *n_dims,
                                     uint64_t shape[8], uint64_t *offset, size_t *bytes);
/* GgufFile::find_tensor (gguf.rs:236). */
HB200_API int hb200_gguf_find_tensor(hb200_gguf_t g, const char *name, size_t *index);
/* GgufFile::tensor_data (gguf.rs:226-230): a pointer into the mapping. */
HB200_API int hb200_gguf_tensor_data(hb200_gguf_t g, size_t index, const uint8_t **data, size_t *bytes);
/* Uploads a one- or two-dimensional tensor as a resident weight: shape[0]
 * columns, shape[1] rows (TensorEntry::n_cols / n_rows,
 * hearth-llm/src/model/tensor.rs:57-71).  Needs hb200_init. */
HB200_API int hb200_gguf_upload_tensor(hb200_gguf_t g, size_t index, hb200_weight_t *out);
/* GgufFile::meta_u32 / meta_u64 / meta_bool, meta_f32, meta_str, meta_array
 * (gguf.rs:240-258).  HB200_ERR_NOT_FOUND for a missing key, HB200_ERR_BAD_DTYPE
 * for a value of another kind. */
HB200_API int hb200_gguf_meta_u64(hb200_gguf_t g, const char *key, uint64_t *out);
HB200_API int hb200_gguf_meta_f64(hb200_gguf_t g, const char *key, double *out);
HB200_API int hb200_gguf_meta_str(hb200_gguf_t g, const char *key, const char **out, size_t *len);
HB200_API int hb200_gguf_meta_array_f32(hb200_gguf_t g, const char *key, float *out, size_t capacity, size_t *count);

#ifdef __cplusplus
}
#endif
#endif /* HB200_H */
