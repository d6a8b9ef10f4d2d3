/* libh3q8 -- B200 (sm_100a) implementation of the int8-weight ("q8") linear
 * layers of the MiniMax-H3 DiT, as a drop-in behind h3cli's GPU operator
 * interface (greg31337/h3cli, src/gpu.h).
 *
 * Two layers, both plain C:
 *   1. h3_gpu_*   the subset of src/gpu.h that the DiT block's linear path
 *                 uses: opaque context + tensors, command scope, and the linear
 *                 operators.  Names, argument meaning, return convention
 *                 (1 = ok, 0 = failure, message via h3_gpu_error) follow the
 *                 reference; each declaration cites the line it replaces.
 *   2. h3q8_*     the raw entry points underneath: device pointers, sizes and
 *                 a CUDA stream, for callers that manage memory themselves.
 *
 * There is no CPU path: every operator runs CUDA kernels or fails with a reason.
 */
#ifndef H3Q8_H
#define H3Q8_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* =====================================================================
 * Host-side weight packing (no GPU involved)
 * ===================================================================== */
#define H3_Q8_VERSION 1 /* src/weights/q8.h:11 -- recipe id, bump when rounding/layout changes */
#define H3_Q8_GROUP 64  /* src/weights/q8.h:12 */
/* src/weights/q8.h:13-16 (src/weights/q8.c:6-56): storage is int8[N,K], zero
 * padding to 4 bytes, float[N, ceil(K/64)]. */
int h3_q8_layout(uint32_t rows, uint32_t columns, size_t *scale_offset, size_t *bytes);
int h3_q8_pack_rows(const uint16_t *source, int8_t *weights, float *scales,
                    uint32_t rows, uint32_t columns);
/* Same recipe with the group width as a parameter (0 = one group per row). */
int h3q8_q8_layout(uint32_t rows, uint32_t columns, uint32_t group, size_t *scale_offset, size_t *bytes);
int h3q8_q8_pack_rows(const uint16_t *source, int8_t *weights, float *scales,
                      uint32_t rows, uint32_t columns, uint32_t group);

/* Weight residency planning (host only) -- src/weights/residency.h:7-33.  The plan says which of
 * the (at most 50) active blocks stay resident and whether two streaming slots are needed. */
enum { H3_WEIGHTS_AUTO, H3_WEIGHTS_RESIDENT, H3_WEIGHTS_STREAM };
typedef struct {
    int mode;
    int max_resident;          /* -1 = uncapped; test-only, never increases capacity */
    uint64_t capacity_limit;   /* test-only total capacity; 0 = uncapped             */
    uint64_t allocation_limit; /* allocation fault injection, not a planner input    */
} h3_weight_options;
typedef struct {
    h3_weight_options options;
    uint64_t active_mask, resident_mask;
    uint64_t free_bytes, live_bytes, reserve_bytes, future_bytes;
    uint64_t block_bytes, resident_bytes, slot_bytes;
    unsigned active_count, resident_count;
    int effective_mode;        /* auto here means partially resident */
} h3_weight_plan;
const char *h3_weight_mode_name(int mode);
int h3_weight_options_read(h3_weight_options *out, int force_stream, char *error, size_t size);
int h3_weight_options_equal(const h3_weight_options *a, const h3_weight_options *b);
int h3_weight_plan_build(h3_weight_plan *out, h3_weight_options options, uint64_t active_mask, uint64_t block_bytes,
                         uint64_t available, uint64_t live, uint64_t future, uint64_t reserve, char *error, size_t size);
int h3_weight_retry_cap(unsigned count);
/* src/weights/residency.h:31-33 for this library's q8 packing: *scale = offset of the fp32 scale plane (16-byte
 * aligned, after the int8 [rows, columns] payload), *global = end of the scale plane (q8 has no global-scale slot),
 * *bytes = blob size rounded up to 256.  mode 1 = W8A16 with the default scale group (H3Q8_GROUP, else 64),
 * mode 2 = W8A8 with per-channel scales; 0 for anything else or a blob beyond 32-bit indexing. */
int h3_weight_packed_size(uint32_t rows, uint32_t columns, int mode, uint64_t *scale, uint64_t *global, uint64_t *bytes);

/* On-disk cache of packed q8 weights (host only), with the guarantees of src/weights/quant_cache.h:14-41 and of the
 * strict mode of src/cuda/cuda_quant.cuh:186-256.  Two kinds of key, both SHA-256:
 *   h3q8_cache_open          source path + file identity and timestamps + offset + shape + group + recipe
 *                            (no weight byte is read to open a hit);
 *   h3q8_cache_open_content  the source matrix bytes + shape + group + recipe (the same weights under any path are
 *                            the same artifact; the artifact also carries a SHA-256 of its payload, verified by every
 *                            read).  h3_gpu_quant_load takes this kind when H3_QUANT_VERIFY=1 (src/weights/quant.c:10-13).
 * Writers hold a per-artifact flock from open to close, publishing is tmp + fsync + rename, a malformed artifact is
 * an error and never a miss.  read: 1 hit, 0 absent, -1 invalid; payload buffers have h3q8_cache_payload_bytes(). */
typedef struct h3q8_cache h3q8_cache;
h3q8_cache *h3q8_cache_open(const char *directory, const char *source, uint64_t offset, uint32_t rows, uint32_t columns,
                            uint32_t group, char *error, size_t size);
h3q8_cache *h3q8_cache_open_content(const char *directory, const char *source, uint64_t offset, uint32_t rows, uint32_t columns,
                                    uint32_t group, char *error, size_t size);
void h3q8_sha256(const void *data, size_t bytes, unsigned char digest[32]);   /* FIPS 180-4, the digest of both key kinds */
int h3q8_cache_read(h3q8_cache *cache, void *payload, char *error, size_t size);
int h3q8_cache_write(h3q8_cache *cache, const void *payload, char *error, size_t size);
int h3q8_cache_unchanged(const h3q8_cache *cache, char *error, size_t size);
size_t h3q8_cache_payload_bytes(const h3q8_cache *cache);
const char *h3q8_cache_artifact(const h3q8_cache *cache);
void h3q8_cache_close(h3q8_cache *cache);

/* =====================================================================
 * Layer 2: raw entry points (device pointers, caller-owned memory)
 * ===================================================================== */
enum { H3Q8_MODE_BF16 = 0, H3Q8_MODE_W8A16 = 1, H3Q8_MODE_W8A8 = 2 };
enum { H3Q8_ACT_NONE = 0, H3Q8_ACT_GELU_TANH = 1,
       /* fc1 + SwiGLU of the real model: weight is [2*output_dim, K] = [gate rows | up rows],
        * out = bf16(silu(bf16(gate)) * up)  (src/metal/shaders.metal:2209-2317,
        * src/cuda/cuda_kernels.cuh:1047-1059); bias, if given, is [2*output_dim] */
       H3Q8_ACT_SWIGLU = 2 };
enum { /* kernel selection; AUTO picks by shape */
    H3Q8_KERNEL_AUTO = 0,
    H3Q8_KERNEL_PLAIN = 1,     /* CUDA-core kernel, any shape                       */
    H3Q8_KERNEL_TCGEN05 = 2,   /* tcgen05/TMA kernel, 128 x 256 tiles               */
    H3Q8_KERNEL_TCGEN05_M256 = 3, /* tcgen05/TMA kernel, 256 x 256 tiles            */
    H3Q8_KERNEL_TCGEN05_N128 = 4, /* tcgen05/TMA kernel, 128 x 128 tiles            */
    H3Q8_KERNEL_TCGEN05_PAIR = 5, /* two-CTA tcgen05 kernels, 256 x 256 tiles per CTA
                                     pair: BF16, W8A8 (per-channel, or scale groups of
                                     128 * n on 256 x 128 tiles), W8A16 with the
                                     dequantisation in the main loop; more than 128 rows */
    H3Q8_KERNEL_TCGEN05_SPLITK = 6, /* skinny M: 128 x 128 tiles, K split over several
                                     CTAs per tile, partial sums in `workspace`, then
                                     a finishing kernel (weight-bandwidth bound)     */
    H3Q8_KERNEL_TCGEN05_SKINNY = 7 /* at most 128 rows: the weight is the MMA's wide
                                     operand, K split over a thread-block cluster,
                                     partial sums reduced through distributed shared
                                     memory; one launch, no workspace                */
};

/* QKV epilogue (src/cuda/cuda_kernels.cuh:988-1045 with the grouped column layout of
 * src/gpu.h:652-653): weight rows / output columns are [head, q|k|v, head_dim]; q and k get
 * the per-head RMS norm (weight q_norm / k_norm) and rotary embedding on dimensions
 * [0, 2*rope_half), v is copied; all are stored as [row, head, head_dim].  Fused form:
 * head_dim 128, rope_half 48 or 64, BF16 or W8A8 per-channel operands. */
typedef struct {
    const uint16_t *q_norm, *k_norm;     /* bf16 [head_dim]            */
    const uint16_t *rope_cos, *rope_sin; /* bf16 [rows, rope_half]     */
    uint16_t *query, *key, *value;       /* bf16 [rows, heads, head_dim] */
    uint32_t heads, head_dim, rope_half;
    float epsilon;
} h3q8_rope_desc;

/* out[M,N] = epilogue(input[M,K] . weight[N,K]^T), everything row-major.
 * Replaces the body of gemm()/quant_gemm() (src/cuda/gpu_cuda.cu:927-1005,
 * src/cuda/cuda_quant.cuh:339-398) and the Metal kernels h3_linear_q8_bf16 /
 * h3_linear_int8_nax_r128 (src/metal/shaders.metal:799-857, 2417-2466), with the
 * separate bias / GELU / gate kernels (src/cuda/cuda_kernels.cuh:879-902,
 * 973-986) folded into the epilogue. */
typedef struct {
    uint32_t mode;            /* H3Q8_MODE_*                                               */
    uint32_t rows;            /* M                                                         */
    uint32_t input_dim;       /* K                                                         */
    uint32_t output_dim;      /* N                                                         */
    const void *input;        /* bf16 [M,K] (BF16, W8A16) or int8 [M,K] (W8A8)             */
    const void *weight;       /* bf16 [N,K] (BF16) or int8 [N,K]                           */
    const float *weight_scales; /* [N, ceil(K/group)] fp32; unused for BF16                */
    uint32_t weight_group;    /* K elements per weight scale; 0 = per output channel       */
    const float *input_scales;/* [M] per-token fp32 scales (W8A8)                          */
    const uint16_t *bias;     /* bf16 [N] or NULL                                          */
    const uint16_t *gate;     /* bf16 [N] or NULL (adaLN gate vector)                      */
    const uint16_t *residual; /* bf16 [M,N] or NULL                                        */
    uint32_t activation;      /* H3Q8_ACT_*                                                */
    uint16_t *output;         /* bf16 [M,N]                                                */
    int32_t *accumulators;    /* optional [M,N] dump: int32 sums (W8A8, per-channel scales)
                                 or fp32 partial sums as bit patterns (bf16 operands)      */
    uint32_t kernel;          /* H3Q8_KERNEL_*                                             */
    uint32_t input_group;     /* W8A8: K elements per activation scale, input_scales is then
                                 [M, K/input_group] (the reference's per-1024 FC2 scales,
                                 src/metal/shaders.metal:2663-2742); 0 = one scale per token   */
    const h3q8_rope_desc *rope; /* optional QKV norm + rotary epilogue; output may then be NULL
                                 (when given it also receives the plain bf16 projection)       */
    void *workspace;          /* device scratch (16-byte aligned) for H3Q8_KERNEL_TCGEN05_SPLITK: splits * rows * output_dim * 4
                                 bytes of partial sums.  AUTO does not need it: problems of at most 128 rows run on the
                                 weight-streaming kernel, which reduces on chip                                         */
    size_t workspace_bytes;
    uint32_t after_producer;  /* 1: an operand of this call (the dequantised weight, the quantised activations) is written
                                 by the kernel enqueued immediately before on the same stream.  The two-CTA kernels are
                                 then launched as a programmatic dependent: their set-up overlaps that kernel's tail and
                                 their first operand load waits for its completion.  0 = ordinary stream order. */
} h3q8_linear_desc;
/* Bytes of workspace that let a rows x output_dim x input_dim problem use every SM (0 when split-K would not help). */
size_t h3q8_linear_workspace_bytes(uint32_t mode, uint32_t rows, uint32_t input_dim, uint32_t output_dim);
int h3q8_linear(const h3q8_linear_desc *desc, void *cuda_stream);
/* Partial sums: a call with `accumulators` set and bf16 operands (BF16, or W8A16 on the one-CTA kernels) stores the raw
 * fp32 accumulators [M,N] there (as bit patterns) before any epilogue term; `output` may then be NULL.  The caller adds
 * partial sums of several K slices in fp32 (on one GPU, or with an all-reduce across GPUs: the tensor-parallel FFN) and
 * h3q8_linear_finish applies bias / GELU-tanh / gate / residual and the single bf16 rounding (no counterpart in the
 * reference, which is single-device: src/cuda/cuda_probe.c:31-40). */
int h3q8_linear_finish(const float *sums, uint32_t rows, uint32_t output_dim, const uint16_t *bias, const uint16_t *gate,
                       const uint16_t *residual, uint32_t activation, uint16_t *output, void *cuda_stream);

/* Several independent problems in one call (video + audio streams of the DiT):
 * every problem is enqueued back to back on the stream with no host sync. */
int h3q8_linear_grouped(const h3q8_linear_desc *problems, uint32_t count, void *cuda_stream);

/* W8A8 projection that allocates nothing (no counterpart in the reference).
 * For callers that may not call cudaMalloc at all -- a render loop that has
 * given all of HBM to its own pools, code running inside another library's
 * callback, a process with a fixed, audited memory budget.  desc->input is the
 * bf16 [M,K] activation matrix; it is quantised per token into a scratch array
 * that is part of the library's device image, then multiplied by the int8
 * weight with the usual fused epilogue.  Limits: rows <= H3Q8_STATIC_MAX_ROWS
 * and rows * input_dim <= H3Q8_STATIC_MAX_ACTIVATION_BYTES (larger problems are
 * refused), per-channel weight scales, input_dim % 16 == 0, output_dim % 8 == 0.
 * Every GPU that loads the library holds that array until exit.  All calls on a
 * device share it: calls that overlap on the GPU race.  The first call on a
 * device looks up the array's address and configures the kernel; make it
 * outside stream capture.  device_status is a zeroed device word of the
 * caller's that receives a code if a bounded wait inside the kernel runs out;
 * with NULL the code goes to a word inside the built-in array, which
 * h3q8_device_status() reads and clears.  desc->rope, desc->workspace and a
 * kernel selector other than AUTO are refused. */
#define H3Q8_STATIC_MAX_ACTIVATION_BYTES (16u << 20)
#define H3Q8_STATIC_MAX_ROWS 16384u
int h3q8_linear_w8a8_static(const h3q8_linear_desc *desc, uint32_t *device_status, void *cuda_stream);

/* Per-token dynamic int8 quantiser (src/metal/shaders.metal:1391-1460):
 * scale = max|x|/127 (1/127 for a zero row), q = clamp(rint(x * (127/max))).
 * Rows in [rows, dispatch_rows) are padding: zero bytes, scale 1. */
int h3q8_quantize_rows(const uint16_t *input, int8_t *output, float *scales, uint32_t rows,
                       uint32_t dispatch_rows, uint32_t columns, float clip, void *cuda_stream);
/* Per-token, per-K-group variant (src/metal/shaders.metal:1552-1598): the same recipe
 * applied to every `group` consecutive columns of a row; scales are [dispatch_rows,
 * columns/group].  columns must be a multiple of group. */
int h3q8_quantize_rows_grouped(const uint16_t *input, int8_t *output, float *scales, uint32_t rows,
                               uint32_t dispatch_rows, uint32_t columns, uint32_t group, void *cuda_stream);
/* Device version of h3q8_q8_pack_rows (bf16 [N,K] -> int8 [N,K] + scales). */
int h3q8_q8_pack_rows_device(const uint16_t *source, int8_t *weights, float *scales, uint32_t rows,
                             uint32_t columns, uint32_t group, void *cuda_stream);
/* bf16(float(q)*scale) for a whole matrix (src/metal/shaders.metal:788-794). */
int h3q8_q8_dequant(const int8_t *weights, const float *scales, uint16_t *output, uint32_t rows,
                    uint32_t columns, uint32_t group, void *cuda_stream);
/* Reads and clears the device error word of the current device (0 = ok);
 * synchronises the stream first.  Bit 31 set: h3q8_quantize_rows[_grouped] or
 * h3q8_q8_pack_rows_device met an Inf or a NaN (the reference rejects both,
 * src/weights/q8.c:38-41).  Otherwise non-zero: a bounded wait inside a kernel
 * ran out (code in the low byte, CTA index above it).  h3q8_last_error() says which. */
uint32_t h3q8_device_status(void *cuda_stream);
/* Failure-path testing, on the host side only (the reference provokes its faults with host flags and budgets too,
 * src/cuda/gpu_cuda.cu:63-66, 603-606): every wait inside the GEMM kernels is bounded, by two seconds' worth of clocks
 * unless wait_limit_cycles says otherwise, and with skip_first_load the TMA producer of the tcgen05 kernels leaves out
 * its very first operand load, so that the MMA issuer's wait runs out, every role unwinds through the kernel's normal
 * exit, and the status word carries the code.  Nothing traps, nothing spins without a limit.  (0, 0) restores normal
 * operation.  No counterpart in the reference. */
void h3q8_fault_injection(uint64_t wait_limit_cycles, uint32_t skip_first_load);
/* Message of the last failed h3q8_* call on this thread. */
const char *h3q8_last_error(void);
/* Launch counter: kernels this library has launched in this process. */
uint64_t h3q8_kernel_launches(void);

/* =====================================================================
 * Layer 1: the reference's GPU operator interface (subset)
 * ===================================================================== */
typedef struct h3_gpu h3_gpu;               /* src/gpu.h:12 */
typedef struct h3_gpu_tensor h3_gpu_tensor; /* src/gpu.h:13 */
typedef struct h3_gpu_event h3_gpu_event;   /* src/gpu.h:14 */
typedef enum { H3_GPU_F32 = 0, H3_GPU_BF16, H3_GPU_I8, H3_GPU_U32, H3_GPU_F16 } h3_gpu_dtype; /* src/gpu.h:16-22 */
typedef enum { H3_GPU_HOST_VISIBLE, H3_GPU_DEVICE_ONLY, H3_GPU_HOST_PINNED } h3_gpu_storage;   /* src/gpu.h:24-25 */
typedef enum { H3_WEIGHT_BF16 = 0, H3_WEIGHT_Q8 = 1 } h3_weight_format;                        /* src/backend.h:9 */

/* h3_gpu_stats: field for field the struct of src/gpu.h:99-142 (same order and types, so that
 * src/denoise/dit.c:3425, 3534, 3865, 3986 can keep passing their own h3_gpu_stats to
 * h3_gpu_get_stats).  This library maintains the counters of the linear / quantisation / streaming
 * path; everything that belongs to other subsystems (Metal layout, attention, convolution, weight
 * cache, sparse routing) stays 0. */
typedef struct {
    uint64_t q8_weights, q8_source_bytes, q8_storage_bytes, q8_dispatches;
    double q8_load_seconds;
    uint64_t layout_prepares, layout_inplace_packs, layout_scan_replaced_bytes, layout_partial_bytes;
    uint64_t allocated_bytes;
    uint64_t live_bytes;
    uint64_t peak_live_bytes;
    uint64_t tensor_allocations;
    uint64_t direct_dispatches;
    uint64_t mps_linear_dispatches;
    uint64_t mps_conv_dispatches;
    uint64_t mps_sdpa_dispatches;
    uint64_t native_attention_dispatches;
    uint64_t metal_current_allocated_bytes;
    uint64_t blit_copies;
    uint64_t submissions;
    double command_encode_seconds;
    double command_wait_seconds;
    double gpu_seconds;
    uint64_t linear_dispatches, conv_dispatches, attention_dispatches;
    uint64_t h2d_bytes, d2h_bytes, d2d_bytes, streamed_bytes;
    uint64_t resident_weight_bytes, stream_slot_bytes, resident_block_mask;
    unsigned resident_blocks, active_weight_blocks;
    uint64_t device_bytes, managed_bytes, pinned_bytes, peak_pinned_bytes;
    uint64_t stream_stalls;
    /* H3_PROFILE categories of src/cuda/gpu_cuda.cu:231-273, harvested at submit while profiling is on:
     * linear_seconds = CUDA-event time of the GEMM launches (0), stream_wait_seconds = slot waits (3),
     * h2d_seconds / d2h_seconds = asynchronous copies (4, 5), quant_conversion_seconds = quantise / dequantise (7) */
    double transfer_seconds, stream_wait_seconds, linear_seconds, attention_seconds;
    double conv_seconds;
    double h2d_seconds, d2h_seconds, slot_wait_seconds, normalization_seconds;
    uint64_t weight_cache_bytes, weight_cache_hits, weight_cache_hit_bytes;
    uint64_t weight_cache_misses, weight_cache_evictions;
    double quant_conversion_seconds;
    uint64_t quant_clipped_values, quant_zeroed_values;
    uint64_t quant_projection_dispatches, quant_cache_hits, quant_cache_misses;
    uint64_t sage2_attention_dispatches, sage3_attention_dispatches, attention_workspace_bytes;
    uint64_t inflight_peak, command_retirements, bounded_waits, pressure_drains;
    uint64_t native_scratch_bytes, native_scratch_allocations, native_scratch_reuses, native_pipeline_count;
    uint64_t main_dense_calls, subblock_calls, subblock_bypass, subblock_protected_calls;
    uint64_t subblock_selected, subblock_possible, subblock_router_calls;
    uint64_t attention_timing_samples, attention_timing_missed;
    double main_attention_seconds, subblock_router_seconds, subblock_kernel_seconds;
} h3_gpu_stats;
/* Counters the reference's struct has no field for (no counterpart in src/gpu.h). */
typedef struct {
    uint64_t linear_kernel_launches;      /* GEMM launches timed under H3_PROFILE category 0       */
    uint64_t conversion_kernel_launches;  /* quantise / dequantise launches timed under category 7 */
} h3q8_gpu_profile;

/* Context -- src/gpu.h:144-145, 180-182, 203, 207, 267-268 */
h3_gpu *h3_gpu_create(const char *shader_source_path, char *error, size_t error_size);
void h3_gpu_free(h3_gpu *gpu);
void h3_gpu_cancel(h3_gpu *gpu);
const char *h3_gpu_error(const h3_gpu *gpu);
/* src/gpu.h:271-272: with H3_PROFILE set, prints the report lines this path feeds (weight placement,
 * quantisation, transfers, GEMM and conversion event seconds) to stderr; silent otherwise. */
void h3_gpu_profile_set_label(h3_gpu *gpu, const char *label);
void h3_gpu_profile_mark(h3_gpu *gpu, const char *phase);
int h3_gpu_get_stats(const h3_gpu *gpu, h3_gpu_stats *stats);
int h3q8_gpu_get_profile(const h3_gpu *gpu, h3q8_gpu_profile *profile);
const char *h3_gpu_backend_name(const h3_gpu *gpu);
int h3_gpu_has_int8_mlp(const h3_gpu *gpu);
/* Command scope -- src/gpu.h:260-266 */
int h3_gpu_begin(h3_gpu *gpu);
int h3_gpu_continue(h3_gpu *gpu);
int h3_gpu_submit(h3_gpu *gpu);
int h3_gpu_synchronize(h3_gpu *gpu);
/* Tensors -- src/gpu.h:26-33, 209-258 */
h3_gpu_tensor *h3_gpu_tensor_alloc(h3_gpu *gpu, size_t elements, h3_gpu_dtype dtype, h3_gpu_storage storage);
void *h3_gpu_tensor_contents(h3_gpu_tensor *tensor);
h3_gpu_tensor *h3_gpu_tensor_new_f32(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_new_bf16(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_new_i8(h3_gpu *gpu, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_f32(h3_gpu *gpu, const float *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_bf16(h3_gpu *gpu, const uint16_t *values, size_t elements);
h3_gpu_tensor *h3_gpu_tensor_from_u32(h3_gpu *gpu, const uint32_t *values, size_t elements);
void h3_gpu_tensor_free(h3_gpu_tensor *tensor);
size_t h3_gpu_tensor_elements(const h3_gpu_tensor *tensor);
h3_gpu_dtype h3_gpu_tensor_dtype(const h3_gpu_tensor *tensor);
int h3_gpu_tensor_read_f32(const h3_gpu_tensor *tensor, float *values, size_t elements);
int h3_gpu_tensor_read_bf16(const h3_gpu_tensor *tensor, uint16_t *values, size_t elements);
int h3_gpu_tensor_read_u32(const h3_gpu_tensor *tensor, uint32_t *values, size_t elements);
int h3_gpu_tensor_write_f32(h3_gpu_tensor *tensor, const float *values, size_t elements);
int h3_gpu_tensor_write_bf16(h3_gpu_tensor *tensor, const uint16_t *values, size_t elements);
int h3_gpu_tensor_write_bf16_range(h3_gpu_tensor *tensor, size_t destination_offset,
                                   const uint16_t *values, size_t elements);
/* Byte-typed transfers for int8 tensors (no reference twin: its int8 tensors
 * are only ever produced on the device). */
int h3_gpu_tensor_read_i8(const h3_gpu_tensor *tensor, int8_t *values, size_t elements);
int h3_gpu_tensor_write_i8(h3_gpu_tensor *tensor, const int8_t *values, size_t elements);
h3_gpu_event *h3_gpu_event_new(h3_gpu *gpu);
int h3_gpu_event_record(h3_gpu *gpu, h3_gpu_event *event);
int h3_gpu_event_wait(h3_gpu *gpu, h3_gpu_event *event);
void h3_gpu_event_free(h3_gpu_event *event);
/* File I/O -- src/gpu.h:221-236.  stream_file may run on an I/O thread while
 * the owner thread enqueues compute (src/cuda/gpu_cuda.cu:761-841). */
h3_gpu_tensor *h3_gpu_tensor_load_bf16(h3_gpu *gpu, const char *path, uint64_t file_offset, size_t elements);
int h3_gpu_tensor_read_file_bf16(h3_gpu_tensor *tensor, const char *path, uint64_t file_offset,
                                 size_t elements, char *error, size_t error_size);
int h3_gpu_tensor_stream_file_bf16(h3_gpu_tensor *tensor, const char *path, uint64_t file_offset,
                                   size_t elements, char *error, size_t error_size);
/* Planning -- src/gpu.h:34-36, 48-50: 0 resident, 1 streamed, -1 insufficient. */
int h3_gpu_plan_weights(h3_gpu *gpu, uint64_t weights, uint64_t activations);
/* src/gpu.h:38-40, 205: per-block residency plan from the device's free memory (reserve = max(1 GiB,
 * 10 % of the device)); retry_cap >= 0 lowers the resident-block ceiling after an out-of-memory retry. */
int h3_gpu_plan_bf16_weights(h3_gpu *gpu, uint64_t active_mask, uint64_t block_bytes, uint64_t future_bytes,
                             int force_stream, int retry_cap, h3_weight_plan *plan);
int h3_gpu_weight_plan_compatible(h3_gpu *gpu, int force_stream);
int h3_gpu_should_retry_streaming(const h3_gpu *gpu);
int h3_gpu_release_weight_cache(h3_gpu *gpu);

/* Linear -- src/gpu.h:501-505.  A weight that carries a q8 descriptor (made by
 * h3_gpu_q8_load / h3_gpu_quant_load) is routed to the int8-weight kernels, as
 * src/cuda/gpu_cuda.cu:927-931 and src/metal/gpu.m:2672-2673 do. */
int h3_gpu_linear_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                       const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                       uint32_t rows, uint32_t input_dim, uint32_t output_dim);
/* Quantised weights -- src/gpu.h:44-47, 74-75.
 * mode: 0 off, 1 W8A16 (int8 weights, bf16 activations), 2 W8A8.  The scale
 * group width comes from H3Q8_GROUP (default 64 for q8_load, per-channel
 * otherwise) or h3q8_gpu_set_group(). */
int h3_gpu_quant_configure(h3_gpu *gpu, int mode, const char *cache, uint64_t bf16_weights,
                           uint64_t activations, int force_stream);
h3_gpu_tensor *h3_gpu_quant_load(h3_gpu *gpu, const char *path, uint64_t offset, uint32_t rows, uint32_t columns);
h3_gpu_tensor *h3_gpu_q8_load(h3_gpu *gpu, const char *path, uint64_t offset, uint32_t rows, uint32_t columns);
int h3q8_gpu_set_group(h3_gpu *gpu, uint32_t group);
/* Bridges between the two layers: the device address behind a tensor and the
 * context's compute stream (a cudaStream_t), for callers that mix h3_gpu
 * tensors with the raw h3q8_* entry points. */
void *h3q8_gpu_tensor_device_pointer(const h3_gpu_tensor *tensor);
void *h3q8_gpu_compute_stream(h3_gpu *gpu);
/* Asynchronous host <-> tensor copies on the context's two copy streams (uploads and downloads
 * have one each, so both PCIe directions run at once), ordered against the
 * compute stream by the tensor's own events (the mechanism of the reference's streamed
 * tensors, src/cuda/gpu_cuda.cu:223-251): an upload waits until compute has released the
 * tensor and marks it ready, operators wait for ready; a download waits until the last
 * operator that touched the tensor is done, and later operators wait for the download.
 * Host memory should be pinned.  h3_gpu_synchronize() waits for all three streams. */
int h3q8_gpu_tensor_upload_async(h3_gpu_tensor *tensor, const void *host, size_t bytes);
int h3q8_gpu_tensor_wait(h3_gpu_tensor *tensor); /* host waits for the tensor's last asynchronous copy only */
int h3q8_gpu_tensor_download_async(h3_gpu_tensor *tensor, void *host, size_t bytes);
/* Rows at or above which a W8A16 linear first dequantises the weight into
 * context scratch and runs the bf16 GEMM (the reference's policy 0,
 * src/metal/q8_host.inc:75-88); 0 = always dequantise in the main loop.  Without this call
 * (and without H3Q8_W8A16_SCRATCH_ROWS in the environment) the policy follows the shape:
 * main-loop dequantisation for at most 1024 rows with input_dim <= 4096, where one pass over
 * the weight costs more than the slower main loop, scratch otherwise.  Problems of at most
 * 128 rows read the int8 weight once with main-loop dequantisation and split-K under every
 * setting (H3Q8_SKINNY_DIRECT=0 turns that off). */
int h3q8_gpu_set_w8a16_scratch_rows(h3_gpu *gpu, uint32_t rows);
/* A linear cut along K, or across GPUs (the tensor-parallel FFN): h3q8_gpu_linear_partial_f32 stores the fp32 partial
 * sums [rows, output_dim] of one K slice (bf16 or W8A16 weights, no epilogue term); the caller adds the slices in fp32
 * (an NCCL all-reduce across GPUs) and h3q8_gpu_linear_finish_bf16 applies bias / GELU-tanh / gate / residual and the
 * single bf16 rounding, so that the result meets the same tolerance as the unsplit call.  No counterpart in the
 * reference (single device). */
int h3q8_gpu_linear_partial_f32(h3_gpu *gpu, h3_gpu_tensor *sums, const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                                uint32_t rows, uint32_t input_dim, uint32_t output_dim);
int h3q8_gpu_linear_finish_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *sums, const h3_gpu_tensor *bias,
                                const h3_gpu_tensor *gate, const h3_gpu_tensor *residual, uint32_t rows, uint32_t output_dim,
                                int activation);
/* Per-kernel CUDA-event timing into h3_gpu_stats (on when H3_PROFILE is set). */
int h3q8_gpu_set_profiling(h3_gpu *gpu, int enabled);
/* Same descriptor built from int8 weights + scales already in host memory. */
h3_gpu_tensor *h3q8_gpu_q8_from_host(h3_gpu *gpu, const int8_t *weights, const float *scales,
                                     uint32_t rows, uint32_t columns, uint32_t group);
/* Packed-weight streaming: a ring of device slots fed from (pinned) host memory on
 * the context's copy stream while the compute stream works on the other slot --
 * the two-slot layer streaming of src/denoise/dit.c:724-843, 2759-2820 and
 * src/cuda/gpu_cuda.cu:761-841, for already packed q8 layers (the reference's
 * quantised path copies synchronously on the compute stream instead,
 * src/cuda/cuda_quant.cuh:346-350).  Per layer:
 *   slot = prefetch(host blob)      copy stream: wait slot 'released', copy, record 'ready'
 *   acquire(slot)                   compute stream waits for 'ready' (with profiling on, waits over 20 us count as stalls)
 *   ... linears on views of the slot ...
 *   release(slot)                   compute stream records 'released'
 * A view is a q8 weight tensor that borrows slot memory (free it like any tensor;
 * the slot memory stays). */
typedef struct h3q8_weight_stream h3q8_weight_stream;
h3q8_weight_stream *h3q8_gpu_weight_stream_create(h3_gpu *gpu, size_t slot_bytes, uint32_t slots);
int h3q8_gpu_weight_stream_prefetch(h3q8_weight_stream *stream, const void *host_blob, size_t bytes);
/* Slots filled by the caller's own stream (e.g. an all-gather of per-rank slices over NVLink): reserve returns the
 * next slot and its device pointer after making producer_stream wait for the slot's release; publish marks it ready. */
int h3q8_gpu_weight_stream_reserve(h3q8_weight_stream *stream, void *producer_stream, void **device_pointer);
int h3q8_gpu_weight_stream_publish(h3q8_weight_stream *stream, int slot, void *producer_stream, size_t bytes);
int h3q8_gpu_weight_stream_acquire(h3q8_weight_stream *stream, int slot);
int h3q8_gpu_weight_stream_release(h3q8_weight_stream *stream, int slot);
h3_gpu_tensor *h3q8_gpu_weight_stream_view(h3q8_weight_stream *stream, int slot, size_t offset, uint32_t rows,
                                           uint32_t columns, uint32_t group);
void h3q8_gpu_weight_stream_free(h3q8_weight_stream *stream);
/* Size of one packed q8 weight as the views expect it (int8 payload, padding to 16
 * bytes, fp32 scales, padded to 256 bytes so that blobs can be concatenated), and
 * the offset of its scale plane. */
size_t h3q8_q8_blob_bytes(uint32_t rows, uint32_t columns, uint32_t group, size_t *scale_offset);

/* W8A8 family -- src/gpu.h:523-537 */
int h3_gpu_quantize_weight_int8(h3_gpu *gpu, h3_gpu_tensor *output, h3_gpu_tensor *scales,
                                const h3_gpu_tensor *input, uint32_t rows, uint32_t columns);
int h3_gpu_linear_int8_bf16(h3_gpu *gpu, h3_gpu_tensor *output, h3_gpu_tensor *quantized_input,
                            h3_gpu_tensor *input_scales, const h3_gpu_tensor *input,
                            const h3_gpu_tensor *weight, const h3_gpu_tensor *weight_scales,
                            uint32_t rows, uint32_t input_dim, uint32_t output_dim,
                            int use_slower_uncached_int8_scales);
/* src/gpu.h:630-642: gate*branch + residual, RMS norm, AdaLN modulation and per-row int8
 * quantisation of the result in one row pass (the producer-side fusion of the activation
 * quantiser; src/metal/shaders.metal:3390-3587).  gated_residual may alias residual. */
int h3_gpu_gate_adaln_quantize_int8(h3_gpu *gpu, h3_gpu_tensor *gated_residual, h3_gpu_tensor *quantized_output,
                                    h3_gpu_tensor *quantized_scales, const h3_gpu_tensor *residual,
                                    const h3_gpu_tensor *branch, const h3_gpu_tensor *norm_weight,
                                    const h3_gpu_tensor *gate_modulation, const h3_gpu_tensor *norm_modulation,
                                    const h3_gpu_tensor *row_map, uint32_t rows, uint32_t padded_rows, uint32_t width,
                                    uint32_t slots, uint32_t gate_slot, uint32_t shift_slot, uint32_t scale_slot,
                                    float epsilon);
/* Fused projection on activations that are already int8 (the `input_is_quantized` route of
 * h3_gpu_mlp_int8_bf16, src/gpu.h:547-563).  weight: q8 descriptor.  input_group: 0 = one
 * scale per row, else K elements per activation scale (the per-1024 FC2 recipe). */
int h3_gpu_linear_fused_int8_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *quantized_input,
                                  const h3_gpu_tensor *input_scales, uint32_t input_group, const h3_gpu_tensor *weight,
                                  const h3_gpu_tensor *bias, const h3_gpu_tensor *gate, const h3_gpu_tensor *residual,
                                  uint32_t rows, uint32_t input_dim, uint32_t output_dim, int activation);
/* The rest of the reference's int8 operator family (src/gpu.h:536-563, 682-702), same argument lists.  Weights are plain
 * int8 tensors with one fp32 scale per output channel; activations are quantised per row on the way in (or arrive
 * quantised from h3_gpu_gate_adaln_quantize_int8 with input_is_quantized = 1).  The use_slower_* switches pick
 * alternative kernels with equal results in the reference; here they are accepted and ignored. */
int h3_gpu_linear_int8_head_major_bf16(h3_gpu *gpu, h3_gpu_tensor *output, h3_gpu_tensor *quantized_input,
                                       h3_gpu_tensor *input_scales, const h3_gpu_tensor *input /* [head, row, dimension] */,
                                       const h3_gpu_tensor *weight, const h3_gpu_tensor *weight_scales, uint32_t rows,
                                       uint32_t heads, uint32_t head_dim, uint32_t output_dim);
int h3_gpu_mlp_int8_bf16(h3_gpu *gpu, h3_gpu_tensor *output, h3_gpu_tensor *activated, h3_gpu_tensor *quantized_activation,
                         h3_gpu_tensor *activation_scales, const h3_gpu_tensor *input, const h3_gpu_tensor *fc1_weight,
                         const h3_gpu_tensor *fc1_scales, const h3_gpu_tensor *fc2_weight, const h3_gpu_tensor *fc2_scales,
                         const h3_gpu_tensor *fc1_bf16, const h3_gpu_tensor *fc2_bf16, uint32_t rows, uint32_t input_dim,
                         uint32_t hidden_dim, uint32_t output_dim, int use_slower_grouped_quantizer, int use_slower_dynamic_fc1_k,
                         int use_int8_row_fc2, int input_is_quantized);
int h3_gpu_grouped_qkv_linear_rope_int8(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key, h3_gpu_tensor *value,
                                        h3_gpu_tensor *quantized_input, h3_gpu_tensor *input_scales, const h3_gpu_tensor *input,
                                        const h3_gpu_tensor *weight, const h3_gpu_tensor *weight_scales, const h3_gpu_tensor *q_norm,
                                        const h3_gpu_tensor *k_norm, const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin,
                                        uint32_t rows, uint32_t input_dim, uint32_t heads, uint32_t head_dim, uint32_t rope_half,
                                        float epsilon, int input_is_quantized, int use_slower_unfused_qkv_rope,
                                        int use_slower_scalar_qkv_rms, int use_slower_uncached_int8_scales);
/* The bf16 side of the block (src/gpu.h:506-511, 586-592, 618-629): RMS norm + AdaLN modulation producing a linear's
 * input, the same after gate * branch + residual, and the MLP with bf16 or q8-descriptor weights (fc1 + SwiGLU fused). */
int h3_gpu_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input, const h3_gpu_tensor *norm_weight,
                      const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                      uint32_t slots, uint32_t shift_slot, uint32_t scale_slot, float epsilon);
int h3_gpu_gate_adaln_bf16(h3_gpu *gpu, h3_gpu_tensor *gated_residual, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                           const h3_gpu_tensor *branch, const h3_gpu_tensor *norm_weight, const h3_gpu_tensor *gate_modulation,
                           const h3_gpu_tensor *norm_modulation, const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width,
                           uint32_t slots, uint32_t gate_slot, uint32_t shift_slot, uint32_t scale_slot, float epsilon);
int h3_gpu_mlp_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input, const h3_gpu_tensor *fc1_weight,
                    const h3_gpu_tensor *fc2_weight, uint32_t rows, uint32_t input_dim, uint32_t hidden_dim, uint32_t output_dim);
/* Unfused epilogue operators kept for comparison -- src/gpu.h:575-577, 612-617, 750-752 */
int h3_gpu_gelu_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input, uint32_t elements, int approximate);
int h3_gpu_gate_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *residual,
                     const h3_gpu_tensor *branch, const h3_gpu_tensor *modulation,
                     const h3_gpu_tensor *row_map, uint32_t rows, uint32_t width, uint32_t slots, uint32_t gate_slot);
/* src/gpu.h:652-664 and 665-683: norm + RoPE on a stored grouped QKV tensor, and the projection
 * fused with it (one kernel when head_dim is 128 and rope_half 48 or 64; qkv may be NULL then,
 * otherwise the projection is stored there first and the separate kernel follows). */
int h3_gpu_grouped_qkv_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key, h3_gpu_tensor *value,
                                 const h3_gpu_tensor *qkv, const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                                 const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin, uint32_t sequence,
                                 uint32_t heads, uint32_t head_dim, uint32_t rope_half, float epsilon);
int h3_gpu_grouped_qkv_linear_rope_bf16(h3_gpu *gpu, h3_gpu_tensor *query, h3_gpu_tensor *key, h3_gpu_tensor *value,
                                        h3_gpu_tensor *qkv, const h3_gpu_tensor *input, const h3_gpu_tensor *weight,
                                        const h3_gpu_tensor *q_norm, const h3_gpu_tensor *k_norm,
                                        const h3_gpu_tensor *rope_cos, const h3_gpu_tensor *rope_sin, uint32_t rows,
                                        uint32_t input_dim, uint32_t heads, uint32_t head_dim, uint32_t rope_half,
                                        float epsilon);
int h3_gpu_swiglu_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *fused, uint32_t rows, uint32_t width); /* src/gpu.h:714-716 */
int h3_gpu_add_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *left,
                    const h3_gpu_tensor *right, uint32_t elements);

/* The fused projection: linear + bias + GELU-tanh | gate*branch + residual in
 * one kernel.  No counterpart in src/gpu.h; modelled on its fused wrappers
 * (h3_gpu_adaln_linear_bf16 :600-611, h3_gpu_gate_adaln_bf16 :618-629).
 * weight may be bf16 or carry a q8 descriptor; with W8A8 configured the
 * activations are quantised per token into context-owned scratch first.
 * bias, gate, residual may be NULL.  activation: H3Q8_ACT_*; with H3Q8_ACT_SWIGLU the weight (and bias)
 * have 2 * output_dim rows, gate rows first (the fc1 of src/denoise/dit.c:2489-2491 in one call). */
int h3_gpu_linear_fused_bf16(h3_gpu *gpu, h3_gpu_tensor *output, const h3_gpu_tensor *input,
                             const h3_gpu_tensor *weight, const h3_gpu_tensor *bias,
                             const h3_gpu_tensor *gate, const h3_gpu_tensor *residual,
                             uint32_t rows, uint32_t input_dim, uint32_t output_dim, int activation);
typedef struct {
    h3_gpu_tensor *output;
    const h3_gpu_tensor *input, *weight, *bias, *gate, *residual;
    uint32_t rows, input_dim, output_dim;
    int activation;
} h3_gpu_linear_problem;
int h3_gpu_linear_grouped_bf16(h3_gpu *gpu, const h3_gpu_linear_problem *problems, uint32_t count);

/* ---------------------------------------------------------------------
 * The linear dispatch of one DiT block (src/denoise/dit.c:2286-2537 and the flags of :1956-1990), as C above the
 * operators: which family runs each projection, and the "input already quantised" state handed from the tail of one
 * block to the QKV projection of the next.  Attention sits between the two calls and stays with the caller.
 * --------------------------------------------------------------------- */
/* src/weights/quant.c:22-40: `requested` for the four projection matrices of a block, 0 for anything else; with the
 * adaptive cache block 0 stays unquantised. */
int h3_quant_projection(const char *name, int requested);
int h3_quant_projection_policy(const char *name, int requested, int adaptive_cache);
typedef struct {
    int int8_qkv, int8_attention_out, int8_mlp;  /* run that projection on the W8A8 operator family                    */
    int head_major_attention_out;                /* the attention output arrives as [head, row, dimension]             */
    int fuse_int8_mlp_input, fuse_int8_qkv_input;/* gate + AdaLN + quantise in one pass in front of that projection    */
    int int8_row_fc2;                            /* per-row instead of per-1024 re-quantisation in front of fc2        */
} h3q8_dit_linear_policy;
typedef struct { uint32_t rows, hidden, heads, head_dim, rope_half, ffn, slots; float epsilon; } h3q8_dit_shape;
typedef struct {
    const h3_gpu_tensor *qkv, *out, *fc1, *fc2;              /* bf16 tensors or quantised descriptors (may be NULL when   */
    const h3_gpu_tensor *qkv_int8, *qkv_scales;              /* the int8 pair of the projection is given, and vice versa) */
    const h3_gpu_tensor *out_int8, *out_scales;
    const h3_gpu_tensor *fc1_int8, *fc1_scales, *fc2_int8, *fc2_scales;
    const h3_gpu_tensor *q_norm, *k_norm, *norm1, *norm2;
} h3q8_dit_block_weights;
typedef struct {                                              /* the block loop's activations, owned by the caller         */
    h3_gpu_tensor *hidden, *mod_attention, *qkv, *query, *key, *value;
    h3_gpu_tensor *attention_heads, *attention_output, *mod_mlp, *mlp_output, *activated;
    h3_gpu_tensor *int8_activation, *int8_activation_scales;
} h3q8_dit_block_buffers;
/* Flags as src/denoise/dit.c:1956-1990 resolves them: the backend's int8 operators, resident (not streamed) weights,
 * rows >= 128 for the attention-side projections, and the H3_DISABLE_* environment switches dit.c reads. */
int h3q8_dit_linear_policy_resolve(const h3_gpu *gpu, uint32_t rows, int streaming, h3q8_dit_linear_policy *policy);
/* (attention AdaLN unless the previous tail did it) -> QKV projection + per-head norm + RoPE into query / key / value. */
int h3q8_dit_block_attention_input(h3_gpu *gpu, const h3q8_dit_linear_policy *policy, const h3q8_dit_shape *shape,
                                   const h3q8_dit_block_weights *weights, const h3q8_dit_block_buffers *buffers,
                                   const h3_gpu_tensor *modulation, const h3_gpu_tensor *row_map, const h3_gpu_tensor *rope_cos,
                                   const h3_gpu_tensor *rope_sin, int attention_adaln_ready, int attention_input_quantized);
/* attention output projection -> gate + MLP AdaLN (+ quantise) -> MLP -> MLP gate, fused with the next block's
 * attention AdaLN (+ quantise) when fuse_next_attention; the two out-flags are the next call's in-flags. */
int h3q8_dit_block_after_attention(h3_gpu *gpu, const h3q8_dit_linear_policy *policy, const h3q8_dit_shape *shape,
                                   const h3q8_dit_block_weights *weights, const h3_gpu_tensor *next_norm1,
                                   const h3q8_dit_block_buffers *buffers, const h3_gpu_tensor *modulation,
                                   const h3_gpu_tensor *next_modulation, const h3_gpu_tensor *row_map, int fuse_next_attention,
                                   int *next_attention_adaln_ready, int *next_attention_input_quantized);

#ifdef __cplusplus
}
#endif
#endif
