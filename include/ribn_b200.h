/*
 * ribn_b200 -- B200 (sm_100a) kernels for the GGUF block-quantized matmul path,
 * behind a C ABI.
 *
 * The reference engine has no C ABI: its seam is the Rust API of its CUDA crate
 * (kernel wrapper objects over a driver binding).  Each entry point below names
 * the reference interface it replaces, by file:line inside the reference
 * project, so a thin `extern "C"` block on the Rust side can swap the wrappers
 * one for one.
 *
 * Conventions kept from the reference:
 *   - the caller owns every buffer; a context owns only its stream handle;
 *   - weights are immutable device bytes in GGUF block layout, GGML dimension
 *     order [K (contiguous input), N (output rows)]      (cuda.rs:154-183,
 *     quantized.rs:138-142);
 *   - activations and outputs are batch-major [members][K] / [members][N]
 *     (quantized.rs:265-267);
 *   - a call validates, enqueues on the context's stream and returns; no
 *     allocation and no host synchronisation on the device-pointer entry
 *     points (quantized.rs:357-362);
 *   - every error is raised before anything is launched and leaves the outputs
 *     untouched (tests/q4_q8_1.rs:298-349);
 *   - a context is not thread-safe: one caller at a time (adapter.rs:16).
 *
 * All pointers named *device* must be device memory of the context's GPU,
 * 16-byte aligned.  There is no CPU fallback anywhere in this library.
 */
#ifndef RIBN_B200_H
#define RIBN_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RIBN_ABI_VERSION 1

/* Mirrors CudaQuantizedKernelError one to one (quantized.rs:90-100); TIMEOUT is
 * the status of a bounded device-side wait that ran out, INVALID_ARGUMENT covers
 * null/misaligned pointers, which the reference's typed slices cannot express. */
typedef enum ribn_status {
    RIBN_OK = 0,
    RIBN_E_DRIVER = 1,             /* Driver(String) */
    RIBN_E_INVALID_WEIGHT = 2,     /* InvalidWeight(String) */
    RIBN_E_UNSUPPORTED_TYPE = 3,   /* UnsupportedValueType { expected, actual } */
    RIBN_E_SHAPE_OVERFLOW = 4,     /* ShapeOverflow */
    RIBN_E_INPUT_LENGTH = 5,       /* InputLength { expected, actual } */
    RIBN_E_OUTPUT_LENGTH = 6,      /* OutputLength { expected, actual } */
    RIBN_E_CONTEXT_MISMATCH = 7,   /* ContextMismatch */
    RIBN_E_TIMEOUT = 8,
    RIBN_E_INVALID_ARGUMENT = 9
} ribn_status;

typedef enum ribn_dtype { RIBN_F32 = 0, RIBN_BF16 = 1 } ribn_dtype;

/* GGML value types on the path (crates/gguf/src/lib.rs:1051-1083). */
#define RIBN_TYPE_Q8_0 8u
#define RIBN_TYPE_Q4_K 12u
#define RIBN_TYPE_Q5_K 13u
#define RIBN_TYPE_Q6_K 14u

/* Largest `members` ribn_gemv accepts (the reference's cap is 8,
 * quantized.rs:12; larger batches go through ribn_gemm). */
#define RIBN_MAX_GEMV_MEMBERS 64u

/* CudaQuantizedWeight (cuda.rs:157-183): opaque encoded bytes on the device +
 * value type + WeightTensorSpec dimensions. */
typedef struct ribn_qweight {
    const void *data;        /* device pointer, GGUF-encoded blocks */
    uint64_t encoded_bytes;  /* exact length of `data` */
    uint32_t value_type;     /* GGML type id */
    uint32_t rank;           /* number of valid entries in `dimensions` */
    uint64_t dimensions[4];  /* GGML order: dimensions[0] = K, dimensions[1] = N */
} ribn_qweight;

typedef struct ribn_ctx ribn_ctx;

/* One owner per (device, stream), like the reference's kernel objects that hold
 * an Arc<CudaStream> (quantized.rs:143-160).  `cuda_stream` is a cudaStream_t /
 * CUstream (NULL = the legacy default stream).  Nothing is compiled at run time:
 * the kernels are built ahead of time for sm_100a (the reference NVRTC-compiles
 * once per process, quantized.rs:76-88, :169-182). */
int ribn_create(int device, void *cuda_stream, ribn_ctx **out);
void ribn_destroy(ribn_ctx *ctx);

/* Block until everything enqueued on the context's stream has finished and report what the kernels flagged in
 * the context's status word (then cleared): a bounded device wait that ran out (RIBN_E_TIMEOUT), or a KV-cache
 * position read from device memory that lay outside the cache (RIBN_E_INVALID_ARGUMENT; nothing was stored
 * there, the attention walk was clamped). */
int ribn_synchronize(ribn_ctx *ctx);

/* Self-test of the bounded-wait machinery, no counterpart in the reference: launches one small kernel that polls,
 * at most `polls` times (1..65536), an mbarrier at which nothing ever arrives and that no copy targets; it gives
 * up, sets the status word and returns.  The next ribn_synchronize must answer RIBN_E_TIMEOUT (and clear it).
 * Nothing is left waiting on the GPU. */
int ribn_selftest_bounded_wait(ribn_ctx *ctx, uint32_t polls);

const char *ribn_status_string(int status);
/* Message of the last failing call on `ctx`, worded like the Display impl of
 * the reference error (quantized.rs:102-137).  Valid until the next call. */
const char *ribn_last_error(const ribn_ctx *ctx);
/* UnsupportedValueType / InputLength / OutputLength carry two numbers. */
void ribn_last_error_detail(const ribn_ctx *ctx, uint64_t *expected, uint64_t *actual);

/* Tuning knobs, the counterpart of the reference's plain option structs
 * (GemvMode, decode.rs:298-307).
 *   "gemv_path":    0 = choose per shape (default), 1 = f32 CUDA-core kernel only,
 *                   2 = integer-dot kernel only (error if the shape does not fit);
 *   "mma_gemv":     1 = calls of up to eight rows per launch (and wider f32 batches, in groups of eight) use the
 *                   half2-unpack + mma.sync kernel where it serves the shape (Q4_K / Q5_K / Q6_K, 16-byte aligned
 *                   rows, at least 16 output rows); 0 = leave them to the integer-dot kernel (default 1);
 *   "mma_image_members": launches of at least this many rows convert their activations in a pre-pass launch,
 *                   narrower ones inside the GEMV kernel (1..9, default 3);
 *   "mma_stages":   ring depth of that kernel, 0 = as many stages as fit (default);
 *   "tc_min_members": smallest bf16 batch ribn_gemv sends to the tcgen05 decode kernel (default 9);
 *   "tc_four_row_bytes": where the mma kernel does not serve a shape, bf16 batches of exactly four rows use the
 *                   tcgen05 kernel when the encoded weights are at least this many bytes (default 8 MiB);
 *   "tc_f32_activations": 1 = f32 batches may use the tcgen05 kernel too (they are rounded to f16; default 0);
 *   "tc_split_operands": 1 = bf16 batches of up to 64 rows use the split-bf16-operand GEMM (the prefill
 *                   kernel) instead of the f16 decode kernel (default 0);
 *   "dp4a_prepass": 0 = calls of 1..4 rows on the integer-dot kernel pack their activations inside it, every CTA
 *                   its own copy, instead of in a launch of their own (default 1);
 *   "pdl":          programmatic dependent launch, process-wide: 0 = off, 1 = every kernel of the path, 2 = the GEMV
 *                   kernels and their pre-passes only (default);
 *   "tc_row_copies": 1 = the tcgen05 kernels fetch raw weight rows with per-row bulk copies even where one tiled
 *                   TMA box per stage would do (the path of shapes whose rows are not 16-byte aligned);
 *   "tc_ksplit":    split-K factor of the tcgen05 kernels, 0 = choose per shape;
 *   "gemv_variant": tile geometry of the f32 kernel, 0 = default, 1..3 = alternatives. */
int ribn_set_option(ribn_ctx *ctx, const char *name, int64_t value);

/* tensor_layout (crates/gguf/src/lib.rs:1051-1083): GGML type -> (elements per
 * block, bytes per block).  RIBN_E_UNSUPPORTED_TYPE for unknown ids. */
int ribn_tensor_layout(uint32_t value_type, uint64_t *block_elements, uint64_t *block_bytes);

/* validate_quantized_geometry (quantized.rs:1755-1804).  `expected_type` 0 means
 * "whatever the weight says, if it is one of the four supported types".  Pure
 * host code, no CUDA call. */
int ribn_validate_quantized_geometry(const ribn_qweight *weight, uint32_t expected_type,
                                     uint64_t *input_size, uint64_t *output_size);

/* Device twin of dequantize_block applied to every block of a tensor
 * (crates/gguf/src/lib.rs:520-547, :589-661): out[n*K + k] as f32, bit-exact
 * with the reference decoder for every finite value.  out_len = N*K. */
int ribn_dequantize(ribn_ctx *ctx, const ribn_qweight *weight, float *out_device, uint64_t out_len);

/* Cuda{Q4K,Q5K,Q6K,Q8_0}Gemv::execute / execute_warp (members = 1) and
 * execute_warp_batch (quantized.rs:1612-1650, :401-487), and
 * QwenGemvKernel::execute* (staging.rs:108-216) when expected_type = 0.
 *   y[m][n] = sum_k dequant(W[n][k]) * x[m][k],  f32 accumulation.
 * x_len / y_len are element counts and must equal members*K / members*N.
 * members = 0 -> RIBN_E_INPUT_LENGTH {expected 1, actual 0}; members >
 * RIBN_MAX_GEMV_MEMBERS -> RIBN_E_INVALID_WEIGHT (quantized.rs:458-469). */
int ribn_gemv(ribn_ctx *ctx, uint32_t expected_type, const ribn_qweight *weight,
              const void *x_device, int x_dtype, uint64_t x_len,
              void *y_device, int y_dtype, uint64_t y_len, uint32_t members);

/* The pair the reference's layer forward always issues back to back -- rms_norm
 * (or rms_norm_batch) then gemv (decode.rs:582-609, :678-696) -- as one call:
 *   y[m][n] = sum_k dequant(W[n][k]) * (x[m][k] * rsqrt(mean(x[m]^2)+eps) * norm_weight[k])
 * Same result contract as ribn_rms_norm followed by ribn_gemv.  For members <= 4
 * the normalisation runs in the GEMV kernel's prologue (no intermediate in
 * memory); larger batches normalise into the context's workspace first. */
int ribn_rms_norm_gemv(ribn_ctx *ctx, uint32_t expected_type, const ribn_qweight *weight,
                       const void *x_device, int x_dtype, uint64_t x_len,
                       const float *norm_weight_device, uint64_t norm_weight_len, float eps,
                       void *y_device, int y_dtype, uint64_t y_len, uint32_t members);

/* Prefill: Y[t][n] = sum_k dequant(W[n][k]) * X[t][k] for any number of tokens,
 * X bf16 [tokens][K], Y bf16 or f32 [tokens][N], on the tensor cores (tcgen05,
 * dequantisation fused into the operand producer).  The reference has no GEMM:
 * it serves prefill as chunks of eight tokens through execute_warp_batch
 * (decode.rs:1953-1977, :2149-2267); this call replaces that loop.  K must be a
 * multiple of 256.  ribn_gemv routes bf16 batches of five or more rows here. */
int ribn_gemm(ribn_ctx *ctx, uint32_t expected_type, const ribn_qweight *weight,
              const void *x_device_bf16, uint64_t x_len,
              void *y_device, int y_dtype, uint64_t y_len, uint64_t tokens);

/* Same operation with HOST activations and outputs: copies x to a staging
 * buffer on the device, runs the GEMV, copies y back and waits.  The staging
 * buffer must have been sized with ribn_reserve_staging first (that call is the
 * only one that allocates). */
int ribn_reserve_staging(ribn_ctx *ctx, uint64_t bytes);
int ribn_gemv_host(ribn_ctx *ctx, uint32_t expected_type, const ribn_qweight *weight,
                   const void *x_host, int x_dtype, uint64_t x_len,
                   void *y_host, int y_dtype, uint64_t y_len, uint32_t members);

/* The same without the final synchronisation: upload, GEMV and download are enqueued on the context's stream and
 * the call returns (the reference's own convention: "a call validates, then enqueues on the owner's stream and
 * returns", quantized.rs:357-362).  y_host is valid after ribn_synchronize; x_host must stay untouched until then.
 * Calls may follow one another without waiting: they share the staging buffer in stream order. */
int ribn_gemv_host_async(ribn_ctx *ctx, uint32_t expected_type, const ribn_qweight *weight,
                   const void *x_host, int x_dtype, uint64_t x_len,
                   void *y_host, int y_dtype, uint64_t y_len, uint32_t members);

/* CudaQwen35Ops::rms_norm / rms_norm_batch (model_ops.rs:1714-1824, kernels
 * :106-199): y[m][i] = x[m][i] * rsqrt(mean_i(x[m]^2) + eps) * weight[i].
 * x_len and y_len must equal members*length, weight_len must equal length. */
int ribn_rms_norm(ribn_ctx *ctx, const void *x_device, int x_dtype, uint64_t x_len,
                  const float *weight_device, uint64_t weight_len,
                  void *y_device, int y_dtype, uint64_t y_len,
                  uint32_t members, uint32_t length, float eps);

/* No counterpart in the reference (its wrappers allocate freely through their
 * driver binding).  The one entry point that allocates nothing, for callers that
 * must not: a serving loop that has given all device memory to its own pools and
 * forbids cudaMalloc after start-up, a latency-critical section that cannot take
 * the implicit synchronisation of an allocation, or a plug-in that may not touch
 * its host's allocator.  It needs no ribn_ctx (ribn_create allocates).
 *
 * Same operation and result as ribn_gemv for members <= 4.  The scratch for the
 * packed activations is a fixed device array inside the library image (about
 * 144 KiB, held by every GPU that loads the library until the process exits),
 * hence the limit: members * K (K rounded up to a multiple of 256) must not
 * exceed RIBN_NOALLOC_MAX_ACTIVATIONS, and the activations must fit the kernel's
 * shared memory; larger calls are refused with RIBN_E_SHAPE_OVERFLOW.
 *
 * The first call on a device resolves the array's device address
 * (cudaGetSymbolAddress) and should therefore be made before any stream
 * capture begins.  All calls share the array and it keeps the previous call's
 * contents; the call clears the one word that must start at zero and rewrites
 * the rest.  Calls whose kernels can overlap on the GPU (other streams, other
 * host threads) race on the array: the caller serialises them.
 *
 * wait != 0: synchronise the stream before returning and report a bounded
 * device wait that ran out as RIBN_E_TIMEOUT.  With wait == 0 nothing reads the status word in this call:
 * ribn_noalloc_status(device, stream) synchronises the stream later and reports it.  error_message (may be NULL)
 * receives the text of a failure.  Buffers that are not device memory of `device` are refused
 * (RIBN_E_CONTEXT_MISMATCH) before anything is enqueued. */
#define RIBN_NOALLOC_MAX_ACTIVATIONS 65536ull
int ribn_gemv_noalloc(int device, void *cuda_stream, const ribn_qweight *weight,
                      const void *x_device, int x_dtype, uint64_t x_len,
                      void *y_device, int y_dtype, uint64_t y_len, uint32_t members, int wait,
                      char *error_message, uint64_t error_capacity);
/* Synchronises `cuda_stream` and reports the status word the last ribn_gemv_noalloc call on `device` left:
 * RIBN_OK, RIBN_E_TIMEOUT after a bounded device wait that ran out.  Allocates nothing.  No counterpart in the reference. */
int ribn_noalloc_status(int device, void *cuda_stream);

/* ribn_gemv_fused: several projections of the same activations behind one activation pre-pass, with the
 * operators the reference launches around them folded in -- the sequences of decode.rs:929-1052:
 *   rms_norm -> q, k, v GEMVs          norm_weight given, three jobs
 *   GEMV -> residual_add               job.accumulate = 1: y += W x (model_ops.rs:600-610)
 *   silu_mul -> down GEMV              RIBN_FUSED_SWIGLU: x is [members][2K], rows [gate | up], the operand is
 *                                      silu(gate) * up (model_ops.rs:316-328)
 * All jobs share K; each is validated like ribn_gemv before anything is launched.  Served by the integer-dot
 * kernel (1..4 member rows per launch) and the tensor-core decode kernel; shapes that only the f32 kernel
 * serves are refused with RIBN_E_INVALID_ARGUMENT (use the separate calls). */
typedef struct ribn_gemv_job {
    uint32_t expected_type;      /* 0 = the weight's own type */
    const ribn_qweight* weight;
    void* y_device;              /* [members][N] */
    int y_dtype;
    uint64_t y_len;
    int accumulate;              /* 0: y = W x;  1: y += W x */
} ribn_gemv_job;
#define RIBN_MAX_FUSED_JOBS 8u
#define RIBN_FUSED_SWIGLU 1u
int ribn_gemv_fused(ribn_ctx* ctx, const ribn_gemv_job* jobs, uint32_t job_count, const void* x_device, int x_dtype,
                    uint64_t x_len, const float* norm_weight_device, uint64_t norm_weight_len, float eps, uint32_t members,
                    uint32_t flags);

/* ---- decoder-layer operators between the GEMVs -------------------------------------------
 * The launches crates/nvidia/src/decode.rs:929-1052 (full_attention_layer) and :544-632 (run_step) make
 * between its projections, for a dense-attention layer with grouped-query attention.  All buffers are
 * f32 device memory except the KV cache (f16) and token / position arrays (32-bit). */

/* ribn_embedding: CudaQ4KEmbedding::execute / execute_batch (quantized.rs:961, :1058 over
 * q4_k.cu:1-67) for any of the four block formats.  weight dims are [hidden, vocabulary]; row `token`
 * is dequantised into out[member][hidden].  A token >= vocabulary leaves its row untouched, as in the
 * reference kernel. */
int ribn_embedding(ribn_ctx* ctx, const ribn_qweight* weight, const uint32_t* tokens_device, uint32_t members,
                   float* out_device, uint64_t out_len);

/* Geometry and buffers of the attention step of one layer.  KV cache layout:
 * [members][kv_heads][max_context][head_dim] f16 (the reference keeps [token][kv_head][dim]). */
typedef struct ribn_attention {
    uint32_t members;          /* sequences decoded together, one new token each */
    uint32_t q_heads;
    uint32_t kv_heads;         /* q_heads / kv_heads in 1..8 */
    uint32_t head_dim;         /* 128 */
    uint32_t rot_dims;         /* rotary dims per head: pairs (p, p + rot_dims/2), the rest passes through */
    float rope_base;
    float eps;                 /* of the per-head RMSNorm */
    const float* q_norm;       /* [head_dim] raw weights, or NULL for no query norm */
    const float* k_norm;
    const int32_t* positions;  /* device, [members]: index of the token being appended */
    void* k_cache;
    void* v_cache;
    uint64_t max_context;      /* tokens the cache holds per (member, head) */
    uint64_t active_context;   /* upper bound of positions[m] + 1 in this call; plans the split of the KV range */
} ribn_attention;

/* strided_rms_norm (model_ops.rs:660-684) on the query and key heads, rope_neox (:393-422) on both, and
 * kv_append_f16 (:1256-1275) of the rotated keys and the values, in one launch.  q is rewritten in place. */
int ribn_qk_norm_rope_append(ribn_ctx* ctx, const ribn_attention* attention, float* q_device, const float* k_device,
                             const float* v_device);

/* attn_score_gqa (model_ops.rs:439-562) without its output gate: softmax(q.K / sqrt(head_dim)).V over tokens
 * 0..positions[m] of every member, f32 accumulation; out is [members][q_heads * head_dim].  The KV range is
 * split over CTAs and merged (partials in the context workspace). */
int ribn_attention_decode(ribn_ctx* ctx, const ribn_attention* attention, const float* q_device, float* out_device);

/* silu_mul (model_ops.rs:316-328): out[m][i] = silu(gate[m][i]) * up[m][i].  gate and up rows are
 * input_row_stride floats apart (so they can be the halves of one [members][2 * length] GEMV output). */
int ribn_silu_mul(ribn_ctx* ctx, const float* gate_device, const float* up_device, float* out_device, uint32_t members,
                  uint64_t length, uint64_t input_row_stride);

/* residual_add (model_ops.rs:600-610): y[i] += x[i]. */
int ribn_residual_add(ribn_ctx* ctx, float* y_device, const float* x_device, uint64_t length);

/* argmax / argmax_batch (model_ops.rs:201-314): index of the largest logit per member; NaN never wins,
 * ties go to the lowest index. */
int ribn_argmax(ribn_ctx* ctx, const float* logits_device, uint32_t members, uint64_t length, uint32_t* out_device);

#ifdef __cplusplus
}
#endif
#endif /* RIBN_B200_H */
