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
 *                   mma.sync kernels where they serve the shape (Q4_K / Q5_K / Q6_K, 16-byte aligned rows, at least
 *                   16 output rows); 0 = leave them to the integer-dot kernel (default 1);
 *   "imma_gemv":    1 = those calls run on the integer instruction (quants as 8-bit operands, activations as
 *                   22-bit integers per 256-value slice); 0 = on the half2-unpack f16 kernel (default 1);
 *                   "imma_max_members": largest such call (1..8, default 8);
 *   "mma_image_members": launches of at least this many rows convert their activations in a pre-pass launch,
 *                   narrower ones inside the GEMV kernel unless K exceeds 24 super-blocks or the input is gated
 *                   (1..9, default 3);
 *   "mma_stages":   ring depth of that kernel, 0 = as many stages as fit (default);
 *   "tc_min_members": smallest bf16 batch ribn_gemv sends to a tcgen05 batch kernel (default 9);
 *   "tmem_gemv":    1 = those batches (Q4_K / Q5_K / Q6_K, up to 64 rows) run on the kernel that unpacks the weights into
 *                   tensor memory (default); 0 = on the f16-tile kernel, which also serves Q8_0;
 *   "tc_four_row_bytes": where the mma kernel does not serve a shape, bf16 batches of exactly four rows use the
 *                   tcgen05 kernel when the encoded weights are at least this many bytes (default 8 MiB);
 *   "tc_f32_activations": 1 = f32 batches may use the tcgen05 kernel too (they are rounded to f16; default 0);
 *   "tc_split_operands": 1 = bf16 batches of up to 64 rows use the prefill GEMM kernel (accumulation over the whole
 *                   K range in tensor memory) instead of the f16 decode kernel (default 0; the name is from when that
 *                   kernel split every weight into two bf16 operands);
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

/* The same without the final synchronisation: the upload runs on a copy stream of the context, the GEMV on the context's
 * stream, the download on a second copy stream, chained by events over four staging slots -- the copies of one call
 * overlap the GEMVs of its neighbours -- and the call returns (the reference's own convention: "a call validates, then
 * enqueues on the owner's stream and returns", quantized.rs:357-362).  y_host is valid after ribn_synchronize; x_host
 * must stay untouched until then.  Calls may follow one another without waiting. */
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
 *   q and k (any two projections of one format) stored as one matrix: one launch, two outputs (split_rows)
 * All jobs share K; each is validated like ribn_gemv before anything is launched.  Served by the kernels ribn_gemv
 * uses (the integer tensor-core kernel for up to eight rows, the batch kernel from nine, the integer-dot kernel for
 * Q8_0); shapes that only the f32 kernel serves are refused with RIBN_E_INVALID_ARGUMENT (use the separate calls). */
typedef struct ribn_gemv_job {
    uint32_t expected_type;      /* 0 = the weight's own type */
    const ribn_qweight* weight;
    void* y_device;              /* [members][N] */
    int y_dtype;
    uint64_t y_len;
    int accumulate;              /* 0: y = W x;  1: y += W x */
    uint64_t split_rows;         /* 0, or a multiple of 128 below N: the weight holds two projections, one after the other */
    void* y2_device;             /* split_rows != 0: rows [0, split_rows) go to y_device as [members][split_rows], rows
                                  * [split_rows, N) to y2_device as [members][N - split_rows]; y_len stays members * N */
} ribn_gemv_job;
#define RIBN_MAX_FUSED_JOBS 8u
#define RIBN_FUSED_SWIGLU 1u
int ribn_gemv_fused(ribn_ctx* ctx, const ribn_gemv_job* jobs, uint32_t job_count, const void* x_device, int x_dtype,
                    uint64_t x_len, const float* norm_weight_device, uint64_t norm_weight_len, float eps, uint32_t members,
                    uint32_t flags);

/* ---- GGUF v3 files: directory reader and staged upload ------------------------------------------
 * GgufFile::open / read_from, tensor_data_range, TensorDataReader (crates/gguf/src/lib.rs:191-280, :324-343,
 * :400-505) and CudaWeightStore::materialize_quantized (crates/nvidia/src/cuda.rs:321-387).  Opening parses the
 * header, the metadata and the tensor directory with the reference's bounds (strings <= 16 MiB, arrays <= 10^6
 * items and 16 levels, <= 16 dimensions, <= 10^7 tensors) and never reads tensor data.  The functions return RIBN_OK,
 * a ribn_status, or one of the codes below, which name the reference's GgufError variants. */
typedef struct ribn_gguf ribn_gguf;

typedef enum ribn_gguf_status {
    RIBN_GGUF_E_IO = 100,
    RIBN_GGUF_E_INVALID_MAGIC = 101,
    RIBN_GGUF_E_UNSUPPORTED_VERSION = 102,
    RIBN_GGUF_E_UNEXPECTED_EOF = 103,
    RIBN_GGUF_E_INVALID_UTF8 = 104,
    RIBN_GGUF_E_INVALID_VALUE_TYPE = 105,
    RIBN_GGUF_E_INVALID_BOOL = 106,
    RIBN_GGUF_E_INVALID_LENGTH = 107,
    RIBN_GGUF_E_ARRAY_NESTING_TOO_DEEP = 108,
    RIBN_GGUF_E_DUPLICATE_METADATA = 109,
    RIBN_GGUF_E_INVALID_DIMENSION_COUNT = 110,
    RIBN_GGUF_E_INVALID_ALIGNMENT = 111,
    RIBN_GGUF_E_TRUNCATED = 112,
    RIBN_GGUF_E_TENSOR_OFFSET_OUT_OF_BOUNDS = 113,
    RIBN_GGUF_E_MISSING_METADATA = 114,
    RIBN_GGUF_E_METADATA_TYPE_MISMATCH = 115,
    RIBN_GGUF_E_MISSING_TENSOR = 116,
    RIBN_GGUF_E_UNSUPPORTED_TENSOR_TYPE = 117,
    RIBN_GGUF_E_ELEMENT_COUNT_OVERFLOW = 118,
    RIBN_GGUF_E_TENSOR_BYTE_LENGTH_OVERFLOW = 119,
    RIBN_GGUF_E_QUANTIZATION_BLOCK_MISMATCH = 120,
    RIBN_GGUF_E_QUANTIZATION_DIMENSION_MISMATCH = 121
} ribn_gguf_status;

#define RIBN_GGUF_MAX_DIMS 16u
#define RIBN_GGUF_SCALAR UINT64_MAX /* `index` of the metadata getters: the value itself, not an array element */

typedef struct ribn_gguf_tensor {
    const char* name;          /* owned by the file object */
    uint32_t value_type;       /* raw GGML type id; unknown ids are kept (lib.rs:103-108) */
    uint32_t n_dims;
    uint64_t dims[RIBN_GGUF_MAX_DIMS];
    uint64_t offset;           /* relative to the aligned tensor-data section */
} ribn_gguf_tensor;

int ribn_gguf_open(const char* path, ribn_gguf** out);
void ribn_gguf_close(ribn_gguf* file);
/* Message of the last failed call on `file`; with NULL, of the last failed ribn_gguf_open on this thread. */
const char* ribn_gguf_last_error(const ribn_gguf* file);
uint32_t ribn_gguf_version(const ribn_gguf* file);
uint64_t ribn_gguf_tensor_count(const ribn_gguf* file);
uint64_t ribn_gguf_metadata_count(const ribn_gguf* file);
uint64_t ribn_gguf_tensor_data_offset(const ribn_gguf* file);
const char* ribn_gguf_metadata_key(const ribn_gguf* file, uint64_t index);   /* keys in sorted order */
/* GGUF value type (0..12) of a key; for arrays (9) also the element type and the item count. */
int ribn_gguf_metadata_type(ribn_gguf* file, const char* key, uint32_t* type, uint32_t* element_type, uint64_t* count);
/* Typed getters with the reference's widening rules (MetadataValue::as_u64 / as_i32 / as_str / as_bool, lib.rs:49-85):
 * u64 takes the unsigned integer types, i64 the signed ones, f64 both float types.  `index` selects an array element,
 * RIBN_GGUF_SCALAR the value itself.  A missing key is RIBN_GGUF_E_MISSING_METADATA, any other miss
 * RIBN_GGUF_E_METADATA_TYPE_MISMATCH. */
int ribn_gguf_metadata_u64(ribn_gguf* file, const char* key, uint64_t index, uint64_t* out);
int ribn_gguf_metadata_i64(ribn_gguf* file, const char* key, uint64_t index, int64_t* out);
int ribn_gguf_metadata_f64(ribn_gguf* file, const char* key, uint64_t index, double* out);
int ribn_gguf_metadata_bool(ribn_gguf* file, const char* key, uint64_t index, int* out);
int ribn_gguf_metadata_string(ribn_gguf* file, const char* key, uint64_t index, const char** data, uint64_t* length);
int ribn_gguf_tensor_info(ribn_gguf* file, uint64_t index, ribn_gguf_tensor* out);
int ribn_gguf_find_tensor(ribn_gguf* file, const char* name, uint64_t* index);
/* Absolute byte range [begin, end) of a tensor's encoding; checks the block layout and the file bounds. */
int ribn_gguf_tensor_data_range(ribn_gguf* file, const char* name, uint64_t* begin, uint64_t* end);
/* Bounded read of a tensor's encoding from byte `offset` of it: never past the tensor's end (*read_out may be short or
 * zero there).  The file is opened for the call and closed before it returns, so no descriptor is held between reads. */
int ribn_gguf_read_tensor(ribn_gguf* file, const char* name, uint64_t offset, void* host_dst, uint64_t bytes, uint64_t* read_out);

/* Shards of a [K, N] tensor for tensor-parallel loading (the reference has one GPU and no shards). */
#define RIBN_SHARD_NONE 0   /* the whole tensor */
#define RIBN_SHARD_ROWS 1   /* output rows [begin, end): one contiguous byte range */
#define RIBN_SHARD_INPUT 2  /* super-blocks of 256 inputs [begin, end) of every row, packed row after row */
int ribn_gguf_shard_bytes(ribn_gguf* file, const char* name, int axis, uint64_t begin, uint64_t end, uint64_t* bytes,
                          uint64_t* k_out, uint64_t* n_out);
/* Copies a tensor's encoding (or a shard of it) from the file to device memory on the context's stream, through two
 * pinned buffers of 8 MiB: the file read of one piece overlaps the copy of the previous one.  dst_bytes must equal the
 * encoding's size (RIBN_E_OUTPUT_LENGTH); an empty encoding is RIBN_E_INVALID_WEIGHT; a file that ends early is
 * RIBN_GGUF_E_UNEXPECTED_EOF (SourceIncomplete in the reference).  On return every piece has left the host buffers;
 * the device copy completes in stream order.  Errors are read with ribn_gguf_last_error(file). */
int ribn_materialize_quantized(ribn_ctx* ctx, ribn_gguf* file, const char* name, int axis, uint64_t begin, uint64_t end,
                               void* device_dst, uint64_t dst_bytes);
/* The device and the stream a context was created on. */
int ribn_context_stream(const ribn_ctx* ctx, int* device, void** cuda_stream);

/* ---- tensor-parallel exchange over peer memory --------------------------------------------------
 * The reference runs on one GPU.  With the weights sharded over `world` GPUs of one node (output rows of q/k/v, gate/up
 * and the output head; input columns of o_proj and ffn_down), two steps of a decode layer need the other ranks:
 * the sum of the column-split projections' partial outputs, and the choice of the next token from per-rank slices of
 * the logits.  Both run as one kernel per rank over memory the peers map: no collective library is called.
 *
 * Every rank creates a link (a block of device memory: two partial slots of slot_bytes plus 4 KiB of flags), hands its
 * 64-byte handle to the peers over any host channel, and connects.  ribn_tp_partial(slot) is where this rank's GEMV
 * writes its partial [members][length] (f32 or bf16); consecutive exchanges must alternate slots 0 and 1.  Waits on
 * peers are bounded (ribn_tp_set_wait, default 1 s): a peer that never arrives makes ribn_synchronize return
 * RIBN_E_TIMEOUT; the GPU is not left waiting.
 *
 * Block layout (part of the contract between ranks; all words little-endian u32): [slot 0][slot 1] then, at byte
 * 2 * slot_bytes: flags[16] (flags[p] = number of the last exchange rank p has published here), select_flags[16] (the
 * same for token selection), pairs[2][64][2] (this rank's best (ordered key of the value, token) per member, generation
 * = exchange number & 1), then words private to the rank. */
typedef struct ribn_tp ribn_tp;
#define RIBN_TP_HANDLE_BYTES 64
/* local_block NULL: the link allocates its block (exportable).  Otherwise the caller's memory of
 * ribn_tp_block_bytes(slot_bytes), 256-byte aligned, zeroed by this call; such links connect by pointers. */
int ribn_tp_create(ribn_ctx* ctx, uint32_t rank, uint32_t world, uint64_t slot_bytes, void* local_block, ribn_tp** out);
void ribn_tp_destroy(ribn_tp* tp);
const char* ribn_tp_last_error(const ribn_tp* tp);
uint64_t ribn_tp_block_bytes(uint64_t slot_bytes);
int ribn_tp_export(ribn_tp* tp, void* handle_out /* RIBN_TP_HANDLE_BYTES */);
int ribn_tp_connect(ribn_tp* tp, const void* handles /* [world][RIBN_TP_HANDLE_BYTES], own entry ignored */);
/* Peers in the same process (peer access enabled by the caller): their blocks' device pointers, own entry ignored. */
int ribn_tp_connect_pointers(ribn_tp* tp, void* const* blocks);
int ribn_tp_set_wait(ribn_tp* tp, uint64_t microseconds);
int ribn_tp_partial(ribn_tp* tp, uint32_t slot, void** device_pointer);
/* hidden[m][i] += sum over ranks, in rank order, of their partials in `slot`; every rank ends with identical bits.
 * Replaces the all-reduce and the residual_add (model_ops.rs:600-610) behind o_proj and ffn_down. */
int ribn_tp_allreduce_residual(ribn_ctx* ctx, ribn_tp* tp, uint32_t slot, float* hidden_device, uint32_t members, uint64_t length,
                               int partial_dtype);
/* argmax / argmax_batch (model_ops.rs:201-314) over a vocabulary split by rows across the ranks: logits_device is this
 * rank's [members][length] slice, whose first column is token index_base.  NaN never wins, ties go to the lowest token. */
int ribn_tp_select_tokens(ribn_ctx* ctx, ribn_tp* tp, const float* logits_device, uint32_t members, uint64_t length,
                          uint32_t index_base, uint32_t* tokens_device);

/* ---- the reference's Q8_1 activation format (compatibility mode) ------------------------------
 * CudaQ8_1Quantizer::execute (crates/nvidia/src/activation.rs:15-88 over activation.cu:3-28): every block of 32
 * floats becomes nine words -- half(max|x|/127) | half(sum x) << 16, then 32 signed bytes round(x / scale).  The
 * output is bit-identical to the reference kernel's (same division, roundf, shuffle tree and cvt.rn).  A batch is one
 * linear stream of blocks.  x_len empty or not a multiple of 32 -> RIBN_E_INPUT_LENGTH; packed_len != x_len/32*9 ->
 * RIBN_E_OUTPUT_LENGTH; more than 2^32-1 values -> RIBN_E_SHAPE_OVERFLOW. */
int ribn_quantize_q8_1(ribn_ctx* ctx, const float* x_device, uint64_t x_len, uint32_t* packed_device, uint64_t packed_len);

/* CudaQ4KQ8_1Gemv::execute / execute_batch and the Q5_K, Q6_K, Q8_0 twins (crates/nvidia/src/q4_q8_1.rs,
 * kernels/quantized/q4_k_q8_1.cu:40-144, q5_k_q8_1.cu, q6_k_q8_1.cu, q8_0_q8_1.cu; CudaIntDotProjector,
 * decode.rs:1341-1478): y[m][n] from Q8_1-packed activations [members][K/32*9] words by exact integer dots, the
 * reference's lossy arithmetic.  members 1..8; 0 -> RIBN_E_INPUT_LENGTH, 9+ -> RIBN_E_INVALID_WEIGHT, both before
 * geometry.  ribn_gemv is the accurate path; this one serves hosts that hold Q8_1 activations already. */
int ribn_gemv_q8_1(ribn_ctx* ctx, uint32_t expected_type, const ribn_qweight* weight, const uint32_t* packed_device,
                   uint64_t packed_len, float* y_device, uint64_t y_len, uint32_t members);

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
    uint32_t shared_cache;     /* 0: member m owns cache slot m.  1: the members are consecutive tokens of ONE sequence (the
                                * prefill chunk of decode.rs:2149-2267, whose attention loop :2945-3021 walks one cache): every
                                * member appends to and reads slot 0 of k_cache / v_cache, causally through positions[m] */
    uint32_t out_dtype;        /* RIBN_F32 or RIBN_BF16: element type of ribn_attention_decode's output */
} ribn_attention;

/* strided_rms_norm (model_ops.rs:660-684) on the query and key heads, rope_neox (:393-422) on both, and
 * kv_append_f16 (:1256-1275) of the rotated keys and the values, in one launch.  q is rewritten in place. */
int ribn_qk_norm_rope_append(ribn_ctx* ctx, const ribn_attention* attention, float* q_device, const float* k_device,
                             const float* v_device);

/* attn_score_gqa (model_ops.rs:439-562) without its output gate: softmax(q.K / sqrt(head_dim)).V over tokens
 * 0..positions[m] of every member, f32 accumulation; out is [members][q_heads * head_dim].  The KV range is
 * split over CTAs and merged (partials in the context workspace). */
int ribn_attention_decode(ribn_ctx* ctx, const ribn_attention* attention, const float* q_device, void* out_device);

/* silu_mul (model_ops.rs:316-328): out[m][i] = silu(gate[m][i]) * up[m][i].  gate and up rows are
 * input_row_stride floats apart (so they can be the halves of one [members][2 * length] GEMV output). */
int ribn_silu_mul(ribn_ctx* ctx, const float* gate_device, const float* up_device, float* out_device, uint32_t members,
                  uint64_t length, uint64_t input_row_stride);
/* The same with a typed output (RIBN_F32 or RIBN_BF16): bf16 feeds ribn_gemm in a prefill chunk. */
int ribn_silu_mul_typed(ribn_ctx* ctx, const float* gate_device, const float* up_device, void* out_device, int out_dtype,
                        uint32_t members, uint64_t length, uint64_t input_row_stride);

/* residual_add (model_ops.rs:600-610): y[i] += x[i]. */
int ribn_residual_add(ribn_ctx* ctx, float* y_device, const float* x_device, uint64_t length);

/* argmax / argmax_batch (model_ops.rs:201-314): index of the largest logit per member; NaN never wins,
 * ties go to the lowest index. */
int ribn_argmax(ribn_ctx* ctx, const float* logits_device, uint32_t members, uint64_t length, uint32_t* out_device);

#ifdef __cplusplus
}
#endif
#endif /* RIBN_B200_H */
