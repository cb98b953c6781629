/*
 * CPU oracle for the GGUF quantized-matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference engine's host-side
 * algorithms for the path.  It exists to check the CUDA kernels and to be the
 * timed CPU baseline; nothing in the shipped library links or calls it.  Only
 * the test-suite, the smoke check and the benchmark's cpu-baseline leg may
 * load it.
 *
 * Reference functions followed (paths are relative to the reference project):
 *   tensor_layout          crates/gguf/src/lib.rs:1051-1083
 *   f16_to_f32 / read_f16  crates/gguf/src/lib.rs:551-567
 *   q4_k_scales            crates/gguf/src/lib.rs:573-587
 *   dequantize_q8_0        crates/gguf/src/lib.rs:589-594
 *   dequantize_q4_k        crates/gguf/src/lib.rs:596-612
 *   dequantize_q5_k        crates/gguf/src/lib.rs:614-633
 *   dequantize_q6_k        crates/gguf/src/lib.rs:635-661
 *   dequantize_block       crates/gguf/src/lib.rs:520-547
 *   gguf_gemv              crates/nvidia/src/qwen_reference.rs:31-40
 *   rms_norm_raw           crates/nvidia/src/qwen_reference.rs:550-556
 *   host_ffn_step (SiLU)   crates/nvidia/src/qwen_reference.rs:523-539
 *
 * Parity pin: the known-answer vectors of the reference's own unit tests
 * (crates/gguf/src/lib.rs:1369-1472) and the structured fixtures of
 * crates/nvidia/tests/q{4,5,6}_q8_1.rs / q8_0_q8_1.rs, whose expected values
 * are closed forms, are replayed against this file by tests/test_oracle.py.
 *
 * Build with -ffp-contract=off: the reference is Rust, which never fuses a
 * multiply and an add, so neither may this file.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define RIBN_ORACLE_OK 0
#define RIBN_ORACLE_UNSUPPORTED_TYPE 1
#define RIBN_ORACLE_INVALID_BLOCK_LENGTH 2
#define RIBN_ORACLE_INVALID_SHAPE 3

/* crates/gguf/src/lib.rs:1051-1083 -- (elements per block, bytes per block).
 * Only the value types the path uses decode here; the size table itself is
 * kept complete for the types the reference lists so shape checks agree. */
int ribn_oracle_tensor_layout(uint32_t value_type, uint64_t *elements, uint64_t *bytes) {
    uint64_t e, b;
    switch (value_type) {
        case 0: case 26: e = 1; b = 4; break;
        case 1: case 25: case 30: e = 1; b = 2; break;
        case 2: case 20: e = 32; b = 18; break;
        case 3: e = 32; b = 20; break;
        case 6: e = 32; b = 22; break;
        case 7: e = 32; b = 24; break;
        case 8: e = 32; b = 34; break;
        case 9: e = 32; b = 36; break;
        case 10: e = 256; b = 84; break;
        case 11: case 21: e = 256; b = 110; break;
        case 12: e = 256; b = 144; break;
        case 13: e = 256; b = 176; break;
        case 14: e = 256; b = 210; break;
        case 15: e = 256; b = 292; break;
        case 16: case 35: e = 256; b = 66; break;
        case 17: e = 256; b = 74; break;
        case 18: e = 256; b = 98; break;
        case 19: e = 256; b = 50; break;
        case 22: e = 256; b = 82; break;
        case 23: e = 256; b = 136; break;
        case 24: e = 1; b = 1; break;
        case 27: case 28: e = 1; b = 8; break;
        case 29: e = 256; b = 56; break;
        case 34: e = 256; b = 54; break;
        case 39: e = 32; b = 17; break;
        case 40: e = 64; b = 36; break;
        case 41: e = 128; b = 18; break;
        case 42: e = 64; b = 18; break;
        default: return RIBN_ORACLE_UNSUPPORTED_TYPE;
    }
    if (elements) *elements = e;
    if (bytes) *bytes = b;
    return RIBN_ORACLE_OK;
}

/* crates/gguf/src/lib.rs:551-563.  Arithmetic form kept on purpose: subnormals
 * are fraction * 2^-24, normals (1 + fraction/1024) * 2^(e-15); every NaN
 * pattern becomes the canonical quiet NaN. */
float ribn_oracle_f16_to_f32(uint16_t bits) {
    const float sign = (bits & 0x8000u) ? -1.0f : 1.0f;
    const int exponent = (bits >> 10) & 0x1f;
    const int fraction = bits & 0x03ff;
    if (exponent == 0) {
        return sign * (float)fraction * ldexpf(1.0f, -24);
    }
    if (exponent == 0x1f) {
        if (fraction == 0) return sign * INFINITY;
        union { uint32_t u; float f; } nan = { 0x7fc00000u };
        return nan.f;
    }
    return sign * (1.0f + (float)fraction / 1024.0f) * ldexpf(1.0f, exponent - 15);
}

static float read_f16(const uint8_t *encoded, size_t offset) {
    return ribn_oracle_f16_to_f32((uint16_t)(encoded[offset] | ((uint16_t)encoded[offset + 1] << 8)));
}

/* crates/gguf/src/lib.rs:573-587.  `packed` is the 12-byte field. */
void ribn_oracle_q4_k_scales(const uint8_t *packed, uint8_t scales[8], uint8_t minima[8]) {
    for (int j = 0; j < 4; ++j) {
        scales[j] = packed[j] & 0x3f;
        scales[j + 4] = (uint8_t)((packed[8 + j] & 0x0f) | ((packed[j] >> 2) & 0x30));
        minima[j] = packed[4 + j] & 0x3f;
        minima[j + 4] = (uint8_t)((packed[8 + j] >> 4) | ((packed[4 + j] >> 2) & 0x30));
    }
}

/* crates/gguf/src/lib.rs:589-594 */
static void dequantize_q8_0(const uint8_t *e, float *out) {
    const float scale = read_f16(e, 0);
    for (int i = 0; i < 32; ++i) out[i] = scale * (float)(int8_t)e[2 + i];
}

/* crates/gguf/src/lib.rs:596-612 */
static void dequantize_q4_k(const uint8_t *e, float *out) {
    const float scale = read_f16(e, 0);
    const float minimum_scale = read_f16(e, 2);
    uint8_t scales[8], minima[8];
    ribn_oracle_q4_k_scales(e + 4, scales, minima);
    for (int group = 0; group < 8; ++group) {
        const int data_offset = 16 + (group / 2) * 32;
        const int shift = (group % 2) * 4;
        const float group_scale = scale * (float)scales[group];
        const float group_minimum = minimum_scale * (float)minima[group];
        for (int i = 0; i < 32; ++i) {
            const int q = (e[data_offset + i] >> shift) & 0x0f;
            out[group * 32 + i] = group_scale * (float)q - group_minimum;
        }
    }
}

/* crates/gguf/src/lib.rs:614-633 */
static void dequantize_q5_k(const uint8_t *e, float *out) {
    const float scale = read_f16(e, 0);
    const float minimum_scale = read_f16(e, 2);
    uint8_t scales[8], minima[8];
    ribn_oracle_q4_k_scales(e + 4, scales, minima);
    const uint8_t *high_bits = e + 16;
    const uint8_t *low_bits = e + 48;
    for (int group = 0; group < 8; ++group) {
        const int data_offset = (group / 2) * 32;
        const int shift = (group % 2) * 4;
        const float group_scale = scale * (float)scales[group];
        const float group_minimum = minimum_scale * (float)minima[group];
        for (int i = 0; i < 32; ++i) {
            const int low = (low_bits[data_offset + i] >> shift) & 0x0f;
            const int high = (high_bits[i] >> group) & 1;
            out[group * 32 + i] = group_scale * (float)(low | (high << 4)) - group_minimum;
        }
    }
}

/* crates/gguf/src/lib.rs:635-661 */
static void dequantize_q6_k(const uint8_t *e, float *out) {
    const uint8_t *low_bits = e;
    const uint8_t *high_bits = e + 128;
    const uint8_t *scales = e + 192;
    const float scale = read_f16(e, 208);
    for (int group = 0; group < 8; ++group) {
        const int chunk = group / 4;
        const int variant = group % 4;
        const int low_offset = chunk * 64 + (variant % 2) * 32;
        const int low_shift = variant < 2 ? 0 : 4;
        const int high_offset = chunk * 32;
        const int high_shift = variant * 2;
        for (int half = 0; half < 2; ++half) {
            const float group_scale = scale * (float)(int8_t)scales[group * 2 + half];
            for (int i = 0; i < 16; ++i) {
                const int p = half * 16 + i;
                const int low = (low_bits[low_offset + p] >> low_shift) & 0x0f;
                const int high = (high_bits[high_offset + p] >> high_shift) & 0x03;
                const int q = (low | (high << 4)) - 32;
                out[group * 32 + p] = group_scale * (float)q;
            }
        }
    }
}

/* crates/gguf/src/lib.rs:520-547.  Decodes exactly one block; `out` must hold
 * the block's element count.  Only value types 0, 1, 8, 12, 13, 14 (the ones on
 * the path) are decoded; anything else the reference also decodes is reported
 * as unsupported here and said so in the design notes. */
int ribn_oracle_dequantize_block(uint32_t value_type, const uint8_t *encoded, uint64_t encoded_len,
                                 float *out) {
    uint64_t elements = 0, bytes = 0;
    int status = ribn_oracle_tensor_layout(value_type, &elements, &bytes);
    if (status != RIBN_ORACLE_OK) return status;
    if (encoded_len != bytes) return RIBN_ORACLE_INVALID_BLOCK_LENGTH;
    switch (value_type) {
        case 0: memcpy(out, encoded, 4); return RIBN_ORACLE_OK;
        case 1: out[0] = read_f16(encoded, 0); return RIBN_ORACLE_OK;
        case 8: dequantize_q8_0(encoded, out); return RIBN_ORACLE_OK;
        case 12: dequantize_q4_k(encoded, out); return RIBN_ORACLE_OK;
        case 13: dequantize_q5_k(encoded, out); return RIBN_ORACLE_OK;
        case 14: dequantize_q6_k(encoded, out); return RIBN_ORACLE_OK;
        default: return RIBN_ORACLE_UNSUPPORTED_TYPE;
    }
}

static int checked_geometry(uint32_t value_type, uint64_t k, uint64_t *elements, uint64_t *bytes) {
    int status = ribn_oracle_tensor_layout(value_type, elements, bytes);
    if (status != RIBN_ORACLE_OK) return status;
    if (value_type != 8 && value_type != 12 && value_type != 13 && value_type != 14)
        return RIBN_ORACLE_UNSUPPORTED_TYPE;
    if (k == 0 || k % *elements != 0) return RIBN_ORACLE_INVALID_SHAPE;
    return RIBN_ORACLE_OK;
}

static void dequantize_row(uint32_t value_type, const uint8_t *row, uint64_t blocks, uint64_t elements,
                           uint64_t bytes, float *out) {
    for (uint64_t b = 0; b < blocks; ++b)
        ribn_oracle_dequantize_block(value_type, row + b * bytes, bytes, out + b * elements);
}

/* Rows are split into contiguous ranges over POSIX threads (no OpenMP runtime
 * is assumed on the host); each row's arithmetic is independent of the split. */
typedef struct {
    uint32_t value_type;
    const uint8_t *data;
    uint64_t k, n, blocks, elements, bytes, members;
    const float *x;
    void *out;
    int mode; /* 0 dequantize, 1 gemv f32, 2 gemv f64, 3 scale */
    uint64_t row_begin, row_end;
} row_job;

/* crates/nvidia/src/qwen_reference.rs:31-40: y[n] = sum_k x[k]*w[n][k], f32,
 * strictly left to right.  Rust's f32 `Sum` folds from -0.0, kept here. */
static float dot_f32_sequential(const float *x, const float *w, uint64_t k) {
    float sum = -0.0f;
    for (uint64_t i = 0; i < k; ++i) sum = sum + x[i] * w[i];
    return sum;
}

static double dot_f64(const float *x, const float *w, uint64_t k) {
    double sum = 0.0;
    for (uint64_t i = 0; i < k; ++i) sum += (double)x[i] * (double)w[i];
    return sum;
}

static void *run_rows(void *arg) {
    const row_job *job = (const row_job *)arg;
    float *scratch = job->mode == 0 ? NULL : (float *)malloc(sizeof(float) * job->k);
    for (uint64_t row = job->row_begin; row < job->row_end; ++row) {
        const uint8_t *encoded = job->data + row * job->blocks * job->bytes;
        if (job->mode == 0) {
            dequantize_row(job->value_type, encoded, job->blocks, job->elements, job->bytes,
                           (float *)job->out + row * job->k);
            continue;
        }
        /* The reference host path: dequantise the row into an f32 scratch first. */
        dequantize_row(job->value_type, encoded, job->blocks, job->elements, job->bytes, scratch);
        for (uint64_t m = 0; m < job->members; ++m) {
            const float *xm = job->x + m * job->k;
            if (job->mode == 1) {
                ((float *)job->out)[m * job->n + row] = dot_f32_sequential(xm, scratch, job->k);
            } else if (job->mode == 2) {
                ((double *)job->out)[m * job->n + row] = dot_f64(xm, scratch, job->k);
            } else {
                double sum = 0.0;
                for (uint64_t i = 0; i < job->k; ++i) {
                    const double p = (double)xm[i] * (double)scratch[i];
                    sum += p * p;
                }
                ((double *)job->out)[m * job->n + row] = sqrt(sum);
            }
        }
    }
    free(scratch);
    return NULL;
}

static int run_job(row_job base, int threads) {
    int status = checked_geometry(base.value_type, base.k, &base.elements, &base.bytes);
    if (status != RIBN_ORACLE_OK) return status;
    base.blocks = base.k / base.elements;
    if (threads < 1) threads = 1;
    if ((uint64_t)threads > base.n) threads = base.n ? (int)base.n : 1;
    if (threads == 1) {
        base.row_begin = 0;
        base.row_end = base.n;
        run_rows(&base);
        return RIBN_ORACLE_OK;
    }
    pthread_t *ids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    row_job *jobs = (row_job *)malloc(sizeof(row_job) * (size_t)threads);
    for (int t = 0; t < threads; ++t) {
        jobs[t] = base;
        jobs[t].row_begin = base.n * (uint64_t)t / (uint64_t)threads;
        jobs[t].row_end = base.n * (uint64_t)(t + 1) / (uint64_t)threads;
        pthread_create(&ids[t], NULL, run_rows, &jobs[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(ids[t], NULL);
    free(ids);
    free(jobs);
    return RIBN_ORACLE_OK;
}

/* Whole tensor [N rows][K] -> f32, block by block in storage order. */
int ribn_oracle_dequantize(uint32_t value_type, const uint8_t *data, uint64_t k, uint64_t n, float *out,
                           int threads) {
    row_job job = { value_type, data, k, n, 0, 0, 0, 0, NULL, out, 0, 0, 0 };
    return run_job(job, threads);
}

/* The reference host path (dequantise a row, sequential f32 dot) for each of
 * `members` activation rows.  x is [members][K] f32, y is [members][N] f32.
 * threads<=1 is the faithful single-threaded form; threads>1 splits rows over
 * host threads with the same arithmetic per row. */
int ribn_oracle_gemv_f32(uint32_t value_type, const uint8_t *data, uint64_t k, uint64_t n,
                         const float *x, uint64_t members, float *y, int threads) {
    row_job job = { value_type, data, k, n, 0, 0, 0, members, x, y, 1, 0, 0 };
    return run_job(job, threads);
}

/* Accuracy oracle: same dequantised f32 weights, f64 products and sums. */
int ribn_oracle_gemv_f64(uint32_t value_type, const uint8_t *data, uint64_t k, uint64_t n,
                         const float *x, uint64_t members, double *y, int threads) {
    row_job job = { value_type, data, k, n, 0, 0, 0, members, x, y, 2, 0, 0 };
    return run_job(job, threads);
}

/* Per-output scale used as the denominator floor of the relative-error metric:
 * sqrt(sum_k (w[n][k]*x[k])^2), the standard deviation a dot product of that
 * row would have under random signs.  f64. */
int ribn_oracle_gemv_scale(uint32_t value_type, const uint8_t *data, uint64_t k, uint64_t n,
                           const float *x, uint64_t members, double *scale, int threads) {
    row_job job = { value_type, data, k, n, 0, 0, 0, members, x, scale, 3, 0, 0 };
    return run_job(job, threads);
}

/* crates/nvidia/src/qwen_reference.rs:550-556.  One vector. */
void ribn_oracle_rms_norm(const float *input, const float *weight, uint64_t length, float eps, float *out) {
    float sum = -0.0f;
    for (uint64_t i = 0; i < length; ++i) sum = sum + input[i] * input[i];
    const float count = (float)length;
    const float inv = 1.0f / sqrtf(sum / count + eps);
    for (uint64_t i = 0; i < length; ++i) out[i] = input[i] * inv * weight[i];
}

/* Batch-major [members][length], the host twin of rms_norm_batch
 * (crates/nvidia/src/model_ops.rs:157-199): the same equation per member. */
void ribn_oracle_rms_norm_batch(const float *input, const float *weight, uint64_t members, uint64_t length,
                                float eps, float *out) {
    for (uint64_t m = 0; m < members; ++m)
        ribn_oracle_rms_norm(input + m * length, weight, length, eps, out + m * length);
}

/* crates/nvidia/src/qwen_reference.rs:531-537: silu(g) * u = g / (1 + exp(-g)) * u */
void ribn_oracle_silu_mul(const float *gate, const float *up, uint64_t length, float *out) {
    for (uint64_t i = 0; i < length; ++i) out[i] = gate[i] / (1.0f + expf(-gate[i])) * up[i];
}

/* bf16 helpers used by tests to build the activation the kernels really see:
 * round-to-nearest-even f32 -> bf16, and exact widening back. */
uint16_t ribn_oracle_f32_to_bf16(float value) {
    union { float f; uint32_t u; } v = { value };
    if ((v.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((v.u >> 16) | 0x0040u);
    const uint32_t rounding = 0x7fffu + ((v.u >> 16) & 1u);
    return (uint16_t)((v.u + rounding) >> 16);
}

float ribn_oracle_bf16_to_f32(uint16_t bits) {
    union { uint32_t u; float f; } v = { (uint32_t)bits << 16 };
    return v.f;
}
