/*
 * CPU oracle for the INT4/INT8 dequantise + matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the GPU kernels are
 * compared against and the code timed as the CPU baseline.  Nothing in the
 * shipped package links, imports or executes it.
 *
 * Each function restates, in plain C, a helper of the reference's own CPU path
 * (its GoogleTest fixture), following the cited lines: same indexing, same
 * formula, same fp32 arithmetic, same k-ascending accumulation order.  The
 * fixture itself cannot be compiled outside macOS (Objective-C++, Metal headers,
 * GoogleTest), hence a restatement.
 *
 * Parity pin: tests/test_oracle_golden.py checks these functions against the
 * reference's known-answer test (INT4_SmallKnownAnswer, expected [-3.3, -9.0])
 * and the formula-seeded INT4/INT8 square-matrix cases of the same test file.
 *
 * Build: make -C oracle      (gcc -O2, no -ffast-math: fp32 results must not
 *                             depend on re-association)
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------- */
/* fp16 <-> fp32 helpers                                                      */
/* ------------------------------------------------------------------------- */

/* Follows tests/cpp/test_dequant_matmul.mm:216-240 (fp16_to_fp32). */
float oracle_fp16_to_fp32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exponent = ((uint32_t)h & 0x7C00u) >> 10;
    uint32_t mantissa = (uint32_t)h & 0x03FFu;
    if (exponent == 0) {
        if (mantissa == 0) return sign ? -0.0f : 0.0f;
        float v = ldexpf((float)mantissa / 1024.0f, -14);
        return sign ? -v : v;
    }
    if (exponent == 31) {
        if (mantissa == 0) return sign ? -INFINITY : INFINITY;
        return NAN;
    }
    uint32_t bits = sign | ((exponent - 15u + 127u) << 23) | (mantissa << 13);
    float out;
    memcpy(&out, &bits, sizeof out);
    return out;
}

/* Follows tests/cpp/test_dequant_matmul.mm:241-259 (fp32_to_fp16): this helper
 * TRUNCATES the mantissa.  Kept only so the fixture's exact input bits can be
 * reproduced; the harness itself creates fp16 data with round-to-nearest-even
 * (oracle_fp32_to_fp16_rn) and hands the same bits to oracle and GPU. */
uint16_t oracle_fp32_to_fp16_trunc(float f)
{
    uint32_t bits;
    memcpy(&bits, &f, sizeof bits);
    uint32_t sign = (bits & 0x80000000u) >> 16;
    int32_t exponent = (int32_t)((bits & 0x7F800000u) >> 23) - 127 + 15;
    uint32_t mantissa = bits & 0x007FFFFFu;
    if (exponent <= 0) {
        if (exponent < -10) return (uint16_t)sign;
        mantissa |= 0x00800000u;
        uint16_t frac = (uint16_t)(mantissa >> (14 - exponent));
        return (uint16_t)(sign | frac);
    }
    if (exponent >= 31) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)exponent << 10) | (mantissa >> 13));
}

/* IEEE round-to-nearest-even fp32 -> fp16 (what `half(x)` / __float2half_rn do). */
uint16_t oracle_fp32_to_fp16_rn(float f)
{
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x0200u : 0u));
    if (absx >= 0x477FF000u) /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    if (absx < 0x33000001u) /* < 2^-25 (or exactly): rounds to zero */
        return (uint16_t)sign;
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x007FFFFFu) | 0x00800000u; /* 24-bit significand */
    int shift;
    uint32_t base;
    if (e >= -14) { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x007FFFFFu; }
    else { shift = 13 + (-14 - e); base = 0; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half_ulp = 1u << (shift - 1);
    if (rem > half_ulp || (rem == half_ulp && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q)); /* carry into the exponent is correct */
}

/* bf16 = high 16 bits of fp32; widening is exact, narrowing rounds to nearest
 * even -- the convention of shaders/common/metal_types.h:17-26. */
float oracle_bf16_to_fp32(uint16_t b)
{
    uint32_t bits = (uint32_t)b << 16;
    float out;
    memcpy(&out, &bits, sizeof out);
    return out;
}

uint16_t oracle_fp32_to_bf16_rn(float f)
{
    uint32_t x;
    memcpy(&x, &f, sizeof x);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

void oracle_fp16_to_fp32_array(const uint16_t* in, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_fp16_to_fp32(in[i]);
}
void oracle_fp32_to_fp16_rn_array(const float* in, uint16_t* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_fp32_to_fp16_rn(in[i]);
}
void oracle_bf16_to_fp32_array(const uint16_t* in, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_bf16_to_fp32(in[i]);
}
void oracle_fp32_to_bf16_rn_array(const float* in, uint16_t* out, size_t n)
{
    for (size_t i = 0; i < n; ++i) out[i] = oracle_fp32_to_bf16_rn(in[i]);
}

/* ------------------------------------------------------------------------- */
/* Packing                                                                    */
/* ------------------------------------------------------------------------- */

/* Follows tests/cpp/test_dequant_matmul.mm:104-116 (pack_int4): values are
 * packed pairwise, element 2j in the low nibble, element 2j+1 in the high one;
 * an odd tail gets a zero high nibble.  `out` holds (count+1)/2 bytes. */
void oracle_pack_int4(const int8_t* values, size_t count, uint8_t* out)
{
    for (size_t i = 0; i < count; i += 2) {
        uint8_t low = (uint8_t)(values[i] & 0x0F);
        uint8_t high = (i + 1 < count) ? (uint8_t)(values[i + 1] & 0x0F) : 0;
        out[i / 2] = (uint8_t)(low | (high << 4));
    }
}

/* ------------------------------------------------------------------------- */
/* Dequantise to fp32, [N, K] row-major                                       */
/* ------------------------------------------------------------------------- */

/* One row of dequant_reference_int4, tests/cpp/test_dequant_matmul.mm:131-153. */
static void dequant_int4_rows(const uint8_t* packed, const float* scales, const float* zeros,
                              uint32_t K, uint32_t group_size, uint32_t n_begin, uint32_t n_end,
                              float* out /* indexed from row 0 */)
{
    uint32_t groups = (K + group_size - 1) / group_size;
    size_t row_bytes = (size_t)((K + 1) / 2);
    for (uint32_t n = n_begin; n < n_end; ++n) {
        for (uint32_t k = 0; k < K; ++k) {
            uint8_t byte = packed[(size_t)n * row_bytes + k / 2];
            int8_t q = (k % 2 == 0) ? (int8_t)(byte & 0x0F) : (int8_t)((byte >> 4) & 0x0F);
            uint32_t g = k / group_size;
            float scale = scales[(size_t)n * groups + g];
            float zero = zeros[(size_t)n * groups + g];
            out[(size_t)n * K + k] = ((float)q - 8.0f) * scale - zero;
        }
    }
}

/* One row of dequant_reference_int8, tests/cpp/test_dequant_matmul.mm:171-184. */
static void dequant_int8_rows(const int8_t* data, const float* scales, const float* zeros,
                              uint32_t K, uint32_t group_size, uint32_t n_begin, uint32_t n_end,
                              float* out)
{
    uint32_t groups = (K + group_size - 1) / group_size;
    for (uint32_t n = n_begin; n < n_end; ++n) {
        for (uint32_t k = 0; k < K; ++k) {
            int8_t q = data[(size_t)n * K + k];
            uint32_t g = k / group_size;
            float scale = scales[(size_t)n * groups + g];
            float zero = zeros[(size_t)n * groups + g];
            out[(size_t)n * K + k] = (float)q * scale - zero;
        }
    }
}

/* tests/cpp/test_dequant_matmul.mm:119-157.  w[n,k] = (float(q) - 8) * s - z,
 * q the unsigned nibble, packed row stride (K+1)/2, scales/zeros [N, ceil(K/g)]. */
void oracle_dequant_int4(const uint8_t* packed, const float* scales, const float* zeros,
                         uint32_t K, uint32_t N, uint32_t group_size, float* out)
{
    dequant_int4_rows(packed, scales, zeros, K, group_size, 0, N, out);
}

/* tests/cpp/test_dequant_matmul.mm:160-188.  w[n,k] = float(q) * s - z. */
void oracle_dequant_int8(const int8_t* data, const float* scales, const float* zeros,
                         uint32_t K, uint32_t N, uint32_t group_size, float* out)
{
    dequant_int8_rows(data, scales, zeros, K, group_size, 0, N, out);
}

/* ------------------------------------------------------------------------- */
/* Naive fp32 matmul                                                          */
/* ------------------------------------------------------------------------- */

static void matmul_cols(const float* A, const float* B, uint32_t M, uint32_t N, uint32_t K,
                        uint32_t n_begin, uint32_t n_end, float* C)
{
    for (uint32_t m = 0; m < M; ++m) {
        for (uint32_t n = n_begin; n < n_end; ++n) {
            float sum = 0.0f;
            for (uint32_t k = 0; k < K; ++k)
                sum += A[(size_t)m * K + k] * B[(size_t)n * K + k];
            C[(size_t)m * N + n] = sum;
        }
    }
}

/* tests/cpp/test_dequant_matmul.mm:191-213.  C[m,n] = sum_k A[m,k] * B[n,k],
 * one fp32 accumulator per output, k ascending. */
void oracle_matmul(const float* A, const float* B, uint32_t M, uint32_t N, uint32_t K, float* C)
{
    matmul_cols(A, B, M, N, K, 0, N, C);
}

/* ------------------------------------------------------------------------- */
/* The whole path, optionally split over N across threads                     */
/* ------------------------------------------------------------------------- */

typedef struct {
    const float* A;
    const void* wq;
    const float* scales;
    const float* zeros;
    uint32_t M, N, K, group_size;
    int quant; /* 0 = int4, 1 = int8 */
    uint32_t n_begin, n_end;
    float* W; /* [N, K] scratch, shared */
    float* C;
} path_job;

static void* path_worker(void* arg)
{
    path_job* j = (path_job*)arg;
    if (j->quant == 0)
        dequant_int4_rows((const uint8_t*)j->wq, j->scales, j->zeros, j->K, j->group_size,
                          j->n_begin, j->n_end, j->W);
    else
        dequant_int8_rows((const int8_t*)j->wq, j->scales, j->zeros, j->K, j->group_size,
                          j->n_begin, j->n_end, j->W);
    matmul_cols(j->A, j->W, j->M, j->N, j->K, j->n_begin, j->n_end, j->C);
    return NULL;
}

/* Dequantise-then-matmul exactly as the fixture's tests do (dequantise the whole
 * weight to fp32, then the naive triple loop), with the N range cut into
 * `threads` contiguous slices.  Every output element is computed by the same
 * instruction sequence whatever `threads` is, so results do not depend on it.
 * `W_scratch` is [N, K] fp32 provided by the caller.  Returns 0, or -1 if a
 * thread could not be started. */
int oracle_dequant_matmul(const float* A, const void* wq, const float* scales, const float* zeros,
                          uint32_t M, uint32_t N, uint32_t K, uint32_t group_size, int quant,
                          int threads, float* W_scratch, float* C)
{
    if (threads < 1) threads = 1;
    if ((uint32_t)threads > N) threads = (int)(N ? N : 1);
    path_job* jobs = (path_job*)calloc((size_t)threads, sizeof *jobs);
    pthread_t* tids = (pthread_t*)calloc((size_t)threads, sizeof *tids);
    if (!jobs || !tids) { free(jobs); free(tids); return -1; }
    int rc = 0, started = 0;
    for (int t = 0; t < threads; ++t) {
        path_job* j = &jobs[t];
        j->A = A; j->wq = wq; j->scales = scales; j->zeros = zeros;
        j->M = M; j->N = N; j->K = K; j->group_size = group_size; j->quant = quant;
        j->n_begin = (uint32_t)(((uint64_t)N * (uint64_t)t) / (uint64_t)threads);
        j->n_end = (uint32_t)(((uint64_t)N * (uint64_t)(t + 1)) / (uint64_t)threads);
        j->W = W_scratch; j->C = C;
        if (threads == 1) { path_worker(j); continue; }
        if (pthread_create(&tids[t], NULL, path_worker, j) != 0) { rc = -1; break; }
        started++;
    }
    for (int t = 0; t < started; ++t) pthread_join(tids[t], NULL);
    free(jobs); free(tids);
    return rc;
}

/* ------------------------------------------------------------------------- */
/* Standalone dequantise kernels (scale only, flat group index)               */
/* ------------------------------------------------------------------------- */

/* shaders/dequantize_kernel.metal:9-22 (and its 8-wide twin :58-96, which
 * computes the same values): out[i] = half(in[i]) * scales[i / group_size],
 * evaluated in half precision.  A product of an 8-bit integer and an 11-bit
 * significand is exact in fp32, so half arithmetic equals one RN to fp16 of the
 * fp32 product.  Output is fp16 bits. */
void oracle_dequantize_flat_int8(const int8_t* in, const uint16_t* scales_fp16, uint16_t* out_fp16,
                                 uint32_t num_elements, uint32_t group_size)
{
    for (uint32_t i = 0; i < num_elements; ++i) {
        float s = oracle_fp16_to_fp32(scales_fp16[i / group_size]);
        out_fp16[i] = oracle_fp32_to_fp16_rn((float)in[i] * s);
    }
}

/* shaders/dequantize_kernel.metal:26-54 (and :100-163): byte j yields
 * out[2j] = half((b & 15) - 8) * s[2j / g], out[2j+1] = half((b >> 4) - 8) * s[(2j+1) / g];
 * no zero-point. */
void oracle_dequantize_flat_int4(const uint8_t* in, const uint16_t* scales_fp16, uint16_t* out_fp16,
                                 uint32_t num_elements, uint32_t group_size)
{
    for (uint32_t i = 0; i < num_elements; i += 2) {
        uint8_t b = in[i / 2];
        int lo = (int)(b & 0x0F) - 8;
        int hi = (int)((b >> 4) & 0x0F) - 8;
        float s_lo = oracle_fp16_to_fp32(scales_fp16[i / group_size]);
        out_fp16[i] = oracle_fp32_to_fp16_rn((float)lo * s_lo);
        if (i + 1 < num_elements) {
            float s_hi = oracle_fp16_to_fp32(scales_fp16[(i + 1) / group_size]);
            out_fp16[i + 1] = oracle_fp32_to_fp16_rn((float)hi * s_hi);
        }
    }
}
