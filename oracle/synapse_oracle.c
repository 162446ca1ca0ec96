/*
 * TEST INFRASTRUCTURE ONLY. This file is the CPU oracle for the B200 backend: a plain-C restatement of
 * the reference's (managedcode/Synapse) CPU arithmetic for the quantized matrix-product path. Only the
 * tests, the smoke check and the benchmark's CPU-baseline leg may load it; the product library never does.
 *
 * Parity pins: the functions below are checked (tests/test_oracle_*.py) against the known-answer vectors
 * held by the reference's own tests: the activation quantiser ties / zero-block / scale vectors
 * (tests/Synapse.IntegrationTests/Features/CpuKernels/ActivationQuantizerTests.cs:28-61), the Q8_0 golden
 * block (tests/Synapse.IntegrationTests/Features/ModelPackages/SourceTensorDecoderTests.cs:56-70), the
 * exhaustive fp16 widening check and the LCG cases with their 2e-5*sum|term| tolerance
 * (native/synapse-kernels/tests/Features/CpuKernels/q8_0_tests.rs:9-62,116,133-140,223-247), and the K-quant
 * geometry (SourceTensorDecoderTests.cs:165-173). The reference itself cannot be built where this oracle is
 * developed (no .NET SDK, no Rust toolchain), so no output of the reference binary is used.
 *
 * Build: -O2 -ffp-contract=off -fno-fast-math (C# and the Rust scalar kernel never contract a*b+c unless they
 * ask for a fused multiply-add explicitly, and where they do this file calls fmaf).
 */
#include <math.h>
#include <pthread.h>
#include <stdatomic.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__)
#include <immintrin.h>
#define ORC_HAVE_AVX2 1 /* compiled per function with target("avx2,fma"); selected at run time */
#define ORC_AVX2_FN __attribute__((target("avx2,fma")))
#else
#define ORC_HAVE_AVX2 0
#endif

#define Q8_BLOCK_VALUES 32
#define Q8_BLOCK_BYTES 34
#define K_SUPER 256
#define Q4K_BYTES 144
#define Q6K_BYTES 210

#define GGML_Q8_0 8u
#define GGML_Q4_K 12u
#define GGML_Q6_K 14u

int orc_have_avx2(void);

/* ------------------------------------------------------------------------------------------------ */
/* fp16 <-> fp32                                                                                      */
/* ------------------------------------------------------------------------------------------------ */

/* Exact half -> float for finite values: magnitude bits shifted by 13, then scaled by 2^112.
 * Follows native/synapse-kernels/src/Features/CpuKernels/q8_0.rs:127-134 and
 * src/Synapse.Runtime/Features/CpuKernels/Fp16.cs:17-22. */
float orc_fp16_to_f32(uint16_t bits)
{
    union { uint32_t u; float f; } magnitude, rescale;
    magnitude.u = (uint32_t)(bits & 0x7fffu) << 13;
    rescale.u = 0x77800000u;
    float value = magnitude.f * rescale.f;
    return (bits & 0x8000u) ? -value : value;
}

/* float -> half, round to nearest even: what C#'s `(Half)value` does
 * (src/Synapse.Runtime/Features/CpuKernels/Q8ActivationQuantizer.cs:56). */
uint16_t orc_f32_to_fp16(float value)
{
    union { uint32_t u; float f; } in;
    in.f = value;
    uint16_t sign = (uint16_t)((in.u >> 16) & 0x8000u);
    uint32_t x = in.u & 0x7fffffffu;
    if (x >= 0x7f800000u) {
        return (uint16_t)(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));
    }
    if (x >= 0x477ff000u) { /* >= 65520 rounds to infinity */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (x < 0x38800000u) { /* below 2^-14: half subnormal = rint(|v| * 2^24), ties to even */
        union { uint32_t u; float f; } mag;
        mag.u = x;
        float scaled = mag.f * 16777216.0f;
        return (uint16_t)(sign | (uint16_t)nearbyintf(scaled));
    }
    uint32_t mantissa = x & 0x7fffffu;
    uint32_t exponent = (x >> 23) - 127u + 15u;
    uint32_t half = (exponent << 10) | (mantissa >> 13);
    uint32_t rest = mantissa & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) {
        half += 1u; /* may carry into the exponent, which is the correct rounding */
    }
    return (uint16_t)(sign | half);
}

static inline float half_at(const uint8_t *p)
{
    return orc_fp16_to_f32((uint16_t)(p[0] | ((uint16_t)p[1] << 8)));
}

/* ------------------------------------------------------------------------------------------------ */
/* O1: activation quantiser                                                                          */
/* ------------------------------------------------------------------------------------------------ */

/* One 32-value block. Follows Q8ActivationQuantizer.cs:34-57 and the scalar restatement in
 * ActivationQuantizerTests.cs:72-95: scale = max|x| / 127, inverse = scale == 0 ? 0 : 1 / scale,
 * code = round_half_even(x * inverse) with the UNROUNDED scale, stored scale = (float)(Half)scale. */
static float quantize_block(const float *x, int8_t *codes)
{
    float amax = 0.0f;
    for (int i = 0; i < Q8_BLOCK_VALUES; ++i) {
        amax = fmaxf(amax, fabsf(x[i]));
    }
    float scale = amax / 127.0f;
    float inverse = scale == 0.0f ? 0.0f : 1.0f / scale;
    for (int i = 0; i < Q8_BLOCK_VALUES; ++i) {
        codes[i] = (int8_t)nearbyintf(x[i] * inverse);
    }
    return orc_fp16_to_f32(orc_f32_to_fp16(scale));
}

/* Returns 0, or 2 when the width is not a positive multiple of 32 (Q8ActivationQuantizer.cs:17-24). */
int orc_q8_quantize_row(const float *x, size_t columns, int8_t *codes, float *scales)
{
    if (columns == 0 || columns % Q8_BLOCK_VALUES != 0) {
        return 2;
    }
    for (size_t b = 0; b < columns / Q8_BLOCK_VALUES; ++b) {
        scales[b] = quantize_block(x + b * Q8_BLOCK_VALUES, codes + b * Q8_BLOCK_VALUES);
    }
    return 0;
}

/* Sum of codes per 16 values; used by the K-quant x Q8 contract (no reference counterpart). */
void orc_q8_group_sums(const int8_t *codes, size_t columns, int16_t *sums16)
{
    for (size_t g = 0; g < columns / 16; ++g) {
        int s = 0;
        for (int i = 0; i < 16; ++i) {
            s += codes[g * 16 + i];
        }
        sums16[g] = (int16_t)s;
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* O2: Q8_0 weights x Q8_0 activations, scalar order                                                 */
/* ------------------------------------------------------------------------------------------------ */

static int32_t q8_block_dot(const uint8_t *block, const int8_t *codes)
{
    int32_t dot = 0;
    for (int i = 0; i < Q8_BLOCK_VALUES; ++i) {
        dot += (int32_t)(int8_t)block[2 + i] * (int32_t)codes[i];
    }
    return dot;
}

/* Status codes of the reference's C ABI (native/synapse-kernels/src/Features/CpuKernels/ffi.rs:10-18). */
enum { ORC_OK = 0, ORC_NULL = 1, ORC_SHAPE = 2, ORC_OVERFLOW = 3 };

static int mul_ok(size_t a, size_t b, size_t *out)
{
    return !__builtin_mul_overflow(a, b, out);
}

/* Shape validation of synapse_q8_0_matmul (ffi.rs:55-84, q8_0.rs:212-246). */
static int q8q8_validate(const void *w, size_t row_bytes, size_t rows, size_t blocks, const void *q,
                         const void *s, size_t tokens, const void *out, size_t stride)
{
    if (!w || !q || !s || !out) {
        return ORC_NULL;
    }
    size_t expect;
    if (rows == 0 || blocks == 0 || tokens == 0 || !mul_ok(blocks, Q8_BLOCK_BYTES, &expect) ||
        expect != row_bytes) {
        return ORC_SHAPE;
    }
    size_t scales, codes, weights, outputs;
    if (!mul_ok(tokens, blocks, &scales) || !mul_ok(scales, Q8_BLOCK_VALUES, &codes) ||
        !mul_ok(rows, row_bytes, &weights) || !mul_ok(tokens - 1, stride, &outputs) ||
        __builtin_add_overflow(outputs, rows, &outputs)) {
        return ORC_OVERFLOW;
    }
    if (tokens > 1 && stride < rows) {
        return ORC_SHAPE;
    }
    return ORC_OK;
}

/* output[t*stride + r] = dot(W[r], A[t]); per block an exact int32 dot, then
 * sum = fma((float)dot, weight_scale * activation_scale, sum) with blocks in order.
 * Follows native/synapse-kernels/src/Features/CpuKernels/scalar.rs:4-48; same signature as
 * synapse_q8_0_matmul (ffi.rs:44-54). */
int orc_q8q8_matmul(const uint8_t *weights, size_t row_bytes, size_t rows, size_t blocks,
                    const int8_t *quants, const float *scales, size_t tokens, float *output, size_t stride)
{
    int status = q8q8_validate(weights, row_bytes, rows, blocks, quants, scales, tokens, output, stride);
    if (status != ORC_OK) {
        return status;
    }
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t *row = weights + r * row_bytes;
        for (size_t t = 0; t < tokens; ++t) {
            const int8_t *codes = quants + t * blocks * Q8_BLOCK_VALUES;
            const float *ascale = scales + t * blocks;
            float sum = 0.0f;
            for (size_t b = 0; b < blocks; ++b) {
                const uint8_t *block = row + b * Q8_BLOCK_BYTES;
                int32_t dot = q8_block_dot(block, codes + b * Q8_BLOCK_VALUES);
                sum = fmaf((float)dot, half_at(block) * ascale[b], sum);
            }
            output[t * stride + r] = sum;
        }
    }
    return ORC_OK;
}

/* The exact integer block dots of O2: dots[(t*rows + r)*blocks + b]. */
void orc_q8q8_block_dots(const uint8_t *weights, size_t rows, size_t blocks, const int8_t *quants,
                         size_t tokens, int32_t *dots)
{
    for (size_t t = 0; t < tokens; ++t) {
        for (size_t r = 0; r < rows; ++r) {
            for (size_t b = 0; b < blocks; ++b) {
                dots[(t * rows + r) * blocks + b] =
                    q8_block_dot(weights + (r * blocks + b) * Q8_BLOCK_BYTES,
                                 quants + (t * blocks + b) * Q8_BLOCK_VALUES);
            }
        }
    }
}

/* FP64 evaluation of O2 with the magnitude sum used to normalise tolerances
 * (q8_0_tests.rs:84-108; tests/Synapse.IntegrationTests/Features/CpuKernels/Q8KernelOracle.cs:67-94). */
void orc_q8q8_exact(const uint8_t *weights, size_t rows, size_t blocks, const int8_t *quants,
                    const float *scales, size_t tokens, double *value, double *magnitude)
{
    for (size_t t = 0; t < tokens; ++t) {
        for (size_t r = 0; r < rows; ++r) {
            double v = 0.0, m = 0.0;
            for (size_t b = 0; b < blocks; ++b) {
                const uint8_t *block = weights + (r * blocks + b) * Q8_BLOCK_BYTES;
                int32_t dot = q8_block_dot(block, quants + (t * blocks + b) * Q8_BLOCK_VALUES);
                double term = (double)half_at(block) * (double)scales[t * blocks + b] * (double)dot;
                v += term;
                m += fabs(term);
            }
            value[t * rows + r] = v;
            magnitude[t * rows + r] = m;
        }
    }
}

/* ------------------------------------------------------------------------------------------------ */
/* O2 (timed baseline): AVX2 + FMA kernel with the reference's row strategy                          */
/* ------------------------------------------------------------------------------------------------ */

#if ORC_HAVE_AVX2
/* Per block: |w| * sign(a, w) through maddubs + madd(1) into eight int32 lanes, converted and fused into
 * eight float lanes with the scalar scale product. Follows avx2.rs:127-147. */
ORC_AVX2_FN static inline __m256 avx2_accumulate(__m256 sum, const uint8_t *block, __m256i values, float ascale)
{
    __m256i w = _mm256_loadu_si256((const __m256i *)(block + 2));
    __m256i magnitudes = _mm256_sign_epi8(w, w);
    __m256i signed_values = _mm256_sign_epi8(values, w);
    __m256i pairs = _mm256_maddubs_epi16(magnitudes, signed_values);
    __m256i dots = _mm256_madd_epi16(pairs, _mm256_set1_epi16(1));
    return _mm256_fmadd_ps(_mm256_cvtepi32_ps(dots), _mm256_set1_ps(half_at(block) * ascale), sum);
}

/* Low + high halves, then pairs, then the last two lanes (avx2.rs:149-156). */
ORC_AVX2_FN static inline float avx2_hsum(__m256 v)
{
    __m128 quad = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
    __m128 pair = _mm_add_ps(quad, _mm_movehl_ps(quad, quad));
    return _mm_cvtss_f32(_mm_add_ss(pair, _mm_shuffle_ps(pair, pair, 1)));
}

/* Rows shorter than 64 blocks go four at a time sharing each activation load; longer rows go one at a
 * time with two accumulators (avx2.rs:19-125, LONG_ROW_BLOCKS = 64). */
ORC_AVX2_FN static void q8q8_avx2_rows(const uint8_t *weights, size_t rows, size_t blocks, const int8_t *quants,
                           const float *scales, size_t tokens, float *output, size_t stride)
{
    const size_t row_bytes = blocks * Q8_BLOCK_BYTES;
    const size_t row_codes = blocks * Q8_BLOCK_VALUES;
    const size_t quad_rows = blocks >= 64 ? 0 : (rows & ~(size_t)3);
    for (size_t r = 0; r < quad_rows; r += 4) {
        for (size_t t = 0; t < tokens; ++t) {
            __m256 sums[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                              _mm256_setzero_ps()};
            for (size_t b = 0; b < blocks; ++b) {
                __m256i values =
                    _mm256_loadu_si256((const __m256i *)(quants + t * row_codes + b * Q8_BLOCK_VALUES));
                float ascale = scales[t * blocks + b];
                for (int lane = 0; lane < 4; ++lane) {
                    sums[lane] = avx2_accumulate(
                        sums[lane], weights + (r + lane) * row_bytes + b * Q8_BLOCK_BYTES, values, ascale);
                }
            }
            for (int lane = 0; lane < 4; ++lane) {
                output[t * stride + r + lane] = avx2_hsum(sums[lane]);
            }
        }
    }
    for (size_t r = quad_rows; r < rows; ++r) {
        const uint8_t *row = weights + r * row_bytes;
        for (size_t t = 0; t < tokens; ++t) {
            const int8_t *codes = quants + t * row_codes;
            const float *ascale = scales + t * blocks;
            __m256 s0 = _mm256_setzero_ps(), s1 = _mm256_setzero_ps();
            size_t unrolled = blocks & ~(size_t)1;
            for (size_t b = 0; b < unrolled; b += 2) {
                s0 = avx2_accumulate(s0, row + b * Q8_BLOCK_BYTES,
                                     _mm256_loadu_si256((const __m256i *)(codes + b * Q8_BLOCK_VALUES)),
                                     ascale[b]);
                s1 = avx2_accumulate(
                    s1, row + (b + 1) * Q8_BLOCK_BYTES,
                    _mm256_loadu_si256((const __m256i *)(codes + (b + 1) * Q8_BLOCK_VALUES)), ascale[b + 1]);
            }
            for (size_t b = unrolled; b < blocks; ++b) {
                s0 = avx2_accumulate(s0, row + b * Q8_BLOCK_BYTES,
                                     _mm256_loadu_si256((const __m256i *)(codes + b * Q8_BLOCK_VALUES)),
                                     ascale[b]);
            }
            output[t * stride + r] = avx2_hsum(s0) + avx2_hsum(s1);
        }
    }
}
#endif

int orc_have_avx2(void)
{
#if ORC_HAVE_AVX2
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
#else
    return 0;
#endif
}

/* ------------------------------------------------------------------------------------------------ */
/* O3: Q8_0 weights x FP32 activations (reference backend)                                           */
/* ------------------------------------------------------------------------------------------------ */

/* Per row: for each block a sequential FP32 blockSum += (float)q * x (separate multiply and add), then
 * sum += scale * blockSum. Follows src/Synapse.Runtime/Features/GraphExecution/Q8Operators.cs:75-96. */
static float q8_f32_row(const uint8_t *row, size_t blocks, const float *x)
{
    float sum = 0.0f;
    for (size_t b = 0; b < blocks; ++b) {
        const uint8_t *block = row + b * Q8_BLOCK_BYTES;
        float scale = half_at(block);
        float block_sum = 0.0f;
        for (int i = 0; i < Q8_BLOCK_VALUES; ++i) {
            block_sum += (float)(int8_t)block[2 + i] * x[b * Q8_BLOCK_VALUES + i];
        }
        sum += scale * block_sum;
    }
    return sum;
}

/* ------------------------------------------------------------------------------------------------ */
/* O4: exact ggml-order block decoders                                                               */
/* ------------------------------------------------------------------------------------------------ */

/* value = scale * (sbyte)code. Follows
 * src/Synapse.Runtime/Features/ModelPackages/SourceFormats/GgufLegacyBlocks.cs:85-92. */
static void decode_q8_0(const uint8_t *block, float *y)
{
    float d = half_at(block);
    for (int i = 0; i < Q8_BLOCK_VALUES; ++i) {
        y[i] = d * (float)(int8_t)block[2 + i];
    }
}

/* 6-bit (scale, min) pair j of a Q4_K super-block; `s` is the 12 packed bytes.
 * Follows GgufKQuantBlocks.cs:149-153. */
static inline void scale_min_k4(int j, const uint8_t *s, int *scale, int *min)
{
    if (j < 4) {
        *scale = s[j] & 63;
        *min = s[j + 4] & 63;
    } else {
        *scale = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        *min = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

/* Four chunks of 64 values: low nibbles then high nibbles of the same 32 bytes;
 * y = (d*scale) * q - (dmin*min), the two products formed first in FP32.
 * Follows GgufKQuantBlocks.cs:99-121. */
static void decode_q4_k(const uint8_t *block, float *y)
{
    float d = half_at(block), dmin = half_at(block + 2);
    const uint8_t *scales = block + 4;
    int out = 0;
    for (int chunk = 0; chunk < 4; ++chunk) {
        const uint8_t *q = block + 16 + chunk * 32;
        int sc1, m1, sc2, m2;
        scale_min_k4(chunk * 2, scales, &sc1, &m1);
        scale_min_k4(chunk * 2 + 1, scales, &sc2, &m2);
        float d1 = d * (float)sc1, mm1 = dmin * (float)m1, d2 = d * (float)sc2, mm2 = dmin * (float)m2;
        for (int l = 0; l < 32; ++l) {
            y[out++] = d1 * (float)(q[l] & 0x0F) - mm1;
        }
        for (int l = 0; l < 32; ++l) {
            y[out++] = d2 * (float)(q[l] >> 4) - mm2;
        }
    }
}

/* Two halves of 128 values; four 6-bit codes share one high-bit byte; value = d * scale * q evaluated
 * left to right. Follows GgufKQuantBlocks.cs:155-177. */
static void decode_q6_k(const uint8_t *block, float *y)
{
    float d = half_at(block + 208);
    for (int half = 0; half < 2; ++half) {
        const uint8_t *ql = block + half * 64;
        const uint8_t *qh = block + 128 + half * 32;
        const int8_t *sc = (const int8_t *)(block + 192 + half * 8);
        float *target = y + half * 128;
        for (int l = 0; l < 32; ++l) {
            int group = l / 16;
            int q1 = ((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
            int q2 = ((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            target[l] = d * (float)sc[group] * (float)q1;
            target[l + 32] = d * (float)sc[group + 2] * (float)q2;
            target[l + 64] = d * (float)sc[group + 4] * (float)q3;
            target[l + 96] = d * (float)sc[group + 6] * (float)q4;
        }
    }
}

static size_t block_values(uint32_t type)
{
    return type == GGML_Q8_0 ? Q8_BLOCK_VALUES : (type == GGML_Q4_K || type == GGML_Q6_K) ? K_SUPER : 0;
}

static size_t block_bytes(uint32_t type)
{
    return type == GGML_Q8_0 ? Q8_BLOCK_BYTES : type == GGML_Q4_K ? Q4K_BYTES : type == GGML_Q6_K ? Q6K_BYTES : 0;
}

/* Bytes of `columns` values, or 0 when the type is unknown or the width is not a whole number of blocks
 * (the reference throws: SourceTensorDecoderTests.cs:165-173). */
size_t orc_row_bytes(uint32_t type, size_t columns)
{
    size_t values = block_values(type);
    if (values == 0 || columns == 0 || columns % values != 0) {
        return 0;
    }
    return columns / values * block_bytes(type);
}

/* Decodes one row of `columns` values. Returns 0, or 2 on an unknown type / ragged width. */
int orc_decode_row(uint32_t type, const uint8_t *row, size_t columns, float *y)
{
    size_t values = block_values(type), bytes = block_bytes(type);
    if (orc_row_bytes(type, columns) == 0) {
        return 2;
    }
    for (size_t b = 0; b < columns / values; ++b) {
        const uint8_t *block = row + b * bytes;
        float *target = y + b * values;
        if (type == GGML_Q8_0) {
            decode_q8_0(block, target);
        } else if (type == GGML_Q4_K) {
            decode_q4_k(block, target);
        } else {
            decode_q6_k(block, target);
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------------ */
/* O5: decoded row x FP32 activations (reference backend for Q4_K / Q6_K)                            */
/* ------------------------------------------------------------------------------------------------ */

/* Decode the row, then sum += w[i] * x[i] for i in index order.
 * Follows src/Synapse.Runtime/Features/GraphExecution/DecodedRowOperators.cs:29-40. */
static float decoded_row_dot(uint32_t type, const uint8_t *row, size_t columns, const float *x, float *scratch)
{
    orc_decode_row(type, row, columns, scratch);
    float sum = 0.0f;
    for (size_t i = 0; i < columns; ++i) {
        sum += scratch[i] * x[i];
    }
    return sum;
}

/* The reference backend's matrix product for one token: Q8_0 takes the per-block path (O3), every other
 * encoding the decode-then-dot path (O5) (Q8Operators.cs:53-57). `x` holds `tokens` rows of `in_stride`
 * floats; y[t*out_stride + r]. The reference runs one token at a time; tokens are independent here. */
int orc_f32_matmul(uint32_t type, const uint8_t *weights, size_t rows, size_t columns, const float *x,
                   size_t tokens, size_t in_stride, float *y, size_t out_stride)
{
    size_t row_bytes = orc_row_bytes(type, columns);
    if (row_bytes == 0 || rows == 0 || tokens == 0) {
        return ORC_SHAPE;
    }
    float *scratch = (float *)malloc(columns * sizeof(float));
    if (!scratch) {
        return ORC_OVERFLOW;
    }
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t *row = weights + r * row_bytes;
        for (size_t t = 0; t < tokens; ++t) {
            const float *xt = x + t * in_stride;
            y[t * out_stride + r] = type == GGML_Q8_0 ? q8_f32_row(row, columns / Q8_BLOCK_VALUES, xt)
                                                      : decoded_row_dot(type, row, columns, xt, scratch);
        }
    }
    free(scratch);
    return ORC_OK;
}

/* FP64 value and sum of |term| of the decoded-weight dot product, any encoding. */
int orc_f32_exact(uint32_t type, const uint8_t *weights, size_t rows, size_t columns, const float *x,
                  size_t tokens, size_t in_stride, double *value, double *magnitude)
{
    size_t row_bytes = orc_row_bytes(type, columns);
    if (row_bytes == 0) {
        return ORC_SHAPE;
    }
    float *scratch = (float *)malloc(columns * sizeof(float));
    if (!scratch) {
        return ORC_OVERFLOW;
    }
    for (size_t r = 0; r < rows; ++r) {
        orc_decode_row(type, weights + r * row_bytes, columns, scratch);
        for (size_t t = 0; t < tokens; ++t) {
            double v = 0.0, m = 0.0;
            for (size_t i = 0; i < columns; ++i) {
                double term = (double)scratch[i] * (double)x[t * in_stride + i];
                v += term;
                m += fabs(term);
            }
            value[t * rows + r] = v;
            magnitude[t * rows + r] = m;
        }
    }
    free(scratch);
    return ORC_OK;
}

/* ------------------------------------------------------------------------------------------------ */
/* O6: K-quant weights x Q8_0-quantised activations (declared contract, no reference counterpart)    */
/* ------------------------------------------------------------------------------------------------ */

/* Integer sums of one Q4_K super-block against one token's codes: for each of the 8 sub-blocks of 32 the
 * dot of the 4-bit codes with the activation codes. dots[8]. Layout as in decode_q4_k. */
static void q4k_block_int(const uint8_t *block, const int8_t *a, int32_t *dots)
{
    for (int chunk = 0; chunk < 4; ++chunk) {
        const uint8_t *q = block + 16 + chunk * 32;
        int32_t lo = 0, hi = 0;
        for (int l = 0; l < 32; ++l) {
            lo += (int32_t)(q[l] & 0x0F) * a[chunk * 64 + l];
            hi += (int32_t)(q[l] >> 4) * a[chunk * 64 + 32 + l];
        }
        dots[chunk * 2] = lo;
        dots[chunk * 2 + 1] = hi;
    }
}

/* Integer sums of one Q6_K super-block: for each of the 16 groups of 16 values the dot of (q - 32) with
 * the activation codes. dots[16], group g covers values 16g..16g+15. Layout as in decode_q6_k. */
static void q6k_block_int(const uint8_t *block, const int8_t *a, int32_t *dots)
{
    for (int g = 0; g < 16; ++g) {
        dots[g] = 0;
    }
    for (int half = 0; half < 2; ++half) {
        const uint8_t *ql = block + half * 64;
        const uint8_t *qh = block + 128 + half * 32;
        const int8_t *ah = a + half * 128;
        for (int l = 0; l < 32; ++l) {
            int group = half * 8 + l / 16;
            int q1 = ((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
            int q2 = ((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            dots[group] += q1 * ah[l];
            dots[group + 2] += q2 * ah[l + 32];
            dots[group + 4] += q3 * ah[l + 64];
            dots[group + 6] += q4 * ah[l + 96];
        }
    }
}

/* The exact integer sub-block dots of O6: Q4_K writes 8 per super-block, Q6_K 16 per super-block, Q8_0 one
 * per block; out[((t*rows + r)*groups_per_row) + g]. Returns groups per row, or 0 on a bad shape. */
size_t orc_int_dots(uint32_t type, const uint8_t *weights, size_t rows, size_t columns, const int8_t *quants,
                    size_t tokens, int32_t *out)
{
    size_t row_bytes = orc_row_bytes(type, columns);
    if (row_bytes == 0) {
        return 0;
    }
    size_t per_block = type == GGML_Q8_0 ? 1 : type == GGML_Q4_K ? 8 : 16;
    size_t blocks = columns / block_values(type);
    size_t groups = blocks * per_block;
    for (size_t t = 0; t < tokens; ++t) {
        for (size_t r = 0; r < rows; ++r) {
            int32_t *target = out + (t * rows + r) * groups;
            for (size_t b = 0; b < blocks; ++b) {
                const uint8_t *block = weights + r * row_bytes + b * block_bytes(type);
                const int8_t *a = quants + t * columns + b * block_values(type);
                if (type == GGML_Q8_0) {
                    target[b] = q8_block_dot(block, a);
                } else if (type == GGML_Q4_K) {
                    q4k_block_int(block, a, target + b * 8);
                } else {
                    q6k_block_int(block, a, target + b * 16);
                }
            }
        }
    }
    return groups;
}

/* O6 result. Q4_K, per sub-block j with activation block scale da and code sum asum:
 *   sum = fma((d*sc_j) * da, (float)dot_j, sum); sum = fma(-((dmin*m_j) * da), (float)asum_j, sum)
 * Q6_K, per group g of 16 inside activation block g/2:
 *   sum = fma((d*(float)sc_g) * da, (float)dot_g, sum)
 * Q8_0: identical to O2. Groups in index order, FP32 throughout. */
int orc_kq_q8_matmul(uint32_t type, const uint8_t *weights, size_t rows, size_t columns, const int8_t *quants,
                     const float *scales, size_t tokens, float *output, size_t stride)
{
    size_t row_bytes = orc_row_bytes(type, columns);
    if (row_bytes == 0 || rows == 0 || tokens == 0 || (tokens > 1 && stride < rows)) {
        return ORC_SHAPE;
    }
    if (type == GGML_Q8_0) {
        return orc_q8q8_matmul(weights, row_bytes, rows, columns / 32, quants, scales, tokens, output, stride);
    }
    size_t blocks = columns / K_SUPER;
    for (size_t r = 0; r < rows; ++r) {
        for (size_t t = 0; t < tokens; ++t) {
            const int8_t *a = quants + t * columns;
            const float *da = scales + t * (columns / 32);
            float sum = 0.0f;
            for (size_t b = 0; b < blocks; ++b) {
                const uint8_t *block = weights + r * row_bytes + b * block_bytes(type);
                const int8_t *ab = a + b * K_SUPER;
                if (type == GGML_Q4_K) {
                    int32_t dots[8];
                    q4k_block_int(block, ab, dots);
                    float d = half_at(block), dmin = half_at(block + 2);
                    for (int j = 0; j < 8; ++j) {
                        int sc, m, asum = 0;
                        scale_min_k4(j, block + 4, &sc, &m);
                        for (int l = 0; l < 32; ++l) {
                            asum += ab[j * 32 + l];
                        }
                        float s = da[b * 8 + j];
                        sum = fmaf((d * (float)sc) * s, (float)dots[j], sum);
                        sum = fmaf(-((dmin * (float)m) * s), (float)asum, sum);
                    }
                } else {
                    int32_t dots[16];
                    q6k_block_int(block, ab, dots);
                    float d = half_at(block + 208);
                    const int8_t *sc = (const int8_t *)(block + 192);
                    for (int g = 0; g < 16; ++g) {
                        sum = fmaf((d * (float)sc[g]) * da[b * 8 + g / 2], (float)dots[g], sum);
                    }
                }
            }
            output[t * stride + r] = sum;
        }
    }
    return ORC_OK;
}

/* FP64 value and sum of |term| of O6 (weights decoded exactly, activations = code * stored scale). */
int orc_kq_q8_exact(uint32_t type, const uint8_t *weights, size_t rows, size_t columns, const int8_t *quants,
                    const float *scales, size_t tokens, double *value, double *magnitude)
{
    size_t row_bytes = orc_row_bytes(type, columns);
    if (row_bytes == 0) {
        return ORC_SHAPE;
    }
    float *scratch = (float *)malloc(columns * sizeof(float));
    if (!scratch) {
        return ORC_OVERFLOW;
    }
    for (size_t r = 0; r < rows; ++r) {
        orc_decode_row(type, weights + r * row_bytes, columns, scratch);
        for (size_t t = 0; t < tokens; ++t) {
            double v = 0.0, m = 0.0;
            for (size_t i = 0; i < columns; ++i) {
                double term = (double)scratch[i] * (double)quants[t * columns + i] *
                              (double)scales[t * (columns / 32) + i / 32];
                v += term;
                m += fabs(term);
            }
            value[t * rows + r] = v;
            magnitude[t * rows + r] = m;
        }
    }
    free(scratch);
    return ORC_OK;
}

/* ------------------------------------------------------------------------------------------------ */
/* Row-chunked thread pool: the reference's intra-op parallelism, for the timed CPU baseline          */
/* ------------------------------------------------------------------------------------------------ */

/* Chunk size rule of ChunkedRowWork (src/Synapse.Runtime/Features/CpuKernels/ChunkedRowWork.cs:41-64):
 * target = threads * 2 chunks, chunk rows = clamp(ceil(rows / target), 16, 4096) rounded up to a multiple
 * of 4; chunks are claimed from an atomic counter. */
size_t orc_chunk_rows(size_t rows, size_t threads)
{
    size_t target = threads * 2;
    size_t chunk = (rows + target - 1) / target;
    if (chunk < 16) {
        chunk = 16;
    }
    if (chunk > 4096) {
        chunk = 4096;
    }
    return (chunk + 3) & ~(size_t)3;
}

typedef struct {
    int kind; /* 0 = q8q8 (AVX2 when available, else scalar), 1 = f32 decoded / Q8_0 reference */
    uint32_t type;
    const uint8_t *weights;
    size_t rows, columns, row_bytes, tokens, in_stride, out_stride, chunk_rows;
    const int8_t *quants;
    const float *scales;
    const float *x;
    float *output;
    atomic_size_t next;
} job_t;

static void *job_worker(void *arg)
{
    job_t *job = (job_t *)arg;
    float *scratch = job->kind == 1 ? (float *)malloc(job->columns * sizeof(float)) : NULL;
    for (;;) {
        size_t start = atomic_fetch_add(&job->next, job->chunk_rows);
        if (start >= job->rows) {
            break;
        }
        size_t count = job->rows - start < job->chunk_rows ? job->rows - start : job->chunk_rows;
        const uint8_t *w = job->weights + start * job->row_bytes;
        if (job->kind == 0) {
#if ORC_HAVE_AVX2
            if (orc_have_avx2()) {
                q8q8_avx2_rows(w, count, job->columns / 32, job->quants, job->scales, job->tokens,
                               job->output + start, job->out_stride);
                continue;
            }
#endif
            orc_q8q8_matmul(w, job->row_bytes, count, job->columns / 32, job->quants, job->scales,
                            job->tokens, job->output + start, job->out_stride);
        } else {
            for (size_t r = 0; r < count; ++r) {
                for (size_t t = 0; t < job->tokens; ++t) {
                    const float *xt = job->x + t * job->in_stride;
                    job->output[t * job->out_stride + start + r] =
                        job->type == GGML_Q8_0
                            ? q8_f32_row(w + r * job->row_bytes, job->columns / 32, xt)
                            : decoded_row_dot(job->type, w + r * job->row_bytes, job->columns, xt, scratch);
                }
            }
        }
    }
    free(scratch);
    return NULL;
}

static int run_job(job_t *job, size_t threads)
{
    if (threads == 0) {
        threads = 1;
    }
    job->chunk_rows = orc_chunk_rows(job->rows, threads);
    atomic_init(&job->next, 0);
    pthread_t *ids = (pthread_t *)malloc(threads * sizeof(pthread_t));
    if (!ids) {
        return ORC_OVERFLOW;
    }
    size_t started = 0;
    for (; started + 1 < threads; ++started) {
        if (pthread_create(&ids[started], NULL, job_worker, job) != 0) {
            break;
        }
    }
    job_worker(job); /* the caller takes part, as in CpuWorkerPool.Run */
    for (size_t i = 0; i < started; ++i) {
        pthread_join(ids[i], NULL);
    }
    free(ids);
    return ORC_OK;
}

/* The `native` CPU backend's matmul over all rows: quantised activations in, row chunks over `threads`
 * threads, AVX2+FMA body where the CPU has it. This is the timed CPU baseline for Q8_0. */
int orc_q8q8_matmul_threads(const uint8_t *weights, size_t rows, size_t blocks, const int8_t *quants,
                            const float *scales, size_t tokens, float *output, size_t stride, size_t threads)
{
    int status = q8q8_validate(weights, blocks * Q8_BLOCK_BYTES, rows, blocks, quants, scales, tokens, output,
                               stride);
    if (status != ORC_OK) {
        return status;
    }
    job_t job;
    memset(&job, 0, sizeof job);
    job.kind = 0;
    job.weights = weights;
    job.rows = rows;
    job.columns = blocks * 32;
    job.row_bytes = blocks * Q8_BLOCK_BYTES;
    job.tokens = tokens;
    job.quants = quants;
    job.scales = scales;
    job.output = output;
    job.out_stride = stride;
    return run_job(&job, threads);
}

/* The `reference` CPU backend's matmul (the only CPU path that accepts Q4_K / Q6_K), rows in parallel as its
 * Parallel.For does (DecodedRowOperators.cs:29; Q8Operators.cs:73). Timed CPU baseline for the K-quants. */
int orc_f32_matmul_threads(uint32_t type, const uint8_t *weights, size_t rows, size_t columns, const float *x,
                           size_t tokens, size_t in_stride, float *y, size_t out_stride, size_t threads)
{
    size_t row_bytes = orc_row_bytes(type, columns);
    if (row_bytes == 0 || rows == 0 || tokens == 0) {
        return ORC_SHAPE;
    }
    job_t job;
    memset(&job, 0, sizeof job);
    job.kind = 1;
    job.type = type;
    job.weights = weights;
    job.rows = rows;
    job.columns = columns;
    job.row_bytes = row_bytes;
    job.tokens = tokens;
    job.x = x;
    job.in_stride = in_stride;
    job.output = y;
    job.out_stride = out_stride;
    return run_job(&job, threads);
}

/* ------------------------------------------------------------------------------------------------ */
/* The reference tests' linear congruential generator                                                */
/* ------------------------------------------------------------------------------------------------ */

/* Builds the Q8_0 x Q8_0 case of q8_0_tests.rs:36-62 from its seed: weights (rows*blocks blocks, fp16 scale
 * bits 0x1000 + next % 0x1400, codes next % 255 - 127), then activation codes, then activation scales
 * (fp16 bits 0x2000 + next % 0x1000 widened to float). state = state * 6364136223846793005 +
 * 1442695040888963407; next = state >> 33 (q8_0_tests.rs:9-23). */
void orc_lcg_case(uint64_t seed, size_t rows, size_t blocks, size_t tokens, uint8_t *weights, int8_t *quants,
                  float *scales)
{
    uint64_t state = seed;
#define LCG_NEXT() (state = state * 6364136223846793005ull + 1442695040888963407ull, (uint32_t)(state >> 33))
    for (size_t b = 0; b < rows * blocks; ++b) {
        uint16_t bits = (uint16_t)(0x1000u + LCG_NEXT() % 0x1400u);
        uint8_t *block = weights + b * Q8_BLOCK_BYTES;
        block[0] = (uint8_t)(bits & 0xff);
        block[1] = (uint8_t)(bits >> 8);
        for (int i = 0; i < Q8_BLOCK_VALUES; ++i) {
            block[2 + i] = (uint8_t)(int8_t)((int64_t)(LCG_NEXT() % 255u) - 127);
        }
    }
    for (size_t i = 0; i < tokens * blocks * Q8_BLOCK_VALUES; ++i) {
        quants[i] = (int8_t)((int64_t)(LCG_NEXT() % 255u) - 127);
    }
    for (size_t i = 0; i < tokens * blocks; ++i) {
        scales[i] = orc_fp16_to_f32((uint16_t)(0x2000u + LCG_NEXT() % 0x1000u));
    }
#undef LCG_NEXT
}

/* ------------------------------------------------------------------------------------------------ */
/* O8: the decode step of the optimized CPU executor (Q8_0-quantised activations everywhere)          */
/* ------------------------------------------------------------------------------------------------ */

#define ORC_NO_TENSOR 0xFFFFFFFFFFFFFFFFull

/* Same field order and sizes as DecoderLayerOffsets (native/synapse-gpu/src/Features/GpuKernels/decoder.rs:61-93). */
typedef struct {
    uint64_t attention_norm, query, key, value, query_bias, key_bias, value_bias, query_norm, key_norm;
    uint64_t attention_output, feed_forward_norm, gate, up, down, encodings;
} orc_layer_offsets;

/* Same field order and sizes as DecoderDesc (decoder.rs:96-131). */
typedef struct {
    const uint8_t *weights;
    uint64_t weights_length;
    const orc_layer_offsets *layers;
    const float *rope_cosines, *rope_sines;
    uint64_t token_embedding, output_norm, output;
    uint32_t layer_count, hidden, feed_forward, heads, kv_heads, head_dim, vocabulary, context, session_slots;
    uint32_t step_tokens, logits_rows;
    float rms_epsilon;
    uint32_t embedding_encoding, rope_layout, activation, kv_precision, kv_growth_positions, output_encoding;
} orc_decoder_desc;

typedef struct {
    orc_decoder_desc desc;
    float *keys, *values; /* [slot][layer][kv_head][position][head_dim] */
    size_t threads;
} orc_decoder;

static uint32_t layer_encoding(const orc_layer_offsets *layer, int matrix)
{
    return (uint32_t)((layer->encodings >> (4 * matrix)) & 0xF);
}

/* RMSNorm with an FP64 sum of squares (GraphExecution/Q8Operators.cs:101-123). */
static void rms_norm(const float *x, const float *w, float epsilon, size_t n, float *out)
{
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) {
        sum += (double)x[i] * x[i];
    }
    float scale = 1.0f / sqrtf((float)(sum / (double)n) + epsilon);
    for (size_t i = 0; i < n; ++i) {
        out[i] = x[i] * scale * w[i];
    }
}

/* The pieces of the step, exported so that the reference's own operator vectors can be replayed against them
 * (ReferenceOperatorsTests.cs:105-164, RopeFrequenciesTests.cs:13-34). */
void orc_rms_norm(const float *x, const float *w, float epsilon, size_t n, float *out) { rms_norm(x, w, epsilon, n, out); }

/* NeoX rotation of one head: element i against element i + head_dim/2 (Qwen2CpuState.cs:85-105). */
void orc_rotate_neox(float *x, size_t head_dim, const float *cosines, const float *sines)
{
    const size_t half = head_dim / 2;
    for (size_t i = 0; i < half; ++i) {
        float a = x[i], b = x[i + half];
        x[i] = a * cosines[i] - b * sines[i];
        x[i + half] = a * sines[i] + b * cosines[i];
    }
}

/* SwiGLU: silu(gate) * up (Qwen2CpuExecutor.cs:189-196). */
void orc_swiglu(const float *gate, const float *up, size_t n, float *out)
{
    for (size_t i = 0; i < n; ++i) {
        float value = gate[i];
        out[i] = value / (1.0f + expf(-value)) * up[i];
    }
}

/* Max-subtracted softmax in place; returns nothing, scores[p] become the weights (Qwen2CpuAttention.cs:120-150). */
void orc_softmax(float *scores, size_t n)
{
    float maximum = -INFINITY;
    for (size_t p = 0; p < n; ++p) {
        maximum = fmaxf(maximum, scores[p]);
    }
    float sum = 0.0f;
    for (size_t p = 0; p < n; ++p) {
        scores[p] = expf(scores[p] - maximum);
        sum += scores[p];
    }
    const float inverse = 1.0f / sum;
    for (size_t p = 0; p < n; ++p) {
        scores[p] *= inverse;
    }
}

/* One quantised-activation product over all rows with the contract of the matching encoding (O2 / O6); large
 * matrices are split into row ranges over threads, which does not change any row's arithmetic. */
typedef struct {
    uint32_t type;
    const uint8_t *weights;
    size_t rows, columns;
    const int8_t *codes;
    const float *scales;
    float *out;
} matmul_slice;

static void *matmul_slice_run(void *arg)
{
    matmul_slice *m = (matmul_slice *)arg;
    orc_kq_q8_matmul(m->type, m->weights, m->rows, m->columns, m->codes, m->scales, 1, m->out, m->rows);
    return NULL;
}

static void decoder_matmul(const orc_decoder *d, uint32_t type, uint64_t offset, size_t rows, size_t columns, const int8_t *codes,
                           const float *scales, float *out)
{
    size_t threads = d->threads;
    if (rows * columns < (1u << 22) || threads < 2) {
        orc_kq_q8_matmul(type, d->desc.weights + offset, rows, columns, codes, scales, 1, out, rows);
        return;
    }
    if (threads > 64) {
        threads = 64;
    }
    pthread_t ids[64];
    matmul_slice slices[64];
    size_t row_bytes = orc_row_bytes(type, columns), per = (rows + threads - 1) / threads, started = 0;
    for (size_t t = 0; t < threads; ++t) {
        size_t first = t * per;
        if (first >= rows) {
            break;
        }
        slices[t] = (matmul_slice){type, d->desc.weights + offset + first * row_bytes, rows - first < per ? rows - first : per, columns, codes,
                                   scales, out + first};
        if (pthread_create(&ids[t], NULL, matmul_slice_run, &slices[t]) != 0) {
            matmul_slice_run(&slices[t]);
            ids[t] = 0;
        }
        started = t + 1;
    }
    for (size_t t = 0; t < started; ++t) {
        if (ids[t]) {
            pthread_join(ids[t], NULL);
        }
    }
}

orc_decoder *orc_decoder_create(const orc_decoder_desc *desc, size_t threads)
{
    orc_decoder *d = (orc_decoder *)calloc(1, sizeof *d);
    if (!d) {
        return NULL;
    }
    d->desc = *desc;
    d->threads = threads ? threads : 1;
    size_t cache = (size_t)desc->session_slots * desc->layer_count * desc->kv_heads * desc->context * desc->head_dim;
    d->keys = (float *)calloc(cache, sizeof(float));
    d->values = (float *)calloc(cache, sizeof(float));
    if (!d->keys || !d->values) {
        free(d->keys);
        free(d->values);
        free(d);
        return NULL;
    }
    return d;
}

void orc_decoder_destroy(orc_decoder *d)
{
    if (d) {
        free(d->keys);
        free(d->values);
        free(d);
    }
}

static size_t kv_index(const orc_decoder_desc *s, uint32_t slot, uint32_t layer, uint32_t kv_head, uint32_t position)
{
    return ((((size_t)slot * s->layer_count + layer) * s->kv_heads + kv_head) * s->context + position) * s->head_dim;
}

/* One token through the whole decoder: embedding row, per layer {RMSNorm -> quantise -> Q/K/V + bias -> NeoX RoPE ->
 * KV store -> softmax attention over the slot's cache -> quantise -> output projection + residual -> RMSNorm ->
 * quantise -> gate/up -> SwiGLU -> quantise -> down + residual}, output norm, quantise, vocabulary projection.
 * Follows Qwen2/Qwen2CpuExecutor.cs:105-244, Qwen2ProjectionWork.cs:7-157, Qwen2CpuState.cs:85-105 (RoPE),
 * Qwen2CpuAttention.cs:82-173. Returns 0, or 2 on an invalid token. logits holds `vocabulary` floats. */
int orc_decoder_forward(orc_decoder *d, int32_t slot, int32_t token, int32_t position, float *logits)
{
    const orc_decoder_desc *s = &d->desc;
    if (slot < 0 || (uint32_t)slot >= s->session_slots || token < 0 || (uint32_t)token >= s->vocabulary || position < 0 ||
        (uint32_t)position >= s->context) {
        return 2;
    }
    const size_t hidden = s->hidden, ffn = s->feed_forward, kvw = (size_t)s->kv_heads * s->head_dim, half = s->head_dim / 2;
    float *h = (float *)malloc(sizeof(float) * (hidden * 4 + kvw * 2 + ffn * 3 + s->context));
    if (!h) {
        return 3;
    }
    float *normed = h + hidden, *q = normed + hidden, *attn = q + hidden, *k = attn + hidden, *v = k + kvw, *gate = v + kvw,
          *up = gate + ffn, *ff = up + ffn, *scores = ff + ffn;
    size_t widest = hidden > ffn ? hidden : ffn;
    int8_t *codes = (int8_t *)malloc(widest);
    float *scales = (float *)malloc(sizeof(float) * (widest / 32));
    orc_decode_row(s->embedding_encoding, s->weights + s->token_embedding + (size_t)token * orc_row_bytes(s->embedding_encoding, hidden),
                   hidden, h);
    const float *cosines = s->rope_cosines + (size_t)position * half, *sines = s->rope_sines + (size_t)position * half;
    const float attention_scale = 1.0f / sqrtf((float)s->head_dim);
    for (uint32_t l = 0; l < s->layer_count; ++l) {
        const orc_layer_offsets *L = &s->layers[l];
        rms_norm(h, (const float *)(s->weights + L->attention_norm), s->rms_epsilon, hidden, normed);
        orc_q8_quantize_row(normed, hidden, codes, scales);
        decoder_matmul(d, layer_encoding(L, 0), L->query, hidden, hidden, codes, scales, q);
        decoder_matmul(d, layer_encoding(L, 1), L->key, kvw, hidden, codes, scales, k);
        decoder_matmul(d, layer_encoding(L, 2), L->value, kvw, hidden, codes, scales, v);
        if (L->query_bias != ORC_NO_TENSOR) {
            const float *bq = (const float *)(s->weights + L->query_bias), *bk = (const float *)(s->weights + L->key_bias),
                        *bv = (const float *)(s->weights + L->value_bias);
            for (size_t i = 0; i < hidden; ++i) q[i] += bq[i];
            for (size_t i = 0; i < kvw; ++i) k[i] += bk[i];
            for (size_t i = 0; i < kvw; ++i) v[i] += bv[i];
        }
        for (uint32_t head = 0; head < s->heads + s->kv_heads; ++head) {
            float *x = head < s->heads ? q + (size_t)head * s->head_dim : k + (size_t)(head - s->heads) * s->head_dim;
            orc_rotate_neox(x, s->head_dim, cosines, sines);
        }
        if (s->kv_precision == 1) {
            /* KvPrecision::F16 (native/synapse-gpu/src/Features/GpuKernels/decoder.rs:43-58): the cache holds the nearest
             * fp16 number of every rotated key and value, and attention -- the current position included -- reads the
             * cache. The CPU executor has no such mode: this branch is this backend's statement of it, not a restatement. */
            for (size_t i = 0; i < kvw; ++i) {
                k[i] = orc_fp16_to_f32(orc_f32_to_fp16(k[i]));
                v[i] = orc_fp16_to_f32(orc_f32_to_fp16(v[i]));
            }
        }
        for (uint32_t kh = 0; kh < s->kv_heads; ++kh) {
            memcpy(d->keys + kv_index(s, (uint32_t)slot, l, kh, (uint32_t)position), k + (size_t)kh * s->head_dim, sizeof(float) * s->head_dim);
            memcpy(d->values + kv_index(s, (uint32_t)slot, l, kh, (uint32_t)position), v + (size_t)kh * s->head_dim, sizeof(float) * s->head_dim);
        }
        const uint32_t group = s->heads / s->kv_heads;
        for (uint32_t head = 0; head < s->heads; ++head) {
            const float *qh = q + (size_t)head * s->head_dim;
            const uint32_t kh = head / group;
            for (int32_t p = 0; p <= position; ++p) {
                const float *kp = d->keys + kv_index(s, (uint32_t)slot, l, kh, (uint32_t)p);
                float dot = 0.0f;
                for (uint32_t i = 0; i < s->head_dim; ++i) dot += qh[i] * kp[i];
                scores[p] = dot * attention_scale;
            }
            orc_softmax(scores, (size_t)position + 1);
            float *out = attn + (size_t)head * s->head_dim;
            for (uint32_t i = 0; i < s->head_dim; ++i) out[i] = 0.0f;
            for (int32_t p = 0; p <= position; ++p) {
                const float *vp = d->values + kv_index(s, (uint32_t)slot, l, kh, (uint32_t)p);
                const float weight = scores[p];
                for (uint32_t i = 0; i < s->head_dim; ++i) out[i] += weight * vp[i];
            }
        }
        orc_q8_quantize_row(attn, hidden, codes, scales);
        decoder_matmul(d, layer_encoding(L, 3), L->attention_output, hidden, hidden, codes, scales, normed);
        for (size_t i = 0; i < hidden; ++i) h[i] += normed[i];
        rms_norm(h, (const float *)(s->weights + L->feed_forward_norm), s->rms_epsilon, hidden, normed);
        orc_q8_quantize_row(normed, hidden, codes, scales);
        decoder_matmul(d, layer_encoding(L, 4), L->gate, ffn, hidden, codes, scales, gate);
        decoder_matmul(d, layer_encoding(L, 5), L->up, ffn, hidden, codes, scales, up);
        orc_swiglu(gate, up, ffn, ff);
        orc_q8_quantize_row(ff, ffn, codes, scales);
        decoder_matmul(d, layer_encoding(L, 6), L->down, hidden, ffn, codes, scales, normed);
        for (size_t i = 0; i < hidden; ++i) h[i] += normed[i];
    }
    rms_norm(h, (const float *)(s->weights + s->output_norm), s->rms_epsilon, hidden, normed);
    orc_q8_quantize_row(normed, hidden, codes, scales);
    decoder_matmul(d, s->output_encoding, s->output, s->vocabulary, hidden, codes, scales, logits);
    free(codes);
    free(scales);
    free(h);
    return 0;
}

/* First maximum (GraphExecution/Q8Operators.cs:152-173). */
int32_t orc_argmax(const float *values, size_t count)
{
    size_t best = 0;
    for (size_t i = 1; i < count; ++i) {
        if (values[i] > values[best]) {
            best = i;
        }
    }
    return (int32_t)best;
}
