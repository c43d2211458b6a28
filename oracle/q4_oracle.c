/*
 * CPU oracle for the affine-Q4 matmul path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the scalar CPU formulas that the reference
 * (baryhuang/cpu-llms-in-c) keeps beside its Metal kernels; each function
 * names the reference lines it follows.  Nothing here is part of the shipped
 * library: it checks the CUDA path and supplies the timed CPU baseline.
 *
 * Parity pin: the conversion helpers, the metadata transform and the fused
 * gate/up and whole-MLP first-8-row values are checked bit-for-bit against the
 * reference's own packer code compiled from its sources (oracle/ref_shim.c),
 * and against vectors that build produced (tests/golden/).
 *
 * Build: gcc -O3 -std=c11 -fopenmp (ISO mode keeps fp contraction off, so the
 * fp32 sums below round exactly as written).
 */
#define _POSIX_C_SOURCE 200809L
#include "q4_oracle.h"

#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ */
/* conversions                                                         */
/* ------------------------------------------------------------------ */

/* Round a finite double to the nearest fp16 (ties to even) in one step.
 * The value is scaled by an exact power of two so that one fp16 ulp is 1.0,
 * rounded with nearbyint (default mode: to nearest even), then re-assembled. */
uint16_t q4o_f64_to_f16(double value) {
    uint16_t sign = signbit(value) ? 0x8000u : 0u;
    if (isnan(value)) {
        return (uint16_t)(sign | 0x7e00u);
    }
    double magnitude = fabs(value);
    if (magnitude >= 65520.0) { /* halfway to 2^16 rounds to infinity */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (magnitude == 0.0) {
        return sign;
    }
    int exponent;
    (void)frexp(magnitude, &exponent); /* magnitude = f * 2^exponent, f in [0.5,1) */
    int unbiased = exponent - 1;       /* floor(log2(magnitude)) */
    if (unbiased < -14) {
        unbiased = -14; /* subnormal range shares the quantum of 2^-14 */
    }
    double scaled = ldexp(magnitude, 10 - unbiased); /* ulp == 1.0 */
    uint32_t integer = (uint32_t)nearbyint(scaled);  /* 0 .. 2048 */
    if (integer >= 2048u) {
        integer = 1024u;
        ++unbiased;
    }
    if (integer < 1024u) { /* subnormal (or rounded up to the first normal) */
        return (uint16_t)(sign | integer);
    }
    if (unbiased > 15) {
        return (uint16_t)(sign | 0x7c00u);
    }
    return (uint16_t)(sign | (uint32_t)(unbiased + 15) << 10 | (integer - 1024u));
}

uint16_t q4o_f32_to_f16(float value) {
    return q4o_f64_to_f16((double)value); /* float -> double is exact */
}

float q4o_f16_to_f32(uint16_t bits) {
    uint32_t exponent = (bits >> 10) & 0x1fu;
    uint32_t mantissa = bits & 0x3ffu;
    float magnitude;
    if (exponent == 0u) {
        magnitude = ldexpf((float)mantissa, -24);
    } else if (exponent == 31u) {
        magnitude = mantissa != 0u ? NAN : INFINITY;
    } else {
        magnitude = ldexpf((float)(mantissa | 0x400u), (int)exponent - 25);
    }
    return (bits & 0x8000u) != 0u ? -magnitude : magnitude;
}

uint16_t q4o_f32_to_bf16(float value) {
    /* benchmarks/minimax_h3_m3_real_gemm.c:18-23 (round to nearest even) */
    uint32_t bits;
    memcpy(&bits, &value, sizeof(bits));
    if ((bits & 0x7f800000u) == 0x7f800000u && (bits & 0x7fffffu) != 0u) {
        return (uint16_t)((bits >> 16) | 0x40u);
    }
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

float q4o_bf16_to_f32(uint16_t bits) {
    uint32_t wide = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &wide, sizeof(value));
    return value;
}

uint16_t q4o_bf16_to_f16(uint16_t bits) {
    /* qwen38_m3_pack.c:173-178: widen to f32, round once to fp16 */
    return q4o_f32_to_f16(q4o_bf16_to_f32(bits));
}

void q4o_round_f16(const float *in, uint16_t *out, size_t count) {
    for (size_t index = 0; index < count; ++index) {
        out[index] = q4o_f32_to_f16(in[index]);
    }
}

int q4o_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ */
/* seeded synthetic inputs                                             */
/* ------------------------------------------------------------------ */

#define Q4O_GOLDEN UINT64_C(0x9E3779B97F4A7C15)

static uint64_t finalize64(uint64_t z) {
    z = (z ^ (z >> 30)) * UINT64_C(0xBF58476D1CE4E5B9);
    z = (z ^ (z >> 27)) * UINT64_C(0x94D049BB133111EB);
    return z ^ (z >> 31);
}

static uint64_t stream_key(uint64_t seed, uint64_t stream) {
    return finalize64(seed * Q4O_GOLDEN + finalize64(stream + 1u));
}

static uint64_t keyed(uint64_t key, uint64_t index) {
    return finalize64(key + (index + 1u) * Q4O_GOLDEN);
}

uint64_t q4o_hash(uint64_t seed, uint64_t stream, uint64_t index) {
    return keyed(stream_key(seed, stream), index);
}

/* Twelve 16-bit uniforms summed: mean 393210, variance 65536^2 (to 1e-9), so
 * (sum - 393210) / 65536 is the classic 12-uniform approximation of N(0,1).
 * Integer arithmetic only, hence identical on every machine. */
static float normal12(uint64_t a, uint64_t b, uint64_t c) {
    uint32_t sum = 0;
    for (int part = 0; part < 4; ++part) {
        sum += (uint32_t)((a >> (16 * part)) & 0xffffu);
        sum += (uint32_t)((b >> (16 * part)) & 0xffffu);
        sum += (uint32_t)((c >> (16 * part)) & 0xffffu);
    }
    return (float)((int32_t)sum - 393210) * (1.0f / 65536.0f);
}

void q4o_synth_codes(uint64_t seed, uint64_t stream, uint32_t *words,
                     size_t word_begin, size_t word_count) {
    uint64_t key = stream_key(seed, stream);
    for (size_t offset = 0; offset < word_count; ++offset) {
        size_t word = word_begin + offset;
        uint64_t bits = keyed(key, word >> 1);
        words[offset] = (uint32_t)(bits >> (32u * (word & 1u)));
    }
}

void q4o_synth_meta(uint64_t seed, uint64_t stream, uint16_t *meta,
                    size_t group_begin, size_t group_count) {
    uint64_t key = stream_key(seed, stream);
    for (size_t offset = 0; offset < group_count; ++offset) {
        uint64_t group = group_begin + offset;
        float uniform = (float)(keyed(key, 4u * group) >> 40) * (1.0f / 16777216.0f);
        /* scale ~ U[5e-4, 4e-3], one fused rounding, then fp16 */
        uint16_t scale = q4o_f32_to_f16(fmaf(uniform, 3.5e-3f, 5.0e-4f));
        float noise = normal12(keyed(key, 4u * group + 1u),
                               keyed(key, 4u * group + 2u),
                               keyed(key, 4u * group + 3u));
        /* bias = -8*scale + N(0, 1e-3); -8*scale is exact */
        float bias = fmaf(noise, 1.0e-3f, -8.0f * q4o_f16_to_f32(scale));
        meta[2 * offset] = scale;
        meta[2 * offset + 1] = q4o_f32_to_f16(bias);
    }
}

void q4o_synth_x(uint64_t seed, uint64_t stream, uint16_t *x_f16, size_t begin,
                 size_t count) {
    uint64_t key = stream_key(seed, stream);
    for (size_t offset = 0; offset < count; ++offset) {
        uint64_t index = begin + offset;
        x_f16[offset] = q4o_f32_to_f16(normal12(keyed(key, 3u * index),
                                                keyed(key, 3u * index + 1u),
                                                keyed(key, 3u * index + 2u)));
    }
}

/* ------------------------------------------------------------------ */
/* the reference's closed-form fixtures                                */
/* ------------------------------------------------------------------ */

static uint32_t xorshift32(uint32_t *state) {
    /* qwen38_m3.m:56-63 */
    uint32_t value = *state;
    value ^= value << 13;
    value ^= value >> 17;
    value ^= value << 5;
    *state = value;
    return value;
}

void q4o_fill_weights_xorshift(uint8_t *quants, uint16_t *meta,
                               size_t group_count, uint32_t seed) {
    /* qwen38_m3.m:64-87: 32 random bytes, then scale from 3 random bits and a
     * bias that depends on the group index */
    uint32_t state = seed;
    for (size_t group = 0; group < group_count; ++group) {
        for (size_t byte = 0; byte < 32; ++byte) {
            quants[group * 32 + byte] = (uint8_t)xorshift32(&state);
        }
        float scale = 0.0035f + 0.00025f * (float)(xorshift32(&state) & 7u);
        float bias = -7.5f * scale + 0.0002f * (float)((int)(group % 5) - 2);
        meta[2 * group] = q4o_f32_to_f16(scale);
        meta[2 * group + 1] = q4o_f32_to_f16(bias);
    }
}

void q4o_activation_sincos(uint16_t *x_f16, size_t count) {
    /* qwen38_m3.m:568-573; qwen38_m3_pack.c:228-231 */
    for (size_t index = 0; index < count; ++index) {
        float value = 0.75f * sinf((float)index * 0.013f) +
                      0.20f * cosf((float)index * 0.031f);
        x_f16[index] = q4o_f32_to_f16(value);
    }
}

void q4o_h3_pattern(uint8_t *quants, uint16_t *meta, size_t rows,
                    size_t groups_per_row, uint16_t *x_f16, size_t x_count,
                    uint32_t input_seed) {
    /* minimax_h3_m3_gemm.m:75-104: bytes, scale and bias are arithmetic
     * functions of the byte / block index */
    size_t blocks = rows * groups_per_row;
    for (size_t block = 0; block < blocks; ++block) {
        for (size_t byte = 0; byte < 32; ++byte) {
            uint32_t index = (uint32_t)(block * 32 + byte);
            uint32_t low = (index * 5u + (index >> 5) * 3u + 3u) & 15u;
            uint32_t high = (index * 7u + (index >> 5) * 11u + 11u) & 15u;
            quants[index] = (uint8_t)(low | (high << 4));
        }
        meta[2 * block] =
            q4o_f32_to_f16(0.0175f + (float)(block % 7u) * 0.0017f);
        meta[2 * block + 1] =
            q4o_f32_to_f16(-0.1875f + (float)(block % 7u) * 0.0078125f);
    }
    for (size_t index = 0; index < x_count; ++index) {
        int value = (int)(((uint32_t)index * 13u + input_seed) % 17u) - 8;
        x_f16[index] = q4o_f32_to_f16((float)value * 0.0625f);
    }
}

/* ------------------------------------------------------------------ */
/* dequantisation                                                      */
/* ------------------------------------------------------------------ */

static unsigned code_at(const uint8_t *group_bytes, size_t within) {
    /* qwen38_m3.m:113-115 */
    uint8_t byte = group_bytes[within >> 1];
    return (within & 1u) == 0u ? (unsigned)(byte & 0x0fu) : (unsigned)(byte >> 4);
}

void q4o_unpack_codes(const uint8_t *quants, size_t rows, size_t groups,
                      uint8_t *codes) {
    size_t blocks = rows * groups;
    for (size_t block = 0; block < blocks; ++block) {
        for (size_t within = 0; within < 64; ++within) {
            codes[block * 64 + within] =
                (uint8_t)code_at(quants + block * 32, within);
        }
    }
}

void q4o_dequant_w32(const uint8_t *quants, const uint16_t *meta, size_t rows,
                     size_t groups, float *w) {
    /* qwen38_m3.m:116: scale * (float)quant + bias, all fp32 */
    size_t blocks = rows * groups;
#pragma omp parallel for schedule(static)
    for (size_t block = 0; block < blocks; ++block) {
        float scale = q4o_f16_to_f32(meta[2 * block]);
        float bias = q4o_f16_to_f32(meta[2 * block + 1]);
        for (size_t within = 0; within < 64; ++within) {
            w[block * 64 + within] =
                scale * (float)code_at(quants + block * 32, within) + bias;
        }
    }
}

void q4o_dequant_w16(const uint8_t *quants, const uint16_t *meta, size_t rows,
                     size_t groups, uint16_t *w_f16) {
    /* qwen38_global.metal:26-27, minimax_h3_m3_gemm.m:97-99: the exact value
     * of scale*q+bias rounded once to fp16 (double holds it exactly) */
    size_t blocks = rows * groups;
#pragma omp parallel for schedule(static)
    for (size_t block = 0; block < blocks; ++block) {
        double scale = (double)q4o_f16_to_f32(meta[2 * block]);
        double bias = (double)q4o_f16_to_f32(meta[2 * block + 1]);
        for (size_t within = 0; within < 64; ++within) {
            w_f16[block * 64 + within] = q4o_f64_to_f16(
                scale * (double)code_at(quants + block * 32, within) + bias);
        }
    }
}

/* ------------------------------------------------------------------ */
/* matmul                                                              */
/* ------------------------------------------------------------------ */

static float load_value(const void *base, int dtype, size_t index) {
    switch (dtype) {
    case Q4O_F16:
        return q4o_f16_to_f32(((const uint16_t *)base)[index]);
    case Q4O_BF16:
        return q4o_bf16_to_f32(((const uint16_t *)base)[index]);
    default:
        return ((const float *)base)[index];
    }
}

/* One row of W against one row of x.  sum32 follows the reference's element
 * order with fp32 adds (qwen38_m3.m:102-121 for fp16 x, qwen38_m3_layer.m:
 * 375-393 for fp32 x; the batched kernel keeps the same order per row,
 * qwen38_prefill.metal:165-173).  sum64 is the same sum in double.  Either
 * pointer may be NULL. */
static void row_dot(const uint8_t *row_quants, const uint16_t *row_meta,
                    size_t groups, const float *x, float *sum32,
                    double *sum64) {
    if (sum32 != NULL) {
        float total = 0.0f;
        for (size_t group = 0; group < groups; ++group) {
            float scale = q4o_f16_to_f32(row_meta[2 * group]);
            float bias = q4o_f16_to_f32(row_meta[2 * group + 1]);
            const uint8_t *packed = row_quants + group * 32;
            const float *xg = x + group * 64;
            for (size_t within = 0; within < 64; ++within) {
                float weight = scale * (float)code_at(packed, within) + bias;
                total += weight * xg[within];
            }
        }
        *sum32 = total;
    }
    if (sum64 != NULL) {
        double wide = 0.0;
        for (size_t group = 0; group < groups; ++group) {
            double scale = (double)q4o_f16_to_f32(row_meta[2 * group]);
            double bias = (double)q4o_f16_to_f32(row_meta[2 * group + 1]);
            const uint8_t *packed = row_quants + group * 32;
            const float *xg = x + group * 64;
            for (size_t within = 0; within < 64; ++within) {
                wide += (scale * (double)code_at(packed, within) + bias) *
                        (double)xg[within];
            }
        }
        *sum64 = wide;
    }
}

static void widen_rows(const void *x, int x_dtype, size_t count, float *out) {
    for (size_t index = 0; index < count; ++index) {
        out[index] = load_value(x, x_dtype, index);
    }
}

#include <stdlib.h>

void q4o_matmul(const uint8_t *quants, const uint16_t *meta, size_t groups,
                size_t row_begin, size_t row_count, const void *x, int x_dtype,
                size_t m_rows, const void *residual, int residual_dtype,
                size_t ld_residual, float *y32, double *y64, size_t ldy,
                int threads) {
    size_t columns = groups * 64;
    float *x32 = malloc(m_rows * columns * sizeof(float));
    if (x32 == NULL) {
        return;
    }
    widen_rows(x, x_dtype, m_rows * columns, x32);
#ifdef _OPENMP
    if (threads <= 0) {
        threads = omp_get_max_threads();
    }
#else
    (void)threads;
#endif
    /* rows split across threads like the reference's CPU GEMV
     * (models/qwen3.5-0.8b/targets/generic/qwen35_task.c:347-361) */
#pragma omp parallel for schedule(static) num_threads(threads)
    for (size_t local = 0; local < row_count; ++local) {
        size_t row = row_begin + local;
        for (size_t m = 0; m < m_rows; ++m) {
            float sum32 = 0.0f;
            double sum64 = 0.0;
            row_dot(quants + row * groups * 32, meta + row * groups * 2, groups,
                    x32 + m * columns, y32 != NULL ? &sum32 : NULL,
                    y64 != NULL ? &sum64 : NULL);
            if (residual != NULL && residual_dtype != Q4O_NONE) {
                /* qwen38_layer.metal:221,253: accumulator + residual */
                float extra = load_value(residual, residual_dtype,
                                         m * ld_residual + local);
                sum32 += extra;
                sum64 += (double)extra;
            }
            if (y32 != NULL) {
                y32[m * ldy + local] = sum32;
            }
            if (y64 != NULL) {
                y64[m * ldy + local] = sum64;
            }
        }
    }
    free(x32);
}

void q4o_gate_up_silu(const uint8_t *gate_quants, const uint16_t *gate_meta,
                      const uint8_t *up_quants, const uint16_t *up_meta,
                      size_t groups, size_t row_begin, size_t row_count,
                      const void *x, int x_dtype, size_t m_rows, float *y32,
                      double *y64, size_t ldy, int threads) {
    size_t columns = groups * 64;
    float *x32 = malloc(m_rows * columns * sizeof(float));
    if (x32 == NULL) {
        return;
    }
    widen_rows(x, x_dtype, m_rows * columns, x32);
#ifdef _OPENMP
    if (threads <= 0) {
        threads = omp_get_max_threads();
    }
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (size_t local = 0; local < row_count; ++local) {
        size_t row = row_begin + local;
        for (size_t m = 0; m < m_rows; ++m) {
            float gate32 = 0.0f, up32 = 0.0f;
            double gate64 = 0.0, up64 = 0.0;
            row_dot(gate_quants + row * groups * 32,
                    gate_meta + row * groups * 2, groups, x32 + m * columns,
                    y32 != NULL ? &gate32 : NULL, y64 != NULL ? &gate64 : NULL);
            row_dot(up_quants + row * groups * 32, up_meta + row * groups * 2,
                    groups, x32 + m * columns, y32 != NULL ? &up32 : NULL,
                    y64 != NULL ? &up64 : NULL);
            if (y32 != NULL) {
                /* qwen38_m3.m:758 */
                y32[m * ldy + local] = (gate32 / (1.0f + expf(-gate32))) * up32;
            }
            if (y64 != NULL) {
                y64[m * ldy + local] = (gate64 / (1.0 + exp(-gate64))) * up64;
            }
        }
    }
    free(x32);
}

void q4o_matmul_bf16(const uint8_t *quants, const uint16_t *scales_bf16,
                     const uint16_t *biases_bf16, size_t groups,
                     size_t row_begin, size_t row_count,
                     const uint16_t *x_bf16, size_t m_rows, float *y32,
                     size_t ldy, int threads) {
    /* benchmarks/minimax_h3_m3_real_gemm.c:25-42 */
    size_t columns = groups * 64;
#ifdef _OPENMP
    if (threads <= 0) {
        threads = omp_get_max_threads();
    }
#else
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (size_t local = 0; local < row_count; ++local) {
        size_t row = row_begin + local;
        for (size_t m = 0; m < m_rows; ++m) {
            float sum = 0.0f;
            for (size_t group = 0; group < groups; ++group) {
                size_t block = row * groups + group;
                float scale = q4o_bf16_to_f32(scales_bf16[block]);
                float bias = q4o_bf16_to_f32(biases_bf16[block]);
                for (size_t within = 0; within < 64; ++within) {
                    float weight = q4o_bf16_to_f32(q4o_f32_to_bf16(
                        scale * (float)code_at(quants + block * 32, within) +
                        bias));
                    sum += q4o_bf16_to_f32(
                               x_bf16[m * columns + group * 64 + within]) *
                           weight;
                }
            }
            y32[m * ldy + local] = sum;
        }
    }
}

/* RMS norm in front of the matmuls: the reference's CPU checks cpu_rms_half and cpu_rms_float
 * (models/qwen3.8-27b/targets/apple-m3-pro/qwen38_m3_layer.m:395-420): the sum of squares in double over the
 * row in index order, inv = 1 / sqrtf((float)(sum / hidden) + epsilon) in float, out = half(x * inv * weight)
 * with both products in float, for every row of [batch][hidden].  input_dtype 0 = fp16, 1 = fp32. */
void q4o_rms_norm(const void *input, int input_dtype, const float *weight,
                  uint16_t *output, size_t hidden, size_t batch, float epsilon) {
    for (size_t row = 0; row < batch; ++row) {
        double squared = 0.0;
        for (size_t index = 0; index < hidden; ++index) {
            float value = load_value(input, input_dtype, row * hidden + index);
            squared += (double)value * value;
        }
        float inv = 1.0f / sqrtf((float)(squared / (double)hidden) + epsilon);
        for (size_t index = 0; index < hidden; ++index) {
            float value = load_value(input, input_dtype, row * hidden + index);
            output[row * hidden + index] = q4o_f32_to_f16(value * inv * weight[index]);
        }
    }
}

/* Affine Q8 (minimax_h3_q8_gemm_bf16_meta, models/minimax-h3/targets/apple-m3-pro/minimax_h3_attention.metal:
 * 594-676): quants [rows][groups][64] code bytes, bf16 scales and biases [rows][groups];
 * weight_tile = half(scale * float(code) + bias) with scale and bias widened to float (:625-633).  The
 * reference has no CPU check of this kernel (its benchmark runs on zero-filled buffers,
 * minimax_h3_m3_gemm.m:464-468), so this restatement of the kernel's own formula is all there is. */
float q4o_q8_w32(uint8_t code, uint16_t scale_bf16, uint16_t bias_bf16) {
    float scale = q4o_bf16_to_f32(scale_bf16), bias = q4o_bf16_to_f32(bias_bf16);
    return scale * (float)code + bias;
}

void q4o_dequant_q8(const uint8_t *quants, const uint16_t *scales_bf16, const uint16_t *biases_bf16,
                    size_t rows, size_t groups, float *w32, uint16_t *w16) {
    for (size_t block = 0; block < rows * groups; ++block) {
        for (size_t k = 0; k < 64; ++k) {
            float value = q4o_q8_w32(quants[block * 64 + k], scales_bf16[block], biases_bf16[block]);
            if (w32 != NULL) w32[block * 64 + k] = value;
            if (w16 != NULL) w16[block * 64 + k] = q4o_f32_to_f16(value);
        }
    }
}

/* y[m][n] = sum_k half(w(n, k)) * x[m][k] for rows row_begin .. row_begin + row_count - 1: the half-rounded
 * weights the kernel multiplies, summed in float (y32) and in double (y64) in column order; x fp16 or fp32. */
void q4o_matmul_q8(const uint8_t *quants, const uint16_t *scales_bf16, const uint16_t *biases_bf16,
                   size_t groups, size_t row_begin, size_t row_count, const void *x, int x_dtype,
                   size_t m_rows, float *y32, double *y64, size_t ldy, int threads) {
    size_t columns = groups * 64;
    if (threads <= 0) threads = q4o_max_threads();
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long long local = 0; local < (long long)row_count; ++local) {
        size_t row = row_begin + (size_t)local;
        for (size_t m = 0; m < m_rows; ++m) {
            float sum32 = 0.0f;
            double sum64 = 0.0;
            for (size_t g = 0; g < groups; ++g) {
                size_t block = row * groups + g;
                for (size_t k = 0; k < 64; ++k) {
                    float weight = q4o_f16_to_f32(q4o_f32_to_f16(
                        q4o_q8_w32(quants[block * 64 + k], scales_bf16[block], biases_bf16[block])));
                    float value = load_value(x, x_dtype, m * columns + g * 64 + k);
                    sum32 += weight * value;
                    sum64 += (double)weight * (double)value;
                }
            }
            if (y32 != NULL) y32[m * ldy + (size_t)local] = sum32;
            if (y64 != NULL) y64[m * ldy + (size_t)local] = sum64;
        }
    }
}

