/*
 * CPU oracle for the affine-Q4 matmul path -- TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the scalar CPU formulas the reference
 * (baryhuang/cpu-llms-in-c) carries next to its Metal kernels.  It is the
 * checker for the CUDA library, never the thing shipped or measured as the
 * product: only the tests, the smoke check and the CPU-baseline leg of the
 * benchmark may call it.
 *
 * Format (models/qwen3.8-27b/targets/apple-m3-pro/qwen38_q4.metal:10-37,
 * qwen38_m3.m:19-22): W[N][K], K % 64 == 0, G = K/64 groups per row.
 *   quants : N*K/2 bytes; byte (n*G+g)*32 + (j>>1), low nibble for even j
 *   meta   : N*G records {uint16 fp16 scale, uint16 fp16 bias}
 *   w(n,k) = scale(n,g)*code(n,k) + bias(n,g)
 */
#ifndef Q4_ORACLE_H
#define Q4_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { Q4O_F16 = 0, Q4O_F32 = 1, Q4O_BF16 = 2, Q4O_NONE = -1 };

/* ---- scalar conversions (own code; pinned against the reference packer's
 * float_to_half_bits / half_bits_to_float / bf16_to_half,
 * compiler/qwen3.8-27b/apple-m3-pro/qwen38_m3_pack.c:110-178) ---- */
uint16_t q4o_f32_to_f16(float value);
uint16_t q4o_f64_to_f16(double value);
float q4o_f16_to_f32(uint16_t bits);
uint16_t q4o_f32_to_bf16(float value);
float q4o_bf16_to_f32(uint16_t bits);
uint16_t q4o_bf16_to_f16(uint16_t bits);

/* ---- seeded synthetic inputs (counter based; the CUDA library carries the
 * same generator so both sides see identical bytes) ---- */
uint64_t q4o_hash(uint64_t seed, uint64_t stream, uint64_t index);
void q4o_synth_codes(uint64_t seed, uint64_t stream, uint32_t *words,
                     size_t word_begin, size_t word_count);
void q4o_synth_meta(uint64_t seed, uint64_t stream, uint16_t *meta,
                    size_t group_begin, size_t group_count);
void q4o_synth_x(uint64_t seed, uint64_t stream, uint16_t *x_f16,
                 size_t begin, size_t count);

/* ---- the reference's own closed-form fixtures, regenerated ---- */
/* xorshift fill of qwen38_m3.m:56-87 (seeds 0x36a110c / 0x27b4c51 / 0x36d027b) */
void q4o_fill_weights_xorshift(uint8_t *quants, uint16_t *meta,
                               size_t group_count, uint32_t seed);
/* activation 0.75 sin(0.013 i) + 0.20 cos(0.031 i), qwen38_m3.m:568-573 */
void q4o_activation_sincos(uint16_t *x_f16, size_t count);
/* arithmetic pattern of minimax_h3_m3_gemm.m:75-104 */
void q4o_h3_pattern(uint8_t *quants, uint16_t *meta, size_t rows,
                    size_t groups_per_row, uint16_t *x_f16, size_t x_count,
                    uint32_t input_seed);

/* ---- dequantisation in isolation (qwen38_global.metal:13-28) ---- */
void q4o_unpack_codes(const uint8_t *quants, size_t rows, size_t groups,
                      uint8_t *codes);
void q4o_dequant_w32(const uint8_t *quants, const uint16_t *meta, size_t rows,
                     size_t groups, float *w);
void q4o_dequant_w16(const uint8_t *quants, const uint16_t *meta, size_t rows,
                     size_t groups, uint16_t *w_f16);

/* ---- matmul: y[m][n] = sum_k w(n,k) * x[m][k] (+ residual[m][n]) ----
 * Rows row_begin .. row_begin+row_count-1 of W are computed; y is indexed
 * [m*ldy + (n - row_begin)].  y32 uses the reference's fp32 accumulation in
 * its element order (qwen38_m3.m:102-121, qwen38_m3_layer.m:354-393); y64
 * accumulates in double.  Either output may be NULL.  threads <= 0 lets
 * OpenMP choose. */
void q4o_matmul(const uint8_t *quants, const uint16_t *meta, size_t groups,
                size_t row_begin, size_t row_count, const void *x, int x_dtype,
                size_t m_rows, const void *residual, int residual_dtype,
                size_t ld_residual, float *y32, double *y64, size_t ldy,
                int threads);

/* fused gate/up: out = silu(g) * u from the un-rounded accumulators
 * (qwen38_q4.metal:129-151, qwen38_m3.m:752-758) */
void q4o_gate_up_silu(const uint8_t *gate_quants, const uint16_t *gate_meta,
                      const uint8_t *up_quants, const uint16_t *up_meta,
                      size_t groups, size_t row_begin, size_t row_count,
                      const void *x, int x_dtype, size_t m_rows, float *y32,
                      double *y64, size_t ldy, int threads);

/* bf16 witness (benchmarks/minimax_h3_m3_real_gemm.c:25-42): separate BF16
 * scale/bias planes, weight rounded to bf16, bf16 x, fp32 sum */
void q4o_matmul_bf16(const uint8_t *quants, const uint16_t *scales_bf16,
                     const uint16_t *biases_bf16, size_t groups,
                     size_t row_begin, size_t row_count,
                     const uint16_t *x_bf16, size_t m_rows, float *y32,
                     size_t ldy, int threads);

void q4o_round_f16(const float *in, uint16_t *out, size_t count);
/* affine Q8 (minimax_h3_attention.metal:594-676): code bytes [rows][groups][64], bf16 scales / biases */
void q4o_dequant_q8(const uint8_t *quants, const uint16_t *scales_bf16, const uint16_t *biases_bf16,
                    size_t rows, size_t groups, float *w32, uint16_t *w16);
void q4o_matmul_q8(const uint8_t *quants, const uint16_t *scales_bf16, const uint16_t *biases_bf16,
                   size_t groups, size_t row_begin, size_t row_count, const void *x, int x_dtype,
                   size_t m_rows, float *y32, double *y64, size_t ldy, int threads);
/* cpu_rms_half / cpu_rms_float (qwen38_m3_layer.m:395-420) over [batch][hidden]; input_dtype 0 = fp16, 1 = fp32 */
void q4o_rms_norm(const void *input, int input_dtype, const float *weight,
                  uint16_t *output, size_t hidden, size_t batch, float epsilon);
int q4o_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
