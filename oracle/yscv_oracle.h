/*
 * CPU oracle for the yscv quantized-matmul hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This is a scalar, loop-for-loop restatement in C of
 * the reference's (enthropy7/YSCV) CPU algorithms; it exists so that the CUDA
 * path can be checked against it. Nothing in the shipped library links,
 * imports or executes it.
 *
 * Build with  -O2 -ffp-contract=off -fno-fast-math : the reference is Rust,
 * which never contracts a*b+c into an FMA and never reassociates.
 *
 * Every function cites the reference file:line it restates (paths are
 * relative to the reference project root).
 */
#ifndef YSCV_ORACLE_H
#define YSCV_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- int4 block-quantized weights -------------------------------------- */

/* crates/yscv-kernels/src/ops/int4_matmul.rs:29-40 */
int8_t yo_unpack_low(uint8_t byte);
int8_t yo_unpack_high(uint8_t byte);

/* crates/yscv-kernels/src/ops/int4_matmul.rs:44-81  packed_int4_gemv_scalar */
void yo_packed_int4_gemv(const uint8_t *weight_packed, const float *scales,
                         const float *activation, float *output,
                         size_t m_w, size_t k, size_t group_size);

/* crates/yscv-kernels/src/ops/int4_matmul.rs:387-435  packed_int4_gemm_scalar */
void yo_packed_int4_gemm(const uint8_t *weight_packed, const float *scales,
                         const float *activation, float *output,
                         size_t m, size_t n, size_t k, size_t group_size);

/* crates/yscv-kernels/src/ops/int4_matmul.rs:611-646  pack_int4_symmetric_per_group */
void yo_pack_int4_symmetric_per_group(const float *weights, size_t m_w, size_t k,
                                      size_t group_size, uint8_t *packed,
                                      float *scales);

/* crates/yscv-onnx/src/quantize/packed_int4.rs:73-85: MatMul weights arrive as
 * [K,N] and are transposed to [N,K] before packing. */
void yo_transpose_kn_to_nk(const float *w_kn, size_t k, size_t n, float *w_nk);

/* crates/yscv-onnx/src/runner/linear.rs:223-278  exec_matmul, int4 branch:
 * M >= 8 -> one GEMM call, else M GEMV calls. */
void yo_exec_matmul_int4(const uint8_t *weight_packed, const float *scales,
                         const float *activation, float *output,
                         size_t m, size_t n, size_t k, size_t group_size);

/* ---- int8 GEMM --------------------------------------------------------- */

/* crates/yscv-kernels/src/ops/int8_matmul.rs:195-208  int8_matmul_scalar */
void yo_int8_matmul(const int8_t *a, const int8_t *b, size_t m, size_t k,
                    size_t n, int32_t *out);

/* crates/yscv-kernels/src/ops/int8_matmul.rs:90-117  transpose_b ([K,N]->[N,K]) */
void yo_transpose_b_i8(const int8_t *b, size_t k, size_t n, int8_t *bt);

/* crates/yscv-kernels/src/ops/int8_matmul.rs:212-227  int8_matmul_prepacked_scalar */
void yo_int8_matmul_prepacked(const int8_t *a, const int8_t *bt, size_t m,
                              size_t k, size_t n, int32_t *out);

/* ---- requantize / quantize --------------------------------------------- */

/* crates/yscv-kernels/src/ops/int8_requant.rs:143-169  requant_scalar.
 * bias may be NULL. Output range is the reference's [-128,127]. */
void yo_requant_i8(const int32_t *acc, size_t len, const int32_t *bias,
                   float composite, float y_zp, int relu, int8_t *out, size_t c);

/* Same formula (separate multiply and add, round-half-even, saturate) with a
 * caller-chosen saturation range, written as int32 so both the int8 and the
 * uint8 output of ONNX QLinearMatMul are covered. */
void yo_requant_range(const int32_t *acc, size_t len, float composite, float y_zp,
                      int32_t lo, int32_t hi, int32_t *out);

/* crates/yscv-kernels/src/ops/int8_requant.rs:537-556  requant_i8_per_channel_scalar */
void yo_requant_i8_per_channel(const int32_t *acc, size_t len, const int32_t *corr,
                               const float *composite, float y_zp, int8_t *out,
                               size_t c);

/* crates/yscv-kernels/src/ops/quantize.rs:242-254  quantize_linear_f32_to_i8_scalar */
void yo_quantize_linear_i8(const float *data, size_t len, float scale,
                           float zero_point, int8_t *out);
/* same formula, uint8 saturation range [0,255] (ONNX QuantizeLinear to uint8) */
void yo_quantize_linear_u8(const float *data, size_t len, float scale,
                           float zero_point, uint8_t *out);

/* crates/yscv-onnx/src/quantize/rewriter.rs:692-706  quantize_tensor_symmetric
 * (inv = 1/scale; round-half-away; clamp [-128,127]) */
void yo_quantize_tensor_symmetric(const float *data, size_t len, float scale,
                                  int8_t *out);

/* crates/yscv-onnx/src/runner/kv_cache.rs:44-60  LayerStorage::append, KvDtype::I8:
 * per row abs_max; scale = abs_max <= EPSILON ? 1.0 : abs_max / 127.0; inv = 1.0 / scale;
 * q = clamp(round_half_away(v * inv), -127, 127). One scale per row. */
void yo_kv_append_i8(const float *src, size_t rows, size_t kv_dim, int8_t *data,
                     float *scales);
/* crates/yscv-onnx/src/runner/kv_cache.rs:63-78  dequantise_to_vec: (q as f32) * scale */
void yo_kv_dequantise_i8(const int8_t *data, const float *scales, size_t rows,
                         size_t kv_dim, float *out);

/* ---- runner-level operator semantics ----------------------------------- */

/* crates/yscv-onnx/src/runner/linear.rs:453-492: QLinearMatMul fast path as the
 * reference runner computes it (f32::round = half away from zero, clamp to
 * [-128,127], result carried as f32). Inputs are f32-encoded integers. */
void yo_runner_qlinear_matmul_fast(const float *a, const float *b, size_t m,
                                   size_t k, size_t n, float a_scale,
                                   float b_scale, float y_scale, float y_zp,
                                   float *out);

/* crates/yscv-onnx/src/runner/linear.rs:648-737: MatMulInteger. Exact integer
 * result of (a - a_zp) x (b - b_zp); the reference reaches it either through
 * the int8 kernel (both zp 0) or an fp32 GEMM + round that is exact whenever
 * all partial sums stay below 2^24. */
void yo_runner_matmul_integer(const float *a, const float *b, size_t m, size_t k,
                              size_t n, float a_zp, float b_zp, float *out);

/* ---- decoder primitives ------------------------------------------------ */

/* crates/yscv-kernels/src/ops/norm.rs:1497-1518  rms_norm_last_dim_row */
void yo_rms_norm(const float *input, size_t rows, size_t hidden, const float *gamma,
                 float epsilon, float *out);

/* crates/yscv-kernels/src/ops/rope.rs:24-117  apply_rotary_embedding (scalar) */
void yo_rope(float *q, float *k, size_t num_q_heads, size_t num_kv_heads,
             size_t d_head, size_t seq_len, size_t seq_offset, float theta);

/* crates/yscv-onnx/src/runner/linear.rs:552-646  exec_grouped_query_attention.
 * causal != 0 limits query sq to keys sk <= sq + (seq_k - seq_q), which is what
 * the exported decoder graphs the reference runs add through their mask. */
void yo_gqa_attention(const float *q, const float *k, const float *v, size_t batch,
                      size_t seq_q, size_t seq_k, size_t num_q_heads,
                      size_t num_kv_heads, size_t d_head, int causal, float *out);

/* crates/yscv-kernels/src/ops/simd/activation.rs:1000-1005  silu scalar */
void yo_silu(const float *input, size_t len, float *out);

/* apps/llm-bench/src/main.rs:538-543: greedy argmax, LAST index among ties */
uint32_t yo_argmax_last(const float *logits, size_t vocab);

/* ---- the reference tests' own input generators ------------------------- */

/* crates/yscv-kernels/src/ops/int4_matmul.rs:652-662 */
void yo_lcg_f32(uint64_t seed, size_t n, float *out);
/* crates/yscv-kernels/src/ops/int8_matmul.rs:2437-2447 */
void yo_lcg_i8(uint64_t seed, size_t n, int8_t *out);

#ifdef __cplusplus
}
#endif
#endif
