/*
 * CPU oracle for the yscv quantized-matmul hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * Scalar C restatement of the reference's CPU algorithms (see yscv_oracle.h for
 * the per-function citations). The shipped CUDA library never calls into this
 * file; only the parity tests, the smoke check and the benchmark's CPU-baseline
 * leg do.
 *
 * Pinned against the reference's own known-answer tests (nibble sign
 * extension, [[1,2],[3,4]]x[[5,6],[7,8]], (-128)^2*128, the round-half-even
 * requant table, saturation, the runner-level QLinearMatMul / MatMulInteger
 * cases): see tests/test_oracle_golden.py.
 *
 * Compile:  gcc -O2 -ffp-contract=off -fno-fast-math -fPIC -shared
 */
#include "yscv_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* Rust `as i8` on a float saturates; values here are already clamped. */
static inline float clampf(float v, float lo, float hi) {
    /* f32::clamp: NaN stays NaN, then `as iN` maps NaN to 0 */
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

static inline float round_ties_even(float v) { return nearbyintf(v); }

/* ---- int4 --------------------------------------------------------------- */

int8_t yo_unpack_low(uint8_t byte) {
    int8_t v = (int8_t)(uint8_t)(byte << 4);
    return (int8_t)(v >> 4);
}

int8_t yo_unpack_high(uint8_t byte) { return (int8_t)(((int8_t)byte) >> 4); }

void yo_packed_int4_gemv(const uint8_t *weight_packed, const float *scales,
                         const float *activation, float *output, size_t m_w,
                         size_t k, size_t group_size) {
    size_t groups = k / group_size;
    for (size_t row = 0; row < m_w; ++row) {
        const uint8_t *row_bytes = weight_packed + row * k / 2;
        const float *row_scales = scales + row * groups;
        float acc = 0.0f;
        for (size_t g = 0; g < groups; ++g) {
            float scale = row_scales[g];
            float group_acc = 0.0f;
            size_t byte_base = g * group_size / 2;
            size_t act_base = g * group_size;
            for (size_t i = 0; i < group_size / 2; ++i) {
                uint8_t byte = row_bytes[byte_base + i];
                float q_lo = (float)yo_unpack_low(byte);
                float q_hi = (float)yo_unpack_high(byte);
                group_acc += q_lo * activation[act_base + 2 * i];
                group_acc += q_hi * activation[act_base + 2 * i + 1];
            }
            acc += scale * group_acc;
        }
        output[row] = acc;
    }
}

void yo_packed_int4_gemm(const uint8_t *weight_packed, const float *scales,
                         const float *activation, float *output, size_t m,
                         size_t n, size_t k, size_t group_size) {
    size_t groups = k / group_size;
    for (size_t i = 0; i < m * n; ++i) output[i] = 0.0f;
    int8_t *unpacked = (int8_t *)malloc(group_size > 256 ? group_size : 256);
    for (size_t nn = 0; nn < n; ++nn) {
        const uint8_t *row_bytes = weight_packed + nn * k / 2;
        const float *row_scales = scales + nn * groups;
        for (size_t g = 0; g < groups; ++g) {
            float scale = row_scales[g];
            size_t byte_base = g * group_size / 2;
            size_t act_base = g * group_size;
            for (size_t i = 0; i < group_size / 2; ++i) {
                uint8_t byte = row_bytes[byte_base + i];
                unpacked[2 * i] = yo_unpack_low(byte);
                unpacked[2 * i + 1] = yo_unpack_high(byte);
            }
            for (size_t mi = 0; mi < m; ++mi) {
                float sum = 0.0f;
                const float *row_act = activation + mi * k + act_base;
                for (size_t j = 0; j < group_size; ++j)
                    sum += (float)unpacked[j] * row_act[j];
                output[mi * n + nn] += scale * sum;
            }
        }
    }
    free(unpacked);
}

void yo_pack_int4_symmetric_per_group(const float *weights, size_t m_w, size_t k,
                                      size_t group_size, uint8_t *packed,
                                      float *scales) {
    size_t groups = k / group_size;
    for (size_t row = 0; row < m_w; ++row) {
        for (size_t g = 0; g < groups; ++g) {
            const float *slice = weights + row * k + g * group_size;
            float abs_max = 0.0f;
            for (size_t i = 0; i < group_size; ++i)
                abs_max = fmaxf(abs_max, fabsf(slice[i]));
            /* f32::EPSILON = 2^-23 */
            float scale = (abs_max <= 1.1920929e-07f) ? 1.0f : abs_max / 7.0f;
            scales[row * groups + g] = scale;
            float inv = 1.0f / scale;
            for (size_t i = 0; i < group_size / 2; ++i) {
                int8_t v0 = (int8_t)clampf(round_ties_even(slice[2 * i] * inv), -8.0f, 7.0f);
                int8_t v1 = (int8_t)clampf(round_ties_even(slice[2 * i + 1] * inv), -8.0f, 7.0f);
                uint8_t byte = (uint8_t)(((uint8_t)v0 & 0x0F) | (((uint8_t)v1 & 0x0F) << 4));
                packed[row * k / 2 + g * group_size / 2 + i] = byte;
            }
        }
    }
}

void yo_transpose_kn_to_nk(const float *w_kn, size_t k, size_t n, float *w_nk) {
    for (size_t kk = 0; kk < k; ++kk)
        for (size_t nn = 0; nn < n; ++nn) w_nk[nn * k + kk] = w_kn[kk * n + nn];
}

void yo_exec_matmul_int4(const uint8_t *weight_packed, const float *scales,
                         const float *activation, float *output, size_t m,
                         size_t n, size_t k, size_t group_size) {
    const size_t GEMM_THRESHOLD = 8;
    if (m >= GEMM_THRESHOLD) {
        yo_packed_int4_gemm(weight_packed, scales, activation, output, m, n, k, group_size);
    } else {
        for (size_t row = 0; row < m; ++row)
            yo_packed_int4_gemv(weight_packed, scales, activation + row * k,
                                output + row * n, n, k, group_size);
    }
}

/* ---- int8 --------------------------------------------------------------- */

void yo_int8_matmul(const int8_t *a, const int8_t *b, size_t m, size_t k, size_t n,
                    int32_t *out) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            for (size_t kk = 0; kk < k; ++kk)
                acc += (int32_t)a[i * k + kk] * (int32_t)b[kk * n + j];
            out[i * n + j] = acc;
        }
}

void yo_transpose_b_i8(const int8_t *b, size_t k, size_t n, int8_t *bt) {
    for (size_t kk = 0; kk < k; ++kk)
        for (size_t j = 0; j < n; ++j) bt[j * k + kk] = b[kk * n + j];
}

void yo_int8_matmul_prepacked(const int8_t *a, const int8_t *bt, size_t m, size_t k,
                              size_t n, int32_t *out) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            for (size_t kk = 0; kk < k; ++kk)
                acc += (int32_t)a[i * k + kk] * (int32_t)bt[j * k + kk];
            out[i * n + j] = acc;
        }
}

/* ---- requant / quantize -------------------------------------------------- */

void yo_requant_i8(const int32_t *acc, size_t len, const int32_t *bias,
                   float composite, float y_zp, int relu, int8_t *out, size_t c) {
    size_t pixels = len / c;
    for (size_t p = 0; p < pixels; ++p)
        for (size_t ch = 0; ch < c; ++ch) {
            int32_t a = acc[p * c + ch];
            if (bias) a = (int32_t)((uint32_t)a + (uint32_t)bias[ch]); /* wrapping_add */
            float v = (float)a * composite;
            v = v + y_zp;
            int8_t q = (int8_t)clampf(round_ties_even(v), -128.0f, 127.0f);
            if (relu && q < 0) q = 0;
            out[p * c + ch] = q;
        }
}

void yo_kv_append_i8(const float *src, size_t rows, size_t kv_dim, int8_t *data,
                     float *scales) {
    for (size_t r = 0; r < rows; ++r) {
        const float *row = src + r * kv_dim;
        float abs_max = 0.0f;
        for (size_t i = 0; i < kv_dim; ++i) {
            float a = fabsf(row[i]);
            if (a > abs_max) abs_max = a; /* f32::max ignores a NaN operand */
        }
        float scale = abs_max <= FLT_EPSILON ? 1.0f : abs_max / 127.0f;
        float inv = 1.0f / scale;
        scales[r] = scale;
        for (size_t i = 0; i < kv_dim; ++i) {
            float v = row[i] * inv;
            float q = roundf(v); /* f32::round: half away from zero */
            if (q < -127.0f) q = -127.0f;
            if (q > 127.0f) q = 127.0f;
            data[r * kv_dim + i] = (v != v) ? (int8_t)0 : (int8_t)q; /* NaN as i8 == 0 */
        }
    }
}

void yo_kv_dequantise_i8(const int8_t *data, const float *scales, size_t rows,
                         size_t kv_dim, float *out) {
    for (size_t r = 0; r < rows; ++r)
        for (size_t i = 0; i < kv_dim; ++i)
            out[r * kv_dim + i] = (float)data[r * kv_dim + i] * scales[r];
}

void yo_requant_range(const int32_t *acc, size_t len, float composite, float y_zp,
                      int32_t lo, int32_t hi, int32_t *out) {
    for (size_t i = 0; i < len; ++i) {
        float v = (float)acc[i] * composite;
        v = v + y_zp;
        out[i] = (int32_t)clampf(round_ties_even(v), (float)lo, (float)hi);
    }
}

void yo_requant_i8_per_channel(const int32_t *acc, size_t len, const int32_t *corr,
                               const float *composite, float y_zp, int8_t *out,
                               size_t c) {
    size_t pixels = len / c;
    for (size_t p = 0; p < pixels; ++p)
        for (size_t ch = 0; ch < c; ++ch) {
            int32_t a = (int32_t)((uint32_t)acc[p * c + ch] + (uint32_t)corr[ch]);
            float v = (float)a * composite[ch];
            v = v + y_zp;
            out[p * c + ch] = (int8_t)clampf(round_ties_even(v), -128.0f, 127.0f);
        }
}

void yo_quantize_linear_i8(const float *data, size_t len, float scale,
                           float zero_point, int8_t *out) {
    for (size_t i = 0; i < len; ++i) {
        float v = data[i] / scale;
        v = v + zero_point;
        out[i] = (int8_t)clampf(round_ties_even(v), -128.0f, 127.0f);
    }
}

void yo_quantize_linear_u8(const float *data, size_t len, float scale,
                           float zero_point, uint8_t *out) {
    for (size_t i = 0; i < len; ++i) {
        float v = data[i] / scale;
        v = v + zero_point;
        out[i] = (uint8_t)clampf(round_ties_even(v), 0.0f, 255.0f);
    }
}

void yo_quantize_tensor_symmetric(const float *data, size_t len, float scale,
                                  int8_t *out) {
    float inv_s = (fabsf(scale) > 1.1920929e-07f) ? 1.0f / scale : 0.0f;
    for (size_t i = 0; i < len; ++i)
        out[i] = (int8_t)clampf(roundf(data[i] * inv_s), -128.0f, 127.0f);
}

/* ---- runner-level -------------------------------------------------------- */

/* Rust `v as i8` for f32 v: truncate toward zero, saturate. */
static inline int8_t f32_as_i8(float v) {
    if (v != v) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v;
}

void yo_runner_qlinear_matmul_fast(const float *a, const float *b, size_t m,
                                   size_t k, size_t n, float a_scale, float b_scale,
                                   float y_scale, float y_zp, float *out) {
    int8_t *a8 = (int8_t *)malloc(m * k);
    int8_t *b8 = (int8_t *)malloc(k * n);
    int32_t *acc = (int32_t *)malloc(m * n * sizeof(int32_t));
    for (size_t i = 0; i < m * k; ++i) a8[i] = f32_as_i8(a[i]);
    for (size_t i = 0; i < k * n; ++i) b8[i] = f32_as_i8(b[i]);
    yo_int8_matmul(a8, b8, m, k, n, acc);
    float composite = (a_scale * b_scale) / y_scale;
    for (size_t i = 0; i < m * n; ++i) {
        float v = (float)acc[i] * composite;
        v = v + y_zp;
        out[i] = clampf(roundf(v), -128.0f, 127.0f);
    }
    free(a8);
    free(b8);
    free(acc);
}

void yo_runner_matmul_integer(const float *a, const float *b, size_t m, size_t k,
                              size_t n, float a_zp, float b_zp, float *out) {
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            int64_t acc = 0;
            for (size_t kk = 0; kk < k; ++kk) {
                int64_t av = (int64_t)(a[i * k + kk] - a_zp);
                int64_t bv = (int64_t)(b[kk * n + j] - b_zp);
                acc += av * bv;
            }
            out[i * n + j] = (float)(int32_t)acc;
        }
}

/* ---- decoder primitives -------------------------------------------------- */

void yo_rms_norm(const float *input, size_t rows, size_t hidden, const float *gamma,
                 float epsilon, float *out) {
    for (size_t r = 0; r < rows; ++r) {
        const float *row = input + r * hidden;
        float sum_sq = 0.0f;
        for (size_t i = 0; i < hidden; ++i) sum_sq += row[i] * row[i];
        float rms = sqrtf(sum_sq / (float)hidden + epsilon);
        float inv_rms = 1.0f / rms;
        for (size_t i = 0; i < hidden; ++i) {
            float t = row[i] * inv_rms;
            out[r * hidden + i] = t * gamma[i];
        }
    }
}

static void rotate_half(float *data, const float *inv_freq, size_t half, float pos) {
    for (size_t i = 0; i < half; ++i) {
        float angle = inv_freq[i] * pos;
        float sin_a = sinf(angle), cos_a = cosf(angle);
        float x0 = data[i], x1 = data[i + half];
        float t0 = x0 * cos_a, t1 = x1 * sin_a;
        float t2 = x0 * sin_a, t3 = x1 * cos_a;
        data[i] = t0 - t1;
        data[i + half] = t2 + t3;
    }
}

void yo_rope(float *q, float *k, size_t num_q_heads, size_t num_kv_heads,
             size_t d_head, size_t seq_len, size_t seq_offset, float theta) {
    size_t half = d_head / 2;
    float *inv_freq = (float *)malloc(half * sizeof(float));
    for (size_t i = 0; i < half; ++i)
        inv_freq[i] = 1.0f / powf(theta, 2.0f * (float)i / (float)d_head);
    for (size_t pos = 0; pos < seq_len; ++pos) {
        float abs_pos = (float)(pos + seq_offset);
        for (size_t h = 0; h < num_q_heads; ++h)
            rotate_half(q + (pos * num_q_heads + h) * d_head, inv_freq, half, abs_pos);
        for (size_t h = 0; h < num_kv_heads; ++h)
            rotate_half(k + (pos * num_kv_heads + h) * d_head, inv_freq, half, abs_pos);
    }
    free(inv_freq);
}

void yo_gqa_attention(const float *q, const float *k, const float *v, size_t batch,
                      size_t seq_q, size_t seq_k, size_t num_q_heads,
                      size_t num_kv_heads, size_t d_head, int causal, float *out) {
    size_t groups = num_q_heads / num_kv_heads;
    float scale = 1.0f / sqrtf((float)d_head);
    float *scores = (float *)malloc(seq_k * sizeof(float));
    for (size_t b = 0; b < batch; ++b) {
        const float *qb = q + b * seq_q * num_q_heads * d_head;
        const float *kb = k + b * seq_k * num_kv_heads * d_head;
        const float *vb = v + b * seq_k * num_kv_heads * d_head;
        float *ob = out + b * seq_q * num_q_heads * d_head;
        for (size_t qh = 0; qh < num_q_heads; ++qh) {
            size_t kv_h = qh / groups;
            for (size_t sq = 0; sq < seq_q; ++sq) {
                size_t limit = causal ? (sq + (seq_k - seq_q) + 1) : seq_k;
                float max_score = -INFINITY;
                for (size_t sk = 0; sk < limit; ++sk) {
                    float dot = 0.0f;
                    for (size_t d = 0; d < d_head; ++d)
                        dot += qb[(sq * num_q_heads + qh) * d_head + d] *
                               kb[(sk * num_kv_heads + kv_h) * d_head + d];
                    float s = dot * scale;
                    if (s > max_score) max_score = s;
                    scores[sk] = s;
                }
                float sum_exp = 0.0f;
                for (size_t sk = 0; sk < limit; ++sk) {
                    scores[sk] = expf(scores[sk] - max_score);
                    sum_exp += scores[sk];
                }
                if (sum_exp > 0.0f) {
                    float inv = 1.0f / sum_exp;
                    for (size_t sk = 0; sk < limit; ++sk) scores[sk] *= inv;
                }
                for (size_t d = 0; d < d_head; ++d) {
                    float acc = 0.0f;
                    for (size_t sk = 0; sk < limit; ++sk)
                        acc += scores[sk] * vb[(sk * num_kv_heads + kv_h) * d_head + d];
                    ob[(sq * num_q_heads + qh) * d_head + d] = acc;
                }
            }
        }
    }
    free(scores);
}

void yo_silu(const float *input, size_t len, float *out) {
    for (size_t i = 0; i < len; ++i) {
        float v = input[i];
        float s = 1.0f / (1.0f + expf(-v));
        out[i] = v * s;
    }
}

uint32_t yo_argmax_last(const float *logits, size_t vocab) {
    /* Iterator::max_by keeps the LAST of several equal maxima. */
    size_t best = 0;
    for (size_t i = 1; i < vocab; ++i)
        if (!(logits[i] < logits[best])) best = i;
    return (uint32_t)best;
}

/* ---- LCG generators of the reference's unit tests ------------------------ */

void yo_lcg_f32(uint64_t seed, size_t n, float *out) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) {
        s = s * 6364136223846793005ULL + 1442695040888963407ULL;
        int64_t r = (int64_t)(s >> 33) % 2001 - 1000;
        out[i] = (float)r * 0.001f;
    }
}

void yo_lcg_i8(uint64_t seed, size_t n, int8_t *out) {
    uint64_t s = seed;
    for (size_t i = 0; i < n; ++i) {
        s = s * 6364136223846793005ULL + 1442695040888963407ULL;
        out[i] = (int8_t)((int64_t)(s >> 33) % 256 - 128);
    }
}
