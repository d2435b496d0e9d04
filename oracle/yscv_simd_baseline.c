/*
 * Timed CPU baseline for the yscv quantized-matmul hot path -- TEST / BENCH
 * INFRASTRUCTURE ONLY, never linked into the shipped library.
 *
 * The reference cannot be built on this machine (it is Rust), so this file
 * restates, with C intrinsics, the SIMD kernels the reference dispatches to on
 * an x86-64 host, with the same run-time gates:
 *   - int4 GEMV : AVX-512 (crates/yscv-kernels/src/ops/int4_matmul.rs:243-307),
 *                 gate avx512bw && group_size % 32 == 0 (:321)
 *   - int4 GEMM : AVX2+FMA (int4_matmul.rs:439-489); the reference has no
 *                 AVX-512 GEMM; gate group_size % 8 == 0 && group_size <= 256 (:562)
 *   - int8 GEMM : AVX-512-VNNI (crates/yscv-kernels/src/ops/int8_matmul.rs:2100-2159)
 *                 with its MR8xNR16 (:2007-2096) and MR4xNR16 (:1850-1925)
 *                 register-blocked variants and the simple B^T row-dot fallback
 * Hosts without these ISA extensions fall back to the scalar oracle and say so
 * through ysb_isa(). Every kernel is single-threaded like the reference's; the
 * *_mt wrappers partition output rows across pthreads ("reference kernel,
 * outer-parallel"), which is how the reference parallelises its int8 path one
 * level up (crates/yscv-onnx/src/runner/conv/quantized.rs:424-447).
 */
#define _GNU_SOURCE
#include <immintrin.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "yscv_oracle.h"

static int has_avx512(void) {
    return __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw");
}
static int has_vnni(void) { return has_avx512() && __builtin_cpu_supports("avx512vnni"); }
static int has_avx2(void) { return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma"); }

const char *ysb_isa(void) {
    if (has_vnni()) return "avx512-vnni";
    if (has_avx512()) return "avx512";
    if (has_avx2()) return "avx2";
    return "scalar";
}

/* ---- int4 GEMV, AVX-512 --------------------------------------------------- */

__attribute__((target("avx512f,avx512bw,avx2"))) static void
int4_gemv_avx512(const uint8_t *wp, const float *scales, const float *act, float *out,
                 size_t m_w, size_t k, size_t gs) {
    size_t groups = k / gs, blocks = gs / 32;
    const __m512i idx_even = _mm512_setr_epi32(0, 2, 4, 6, 8, 10, 12, 14, 16, 18, 20, 22, 24, 26, 28, 30);
    const __m512i idx_odd = _mm512_setr_epi32(1, 3, 5, 7, 9, 11, 13, 15, 17, 19, 21, 23, 25, 27, 29, 31);
    for (size_t row = 0; row < m_w; ++row) {
        const uint8_t *rb = wp + row * k / 2;
        const float *rs = scales + row * groups;
        __m512 acc_total = _mm512_setzero_ps();
        for (size_t g = 0; g < groups; ++g) {
            __m512 scale_v = _mm512_set1_ps(rs[g]);
            __m512 group_acc = _mm512_setzero_ps();
            for (size_t blk = 0; blk < blocks; ++blk) {
                const uint8_t *p = rb + g * gs / 2 + blk * 16;
                const float *a = act + g * gs + blk * 32;
                __m256i p16 = _mm256_cvtepu8_epi16(_mm_loadu_si128((const __m128i *)p));
                __m256i lo = _mm256_srai_epi16(_mm256_slli_epi16(p16, 12), 12);
                __m256i hi = _mm256_srai_epi16(_mm256_slli_epi16(p16, 8), 12);
                __m512 lo_f = _mm512_cvtepi32_ps(_mm512_cvtepi16_epi32(lo));
                __m512 hi_f = _mm512_cvtepi32_ps(_mm512_cvtepi16_epi32(hi));
                __m512 a0 = _mm512_loadu_ps(a), a1 = _mm512_loadu_ps(a + 16);
                __m512 a_even = _mm512_permutex2var_ps(a0, idx_even, a1);
                __m512 a_odd = _mm512_permutex2var_ps(a0, idx_odd, a1);
                group_acc = _mm512_fmadd_ps(lo_f, a_even, group_acc);
                group_acc = _mm512_fmadd_ps(hi_f, a_odd, group_acc);
            }
            acc_total = _mm512_fmadd_ps(group_acc, scale_v, acc_total);
        }
        out[row] = _mm512_reduce_add_ps(acc_total);
    }
}

void ysb_int4_gemv(const uint8_t *wp, const float *scales, const float *act, float *out,
                   size_t m_w, size_t k, size_t gs) {
    if (has_avx512() && gs % 32 == 0)
        int4_gemv_avx512(wp, scales, act, out, m_w, k, gs);
    else
        yo_packed_int4_gemv(wp, scales, act, out, m_w, k, gs);
}

/* ---- int4 GEMM, AVX2 + FMA ------------------------------------------------ */

__attribute__((target("avx2,fma"))) static void
int4_gemm_avx2(const uint8_t *wp, const float *scales, const float *act, float *out,
               size_t m, size_t n, size_t k, size_t gs) {
    size_t groups = k / gs;
    float unpacked[256];
    memset(out, 0, m * n * sizeof(float));
    for (size_t nn = 0; nn < n; ++nn) {
        const uint8_t *rb = wp + nn * k / 2;
        const float *rs = scales + nn * groups;
        for (size_t g = 0; g < groups; ++g) {
            float scale = rs[g];
            for (size_t i = 0; i < gs / 2; ++i) {
                uint8_t b = rb[g * gs / 2 + i];
                unpacked[2 * i] = (float)yo_unpack_low(b);
                unpacked[2 * i + 1] = (float)yo_unpack_high(b);
            }
            for (size_t mi = 0; mi < m; ++mi) {
                const float *ar = act + mi * k + g * gs;
                __m256 acc = _mm256_setzero_ps();
                for (size_t j = 0; j + 8 <= gs; j += 8)
                    acc = _mm256_fmadd_ps(_mm256_loadu_ps(unpacked + j), _mm256_loadu_ps(ar + j), acc);
                float buf[8], sum = 0.0f;
                _mm256_storeu_ps(buf, acc);
                for (int t = 0; t < 8; ++t) sum += buf[t];
                out[mi * n + nn] += scale * sum;
            }
        }
    }
}

/* column slice [n0,n1) of the GEMM, used by the outer-parallel wrapper */
static void int4_gemm_cols(const uint8_t *wp, const float *scales, const float *act,
                           float *out, size_t m, size_t n, size_t k, size_t gs,
                           size_t n0, size_t n1) {
    size_t cols = n1 - n0, groups = k / gs;
    float *tmp = (float *)malloc(m * cols * sizeof(float));
    if (has_avx2() && gs % 8 == 0 && gs <= 256)
        int4_gemm_avx2(wp + n0 * k / 2, scales + n0 * groups, act, tmp, m, cols, k, gs);
    else
        yo_packed_int4_gemm(wp + n0 * k / 2, scales + n0 * groups, act, tmp, m, cols, k, gs);
    for (size_t mi = 0; mi < m; ++mi)
        memcpy(out + mi * n + n0, tmp + mi * cols, cols * sizeof(float));
    free(tmp);
}

void ysb_int4_gemm(const uint8_t *wp, const float *scales, const float *act, float *out,
                   size_t m, size_t n, size_t k, size_t gs) {
    if (has_avx2() && gs % 8 == 0 && gs <= 256)
        int4_gemm_avx2(wp, scales, act, out, m, n, k, gs);
    else
        yo_packed_int4_gemm(wp, scales, act, out, m, n, k, gs);
}

/* ---- int8 GEMM, AVX-512-VNNI ---------------------------------------------- */

/* bp[jp][g][c][r] = b[(4g+r)*n + 16jp + c]   (int8_matmul.rs:1815-1835) */
static int8_t *pack_b_vnni_4x16(const int8_t *b, size_t k, size_t n, size_t *k4_full) {
    size_t k4 = (k / 4) * 4, groups = k4 / 4, panels = n / 16;
    int8_t *bp = (int8_t *)malloc(panels * groups * 64 + 64);
    for (size_t jp = 0; jp < panels; ++jp)
        for (size_t g = 0; g < groups; ++g)
            for (size_t c = 0; c < 16; ++c)
                for (size_t r = 0; r < 4; ++r)
                    bp[(jp * groups + g) * 64 + c * 4 + r] = b[(g * 4 + r) * n + jp * 16 + c];
    *k4_full = k4;
    return bp;
}

#define VNNI_BLOCKED(NAME, MR)                                                          \
    __attribute__((target("avx512f,avx512bw,avx512vnni"))) static void NAME(           \
        const int8_t *a, const int8_t *b, size_t m, size_t k, size_t n, int32_t *out) { \
        size_t k4_full;                                                                 \
        int8_t *bp = pack_b_vnni_4x16(b, k, n, &k4_full);                               \
        size_t groups = k4_full / 4, panels = n / 16;                                   \
        int32_t *col_sum = (int32_t *)malloc(n * sizeof(int32_t));                      \
        for (size_t j = 0; j < n; ++j) {                                                \
            int32_t s = 0;                                                              \
            for (size_t kk = 0; kk < k4_full; ++kk) s += b[kk * n + j];                 \
            col_sum[j] = s;                                                             \
        }                                                                               \
        const __m512i bias_xor = _mm512_set1_epi8((char)-128);                          \
        for (size_t ib = 0; ib < m; ib += MR)                                           \
            for (size_t jp = 0; jp < panels; ++jp) {                                    \
                __m512i acc[MR];                                                        \
                for (int r = 0; r < MR; ++r) acc[r] = _mm512_setzero_si512();           \
                const int8_t *panel = bp + jp * groups * 64;                            \
                for (size_t g = 0; g < groups; ++g) {                                   \
                    __m512i bv = _mm512_loadu_si512((const void *)(panel + g * 64));    \
                    for (int r = 0; r < MR; ++r) {                                      \
                        int32_t ap;                                                     \
                        memcpy(&ap, a + (ib + r) * k + g * 4, 4);                       \
                        __m512i av = _mm512_xor_si512(_mm512_set1_epi32(ap), bias_xor); \
                        acc[r] = _mm512_dpbusd_epi32(acc[r], av, bv);                   \
                    }                                                                   \
                }                                                                       \
                int32_t buf[16];                                                        \
                for (int r = 0; r < MR; ++r) {                                          \
                    _mm512_storeu_si512((void *)buf, acc[r]);                           \
                    for (int c = 0; c < 16; ++c) {                                      \
                        size_t j = jp * 16 + c;                                         \
                        int32_t v = buf[c] - 128 * col_sum[j];                          \
                        for (size_t kk = k4_full; kk < k; ++kk)                         \
                            v += (int32_t)a[(ib + r) * k + kk] * (int32_t)b[kk * n + j]; \
                        out[(ib + r) * n + j] = v;                                      \
                    }                                                                   \
                }                                                                       \
            }                                                                           \
        free(col_sum);                                                                  \
        free(bp);                                                                       \
    }

VNNI_BLOCKED(int8_vnni_mr4, 4)
VNNI_BLOCKED(int8_vnni_mr8, 8)

/* simple B^T row-dot path with the XOR-0x80 bias shift (int8_matmul.rs:2125-2158).
 * bt/col_sum may be supplied by the caller (prepacked) or NULL (built here). */
__attribute__((target("avx512f,avx512bw,avx512vnni"))) static void
int8_vnni_simple(const int8_t *a, const int8_t *bt, const int32_t *col_sum, size_t m,
                 size_t k, size_t n, int32_t *out) {
    const __m512i bias128 = _mm512_set1_epi8((char)-128);
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            __m512i acc = _mm512_setzero_si512();
            size_t kk = 0;
            for (; kk + 64 <= k; kk += 64) {
                __m512i av = _mm512_loadu_si512((const void *)(a + i * k + kk));
                __m512i bv = _mm512_loadu_si512((const void *)(bt + j * k + kk));
                acc = _mm512_dpbusd_epi32(acc, _mm512_xor_si512(av, bias128), bv);
            }
            int32_t tail = _mm512_reduce_add_epi32(acc) - 128 * col_sum[j];
            for (; kk < k; ++kk) tail += (int32_t)a[i * k + kk] * (int32_t)bt[j * k + kk];
            out[i * n + j] = tail;
        }
}

static void col_sums_bt(const int8_t *bt, size_t k, size_t n, int32_t *col_sum) {
    size_t k_vnni = (k / 64) * 64;
    for (size_t j = 0; j < n; ++j) {
        int32_t s = 0;
        for (size_t kk = 0; kk < k_vnni; ++kk) s += bt[j * k + kk];
        col_sum[j] = s;
    }
}

/* int8_matmul_dispatch: B arrives [K,N]; transpose / pack happens per call,
 * exactly as in the reference's non-prepacked entry point. */
void ysb_int8_matmul(const int8_t *a, const int8_t *b, size_t m, size_t k, size_t n,
                     int32_t *out) {
    if (!has_vnni()) {
        yo_int8_matmul(a, b, m, k, n, out);
        return;
    }
    if (m >= 8 && m % 8 == 0 && n % 16 == 0 && k >= 8000 && n <= 2048) {
        int8_vnni_mr8(a, b, m, k, n, out);
        return;
    }
    if (m >= 4 && m % 4 == 0 && n % 16 == 0 && k >= 4 && (k * n <= 1000000 || n >= 16384)) {
        int8_vnni_mr4(a, b, m, k, n, out);
        return;
    }
    int8_t *bt = (int8_t *)malloc(k * n);
    int32_t *col_sum = (int32_t *)malloc(n * sizeof(int32_t));
    yo_transpose_b_i8(b, k, n, bt);
    col_sums_bt(bt, k, n, col_sum);
    int8_vnni_simple(a, bt, col_sum, m, k, n, out);
    free(col_sum);
    free(bt);
}

/* prepacked form: B^T [N,K] and its column sums are built once by the caller
 * (PackedI8B, int8_matmul.rs:128-191) and only the row-dot runs per call. */
void ysb_int8_matmul_prepacked(const int8_t *a, const int8_t *bt, size_t m, size_t k,
                               size_t n, int32_t *out) {
    if (!has_vnni()) {
        yo_int8_matmul_prepacked(a, bt, m, k, n, out);
        return;
    }
    int32_t *col_sum = (int32_t *)malloc(n * sizeof(int32_t));
    col_sums_bt(bt, k, n, col_sum);
    int8_vnni_simple(a, bt, col_sum, m, k, n, out);
    free(col_sum);
}

/* ---- outer-parallel wrappers --------------------------------------------- */

typedef struct {
    int kind; /* 0 gemv rows, 1 gemm cols, 2 int8 prepacked rows */
    const void *p0, *p1, *p2;
    void *out;
    size_t m, n, k, gs, lo, hi;
} job_t;

static void *job_main(void *arg) {
    job_t *j = (job_t *)arg;
    if (j->lo >= j->hi) return NULL;
    if (j->kind == 0) {
        size_t groups = j->k / j->gs;
        for (size_t mi = 0; mi < j->m; ++mi)
            ysb_int4_gemv((const uint8_t *)j->p0 + j->lo * j->k / 2,
                          (const float *)j->p1 + j->lo * groups,
                          (const float *)j->p2 + mi * j->k,
                          (float *)j->out + mi * j->n + j->lo, j->hi - j->lo, j->k, j->gs);
    } else if (j->kind == 1) {
        int4_gemm_cols((const uint8_t *)j->p0, (const float *)j->p1, (const float *)j->p2,
                       (float *)j->out, j->m, j->n, j->k, j->gs, j->lo, j->hi);
    } else {
        ysb_int8_matmul_prepacked((const int8_t *)j->p0 + j->lo * j->k, (const int8_t *)j->p1,
                                  j->hi - j->lo, j->k, j->n, (int32_t *)j->out + j->lo * j->n);
    }
    return NULL;
}

static void run_jobs(job_t proto, size_t extent, int threads) {
    if (threads < 1) threads = 1;
    pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    job_t *jobs = (job_t *)malloc(sizeof(job_t) * (size_t)threads);
    for (int t = 0; t < threads; ++t) {
        jobs[t] = proto;
        jobs[t].lo = extent * (size_t)t / (size_t)threads;
        jobs[t].hi = extent * (size_t)(t + 1) / (size_t)threads;
        pthread_create(&tid[t], NULL, job_main, &jobs[t]);
    }
    for (int t = 0; t < threads; ++t) pthread_join(tid[t], NULL);
    free(jobs);
    free(tid);
}

/* exec_matmul int4 branch (crates/yscv-onnx/src/runner/linear.rs:242-267) with
 * the weight rows split across `threads`: M < 8 -> M GEMV calls per slice,
 * else one GEMM per slice. */
void ysb_exec_matmul_int4_mt(const uint8_t *wp, const float *scales, const float *act,
                             float *out, size_t m, size_t n, size_t k, size_t gs,
                             int threads) {
    job_t j = {m >= 8 ? 1 : 0, wp, scales, act, out, m, n, k, gs, 0, 0};
    run_jobs(j, n, threads);
}

/* int8 GEMM against a prepacked B^T, rows of A split across `threads` */
void ysb_int8_matmul_prepacked_mt(const int8_t *a, const int8_t *bt, size_t m, size_t k,
                                  size_t n, int32_t *out, int threads) {
    job_t j = {2, a, bt, NULL, out, m, n, k, 0, 0, 0};
    run_jobs(j, m, threads);
}
