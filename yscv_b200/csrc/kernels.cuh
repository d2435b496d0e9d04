// Internal launch wrappers shared between the kernel files and the C ABI.
#pragma once
#include <stddef.h>
#include <stdint.h>

struct yscv_cuda_ctx;
struct yscv_cuda_i8b;

namespace yscv {

// int4_gemv.cu
bool int4_gemv_fast_supported(size_t m, size_t n, size_t k, size_t gs);
size_t int4_gemv_scratch_bytes(size_t m, size_t k);
// fp32 matmul out[m][n] = sum_k x[m][k] w[n][k] for m > 8 as three TF32 products per fp32 product
// on the tensor cores (f32_gemm_tf32x3.cu)
bool f32_gemm_tc_supported(const float *d_w, const float *d_x, size_t m, size_t n, size_t k);
size_t f32_gemm_tc_scratch_bytes(size_t m, size_t k);
int f32_gemm_tc(yscv_cuda_ctx *ctx, const float *d_w, const float *d_x, size_t m, size_t n, size_t k,
                float *d_out, void *scratch);
int int4_gemv_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales, const float *act,
                   float *out, size_t m, size_t n, size_t k, void *scratch);
int int4_gemv_generic(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                      const float *act, float *out, size_t m, size_t n, size_t k, size_t gs);

// int4_prefill_gemm.cu
bool int4_prefill_supported(size_t m, size_t n, size_t k, size_t gs);
size_t int4_prefill_scratch_bytes(size_t m, size_t k);
int int4_prefill_gemm(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales, const float *act,
                      float *out, size_t m, size_t n, size_t k, void *scratch, const void *act_bf16 = nullptr);

// int4_pack.cu
int pack_int4(yscv_cuda_ctx *ctx, const float *d_weights, size_t m_w, size_t k, size_t gs,
              uint8_t *d_packed, float *d_scales);

int int4_from_matmulnbits(yscv_cuda_ctx *ctx, const uint8_t *d_src, uint8_t *d_dst, size_t bytes);

// int8_gemm.cu
int pack_i8_b(yscv_cuda_ctx *ctx, const int8_t *d_b, size_t k, size_t n, int8_t *d_bt,
              int32_t *d_colsum, size_t kp);
int int8_gemm(yscv_cuda_ctx *ctx, const void *d_a, const yscv_cuda_i8b *b, size_t m, void *d_out,
              int a_unsigned, int a_zp, int mode, float composite, float y_zp, int qmin, int qmax,
              int round_mode, const int32_t *d_corr = nullptr, const float *d_comp_pc = nullptr,
              int relu = 0);

}  // namespace yscv
