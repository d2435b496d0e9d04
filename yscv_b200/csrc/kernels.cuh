// Internal launch wrappers shared between the kernel files and the C ABI.
#pragma once
#include <stddef.h>
#include <stdint.h>

struct yscv_cuda_ctx;

namespace yscv {

// int4_gemv.cu
bool int4_gemv_fast_supported(size_t m, size_t n, size_t k, size_t gs);
size_t int4_gemv_scratch_bytes(size_t m, size_t k);
int int4_gemv_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales, const float *act,
                   float *out, size_t m, size_t n, size_t k, void *scratch);
int int4_gemv_generic(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                      const float *act, float *out, size_t m, size_t n, size_t k, size_t gs);

// int4_pack.cu
int pack_int4(yscv_cuda_ctx *ctx, const float *d_weights, size_t m_w, size_t k, size_t gs,
              uint8_t *d_packed, float *d_scales);

}  // namespace yscv
