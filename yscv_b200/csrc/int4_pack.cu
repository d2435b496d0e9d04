// pack_int4_symmetric_per_group on the GPU
// (reference: crates/yscv-kernels/src/ops/int4_matmul.rs:611-646).
//
// Bit-identical to the reference packer: abs-max per (row, group), scale =
// abs_max / 7 (1.0 when abs_max <= f32::EPSILON), inv = 1 / scale, and each
// element is quantised as clamp(round_ties_even(x * inv), -8, 7). Every float
// operation is a single IEEE round-to-nearest op (no FMA contraction, no
// approximate division), so packed bytes and scales match the CPU result
// exactly. One warp per (row, group).
#include "common.cuh"
#include "kernels.cuh"

namespace yscv {

__global__ void __launch_bounds__(256)
pack_int4_kernel(const float *__restrict__ w, uint8_t *__restrict__ packed,
                 float *__restrict__ scales, long long m_w, int k, int gs) {
    const int lane = threadIdx.x & 31;
    const int groups = k / gs;
    const long long total = m_w * groups;
    const long long wpb = blockDim.x >> 5;
    for (long long item = blockIdx.x * wpb + (threadIdx.x >> 5); item < total;
         item += (long long)gridDim.x * wpb) {
        const long long row = item / groups;
        const int g = (int)(item % groups);
        const float *slice = w + row * k + (long long)g * gs;
        float amax = 0.0f;
        for (int i = lane; i < gs; i += 32) amax = fmaxf(amax, fabsf(slice[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = (amax <= 1.1920929e-07f) ? 1.0f : __fdiv_rn(amax, 7.0f);
        const float inv = __fdiv_rn(1.0f, scale);
        if (lane == 0) scales[item] = scale;
        uint8_t *dst = packed + row * (k / 2) + (long long)g * (gs / 2);
        for (int i = lane; i < gs / 2; i += 32) {
            const float x0 = __fmul_rn(slice[2 * i], inv), x1 = __fmul_rn(slice[2 * i + 1], inv);
            // NaN -> 0, as Rust's saturating float-to-int cast does
            const int v0 = (x0 != x0) ? 0 : (int)fminf(fmaxf(rintf(x0), -8.0f), 7.0f);
            const int v1 = (x1 != x1) ? 0 : (int)fminf(fmaxf(rintf(x1), -8.0f), 7.0f);
            dst[i] = (uint8_t)((v0 & 0x0F) | ((v1 & 0x0F) << 4));
        }
    }
}

int pack_int4(yscv_cuda_ctx *ctx, const float *d_weights, size_t m_w, size_t k, size_t gs,
              uint8_t *d_packed, float *d_scales) {
    const long long total = (long long)m_w * (long long)(k / gs);
    const int blocks = (int)((total + 7) / 8 < (long long)(32 * ctx->sm_count)
                                 ? (total + 7) / 8
                                 : (long long)(32 * ctx->sm_count));
    pack_int4_kernel<<<blocks > 0 ? blocks : 1, 256, 0, ctx->stream>>>(
        d_weights, d_packed, d_scales, (long long)m_w, (int)k, (int)gs);
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    ctx->last_kernel = "pack_int4";
    return YSCV_CUDA_OK;
}

// MatMulNBits (4 bits, zero point 8) bytes -> two's-complement nibbles: every nibble q_u in
// [0,15] stands for q_u - 8, whose two's-complement nibble is q_u ^ 8.
__global__ void nbits_xor_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t bytes) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < bytes; i += stride)
        dst[i] = src[i] ^ 0x88u;
}

int int4_from_matmulnbits(yscv_cuda_ctx *ctx, const uint8_t *d_src, uint8_t *d_dst, size_t bytes) {
    if (bytes == 0) return YSCV_CUDA_OK;
    const size_t want = (bytes + 255) / 256;
    const int blocks = (int)(want < (size_t)(32 * ctx->sm_count) ? want : (size_t)(32 * ctx->sm_count));
    nbits_xor_kernel<<<blocks, 256, 0, ctx->stream>>>(d_src, d_dst, bytes);
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    return YSCV_CUDA_OK;
}

}  // namespace yscv
