// fp32 x fp32 matmul for a wide decode batch (the fp32 LM head of the decoder,
// out[m][n] = sum_k x[m][k] * w[n][k], m > 8) on the 5th-generation tensor cores, keeping fp32
// accuracy: every operand is split into a TF32 part and a remainder,
//     x = x_hi + x_lo,   w = w_hi + w_lo,   x_hi = x with the low 13 mantissa bits cleared,
// and the product is accumulated in fp32 (TMEM) as w_hi*x_hi + w_hi*x_lo + w_lo*x_hi by
// tcgen05.mma.kind::tf32. The parts with cleared bits are exact TF32 values whatever the
// hardware does with the bits it does not use; the remainders keep 11 of their 13 significant
// bits: the relative error of a product is ~2^-21, that of the dropped w_lo*x_lo term 2^-22.
//
// Same orientation as the packed-int4 prefill GEMM: the weight rows are the MMA's M side (128 per
// tile), the batch rows its N side (BT <= 128 per pass). Per block of 32 k: TMA brings the weight
// tile [128][32] fp32 and the two activation tiles [BT][32] (x_hi, x_lo come from a small pre-pass
// over the activations), four warps split the weight tile (w_hi back in place, w_lo into one of two
// buffers; an element-wise pass, so the 128-byte swizzle of the tiles never has to be undone), one
// thread issues 12 MMAs (4 k steps of 8 x 3 products). The weights are read from HBM once.
//
// The tensor core adds into its fp32 accumulator by truncation, so a long chain of accumulations
// drifts toward zero: one accumulator over K = 2048 (768 MMAs) came out with a relative error of
// 1.8e-5, over K = 8192 with 6e-5, ten to thirty times what fp32 FMAs leave. So an accumulator
// only ever collects FT_KC blocks (64 k, 24 MMAs); the epilogue warps drain it into fp32 registers
// with ordinary rounded adds while the MMAs fill the other buffer, and store once per tile. That
// bounds the drift by the chunk length, whatever K is (measured ~1e-6).
// Persistent CTAs, all waits bounded.
#include "common.cuh"
#include "kernels.cuh"
#include "tma.cuh"

namespace yscv {

constexpr int FT_BM = 128;       // weight rows per tile
constexpr int FT_BK = 32;        // fp32 per 128-byte swizzle row
constexpr int FT_SPLIT_WARPS = 4;
constexpr int FT_EPI_WARPS = 8;  // two per TMEM lane quadrant: columns 0..63 and 64..127 of the accumulator
constexpr int FT_THREADS = (2 + FT_SPLIT_WARPS + FT_EPI_WARPS) * 32;
constexpr int FT_KC = 2;         // k blocks per accumulator chunk
constexpr int FT_MIN_STAGES2 = 2; // ring stages needed to carry two blocks per stage
constexpr int FT_BT_MAX = 128;   // batch rows per pass: 64 accumulator columns per epilogue thread
constexpr int FT_W_BYTES = FT_BM * FT_BK * 4;   // 16 KB

struct FTParams {
    int M, N, K;
    int BT;                 // batch rows per pass (multiple of 16, <= FT_BT_MAX)
    int n_tiles, t_chunks, k_blocks;   // k_blocks counts ring stages (KSUB blocks of 32 k each)
    int stages, stage_bytes;
};

__device__ __forceinline__ void ft_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void ft_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// K-major tile, 128-byte swizzle, rows 128 bytes apart, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t ft_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void ft_mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void ft_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void ft_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

constexpr uint32_t FT_HI_MASK = 0xFFFFE000u;   // sign, exponent, 10 mantissa bits

// activations -> x_hi (low 13 mantissa bits cleared) and x_lo = x - x_hi (exact)
__global__ void __launch_bounds__(256) ft_split_act_kernel(const float4 *__restrict__ x, float4 *__restrict__ hi,
                                                           float4 *__restrict__ lo, size_t n4) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = x[i];
        float4 h;
        h.x = __uint_as_float(__float_as_uint(v.x) & FT_HI_MASK);
        h.y = __uint_as_float(__float_as_uint(v.y) & FT_HI_MASK);
        h.z = __uint_as_float(__float_as_uint(v.z) & FT_HI_MASK);
        h.w = __uint_as_float(__float_as_uint(v.w) & FT_HI_MASK);
        hi[i] = h;
        lo[i] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
    }
}

// KSUB = blocks of 32 k per ring stage and hand-over (split tile -> MMA -> buffer back): 2 whenever K
// allows, a hand-over costs over a thousand cycles whatever it carries. A stage holds
// [KSUB weight tiles][KSUB x_hi tiles][KSUB x_lo tiles], a remainder buffer KSUB tiles.
template <int KSUB>
__global__ void __launch_bounds__(FT_THREADS, 1)
f32_gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_xh,
                       const __grid_constant__ CUtensorMap tm_xl, float *__restrict__ out, FTParams p,
                       int *__restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = smem_u32(smem);
    // [w_lo buffer 0][w_lo buffer 1][stages x {weight tile | x_hi tile | x_lo tile}][barriers][tmem slot]
    constexpr int LO_BUF = KSUB * FT_W_BYTES;
    constexpr int CHUNK_STAGES = FT_KC / KSUB;   // ring stages per accumulator chunk
    const uint32_t lo_tiles = smem_base;
    const uint32_t ring = smem_base + 2 * LO_BUF;
    const int x_bytes = p.BT * 128;
    const uint32_t bars = ring + (uint32_t)p.stages * p.stage_bytes;
    const uint32_t bar_full = bars, bar_empty = bars + 64, bar_afull = bars + 128, bar_aempty = bars + 144;
    const uint32_t bar_tfull = bars + 160, bar_tempty = bars + 176;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 2 * LO_BUF + (size_t)p.stages * p.stage_bytes + 192);
    const int tiles = p.n_tiles * p.t_chunks;

    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(bar_full + i * 8, 1);
            mbar_init(bar_empty + i * 8, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_afull + i * 8, FT_SPLIT_WARPS);
            mbar_init(bar_aempty + i * 8, 1);
            mbar_init(bar_tfull + i * 8, 1);
            mbar_init(bar_tempty + i * 8, FT_EPI_WARPS);
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    ft_fence_before();
    __syncthreads();
    ft_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the activation parts come from the pre-pass, the output may still be read by a predecessor
    pdl_wait();
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
                const int nt_i = t % p.n_tiles, tc = t / p.n_tiles;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    alive = mbar_wait(bar_empty + slot * 8, phase ^ 1u, status);
                    if (!alive) break;
                    const uint32_t st = ring + (uint32_t)slot * p.stage_bytes;
                    const uint32_t full = bar_full + slot * 8;
                    mbar_expect_tx(full, (uint32_t)(KSUB * (FT_W_BYTES + 2 * x_bytes)));
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        const int kx = (kb * KSUB + sub) * FT_BK;
                        tma_load_2d(st + sub * FT_W_BYTES, &tm_w, kx, nt_i * FT_BM, full);
                        tma_load_2d(st + KSUB * FT_W_BYTES + sub * x_bytes, &tm_xh, kx, tc * p.BT, full);
                        tma_load_2d(st + KSUB * FT_W_BYTES + (KSUB + sub) * x_bytes, &tm_xl, kx, tc * p.BT, full);
                    }
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // D fp32, A and B TF32, both K-major, N = BT, M = 128
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(p.BT >> 3) << 17) |
                                   ((uint32_t)(FT_BM >> 4) << 24);
            int slot = 0, abuf = 0, tbuf = 0;
            uint32_t phase = 0, aphase = 0, tphase = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    const bool chunk_start = kb % CHUNK_STAGES == 0;
                    if (chunk_start) {
                        // the epilogue has drained this accumulator buffer
                        alive = mbar_wait(bar_tempty + tbuf * 8, tphase ^ 1u, status);
                        if (!alive) break;
                    }
                    alive = mbar_wait(bar_afull + abuf * 8, aphase, status);   // implies the stage has landed
                    if (!alive) break;
                    ft_fence_after();
                    const uint32_t tacc = tmem_base + (uint32_t)tbuf * FT_BT_MAX;
                    const uint32_t st = ring + (uint32_t)slot * p.stage_bytes;
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        const uint64_t d_whi = ft_desc_sw128(st + sub * FT_W_BYTES);
                        const uint64_t d_wlo = ft_desc_sw128(lo_tiles + abuf * LO_BUF + sub * FT_W_BYTES);
                        const uint64_t d_xhi = ft_desc_sw128(st + KSUB * FT_W_BYTES + sub * x_bytes);
                        const uint64_t d_xlo = ft_desc_sw128(st + KSUB * FT_W_BYTES + (KSUB + sub) * x_bytes);
#pragma unroll
                        for (int kk = 0; kk < FT_BK / 8; ++kk) {   // K = 8 per instruction: +32 bytes
                            const uint64_t o = (uint64_t)(kk * 2);
                            ft_mma_tf32(tacc, d_wlo + o, d_xhi + o, idesc, (!chunk_start || sub > 0 || kk > 0) ? 1u : 0u);
                            ft_mma_tf32(tacc, d_whi + o, d_xlo + o, idesc, 1u);
                            ft_mma_tf32(tacc, d_whi + o, d_xhi + o, idesc, 1u);
                        }
                    }
                    ft_commit(bar_empty + slot * 8);
                    ft_commit(bar_aempty + abuf * 8);
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                    if (++abuf == 2) { abuf = 0; aphase ^= 1u; }
                    if (kb % CHUNK_STAGES == CHUNK_STAGES - 1 || kb == p.k_blocks - 1) {
                        ft_commit(bar_tfull + tbuf * 8);   // chunk complete
                        if (++tbuf == 2) { tbuf = 0; tphase ^= 1u; }
                    }
                }
            }
        }
    } else if (warp < 2 + FT_SPLIT_WARPS) {
        // ------- split: thread r owns weight row r of the tile (128 bytes = eight 16-byte pieces) -------
        const int r = (warp - 2) * 32 + lane;
        int slot = 0, abuf = 0;
        uint32_t phase = 0, aphase = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                alive = mbar_wait(bar_full + slot * 8, phase, status) &&
                        mbar_wait(bar_aempty + abuf * 8, aphase ^ 1u, status);
                if (!alive) break;
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub) {
                    unsigned char *wrow = smem + 2 * LO_BUF + (size_t)slot * p.stage_bytes + (size_t)sub * FT_W_BYTES + (size_t)r * 128;
                    unsigned char *lrow = smem + (size_t)abuf * LO_BUF + (size_t)sub * FT_W_BYTES + (size_t)r * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        // an element-wise pass: the pieces of a row in an order that spreads a quarter warp over all banks
                        const int off = ((c + r) & 7) << 4;
                        const uint4 v = *reinterpret_cast<const uint4 *>(wrow + off);
                        uint4 h, l;
                        h.x = v.x & FT_HI_MASK; h.y = v.y & FT_HI_MASK; h.z = v.z & FT_HI_MASK; h.w = v.w & FT_HI_MASK;
                        l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(h.x));
                        l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(h.y));
                        l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(h.z));
                        l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(h.w));
                        *reinterpret_cast<uint4 *>(wrow + off) = h;
                        *reinterpret_cast<uint4 *>(lrow + off) = l;
                    }
                }
                // make the generic-proxy writes visible to the tensor core's async proxy
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_afull + abuf * 8);
                if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                if (++abuf == 2) { abuf = 0; aphase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue: eight warps, TMEM lanes 32*(warp%4).., columns 64*half.. ----------------
        const int q = warp & 3, half = (warp - 2 - FT_SPLIT_WARPS) >> 2;
        const int col_base = half * 64;
        const int n_chunks = (p.k_blocks + CHUNK_STAGES - 1) / CHUNK_STAGES;
        int tbuf = 0;
        uint32_t tphase = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
            const int nt_i = t % p.n_tiles, tc = t / p.n_tiles;
            float acc[2][32];
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[c][j] = 0.0f;
            for (int ch = 0; ch < n_chunks && alive; ++ch) {
                alive = mbar_wait(bar_tfull + tbuf * 8, tphase, status);
                if (!alive) break;
                ft_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(tbuf * FT_BT_MAX + col_base);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    if (col_base + c * 32 < p.BT) {   // the same for the whole warp
                        uint32_t rr[32];
                        ft_tmem_ld32(taddr + c * 32, rr);
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[c][j] += __uint_as_float(rr[j]);
                    }
                }
                ft_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_tempty + tbuf * 8);
                if (++tbuf == 2) { tbuf = 0; tphase ^= 1u; }
            }
            if (!alive) break;
            const int n = nt_i * FT_BM + q * 32 + lane;   // output column (weight row) of this lane
            if (n < p.N) {
#pragma unroll
                for (int c = 0; c < 2; ++c) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = col_base + c * 32 + j, row = tc * p.BT + col;
                        if (col < p.BT && row < p.M) out[(size_t)row * p.N + n] = acc[c][j];
                    }
                }
            }
        }
    }

    ft_fence_before();
    __syncthreads();
    if (warp == 1) {
        ft_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

bool f32_gemm_tc_supported(const float *d_w, const float *d_x, size_t m, size_t n, size_t k) {
    return tensor_map_encoder() != nullptr && m > 8 && n >= 1 && k >= FT_BK && k % FT_BK == 0 &&
           ((reinterpret_cast<uintptr_t>(d_w) | reinterpret_cast<uintptr_t>(d_x)) & 15) == 0 &&
           m < (1u << 30) && n < (1u << 30) && k < (1u << 30);
}

size_t f32_gemm_tc_scratch_bytes(size_t m, size_t k) { return 2 * m * k * sizeof(float) + 256; }

// d_w [n][k], d_x [m][k], d_out [m][n]; scratch: f32_gemm_tc_scratch_bytes(m, k)
int f32_gemm_tc(yscv_cuda_ctx *ctx, const float *d_w, const float *d_x, size_t m, size_t n, size_t k,
                float *d_out, void *scratch) {
    FTParams p = {};
    p.M = (int)m;
    p.N = (int)n;
    p.K = (int)k;
    const int m16 = (int)((m + 15) / 16 * 16);
    p.BT = m16 <= FT_BT_MAX ? m16 : FT_BT_MAX;
    p.n_tiles = (p.N + FT_BM - 1) / FT_BM;
    p.t_chunks = (p.M + p.BT - 1) / p.BT;
    // two blocks per stage and hand-over when K allows and the ring still has at least two such stages
    int ksub = p.K % (2 * FT_BK) == 0 ? 2 : 1;
    for (;; ksub = 1) {
        p.stage_bytes = ((ksub * (FT_W_BYTES + 2 * p.BT * 128) + 1023) / 1024) * 1024;
        p.stages = (227 * 1024 - 2 * ksub * FT_W_BYTES - 1024) / p.stage_bytes;
        if (p.stages >= FT_MIN_STAGES2 || ksub == 1) break;
    }
    p.k_blocks = p.K / (FT_BK * ksub);
    if (p.stages > 8) p.stages = 8;
    const int smem = 2 * ksub * FT_W_BYTES + p.stages * p.stage_bytes + 256;

    float *x_hi = reinterpret_cast<float *>(scratch), *x_lo = x_hi + m * k;
    const size_t n4 = m * k / 4;
    const unsigned sb = (unsigned)((n4 + 255) / 256 < 2368 ? (n4 + 255) / 256 : 2368);
    YSCV_CUDA_TRY(launch_pdl(ft_split_act_kernel, dim3(sb), dim3(256), 0, ctx->stream,
                             reinterpret_cast<const float4 *>(d_x), reinterpret_cast<float4 *>(x_hi),
                             reinterpret_cast<float4 *>(x_lo), n4));
    ctx->launches++;

    CUtensorMap tm_w, tm_xh, tm_xl;
    int rc = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, d_w, n, k, k * 4, FT_BM, FT_BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = encode_2d(&tm_xh, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x_hi, m, k, k * 4, (uint32_t)p.BT, FT_BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = encode_2d(&tm_xl, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, x_lo, m, k, k * 4, (uint32_t)p.BT, FT_BK, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    auto kern = ksub == 2 ? f32_gemm_tf32x3_kernel<2> : f32_gemm_tf32x3_kernel<1>;
    rc = ensure_dynamic_smem(reinterpret_cast<const void *>(kern), ctx->device, 227 * 1024);
    if (rc) return rc;
    const int tiles = p.n_tiles * p.t_chunks;
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    YSCV_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(FT_THREADS), (size_t)smem, ctx->stream, tm_w, tm_xh, tm_xl, d_out, p,
                             ctx->d_status));
    ctx->launches++;
    return YSCV_CUDA_OK;
}

}  // namespace yscv
