// Decode-shaped (M <= 16) packed-int4 x fp32 matmul for sm_100a.
//
// Replaces packed_int4_gemv_dispatch / the M < GEMM_THRESHOLD loop of the
// reference (crates/yscv-kernels/src/ops/int4_matmul.rs:44-81, 310-377;
// crates/yscv-onnx/src/runner/linear.rs:242-267). Same operands and layouts:
// weights [N][K/2] bytes (two's-complement nibbles, low nibble = even k),
// scales [N][K/group] f32, activations [M][K] f32, output [M][N] f32.
//
// Two kernels:
//
//  * int4_gemv_generic_kernel: any even group size, any K. One warp per weight
//    row, fp32 FMAs, warp-shuffle K reduction. Used for shapes the fast kernel
//    does not take (group != 32, K % 256 != 0).
//
//  * int4_gemv_fast_kernel: group 32, K % 256 == 0. The op is HBM-bound, and
//    on a B200 a nibble has to cost less than ~2 issue slots for the SMs to
//    keep up with 6.5 TB/s. Unpacking to fp32 on the CUDA cores costs >= 3
//    (isolate, convert, FMA) per nibble *per activation row*, so the dot
//    products run on the integer tensor path instead, without giving up fp32
//    accuracy: each group of 32 activations is turned once (act_quant_kernel)
//    into a 22-bit block-fixed-point number, split into three signed 8-bit
//    digit planes; the per-group integer dot  sum_j q_j * afix_j  is then exact
//    in int32 (three mma.sync.m16n8k32.u8.s8 with a x256 between them), and only
//    the per-(row,group) scale is applied in fp32. Weights are staged through
//    shared memory by 16-byte cp.async in a multi-stage ring (coalesced 128-bit
//    loads, no register cost for bytes in flight), read back conflict-free
//    through an XOR swizzle, and turned into MMA fragments with 3 logic ops per
//    8 nibbles. One persistent CTA per SM owns a contiguous row range; inside
//    the CTA the K range of a stage is split across warps and the partial sums
//    are combined in a fixed order (deterministic, no atomics).
#include "common.cuh"
#include "kernels.cuh"

namespace yscv {

// ---------------------------------------------------------------------------
// Generic kernel
// ---------------------------------------------------------------------------

__device__ __forceinline__ float nib_lo(uint32_t w, int j) {
    // sign-extended nibble j (0..7) of a 32-bit word
    return (float)(((int32_t)(w << (28 - 4 * j))) >> 28);
}

template <int MT>
__global__ void __launch_bounds__(256)
int4_gemv_generic_kernel(const uint8_t *__restrict__ wq, const float *__restrict__ scales,
                         const float *__restrict__ act, float *__restrict__ out, int m0,
                         int M, int N, int K, int gs, int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    const int groups = K / gs;
    const int mt = min(MT, M - m0);
    for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < N;
         row += gridDim.x * warps_per_block) {
        const uint8_t *rb = wq + (size_t)row * (K / 2);
        const float *rs = scales + (size_t)row * groups;
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
        if (vec_ok) {
            // 16 bytes = 32 nibbles per step; gs % 32 == 0 keeps them in one group
            for (int c = lane; c < K / 32; c += 32) {
                const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(rb) + c);
                const float s = __ldg(rs + (c * 32) / gs);
                const uint32_t w4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    if (i < mt) {
                        const float4 *a4 =
                            reinterpret_cast<const float4 *>(act + (size_t)(m0 + i) * K + c * 32);
                        float g = 0.0f;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 x0 = __ldg(a4 + 2 * q), x1 = __ldg(a4 + 2 * q + 1);
                            const uint32_t w = w4[q];
                            g = fmaf(nib_lo(w, 0), x0.x, g);
                            g = fmaf(nib_lo(w, 1), x0.y, g);
                            g = fmaf(nib_lo(w, 2), x0.z, g);
                            g = fmaf(nib_lo(w, 3), x0.w, g);
                            g = fmaf(nib_lo(w, 4), x1.x, g);
                            g = fmaf(nib_lo(w, 5), x1.y, g);
                            g = fmaf(nib_lo(w, 6), x1.z, g);
                            g = fmaf(nib_lo(w, 7), x1.w, g);
                        }
                        acc[i] = fmaf(s, g, acc[i]);
                    }
                }
            }
        } else {
            for (int b = lane; b < K / 2; b += 32) {
                const uint32_t byte = rb[b];
                const float s = rs[(2 * b) / gs];
                const float lo = nib_lo(byte, 0), hi = nib_lo(byte, 1);
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    if (i < mt) {
                        const float *a = act + (size_t)(m0 + i) * K + 2 * b;
                        acc[i] = fmaf(s, fmaf(hi, a[1], lo * a[0]), acc[i]);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            float v = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && i < mt) out[(size_t)(m0 + i) * N + row] = v;
        }
    }
}

// ---------------------------------------------------------------------------
// Activation -> digit planes
// ---------------------------------------------------------------------------
//
// For activation row m and group G (32 consecutive k):
//   e     : max|a| < 2^e
//   afix_j = rint(a_j * 2^(21-e))                 |afix| <= 2^21
//   afix  = d2*65536 + d1*256 + d0                d0,d1 in [-128,127], |d2| <= 32
// Output layout (uint4 = 4 words):
//   digits[((G*2 + h)*MP + m)*4 + t]  h=0: {d2.b0, d2.b1, d1.b0, d1.b1}
//                                     h=1: {d0.b0, d0.b1, 0, 0}
//     b0 = digits of k = 8t+{0,2,4,6}, b1 = digits of k = 8t+{1,3,5,7}
//     (the B fragment of mma.m16n8k32 for column m, thread-in-quad t)
//   meta[G*MP + m] = { 2^(e-21) as float, 8 * sum_j afix_j as int }
// Rows m >= M (padding up to MP) are written as zeros.
__global__ void __launch_bounds__(256)
act_quant_kernel(const float *__restrict__ act, uint4 *__restrict__ digits,
                 int2 *__restrict__ meta, int M, int MP, int K) {
    const int lane = threadIdx.x & 31;
    const int groups = K / 32;
    const int total = groups * MP;
    for (int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < total;
         item += gridDim.x * (blockDim.x >> 5)) {
        const int G = item / MP, m = item % MP;
        const float v = (m < M) ? act[(size_t)m * K + G * 32 + lane] : 0.0f;
        float gmax = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
        // a non-finite activation poisons the whole group, as it would in fp32
        const bool bad = !(gmax <= 3.0e38f) || (__ballot_sync(0xffffffffu, v != v) != 0u);
        int e = 0;
        if (gmax > 0.0f && !bad) (void)frexpf(gmax, &e);
        e = max(e, -100);  // keeps 2^(21-e) finite for vanishing groups
        const float up = ldexpf(1.0f, 21 - e);
        int fx = bad ? 0 : __float2int_rn(v * up);
        int sum = fx;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const int d0 = ((fx + 128) & 255) - 128;
        const int r1 = (fx - d0) >> 8;
        const int d1 = ((r1 + 128) & 255) - 128;
        const int d2 = (r1 - d1) >> 8;
        const uint32_t dp = (uint32_t)(d0 & 255) | ((uint32_t)(d1 & 255) << 8) |
                            ((uint32_t)(d2 & 255) << 16);
        const int t = lane & 3;
        uint32_t b0[3] = {0, 0, 0}, b1[3] = {0, 0, 0};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t ev = __shfl_sync(0xffffffffu, dp, 8 * t + 2 * i);
            const uint32_t od = __shfl_sync(0xffffffffu, dp, 8 * t + 2 * i + 1);
#pragma unroll
            for (int d = 0; d < 3; ++d) {
                b0[d] |= ((ev >> (8 * d)) & 255u) << (8 * i);
                b1[d] |= ((od >> (8 * d)) & 255u) << (8 * i);
            }
        }
        if (lane < 4) {
            digits[((size_t)(G * 2 + 0) * MP + m) * 4 + t] = make_uint4(b0[2], b1[2], b0[1], b1[1]);
            digits[((size_t)(G * 2 + 1) * MP + m) * 4 + t] = make_uint4(b0[0], b1[0], 0u, 0u);
        }
        if (lane == 0) {
            const float as = bad ? __int_as_float(0x7fc00000) : ldexpf(1.0f, e - 21);
            meta[(size_t)G * MP + m] = make_int2(__float_as_int(as), 8 * sum);
        }
    }
}

// ---------------------------------------------------------------------------
// Fast kernel
// ---------------------------------------------------------------------------

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int sz = valid ? 16 : 0;  // src-size 0 => 16 bytes of zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_dyn(int n) {
    switch (n) {
        case 0: asm volatile("cp.async.wait_group 0;\n" ::); break;
        case 1: asm volatile("cp.async.wait_group 1;\n" ::); break;
        case 2: asm volatile("cp.async.wait_group 2;\n" ::); break;
        case 3: asm volatile("cp.async.wait_group 3;\n" ::); break;
        case 4: asm volatile("cp.async.wait_group 4;\n" ::); break;
        case 5: asm volatile("cp.async.wait_group 5;\n" ::); break;
        case 6: asm volatile("cp.async.wait_group 6;\n" ::); break;
        default: asm volatile("cp.async.wait_group 7;\n" ::); break;
    }
}

__device__ __forceinline__ void mma_u8s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// (w ^ 0x88888888) & 0x0f0f0f0f in one LOP3: unsigned nibbles q+8 as bytes
__device__ __forceinline__ uint32_t nib_u8(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x88888888, 0x0f0f0f0f, 0x28;\n" : "=r"(r) : "r"(w));
    return r;
}

struct FastGeom {
    int tiles;        // 16-row tiles per row block (1..8)
    int tiles_pow2;   // next power of two
    int kslices;      // warps sharing one tile along K
    int stages;       // ring depth
    int w_bytes, s_bytes, d_bytes, a_bytes, stage_bytes;
    int s_pitch;      // floats per row in the scale tile
};

// GS = groups (of 32 k) per stage: 16 (512 k) or 8 (256 k). MP = padded M.
template <int MP, int GS>
__global__ void __launch_bounds__(512, 1)
int4_gemv_fast_kernel(const uint8_t *__restrict__ wq, const float *__restrict__ scales,
                      const uint4 *__restrict__ digits, const int2 *__restrict__ meta,
                      float *__restrict__ out, int M, int N, int K, FastGeom g) {
    constexpr int NT = (MP > 8) ? 2 : 1;
    constexpr int ATOMS = GS / 8;  // 128-byte swizzle atoms per row per stage
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t = lane & 3;

    const int r0 = (int)(((long long)N * blockIdx.x) / gridDim.x);
    const int r1 = (int)(((long long)N * (blockIdx.x + 1)) / gridDim.x);
    if (r0 >= r1) return;
    const int rb_rows = g.tiles * 16;
    const int n_rb = (r1 - r0 + rb_rows - 1) / rb_rows;
    const int k_stages = K / (GS * 32);
    const int total = n_rb * k_stages;
    const int groups = K / 32;

    float *red = reinterpret_cast<float *>(smem + (size_t)g.stages * g.stage_bytes);

    auto issue = [&](int it) {
        const int rb = it / k_stages, ks = it % k_stages;
        const int row0 = r0 + rb * rb_rows;
        unsigned char *st = smem + (size_t)(it % g.stages) * g.stage_bytes;
        // weights: rb_rows x (GS*16) bytes, 16-byte chunks, chunk ^= row&7 inside each atom
        const int wchunks = rb_rows * GS;
        for (int i = tid; i < wchunks; i += 512) {
            const int r = i / GS, c = i % GS;
            const int atom = c >> 3, cc = c & 7;
            unsigned char *dst = st + atom * (rb_rows * 128) + r * 128 + ((cc ^ (r & 7)) << 4);
            const int row = row0 + r;
            const bool ok = row < r1;
            const uint8_t *src = wq + (size_t)(ok ? row : r0) * (K / 2) + (size_t)ks * (GS * 16) + c * 16;
            cp_async16(dst, src, ok);
        }
        // scales: rb_rows x GS floats, row pitch s_pitch floats
        unsigned char *ss = st + g.w_bytes;
        const int schunks = rb_rows * (GS / 4);
        for (int i = tid; i < schunks; i += 512) {
            const int r = i / (GS / 4), c = i % (GS / 4);
            const int row = row0 + r;
            const bool ok = row < r1;
            const float *src = scales + (size_t)(ok ? row : r0) * groups + ks * GS + c * 4;
            cp_async16(ss + r * (g.s_pitch * 4) + c * 16, src, ok);
        }
        // digit planes of this K range: GS*2*MP*4 uint4, contiguous
        unsigned char *ds = ss + g.s_bytes;
        const int dchunks = GS * 2 * MP * 4;
        const uint4 *dsrc = digits + (size_t)ks * dchunks;
        for (int i = tid; i < dchunks; i += 512) cp_async16(ds + i * 16, dsrc + i, true);
        // meta: GS*MP int2
        unsigned char *as = ds + g.d_bytes;
        const int achunks = (GS * MP * 8 + 15) / 16;
        const unsigned char *asrc = reinterpret_cast<const unsigned char *>(meta + (size_t)ks * GS * MP);
        for (int i = tid; i < achunks; i += 512) cp_async16(as + i * 16, asrc + i * 16, true);
    };

    for (int p = 0; p < g.stages - 1; ++p) {
        if (p < total) issue(p);
        cp_async_commit();
    }

    const int tile = warp % g.tiles_pow2;
    const int kslice = warp / g.tiles_pow2;
    const bool active = (tile < g.tiles) && (kslice < g.kslices);
    const int gpw = GS / g.kslices;  // groups per warp per stage

    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[n][j] = 0.0f;

    for (int it = 0; it < total; ++it) {
        cp_async_wait_dyn(g.stages - 2);
        __syncthreads();
        {
            const int nxt = it + g.stages - 1;
            if (nxt < total) issue(nxt);
            cp_async_commit();
        }
        const unsigned char *st = smem + (size_t)(it % g.stages) * g.stage_bytes;
        if (active) {
            const float *ss = reinterpret_cast<const float *>(st + g.w_bytes);
            const uint4 *ds = reinterpret_cast<const uint4 *>(st + g.w_bytes + g.s_bytes);
            const int2 *as = reinterpret_cast<const int2 *>(st + g.w_bytes + g.s_bytes + g.d_bytes);
            const int rowA = tile * 16 + gq, rowB = rowA + 8;
#pragma unroll 4
            for (int gi = 0; gi < gpw; ++gi) {
                const int G = kslice * gpw + gi;
                const int atom = G >> 3, cc = G & 7;
                const unsigned char *wa = st + atom * (rb_rows * 128);
                const uint32_t wA = *reinterpret_cast<const uint32_t *>(
                    wa + rowA * 128 + ((cc ^ (rowA & 7)) << 4) + t * 4);
                const uint32_t wB = *reinterpret_cast<const uint32_t *>(
                    wa + rowB * 128 + ((cc ^ (rowB & 7)) << 4) + t * 4);
                uint32_t a[4];
                a[0] = nib_u8(wA);
                a[1] = nib_u8(wB);
                a[2] = nib_u8(wA >> 4);
                a[3] = nib_u8(wB >> 4);
                const float sA = ss[rowA * g.s_pitch + G], sB = ss[rowB * g.s_pitch + G];
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const int mcol = n * 8 + gq;  // activation row this thread feeds as B column
                    uint4 h0 = make_uint4(0, 0, 0, 0), h1 = make_uint4(0, 0, 0, 0);
                    if (mcol < MP) {
                        h0 = ds[((G * 2 + 0) * MP + mcol) * 4 + t];
                        h1 = ds[((G * 2 + 1) * MP + mcol) * 4 + t];
                    }
                    // columns of the accumulator fragment this thread owns: 2t, 2t+1
                    const int c0 = n * 8 + 2 * t;
                    int2 m0 = make_int2(0, 0), m1 = make_int2(0, 0);
                    if (c0 < MP) m0 = as[G * MP + c0];
                    if (c0 + 1 < MP) m1 = as[G * MP + c0 + 1];
                    int c[4] = {0, 0, 0, 0};
                    mma_u8s8(c, a, h0.x, h0.y);  // d2
                    c[0] <<= 8; c[1] <<= 8; c[2] <<= 8; c[3] <<= 8;
                    mma_u8s8(c, a, h0.z, h0.w);  // d1
                    c[0] = c[0] * 256 - m0.y;    // fold the -8*sum(afix) of the +8 nibble bias
                    c[1] = c[1] * 256 - m1.y;
                    c[2] = c[2] * 256 - m0.y;
                    c[3] = c[3] * 256 - m1.y;
                    mma_u8s8(c, a, h1.x, h1.y);  // d0
                    const float as0 = __int_as_float(m0.x), as1 = __int_as_float(m1.x);
                    acc[n][0] = fmaf(sA * as0, (float)c[0], acc[n][0]);
                    acc[n][1] = fmaf(sA * as1, (float)c[1], acc[n][1]);
                    acc[n][2] = fmaf(sB * as0, (float)c[2], acc[n][2]);
                    acc[n][3] = fmaf(sB * as1, (float)c[3], acc[n][3]);
                }
            }
        }
        if ((it % k_stages) == k_stages - 1) {
            // end of a row block: combine the K slices in a fixed order and store
            if (active) {
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        red[(((kslice * g.tiles + tile) * NT + n) * 4 + j) * 32 + lane] = acc[n][j];
            }
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[n][j] = 0.0f;
            __syncthreads();
            const int row0 = r0 + (it / k_stages) * rb_rows;
            const int items = g.tiles * NT * 128;
            for (int i = tid; i < items; i += 512) {
                const int l = i & 31, j = (i >> 5) & 3, n = (i >> 7) % NT, tl = (i >> 7) / NT;
                float v = 0.0f;
                for (int ks = 0; ks < g.kslices; ++ks)
                    v += red[(((ks * g.tiles + tl) * NT + n) * 4 + j) * 32 + l];
                const int row = row0 + tl * 16 + (l >> 2) + ((j & 2) ? 8 : 0);
                const int m = n * 8 + 2 * (l & 3) + (j & 1);
                if (row < r1 && m < M) out[(size_t)m * N + row] = v;
            }
            // `red` is next written after at least one more __syncthreads (top of the loop)
        }
    }
    cp_async_wait_dyn(0);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

static int padded_m(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16; }

size_t int4_gemv_scratch_bytes(size_t m, size_t k) {
    const size_t mp = (size_t)padded_m((int)m);
    return (k / 32) * 2 * mp * 4 * 16 + (k / 32) * mp * 8 + 256;
}

bool int4_gemv_fast_supported(size_t m, size_t n, size_t k, size_t gs) {
    return gs == 32 && k % 256 == 0 && k >= 256 && m >= 1 && m <= 16 && n >= 1 &&
           n < (1u << 30) && k < (1u << 24);
}

template <int MP, int GS>
static int launch_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                       const uint4 *digits, const int2 *meta, float *out, int M, int N, int K) {
    const int grid = ctx->sm_count;
    const int rows_per_cta = (N + grid - 1) / grid;
    FastGeom g;
    g.tiles = min(8, (rows_per_cta + 15) / 16);
    g.tiles_pow2 = 1;
    while (g.tiles_pow2 < g.tiles) g.tiles_pow2 <<= 1;
    g.kslices = min(16 / g.tiles_pow2, GS);
    const int rb_rows = g.tiles * 16;
    g.w_bytes = rb_rows * GS * 16;
    g.s_pitch = GS + 4;  // 20 or 12 floats: rows land on distinct banks for 128-bit reads
    g.s_bytes = rb_rows * g.s_pitch * 4;
    g.d_bytes = GS * 2 * MP * 4 * 16;
    g.a_bytes = ((GS * MP * 8 + 15) / 16) * 16;
    g.stage_bytes = ((g.w_bytes + g.s_bytes + g.d_bytes + g.a_bytes + 127) / 128) * 128;
    const int red_bytes = 16 * 2 * 4 * 32 * 4;
    const int budget = 227 * 1024 - red_bytes;
    g.stages = max(2, min(8, budget / g.stage_bytes));
    const int smem = g.stages * g.stage_bytes + red_bytes;
    auto kern = int4_gemv_fast_kernel<MP, GS>;
    static int smem_set[16] = {0};  // per device: opt-in shared memory size already raised
    if (ctx->device >= 16 || !smem_set[ctx->device]) {
        YSCV_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           227 * 1024));
        if (ctx->device < 16) smem_set[ctx->device] = 1;
    }
    ctx->prof_begin();
    kern<<<grid, 512, smem, ctx->stream>>>(wq, scales, digits, meta, out, M, N, K, g);
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    return YSCV_CUDA_OK;
}

int int4_gemv_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales, const float *act,
                   float *out, size_t m, size_t n, size_t k, void *scratch) {
    const int M = (int)m, N = (int)n, K = (int)k;
    const int MP = padded_m(M);
    uint4 *digits = reinterpret_cast<uint4 *>(scratch);
    int2 *meta = reinterpret_cast<int2 *>(reinterpret_cast<unsigned char *>(scratch) +
                                          (size_t)(K / 32) * 2 * MP * 4 * 16);
    const int items = (K / 32) * MP;
    const int qblocks = min((items + 7) / 8, 4 * ctx->sm_count);
    act_quant_kernel<<<qblocks, 256, 0, ctx->stream>>>(act, digits, meta, M, MP, K);
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    const bool wide = (K % 512 == 0) && MP <= 4;
    ctx->last_kernel = "int4_gemv_fast(imma,cp.async)";
    switch (MP) {
        case 1: return wide ? launch_fast<1, 16>(ctx, wq, scales, digits, meta, out, M, N, K)
                            : launch_fast<1, 8>(ctx, wq, scales, digits, meta, out, M, N, K);
        case 2: return wide ? launch_fast<2, 16>(ctx, wq, scales, digits, meta, out, M, N, K)
                            : launch_fast<2, 8>(ctx, wq, scales, digits, meta, out, M, N, K);
        case 4: return wide ? launch_fast<4, 16>(ctx, wq, scales, digits, meta, out, M, N, K)
                            : launch_fast<4, 8>(ctx, wq, scales, digits, meta, out, M, N, K);
        case 8: return launch_fast<8, 8>(ctx, wq, scales, digits, meta, out, M, N, K);
        default: return launch_fast<16, 8>(ctx, wq, scales, digits, meta, out, M, N, K);
    }
}

int int4_gemv_generic(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                      const float *act, float *out, size_t m, size_t n, size_t k, size_t gs) {
    const int vec_ok = (k % 32 == 0) && (gs % 32 == 0) &&
                       ((reinterpret_cast<uintptr_t>(wq) & 15) == 0) &&
                       ((reinterpret_cast<uintptr_t>(act) & 15) == 0);
    const int blocks = (int)min((size_t)(8 * ctx->sm_count), (n + 7) / 8);
    for (size_t m0 = 0; m0 < m; m0 += 4) {
        int4_gemv_generic_kernel<4><<<blocks, 256, 0, ctx->stream>>>(
            wq, scales, act, out, (int)m0, (int)m, (int)n, (int)k, (int)gs, vec_ok);
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
    }
    ctx->last_kernel = vec_ok ? "int4_gemv_generic(vec128)" : "int4_gemv_generic(bytewise)";
    return YSCV_CUDA_OK;
}

}  // namespace yscv
