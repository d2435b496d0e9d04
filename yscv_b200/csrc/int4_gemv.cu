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
//   e      : max|a| < 2^e
//   afix_j = rint(a_j * 2^(21-e))                 |afix| <= 2^21
//   afix   = d2*65536 + d1*256 + d0               d0,d1 in [-128,127], |d2| <= 32
//   as     = 2^(e-21),  corr = 8 * sum_j afix_j   (undoes the +8 bias of the nibbles)
// A digit plane of one (m, G) is stored as the B fragment of mma.m16n8k32 for
// one column: per thread-in-quad t two words, b0 = digits of k = 8t+{0,2,4,6},
// b1 = digits of k = 8t+{1,3,5,7} (the order in which the nibbles of weight
// word t come out of the unpack).
//
// The output is one contiguous blob per K stage (GS groups), in the exact
// layout the matmul kernel keeps in shared memory:
//
//  "columns" form, M <= 2 (one MMA per group does all three planes):
//    frag[GS][8 cols][4 t] uint4 = {b0, b1, as, nc}
//      b0,b1 : col 0/1/2 = d2/d1/d0 of m=0, col 4/5/6 of m=1, cols 3 and 7 zero
//      as,nc : what accumulator thread t needs, repeated for every col:
//              t even: {as(m=t/2), -corr(m=t/2)}; t odd: {as(m=t/2), 0}
//
//  "planes" form, M >= 4 (three MMAs per group and 8 activation rows):
//    h0[GS][MS][4 t] uint4 = {d2.b0, d2.b1, d1.b0, d1.b1}
//    h1[GS][MS][4 t] uint2 = {d0.b0, d0.b1}
//    meta[GS][MC] int2     = {as, -corr}
//    MS = M slots incl. one all-zero slot for lanes without a row (MP=4: 5),
//    MC = meta slots (8 or 16), zero beyond M.
struct QuantLayout {
    int mp, gs;          // padded M, groups per stage
    int ms, mc;          // planes form: fragment slots, meta slots
    int blob_bytes;      // bytes per K stage
    int off_h1, off_meta;
};

static QuantLayout quant_layout(int mp, int gs) {
    QuantLayout q;
    q.mp = mp;
    q.gs = gs;
    if (mp <= 2) {
        q.ms = 8;
        q.mc = 4;
        q.off_h1 = 0;
        q.off_meta = 0;
        q.blob_bytes = gs * 8 * 4 * 16;
    } else {
        q.ms = (mp < 8) ? mp + 1 : mp;
        q.mc = (mp <= 8) ? 8 : 16;
        q.off_h1 = gs * q.ms * 4 * 16;
        q.off_meta = q.off_h1 + gs * q.ms * 4 * 8;
        q.blob_bytes = q.off_meta + gs * q.mc * 8;
    }
    return q;
}

__global__ void __launch_bounds__(256)
act_quant_kernel(const float *__restrict__ act, unsigned char *__restrict__ blobs, int M, int K,
                 QuantLayout q) {
    const int lane = threadIdx.x & 31;
    const int groups = K / 32;
    const int slots = (q.mp <= 2) ? 2 : max(q.ms, q.mc);  // rows to visit per group (incl. zero rows)
    const int total = groups * slots;
    for (int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < total;
         item += gridDim.x * (blockDim.x >> 5)) {
        const int Gabs = item / slots, m = item % slots;
        const int ks = Gabs / q.gs, G = Gabs % q.gs;
        unsigned char *blob = blobs + (size_t)ks * q.blob_bytes;
        const float v = (m < M) ? act[(size_t)m * K + Gabs * 32 + lane] : 0.0f;
        float gmax = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, o));
        // a non-finite activation poisons the whole group, as it would in fp32
        const bool bad = !(gmax <= 3.0e38f) || (__ballot_sync(0xffffffffu, v != v) != 0u);
        int e = 0;
        if (gmax > 0.0f && !bad) (void)frexpf(gmax, &e);
        e = max(e, -100);  // keeps 2^(21-e) finite for vanishing groups
        const float up = ldexpf(1.0f, 21 - e);
        const int fx = bad ? 0 : __float2int_rn(v * up);
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
        const float as = (m < M) ? (bad ? __int_as_float(0x7fc00000) : ldexpf(1.0f, e - 21)) : 0.0f;
        const int ncorr = -8 * sum;
        if (q.mp <= 2) {
            uint32_t *frag = reinterpret_cast<uint32_t *>(blob);  // [G][col][t][4 words]
            if (lane < 4) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int d = 2 - c;  // col 0,1,2 = planes 2,1,0; col 3 = zero
                    uint32_t *w = frag + ((G * 8 + 4 * m + c) * 4 + t) * 4;
                    w[0] = (c < 3) ? b0[d < 0 ? 0 : d] : 0u;
                    w[1] = (c < 3) ? b1[d < 0 ? 0 : d] : 0u;
                }
            }
            if (lane < 16) {
                // accumulator threads t = 2m (gets -corr) and 2m+1 (gets 0), in all 8 columns
                const int col = lane >> 1, tt = 2 * m + (lane & 1);
                uint32_t *w = frag + ((G * 8 + col) * 4 + tt) * 4;
                w[2] = __float_as_uint(as);
                w[3] = (lane & 1) ? 0u : (uint32_t)ncorr;
            }
        } else {
            uint4 *h0 = reinterpret_cast<uint4 *>(blob);
            uint2 *h1 = reinterpret_cast<uint2 *>(blob + q.off_h1);
            int2 *meta = reinterpret_cast<int2 *>(blob + q.off_meta);
            if (lane < 4 && m < q.ms) {
                h0[(G * q.ms + m) * 4 + t] = make_uint4(b0[2], b1[2], b0[1], b1[1]);
                h1[(G * q.ms + m) * 4 + t] = make_uint2(b0[0], b1[0]);
            }
            if (lane == 0 && m < q.mc) meta[G * q.mc + m] = make_int2(__float_as_int(as), ncorr);
        }
    }
}

// ---------------------------------------------------------------------------
// Fast kernel
// ---------------------------------------------------------------------------

__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void *gsrc, bool valid) {
    const int sz = valid ? 16 : 0;  // src-size 0 => 16 bytes of zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_dst), "l"(gsrc), "r"(sz));
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

// D = A(u8, 16x32) * B(s8, 32x8) + C, int32 accumulate
__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1, int c0, int c1, int c2, int c3) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2),
          "r"(c3));
}

// (w ^ 0x88888888) & 0x0f0f0f0f in one LOP3: unsigned nibbles q+8 as bytes
__device__ __forceinline__ uint32_t nib_u8(uint32_t w) {
    uint32_t r;
    asm("lop3.b32 %0, %1, 0x88888888, 0x0f0f0f0f, 0x28;\n" : "=r"(r) : "r"(w));
    return r;
}

// Shared-memory reads go through ordinary pointers (not volatile asm) so that the
// compiler can hoist the loads of all the groups a warp handles in a stage above
// the first MMA; `off` is a byte offset from the start of dynamic shared memory.
__device__ __forceinline__ uint32_t lds32(const unsigned char *base, uint32_t off) {
    return *reinterpret_cast<const uint32_t *>(base + off);
}
__device__ __forceinline__ float lds_f32(const unsigned char *base, uint32_t off) {
    return *reinterpret_cast<const float *>(base + off);
}
__device__ __forceinline__ uint2 lds64(const unsigned char *base, uint32_t off) {
    return *reinterpret_cast<const uint2 *>(base + off);
}
__device__ __forceinline__ uint4 lds128(const unsigned char *base, uint32_t off) {
    return *reinterpret_cast<const uint4 *>(base + off);
}

struct FastGeom {
    int tiles;        // 16-row tiles per row block (1..TP2)
    int stages;       // ring depth
    int w_bytes, s_bytes, stage_bytes;
    QuantLayout q;
};

// MP  = padded M (1,2,4,8,16)
// GS  = groups of 32 k per stage: 16 (512 k) or 8 (256 k)
// TP2 = warps along the rows of a row block (2 or 8); the other 16/TP2 warps of
//       a tile split the stage's groups between them
template <int MP, int GS, int TP2>
__global__ void __launch_bounds__(512, 1)
int4_gemv_fast_kernel(const uint8_t *__restrict__ wq, const float *__restrict__ scales,
                      const unsigned char *__restrict__ blobs, float *__restrict__ out, int M,
                      int N, int K, FastGeom g) {
    constexpr bool COLS = (MP <= 2);           // digit planes in MMA columns
    constexpr int NT = (MP > 8) ? 2 : 1;       // 8-wide activation tiles (planes form)
    constexpr int NACC = COLS ? 2 : NT * 4;
    constexpr int KSL = (16 / TP2 < GS) ? 16 / TP2 : GS;  // K slices per tile
    constexpr int GPW = GS / KSL;              // groups per warp per stage
    constexpr int S_PITCH = (GS + 4) * 4;      // bytes per row of the scale tile (80 / 48)
    extern __shared__ __align__(1024) unsigned char smem[];
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
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    float *red = reinterpret_cast<float *>(smem + (size_t)g.stages * g.stage_bytes);

    // ---- producer state: every thread owns up to 4 weight chunks, 1 scale chunk and
    // ---- 2 digit-blob chunks per stage; pointers advance by one stage of K per issue
    const int wchunks = rb_rows * GS;
    const uint8_t *w_ptr[4];
    uint32_t w_dst[4];
    int w_row[4];
    unsigned w_ok = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = tid + 512 * j;
        const int r = i / GS, c = i % GS;
        w_row[j] = (i < wchunks) ? r : -1;
        w_dst[j] = (c >> 3) * (rb_rows * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
        w_ptr[j] = wq + c * 16;
    }
    const int s_row = (tid < rb_rows * (GS / 4)) ? tid / (GS / 4) : -1;
    const uint32_t s_dst = g.w_bytes + (tid / (GS / 4)) * S_PITCH + (tid % (GS / 4)) * 16;
    const float *s_ptr = scales + (tid % (GS / 4)) * 4;
    bool s_ok = false;
    const int bchunks = g.q.blob_bytes / 16;
    const uint32_t b_off = g.w_bytes + g.s_bytes;

    int p_slot = 0, p_ks = 0, p_rb = 0;  // next stage to issue
    auto issue = [&]() {
        if (p_ks == 0) {  // (re)aim the pointers at the first K stage of row block p_rb
            const int row0 = r0 + p_rb * rb_rows;
            w_ok = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = row0 + w_row[j];
                const bool ok = (w_row[j] >= 0) && (row < r1);
                w_ok |= (ok ? 1u : 0u) << j;
                const int i = tid + 512 * j;
                w_ptr[j] = wq + (size_t)(ok ? row : r0) * (K / 2) + (i % GS) * 16;
            }
            const int srow = row0 + s_row;
            s_ok = (s_row >= 0) && (srow < r1);
            s_ptr = scales + (size_t)(s_ok ? srow : r0) * groups + (tid % (GS / 4)) * 4;
        }
        const uint32_t st = smem_base + (uint32_t)p_slot * g.stage_bytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (w_row[j] >= 0) cp_async16(st + w_dst[j], w_ptr[j], (w_ok >> j) & 1u);
            w_ptr[j] += GS * 16;
        }
        if (s_row >= 0) cp_async16(st + s_dst, s_ptr, s_ok);
        s_ptr += GS;
        const unsigned char *bsrc = blobs + (size_t)p_ks * g.q.blob_bytes;
        for (int i = tid; i < bchunks; i += 512) cp_async16(st + b_off + i * 16, bsrc + i * 16, true);
        if (++p_slot == g.stages) p_slot = 0;
        if (++p_ks == k_stages) { p_ks = 0; ++p_rb; }
    };

    for (int p = 0; p < g.stages - 1; ++p) {
        if (p < total) issue();
        cp_async_commit();
    }

    const int tile = warp % TP2;
    const int kslice = warp / TP2;
    const bool active = (tile < g.tiles) && (kslice < KSL);
    const int G0 = kslice * GPW;  // first group of this warp inside a stage

    // ---- consumer offsets, constant for the whole kernel (relative to the stage base) ----
    // weight word of (row gq of this warp's tile, group G0+gi, thread-in-quad t); the row 8
    // below is 1024 bytes further with the same swizzle phase.
    uint32_t w_off[GPW];
#pragma unroll
    for (int gi = 0; gi < GPW; ++gi) {
        const int G = G0 + gi;
        w_off[gi] = (uint32_t)(G >> 3) * (rb_rows * 128) + (uint32_t)(tile * 16 + gq) * 128 +
                    ((((uint32_t)G & 7u) ^ (uint32_t)gq) << 4) + t * 4;
    }
    const uint32_t sA_off = g.w_bytes + (uint32_t)(tile * 16 + gq) * S_PITCH + G0 * 4;
    // columns form: one uint4 per unit; planes form: h0 / h1 / meta
    const int mslot = (MP < 8) ? min(gq, g.q.ms - 1) : gq;
    const uint32_t f_off = COLS ? b_off + (uint32_t)((G0 * 8 + gq) * 4 + t) * 16
                                : b_off + (uint32_t)((G0 * g.q.ms + mslot) * 4 + t) * 16;
    const uint32_t h1_off = b_off + g.q.off_h1 + (uint32_t)((G0 * g.q.ms + mslot) * 4 + t) * 8;
    const uint32_t mt_off = b_off + g.q.off_meta + (uint32_t)(G0 * g.q.mc + 2 * t) * 8;
    const uint32_t f_step = COLS ? 8 * 4 * 16 : g.q.ms * 4 * 16;  // bytes per group
    const uint32_t h1_step = g.q.ms * 4 * 8, mt_step = g.q.mc * 8;
    const int mul_hi = (t & 1) ? 1 : 65536;  // columns form: plane weight of this thread's c0

    float acc[NACC];
#pragma unroll
    for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;

    int c_slot = 0, c_ks = 0, c_rb = 0;  // stage being consumed
    for (int it = 0; it < total; ++it) {
        cp_async_wait_dyn(g.stages - 2);
        __syncthreads();
        if (it + g.stages - 1 < total) issue();
        cp_async_commit();
        if (active) {
            const unsigned char *st = smem + (size_t)c_slot * g.stage_bytes;
            float sA[GPW], sB[GPW];
            if constexpr (GPW % 4 == 0) {
#pragma unroll
                for (int gi = 0; gi < GPW; gi += 4) {
                    const uint4 x = lds128(st, sA_off + gi * 4);
                    const uint4 y = lds128(st, sA_off + 8 * S_PITCH + gi * 4);
                    sA[gi] = __uint_as_float(x.x); sA[gi + 1] = __uint_as_float(x.y);
                    sA[gi + 2] = __uint_as_float(x.z); sA[gi + 3] = __uint_as_float(x.w);
                    sB[gi] = __uint_as_float(y.x); sB[gi + 1] = __uint_as_float(y.y);
                    sB[gi + 2] = __uint_as_float(y.z); sB[gi + 3] = __uint_as_float(y.w);
                }
            } else {
#pragma unroll
                for (int gi = 0; gi < GPW; ++gi) {
                    sA[gi] = lds_f32(st, sA_off + gi * 4);
                    sB[gi] = lds_f32(st, sA_off + 8 * S_PITCH + gi * 4);
                }
            }
#pragma unroll
            for (int gi = 0; gi < GPW; ++gi) {
                const uint32_t wA = lds32(st, w_off[gi]), wB = lds32(st, w_off[gi] + 1024);
                uint32_t a[4];
                a[0] = nib_u8(wA);
                a[1] = nib_u8(wB);
                a[2] = nib_u8(wA >> 4);
                a[3] = nib_u8(wB >> 4);
                if constexpr (COLS) {
                    const uint4 f = lds128(st, f_off + gi * f_step);
                    int c[4];
                    mma_u8s8(c, a, f.x, f.y, 0, 0, 0, 0);
                    const int vA = c[0] * mul_hi + (c[1] * 256 + (int)f.w);
                    const int vB = c[2] * mul_hi + (c[3] * 256 + (int)f.w);
                    const float as = __uint_as_float(f.z);
                    acc[0] = fmaf(sA[gi] * as, (float)vA, acc[0]);
                    acc[1] = fmaf(sB[gi] * as, (float)vB, acc[1]);
                } else {
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        const uint4 h0 = lds128(st, f_off + gi * f_step + n * (8 * 4 * 16));
                        const uint2 h1 = lds64(st, h1_off + gi * h1_step + n * (8 * 4 * 8));
                        const uint4 mt = lds128(st, mt_off + gi * mt_step + n * (8 * 8));
                        int c2[4], c1[4], c0[4];
                        mma_u8s8(c2, a, h0.x, h0.y, 0, 0, 0, 0);
                        mma_u8s8(c1, a, h0.z, h0.w, 0, 0, 0, 0);
                        mma_u8s8(c0, a, h1.x, h1.y, (int)mt.y, (int)mt.w, (int)mt.y, (int)mt.w);
                        const float as0 = __uint_as_float(mt.x), as1 = __uint_as_float(mt.z);
                        const int v0 = c2[0] * 65536 + (c1[0] * 256 + c0[0]);
                        const int v1 = c2[1] * 65536 + (c1[1] * 256 + c0[1]);
                        const int v2 = c2[2] * 65536 + (c1[2] * 256 + c0[2]);
                        const int v3 = c2[3] * 65536 + (c1[3] * 256 + c0[3]);
                        acc[n * 4 + 0] = fmaf(sA[gi] * as0, (float)v0, acc[n * 4 + 0]);
                        acc[n * 4 + 1] = fmaf(sA[gi] * as1, (float)v1, acc[n * 4 + 1]);
                        acc[n * 4 + 2] = fmaf(sB[gi] * as0, (float)v2, acc[n * 4 + 2]);
                        acc[n * 4 + 3] = fmaf(sB[gi] * as1, (float)v3, acc[n * 4 + 3]);
                    }
                }
            }
        }
        if (++c_slot == g.stages) c_slot = 0;
        if (++c_ks == k_stages) {
            c_ks = 0;
            // end of a row block: combine the K slices in a fixed order and store
            if (active) {
#pragma unroll
                for (int j = 0; j < NACC; ++j)
                    red[((kslice * g.tiles + tile) * NACC + j) * 32 + lane] = acc[j];
            }
#pragma unroll
            for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;
            __syncthreads();
            const int row0 = r0 + c_rb * rb_rows;
            if constexpr (COLS) {
                // element (tile, half, gq, m): sum over K slices and the thread pair t=2m,2m+1
                const int items = g.tiles * 2 * 8 * MP;
                for (int i = tid; i < items; i += 512) {
                    const int m = i % MP, q8 = (i / MP) & 7, half = (i / (MP * 8)) & 1, tl = i / (MP * 16);
                    float v = 0.0f;
                    for (int ks = 0; ks < KSL; ++ks) {
                        const float *p = red + ((ks * g.tiles + tl) * NACC + half) * 32 + q8 * 4 + 2 * m;
                        v += p[0] + p[1];
                    }
                    const int row = row0 + tl * 16 + q8 + half * 8;
                    if (row < r1 && m < M) out[(size_t)m * N + row] = v;
                }
            } else {
                const int items = g.tiles * NACC * 32;
                for (int i = tid; i < items; i += 512) {
                    const int l = i & 31, j = (i >> 5) % NACC, tl = (i >> 5) / NACC;
                    float v = 0.0f;
                    for (int ks = 0; ks < KSL; ++ks)
                        v += red[((ks * g.tiles + tl) * NACC + j) * 32 + l];
                    const int row = row0 + tl * 16 + (l >> 2) + ((j & 2) ? 8 : 0);
                    const int m = (j >> 2) * 8 + 2 * (l & 3) + (j & 1);
                    if (row < r1 && m < M) out[(size_t)m * N + row] = v;
                }
            }
            ++c_rb;
            // `red` is next written after at least one more __syncthreads (top of the loop)
        }
    }
    cp_async_wait_dyn(0);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------

static int padded_m(int m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16; }
static int stage_groups(int mp, int k) { return (k % 512 == 0 && mp <= 4) ? 16 : 8; }

size_t int4_gemv_scratch_bytes(size_t m, size_t k) {
    // worst case over every padded M up to the one requested
    size_t worst = 0;
    for (int mp = 1; mp <= padded_m((int)m); mp *= 2) {
        const int gs = stage_groups(mp, (int)k);
        const QuantLayout q = quant_layout(mp, gs);
        const size_t b = (k / (32 * (size_t)gs)) * (size_t)q.blob_bytes;
        worst = b > worst ? b : worst;
    }
    return worst + 256;
}

bool int4_gemv_fast_supported(size_t m, size_t n, size_t k, size_t gs) {
    return gs == 32 && k % 256 == 0 && k >= 256 && m >= 1 && m <= 16 && n >= 1 &&
           n < (1u << 30) && k < (1u << 24);
}

template <int MP, int GS, int TP2>
static int launch_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                       const unsigned char *blobs, float *out, int M, int N, int K,
                       const QuantLayout &q) {
    const int grid = ctx->sm_count;
    const int rows_per_cta = (N + grid - 1) / grid;
    FastGeom g;
    g.q = q;
    g.tiles = min(TP2, (rows_per_cta + 15) / 16);
    const int rb_rows = g.tiles * 16;
    g.w_bytes = rb_rows * GS * 16;
    g.s_bytes = rb_rows * (GS + 4) * 4;  // 80- or 48-byte rows land on distinct banks
    g.stage_bytes = ((g.w_bytes + g.s_bytes + q.blob_bytes + 1023) / 1024) * 1024;
    const int red_bytes = 16 * 8 * 32 * 4;
    const int budget = 227 * 1024 - red_bytes - 1024;
    g.stages = max(2, min(8, budget / g.stage_bytes));
    const int smem = g.stages * g.stage_bytes + red_bytes;
    auto kern = int4_gemv_fast_kernel<MP, GS, TP2>;
    static int smem_set[16] = {0};  // per device: opt-in shared memory size already raised
    if (ctx->device >= 16 || !smem_set[ctx->device]) {
        YSCV_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           227 * 1024));
        if (ctx->device < 16) smem_set[ctx->device] = 1;
    }
    ctx->prof_begin();
    kern<<<grid, 512, smem, ctx->stream>>>(wq, scales, blobs, out, M, N, K, g);
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    return YSCV_CUDA_OK;
}

template <int MP, int GS>
static int launch_fast_tp(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                          const unsigned char *blobs, float *out, int M, int N, int K,
                          const QuantLayout &q) {
    const int rows_per_cta = (N + ctx->sm_count - 1) / ctx->sm_count;
    if (rows_per_cta <= 32) return launch_fast<MP, GS, 2>(ctx, wq, scales, blobs, out, M, N, K, q);
    return launch_fast<MP, GS, 8>(ctx, wq, scales, blobs, out, M, N, K, q);
}

int int4_gemv_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales, const float *act,
                   float *out, size_t m, size_t n, size_t k, void *scratch) {
    const int M = (int)m, N = (int)n, K = (int)k;
    const int MP = padded_m(M);
    const int GS = stage_groups(MP, K);
    const QuantLayout q = quant_layout(MP, GS);
    unsigned char *blobs = reinterpret_cast<unsigned char *>(scratch);
    const int items = (K / 32) * ((MP <= 2) ? 2 : max(q.ms, q.mc));
    const int qblocks = min((items + 7) / 8, 4 * ctx->sm_count);
    act_quant_kernel<<<qblocks, 256, 0, ctx->stream>>>(act, blobs, M, K, q);
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    ctx->last_kernel = "int4_gemv_fast(imma,cp.async)";
    switch (MP) {
        case 1: return GS == 16 ? launch_fast_tp<1, 16>(ctx, wq, scales, blobs, out, M, N, K, q)
                                : launch_fast_tp<1, 8>(ctx, wq, scales, blobs, out, M, N, K, q);
        case 2: return GS == 16 ? launch_fast_tp<2, 16>(ctx, wq, scales, blobs, out, M, N, K, q)
                                : launch_fast_tp<2, 8>(ctx, wq, scales, blobs, out, M, N, K, q);
        case 4: return GS == 16 ? launch_fast_tp<4, 16>(ctx, wq, scales, blobs, out, M, N, K, q)
                                : launch_fast_tp<4, 8>(ctx, wq, scales, blobs, out, M, N, K, q);
        case 8: return launch_fast_tp<8, 8>(ctx, wq, scales, blobs, out, M, N, K, q);
        default: return launch_fast_tp<16, 8>(ctx, wq, scales, blobs, out, M, N, K, q);
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
