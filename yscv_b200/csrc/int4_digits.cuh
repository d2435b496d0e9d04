// Device-side pieces shared by the W4 decode kernels: the block-fixed-point digit planes
// the activations are turned into, and the fragment helpers of the integer MMA path.
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

namespace yscv {

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
//    frag[GS][C cols][4 t] uint4 = {b0, b1, as, nc},  C = 4 (M=1) or 8 (M=2)
//      b0,b1 : col 0/1/2 = d2/d1/d0 of m=0, col 4/5/6 of m=1, cols 3 and 7 zero
//              (with C = 4, MMA columns 4..7 re-read columns 0..3; their products
//              land in accumulator threads t = 2,3 whose `as` is zero)
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

__host__ __device__ inline QuantLayout quant_layout(int mp, int gs) {
    QuantLayout q;
    q.mp = mp;
    q.gs = gs;
    if (mp <= 2) {
        q.ms = (mp == 1) ? 4 : 8;  // columns stored per group
        q.mc = 4;
        q.off_h1 = 0;
        q.off_meta = 0;
        q.blob_bytes = gs * q.ms * 4 * 16;
    } else {
        q.ms = (mp < 8) ? mp + 1 : mp;
        q.mc = (mp <= 8) ? 8 : 16;
        q.off_h1 = gs * q.ms * 4 * 16;
        q.off_meta = q.off_h1 + gs * q.ms * 4 * 8;
        q.blob_bytes = q.off_meta + gs * q.mc * 8;
    }
    return q;
}

__device__ __forceinline__ void quantize_group_values(const float (&v)[8], unsigned char *blobs,
                                                      const struct QuantLayout &q, int Gabs, int m, int t,
                                                      bool valid);

// A quad (4 consecutive lanes) turns the 32 activations of (row m, group Gabs) into
// digit planes and writes them into the blob of their K stage. Lane t of the quad
// owns k = 8t..8t+7, which is exactly what fragment thread t needs, so the only
// cross-lane traffic is the quad-wide max and sum. `blobs` may point to global or
// shared memory. `src` (this lane's 8 floats) is null for padding rows (m >= M),
// which produce zeros. All 32 lanes of the warp must call this together; lanes
// whose item is out of range pass valid = false.
template <bool SMEM_SRC = false>
__device__ __forceinline__ void quantize_group(const float *__restrict__ src, unsigned char *blobs,
                                               const QuantLayout &q, int Gabs, int m, int t,
                                               bool valid) {
    if (!src) {
        // padding row (m >= M): all digits, the scale factor and the correction are zero.
        // A warp's eight quads belong to the same row (K/32 is a multiple of 8), so the whole
        // warp takes this branch together and skips the shuffles below.
        if (!valid) return;
        const int ks = Gabs / q.gs, G = Gabs % q.gs;
        unsigned char *blob = blobs + (size_t)ks * q.blob_bytes;
        if (q.mp <= 2) {
            uint2 *frag = reinterpret_cast<uint2 *>(blob);
            const int C = q.ms;
            if (4 * m < C)
                for (int c = 0; c < 4; ++c) frag[((G * C + 4 * m + c) * 4 + t) * 2] = make_uint2(0u, 0u);
            for (int col = t; col < C; col += 4) {
                frag[((G * C + col) * 4 + 2 * m) * 2 + 1] = make_uint2(0u, 0u);
                frag[((G * C + col) * 4 + 2 * m + 1) * 2 + 1] = make_uint2(0u, 0u);
            }
        } else {
            if (m < q.ms) {
                reinterpret_cast<uint4 *>(blob)[(G * q.ms + m) * 4 + t] = make_uint4(0u, 0u, 0u, 0u);
                reinterpret_cast<uint2 *>(blob + q.off_h1)[(G * q.ms + m) * 4 + t] = make_uint2(0u, 0u);
            }
            if (t == 0 && m < q.mc) reinterpret_cast<int2 *>(blob + q.off_meta)[G * q.mc + m] = make_int2(0, 0);
        }
        return;
    }
    float v[8];
    if (src && valid) {
        float4 x, y;
        if constexpr (SMEM_SRC) {  // staged in shared memory by the producer
            x = *reinterpret_cast<const float4 *>(src);
            y = *(reinterpret_cast<const float4 *>(src) + 1);
        } else {
            x = __ldg(reinterpret_cast<const float4 *>(src));
            y = __ldg(reinterpret_cast<const float4 *>(src) + 1);
        }
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
        v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
    quantize_group_values(v, blobs, q, Gabs, m, t, valid);
}

// The same for eight activations the lane already holds in registers (k = 8t .. 8t+7 of group
// Gabs, row m). All 32 lanes of the warp call it together; lanes without an item pass
// valid = false (and any values).
__device__ __forceinline__ void quantize_group_values(const float (&v)[8], unsigned char *blobs,
                                                      const QuantLayout &q, int Gabs, int m, int t,
                                                      bool valid) {
    float gmax = 0.0f;
    int nan = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        gmax = fmaxf(gmax, fabsf(v[i]));
        nan |= (v[i] != v[i]) ? 1 : 0;
    }
    gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 1));
    gmax = fmaxf(gmax, __shfl_xor_sync(0xffffffffu, gmax, 2));
    nan |= __shfl_xor_sync(0xffffffffu, nan, 1);
    nan |= __shfl_xor_sync(0xffffffffu, nan, 2);
    // a non-finite activation poisons the whole group, as it would in fp32
    const bool bad = nan || !(gmax <= 3.0e38f);
    int e = 0;
    if (gmax > 0.0f && !bad) e = ((__float_as_int(gmax) >> 23) & 255) - 126;  // gmax < 2^e
    e = max(e, -100);  // keeps 2^(21-e) finite for vanishing (or subnormal) groups
    const float up = __int_as_float((127 + 21 - e) << 23);  // 2^(21-e)
    int sum = 0;
    // The balanced digits d0, d1 (in [-128, 127]) and the remainder d2 of afix are the three low
    // bytes of (afix + 0x8080) ^ 0x8080: adding 128 at a digit's position lets the carry into the
    // next digit do the rounding, and flipping bit 7 turns the biased byte into two's complement.
    uint32_t z[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int fx = bad ? 0 : __float2int_rn(v[i] * up);
        sum += fx;
        z[i] = (uint32_t)(fx + 0x8080) ^ 0x8080u;
    }
    uint32_t b0[3], b1[3];  // per plane: the digits of k = 0,2,4,6 / k = 1,3,5,7, one per byte
#pragma unroll
    for (int pl = 0; pl < 3; ++pl) {
        const uint32_t sel = (uint32_t)pl | ((uint32_t)(4 + pl) << 4);
        b0[pl] = __byte_perm(__byte_perm(z[0], z[2], sel), __byte_perm(z[4], z[6], sel), 0x5410);
        b1[pl] = __byte_perm(__byte_perm(z[1], z[3], sel), __byte_perm(z[5], z[7], sel), 0x5410);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (!valid) return;
    const int ks = Gabs / q.gs, G = Gabs % q.gs;
    unsigned char *blob = blobs + (size_t)ks * q.blob_bytes;
    const float as = bad ? __int_as_float(0x7fc00000) : __int_as_float((127 + e - 21) << 23);  // 2^(e-21)
    const int ncorr = -8 * sum;
    if (q.mp <= 2) {
        uint2 *frag = reinterpret_cast<uint2 *>(blob);  // [G][col][t] x {b0,b1 | as,nc}
        const int C = q.ms;
        if (4 * m < C) {
#pragma unroll
            for (int c = 0; c < 3; ++c)  // col 0,1,2 = planes 2,1,0
                frag[((G * C + 4 * m + c) * 4 + t) * 2] = make_uint2(b0[2 - c], b1[2 - c]);
            frag[((G * C + 4 * m + 3) * 4 + t) * 2] = make_uint2(0u, 0u);
        }
        // accumulator threads 2m (gets -corr) and 2m+1 (gets 0), in every column; the four
        // lanes of the quad share the columns between them
        for (int col = t; col < C; col += 4) {
            frag[((G * C + col) * 4 + 2 * m) * 2 + 1] = make_uint2(__float_as_uint(as), (uint32_t)ncorr);
            frag[((G * C + col) * 4 + 2 * m + 1) * 2 + 1] = make_uint2(__float_as_uint(as), 0u);
        }
    } else {
        uint4 *h0 = reinterpret_cast<uint4 *>(blob);
        uint2 *h1 = reinterpret_cast<uint2 *>(blob + q.off_h1);
        int2 *meta = reinterpret_cast<int2 *>(blob + q.off_meta);
        if (m < q.ms) {
            h0[(G * q.ms + m) * 4 + t] = make_uint4(b0[2], b1[2], b0[1], b1[1]);
            h1[(G * q.ms + m) * 4 + t] = make_uint2(b0[0], b1[0]);
        }
        if (t == 0 && m < q.mc) meta[G * q.mc + m] = make_int2(__float_as_int(as), ncorr);
    }
}

// rows to visit per group, padding rows included
__host__ __device__ inline int quant_slots(const QuantLayout &q) {
    return (q.mp <= 2) ? 2 : (q.ms > q.mc ? q.ms : q.mc);
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

}  // namespace yscv
