// int8 x int8 -> int32 GEMM on the 5th-generation tensor cores (tcgen05, sm_100a),
// with the MatMulInteger / QLinearMatMul epilogues fused behind it.
//
// Replaces int8_matmul_dispatch / int8_matmul_prepacked_dispatch and the
// requantisation pass that follows them in the reference
// (crates/yscv-kernels/src/ops/int8_matmul.rs:195-227, 2407-2425;
//  crates/yscv-kernels/src/ops/int8_requant.rs:143-169;
//  crates/yscv-onnx/src/runner/linear.rs:438-537, 648-737).
//
// Operands: A [M][K] row-major (i8, or u8 with a zero point), B prepacked once
// as B^T [N][Kp] (K-major, Kp = K rounded up to 16, zero padded) together with
// its column sums; both are exactly what the MMA wants: K-major tiles fetched by
// TMA with the 128-byte swizzle. Integer accumulation is exact, so the result
// is bit-identical to the scalar CPU kernel in any order.
//
// Kernel: persistent, one CTA per SM, 192 threads, warp-specialised:
//   warp 0      TMA producer: A tile [128][128 B] + B tile [BN][128 B] per stage
//   warp 1      allocates TMEM, issues tcgen05.mma.kind::i8 (M=128, N=BN, K=32,
//               four per stage), commits stages back to the producer and
//               finished accumulators to the epilogue
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, subtract
//               a_zp * colsum[n], then either store int32 or requantise
//               ((float)acc * composite + y_zp with separate multiply and add,
//               round, saturate) and store bytes
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of
// tile i overlaps the main loop of tile i+1. All mbarrier waits are bounded; a
// wait that runs out sets the context's status word and every role falls through
// to the common exit, where TMEM is released.
#include "common.cuh"
#include "kernels.cuh"
#include "tma.cuh"

namespace yscv {

constexpr int G8_BM = 128;
constexpr int G8_BK = 128;  // bytes of K per stage = one 128-byte swizzle row
constexpr int G8_THREADS = 192;

struct G8Params {
    int M, N, K;            // logical sizes (K = padded K of the prepacked B)
    int m_blocks, n_blocks, k_blocks;
    int stages;
    int a_unsigned;         // A holds u8
    int a_zp;               // subtracted through a_zp * colsum[n]
    int mode;               // 0: int32 out, 1: requantised byte out
    float composite, y_zp;
    int qmin, qmax;
    int round_mode;         // 0: ties to even, 1: half away from zero
    long long ldc;          // elements per output row
    // requantised output only, all optional: corr[n] is added to the accumulator (wrapping, as
    // the reference's per-channel requant does with bias - x_zp * colsum), comp_pc[n] replaces
    // the scalar composite, relu clamps negative outputs to zero after the saturation
    const int32_t *corr;
    const float *comp_pc;
    int relu;
    // zero point of B: (a - a_zp)(b - b_zp) summed over k = acc - a_zp * colsum[n]
    //                  - b_zp * rowsum[m] + k_true * a_zp * b_zp, all modulo 2^32
    int b_zp;
    const int32_t *rowsum;  // row sums of A over k (only when b_zp != 0)
    int k_true;
    // K split (one-CTA kernel, shapes with far fewer tiles than SMs and a long K): the K loops of
    // the tiles from `tail_first` on are cut into runs of `tail_units` K blocks, one run per CTA,
    // laid end to end over those tiles. The CTA that holds a tile's first K block owns the tile;
    // the others leave their int32 partial sums in slot blockIdx.x of `ws` and publish `epoch`
    // in ws_flag[4 * blockIdx.x + epilogue warp]. Integer addition is exact and commutative, so
    // the result does not depend on the split. tail_first == tiles: no split.
    int tail_first, tail_units;
    int32_t *ws;
    int *ws_flag;
    int epoch;
};

// One piece of work of a CTA: K blocks [kb0, kb1) of output tile `tile`.
struct G8Item {
    int tile, kb0, kb1;
};

// The pieces of one CTA in the order every role walks them: its run of the split tiles (at most
// one tile boundary inside a run, since a run is never longer than a tile's K loop), the part it
// does not own first, then whole tiles.
struct G8Walk {
    int t, u, u1;
    __device__ explicit G8Walk(const G8Params &p) {
        const int tail_total = (p.m_blocks * p.n_blocks - p.tail_first) * p.k_blocks;
        t = blockIdx.x;
        u = min((int)blockIdx.x * p.tail_units, tail_total);
        u1 = min(u + p.tail_units, tail_total);
    }
    __device__ bool next(const G8Params &p, G8Item &it) {
        if (u < u1) {
            const int tl = u / p.k_blocks, kb0 = u - tl * p.k_blocks;
            const int n = min(u1 - u, p.k_blocks - kb0);
            it.tile = p.tail_first + tl; it.kb0 = kb0; it.kb1 = kb0 + n;
            u += n;
            return true;
        }
        if (t < p.tail_first) {
            it.tile = t; it.kb0 = 0; it.kb1 = p.k_blocks;
            t += gridDim.x;
            return true;
        }
        return false;
    }
};

__device__ __forceinline__ int ld_acquire_gpu(const int *p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int *p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}

// K-major operand tile in shared memory, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (what a TMA box [rows][128 B] with SWIZZLE_128B writes).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);        // start address
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused, K-major swizzled)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset: 8 rows
    d |= (uint64_t)1 << 46;                            // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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

// Words per row of an epilogue warp's transposition scratch: 32 columns + 4 of padding, so that
// 16-byte accesses by row (one thread, eight pieces) and by piece (eight threads, one row) both
// spread over all banks.
constexpr int G8_XP_PITCH = 36;
constexpr int G8_XP_BYTES = 4 * 32 * G8_XP_PITCH * 4;   // four epilogue warps

// fp32 -> integer in [lo, hi], round to nearest even. Clamping first and rounding second gives
// the same integer as rint-then-clamp for integer bounds; the rounding itself is the fp32 add of
// 1.5 * 2^23 (exact for |v| < 2^22), whose low mantissa bits are the integer in two's complement:
// no conversion instruction (a quarter-rate pipe) on the way out.
__device__ __forceinline__ int round_clamped(float v, float lo, float hi) {
    v = fminf(fmaxf(v, lo), hi);
    return __float_as_int(__fadd_rn(v, 12582912.0f)) - 0x4B400000;
}

// Epilogue of one accumulator row: the thread owns output row `row`, whose BN int32 sums sit in
// TMEM at `taddr` (this warp's lane group, the tile's first column); columns nb * BN ... of the
// output. Subtracts the zero-point terms, then stores int32 or requantises and stores bytes.
// int32 rows go through `xpose` (this warp's 32 x G8_XP_PITCH words of shared memory) so that a
// store instruction writes four 128-byte row segments instead of 16 bytes of 32 different rows.
// [c_first, c_last]: CTAs whose partial sums of this tile (slots of p.ws, row `rt` of the tile) are
// added first; empty range when the tile was not split.
template <int BN>
__device__ __forceinline__ void epilogue_row(const G8Params &p, const int32_t *__restrict__ colsum,
                                             void *__restrict__ out, int row, uint32_t taddr, int nb,
                                             uint32_t *xpose, int rt = 0, int c_first = 0, int c_last = -1) {
    const int lane = threadIdx.x & 31;
    const bool general = p.corr != nullptr || p.comp_pc != nullptr || p.relu != 0 || p.b_zp != 0;
    // 16-byte vector stores need a 16-byte aligned output (rows then stay aligned through
    // the pitch conditions below); anything else takes scalar stores
    const bool out_vec_ok = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    const bool live = row < p.M;
    const float lo = (float)p.qmin, hi = (float)p.qmax;
    // what the zero point of B adds to every element of this row
    int row_term = 0;
    if (p.b_zp != 0 && live)
        row_term = (int)((uint32_t)p.k_true * (uint32_t)p.a_zp * (uint32_t)p.b_zp -
                         (uint32_t)p.b_zp * (uint32_t)__ldg(p.rowsum + row));
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        const int col0 = nb * BN + c0;
        if (col0 >= p.N) continue;   // the same for the whole warp
        if (live) {
            // partial sums: 16-byte piece (4 columns) j of row rt sits at piece index j * 128 + rt of
            // the slot, so a warp reads 512 contiguous bytes; two slots are in flight at a time
            for (int c = c_first; c <= c_last; c += 2) {
                const bool two = c + 1 <= c_last;
                const int4 *s0 = reinterpret_cast<const int4 *>(p.ws) + (size_t)c * (G8_BM * BN / 4) + (c0 / 4) * G8_BM + rt;
                const int4 *s1 = s0 + (two ? G8_BM * BN / 4 : 0);
                int4 v0[8], v1[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v0[j] = __ldcg(s0 + j * G8_BM);  // another CTA wrote them: L2, not L1
#pragma unroll
                for (int j = 0; j < 8; ++j) v1[j] = two ? __ldcg(s1 + j * G8_BM) : make_int4(0, 0, 0, 0);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    r[4 * j] += (uint32_t)(v0[j].x + v1[j].x); r[4 * j + 1] += (uint32_t)(v0[j].y + v1[j].y);
                    r[4 * j + 2] += (uint32_t)(v0[j].z + v1[j].z); r[4 * j + 3] += (uint32_t)(v0[j].w + v1[j].w);
                }
            }
        }
        if (p.mode == 0) {
            int32_t *o = reinterpret_cast<int32_t *>(out) + (size_t)row * p.ldc + col0;
            if (col0 + 32 <= p.N && (p.ldc & 3) == 0 && out_vec_ok) {
                // every lane takes part (rows past M carry sums of zero rows and are not stored)
                int4 *mine = reinterpret_cast<int4 *>(xpose + lane * G8_XP_PITCH);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    int4 v;
                    v.x = (int)r[j] - p.a_zp * __ldg(colsum + col0 + j) + row_term;
                    v.y = (int)r[j + 1] - p.a_zp * __ldg(colsum + col0 + j + 1) + row_term;
                    v.z = (int)r[j + 2] - p.a_zp * __ldg(colsum + col0 + j + 2) + row_term;
                    v.w = (int)r[j + 3] - p.a_zp * __ldg(colsum + col0 + j + 3) + row_term;
                    mine[j >> 2] = v;
                }
                __syncwarp();
                const int row0 = row - lane, piece = lane & 7;
                int32_t *ob = reinterpret_cast<int32_t *>(out) + col0 + 4 * piece;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = 4 * i + (lane >> 3);
                    const int4 v = *reinterpret_cast<const int4 *>(xpose + rr * G8_XP_PITCH + 4 * piece);
                    if (row0 + rr < p.M) *reinterpret_cast<int4 *>(ob + (size_t)(row0 + rr) * p.ldc) = v;
                }
                __syncwarp();
            } else if (live) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.N) o[j] = (int)r[j] - p.a_zp * __ldg(colsum + col0 + j) + row_term;
            }
        } else if (live) {
            uint8_t *o = reinterpret_cast<uint8_t *>(out) + (size_t)row * p.ldc + col0;
            uint32_t packed[8];
            if (general) {
                // per-channel vectors, bias, ReLU or a zero point on B
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int cc = (col0 + j < p.N) ? col0 + j : col0;
                    int acc = (int)r[j] - p.a_zp * __ldg(colsum + cc) + row_term;
                    float comp = p.composite;
                    if (p.corr) acc = (int)((uint32_t)acc + (uint32_t)__ldg(p.corr + cc));
                    if (p.comp_pc) comp = __ldg(p.comp_pc + cc);
                    // separate multiply and add: the CPU kernel does not fuse them
                    const float v = __fadd_rn(__fmul_rn((float)acc, comp), p.y_zp);
                    int qv = p.round_mode ? (int)fminf(fmaxf(roundf(v), lo), hi) : round_clamped(v, lo, hi);
                    if (p.relu && qv < 0) qv = 0;
                    if ((j & 3) == 0) packed[j >> 2] = 0;
                    packed[j >> 2] |= ((uint32_t)qv & 255u) << (8 * (j & 3));
                }
            } else if (p.round_mode == 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int cc = (col0 + j < p.N) ? col0 + j : col0;
                    const int acc = (int)r[j] - p.a_zp * __ldg(colsum + cc);
                    // separate multiply and add: the CPU kernel does not fuse them
                    const float v = __fadd_rn(__fmul_rn((float)acc, p.composite), p.y_zp);
                    const int qv = round_clamped(v, lo, hi);
                    if ((j & 3) == 0) packed[j >> 2] = 0;
                    packed[j >> 2] |= ((uint32_t)qv & 255u) << (8 * (j & 3));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int cc = (col0 + j < p.N) ? col0 + j : col0;
                    const int acc = (int)r[j] - p.a_zp * __ldg(colsum + cc);
                    const float v = __fadd_rn(__fmul_rn((float)acc, p.composite), p.y_zp);
                    const int qv = (int)fminf(fmaxf(roundf(v), lo), hi);
                    if ((j & 3) == 0) packed[j >> 2] = 0;
                    packed[j >> 2] |= ((uint32_t)qv & 255u) << (8 * (j & 3));
                }
            }
            if (col0 + 32 <= p.N && (p.ldc & 15) == 0 && out_vec_ok) {
                *reinterpret_cast<uint4 *>(o) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4 *>(o + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.N) o[j] = (uint8_t)(packed[j >> 2] >> (8 * (j & 3)));
            }
        }
    }
}

// A non-owner's piece of a split tile: the raw int32 sums of row `rt` go to this CTA's slot.
template <int BN>
__device__ __forceinline__ void dump_row(const G8Params &p, int row, uint32_t taddr, int nb, int rt) {
    int4 *dst = reinterpret_cast<int4 *>(p.ws) + (size_t)blockIdx.x * (G8_BM * BN / 4) + rt;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        if (row < p.M && nb * BN + c0 < p.N) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                __stcg(dst + (c0 / 4 + j) * G8_BM,
                       make_int4((int)r[4 * j], (int)r[4 * j + 1], (int)r[4 * j + 2], (int)r[4 * j + 3]));
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(G8_THREADS, 1)
int8_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const int32_t *__restrict__ colsum, void *__restrict__ out, G8Params p,
                    int *__restrict__ status) {
    constexpr int A_BYTES = G8_BM * G8_BK;  // 16 KB
    constexpr int B_BYTES = BN * G8_BK;     // 32 / 16 KB
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bars = smem_base + (uint32_t)p.stages * STAGE_BYTES;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * 8;
    const uint32_t bar_tfull = bars + 16 * 8, bar_tempty = bars + 18 * 8;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (size_t)p.stages * STAGE_BYTES + 20 * 8);
    // transposition scratch of the epilogue warps, behind the 256 bytes of barriers
    uint32_t *xpose_all = reinterpret_cast<uint32_t *>(smem + (size_t)p.stages * STAGE_BYTES + 256);

    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(bar_full + i * 8, 1);
            mbar_init(bar_empty + i * 8, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + i * 8, 1);
            mbar_init(bar_tempty + i * 8, 4);  // one arrival per epilogue warp
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        // 2 x BN columns of TMEM (power of two >= 32); released at the common exit below
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(2 * BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // programmatic dependent launch: the set-up above may overlap the tail of the previous kernel of
    // the stream; everything below reads what it may have written or writes what it may still read
    pdl_wait();
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_a));
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_b));
            int slot = 0;
            uint32_t phase = 0;
            bool alive = true;
            G8Walk walk(p);
            G8Item it;
            while (alive && walk.next(p, it)) {
                const int mb = it.tile % p.m_blocks, nb = it.tile / p.m_blocks;
                for (int kb = it.kb0; kb < it.kb1; ++kb) {
                    alive = mbar_wait(bar_empty + slot * 8, phase ^ 1u, status);
                    if (!alive) break;
                    const uint32_t st = smem_base + (uint32_t)slot * STAGE_BYTES;
                    const uint32_t full = bar_full + slot * 8;
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(st, &tm_a, kb * G8_BK, mb * G8_BM, full);
                    tma_load_2d(st + A_BYTES, &tm_b, kb * G8_BK, nb * BN, full);
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = (2u << 4) | ((p.a_unsigned ? 0u : 1u) << 7) | (1u << 10) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(G8_BM >> 4) << 24);
            int slot = 0, abuf = 0;
            uint32_t phase = 0, aphase = 0;
            bool alive = true;
            G8Walk walk(p);
            G8Item it;
            while (alive && walk.next(p, it)) {
                // the epilogue must have drained this accumulator buffer
                alive = mbar_wait(bar_tempty + abuf * 8, aphase ^ 1u, status);
                if (!alive) break;
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)abuf * BN;
                for (int kb = it.kb0; kb < it.kb1; ++kb) {
                    alive = mbar_wait(bar_full + slot * 8, phase, status);
                    if (!alive) break;
                    tc_fence_after();
                    const uint32_t st = smem_base + (uint32_t)slot * STAGE_BYTES;
                    const uint64_t da = umma_desc_sw128(st), db = umma_desc_sw128(st + A_BYTES);
#pragma unroll
                    for (int j = 0; j < G8_BK / 32; ++j)  // K = 32 per instruction: +32 bytes in the row
                        umma_i8(tacc, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc,
                                (kb > it.kb0 || j > 0) ? 1u : 0u);
                    umma_commit(bar_empty + slot * 8);  // stage free once these MMAs have read it
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                }
                if (!alive) break;
                umma_commit(bar_tfull + abuf * 8);  // accumulator complete
                if (++abuf == 2) { abuf = 0; aphase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lanes 32*(warp%4).. ----------------
        const int q = warp & 3;
        uint32_t *xpose = xpose_all + q * 32 * G8_XP_PITCH;
        int abuf = 0;
        uint32_t aphase = 0;
        bool alive = true;
        G8Walk walk(p);
        G8Item it;
        while (alive && walk.next(p, it)) {
            const int mb = it.tile % p.m_blocks, nb = it.tile / p.m_blocks;
            alive = mbar_wait(bar_tfull + abuf * 8, aphase, status);
            if (!alive) break;
            tc_fence_after();
            const int rt = q * 32 + lane;
            const int row = mb * G8_BM + rt;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)abuf * BN;
            if (it.kb0 > 0) {
                // a later part of a split tile: leave the partial sums for the tile's owner
                dump_row<BN>(p, row, taddr, nb, rt);
                __threadfence();
                __syncwarp();
                if (lane == 0) st_release_gpu(p.ws_flag + 4 * blockIdx.x + q, p.epoch);
            } else if (it.kb1 < p.k_blocks) {
                // the first part of a split tile: this CTA owns it. The other parts belong to the
                // CTAs that follow, which compute them at the start of their runs; wait (bounded)
                // for the same warp of each, whose threads wrote the rows this warp reads.
                const int u_end = (it.tile - p.tail_first + 1) * p.k_blocks - 1;
                const int c_first = (int)blockIdx.x + 1, c_last = u_end / p.tail_units;
                for (int c = c_first; c <= c_last && alive; ++c) {
                    const int *f = p.ws_flag + 4 * c + q;
                    bool seen = false;
                    for (uint32_t i = 0; i < (1u << 22) && !seen; ++i) seen = ld_acquire_gpu(f) == p.epoch;
                    if (!seen) {
                        atomicExch(status, 2 /* YSCV_DEV_FLAG_TIMEOUT */);
                        alive = false;
                    }
                }
                alive = __all_sync(0xffffffffu, alive);
                if (alive) epilogue_row<BN>(p, colsum, out, row, taddr, nb, xpose, rt, c_first, c_last);
            } else {
                epilogue_row<BN>(p, colsum, out, row, taddr, nb, xpose);
            }
            // all columns of this buffer have been read: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + abuf * 8);
            if (++abuf == 2) { abuf = 0; aphase ^= 1u; }
        }
    }

    // ---------------- common exit: release TMEM ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * BN));
    }
}

// ---------------------------------------------------------------------------
// CTA-pair kernel: tcgen05.mma.cta_group::2
// ---------------------------------------------------------------------------
//
// Two CTAs on the two SMs of a TPC (a cluster of 2) share one 256 x 256 output tile. Per K
// step each CTA stages its own 128 rows of A and its own 128 rows of the B^T tile (plain TMA
// loads, no multicast); the leader CTA (cluster rank 0) issues one MMA of M = 256, N = 256 that
// reads both CTAs' shared memory and accumulates rows 0..127 into its own TMEM and rows
// 128..255 into the peer's. Against the one-CTA kernel a tensor core then reads 8 KB instead of
// 12 KB of shared memory per instruction and each SM pulls 32 KB instead of 48 KB per K step
// from L2 for the same flops: shared-memory bandwidth (TMA fill + MMA operand reads on one
// 128 B/clk port) is what holds the one-CTA kernel at ~60 % of the tensor rate.
//
// Signalling (no multicast form is used anywhere; every cross-CTA signal is raised by the
// hardware unit that finishes the work, never relayed by a polling thread):
//   full[s]    leader only, one arrival (the leader's expect_tx of BOTH CTAs' bytes): the peer's
//              TMA loads are issued with .cta_group::2 and complete their bytes on the leader's
//              barrier (address through mapa), so the MMA issuer waits on one barrier
//   empty[s]   each CTA its own: the leader commits the MMAs of stage s twice, once to its own
//              barrier and once to the peer's (a plain tcgen05.commit to a shared::cluster address)
//   tfull[b]   each CTA its own, committed twice the same way after the last K step
//   tempty[b]  leader only, 8 arrivals: the four epilogue warps of both CTAs drained buffer b
//              (remote mbarrier.arrive from the peer's warps, once per tile)
// All waits are bounded; a wait that runs out sets the status word, the roles fall through to the
// cluster-wide barrier at the end, and TMEM is released.
constexpr int G8P_BN = 256;           // columns of the pair tile
constexpr int G8P_STAGE = 2 * G8_BM * G8_BK;  // per CTA: 128 rows of A + 128 rows of B^T

__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}

__global__ void __launch_bounds__(G8_THREADS, 1)
int8_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const int32_t *__restrict__ colsum, void *__restrict__ out, G8Params p,
                      int *__restrict__ status) {
    constexpr int BN = G8P_BN;
    constexpr int HALF_BYTES = G8_BM * G8_BK;   // 16 KB: one CTA's rows of A, or of B^T
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();       // 0: leader (issues the MMAs), 1: peer
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bars = smem_base + (uint32_t)p.stages * G8P_STAGE;
    const uint32_t bar_full = bars, bar_empty = bars + 8 * 8;
    const uint32_t bar_tfull = bars + 24 * 8, bar_tempty = bars + 26 * 8;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + (size_t)p.stages * G8P_STAGE + 28 * 8);
    uint32_t *xpose_all = reinterpret_cast<uint32_t *>(smem + (size_t)p.stages * G8P_STAGE + 256);
    const int tiles = p.m_blocks * p.n_blocks;   // pair tiles of 256 x 256

    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(bar_full + i * 8, 1);
            mbar_init(bar_empty + i * 8, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_tfull + i * 8, 1);
            mbar_init(bar_tempty + i * 8, 8);  // four epilogue warps of each CTA
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        // 2 x 256 columns in each CTA of the pair; released after the cluster barrier at the end
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(2 * BN));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
    }
    tc_fence_before();
    cluster_sync_all();   // both CTAs' barriers exist before anyone arrives on a remote one
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();      // as in the one-CTA kernel
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs): own 128 rows of A, own 128 rows of B^T ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_a));
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_b));
            int slot = 0;
            uint32_t phase = 0;
            bool alive = true;
            const uint32_t leader_full = map_to_cta(bar_full, 0);
            for (int t = pair; t < tiles && alive; t += n_pairs) {
                const int mb = t % p.m_blocks, nb = t / p.m_blocks;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    alive = mbar_wait(bar_empty + slot * 8, phase ^ 1u, status);
                    if (!alive) break;
                    const uint32_t st = smem_base + (uint32_t)slot * G8P_STAGE;
                    const uint32_t full = leader_full + slot * 8;
                    if (rank == 0) mbar_expect_tx(bar_full + slot * 8, 2 * G8P_STAGE);
                    tma_load_2d_pair(st, &tm_a, kb * G8_BK, mb * 256 + (int)rank * G8_BM, full);
                    tma_load_2d_pair(st + HALF_BYTES, &tm_b, kb * G8_BK, nb * BN + (int)rank * G8_BM, full);
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---------------- MMA issuer (leader only) ----------------
            const uint32_t idesc = (2u << 4) | ((p.a_unsigned ? 0u : 1u) << 7) | (1u << 10) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int slot = 0, abuf = 0;
            uint32_t phase = 0, aphase = 0;
            bool alive = true;
            const uint32_t peer_empty = map_to_cta(bar_empty, 1), peer_tfull = map_to_cta(bar_tfull, 1);
            for (int t = pair; t < tiles && alive; t += n_pairs) {
                alive = mbar_spin_cluster(bar_tempty + abuf * 8, aphase ^ 1u, status);
                if (!alive) break;
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)abuf * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    alive = mbar_wait_cluster(bar_full + slot * 8, phase, status);
                    if (!alive) break;
                    tc_fence_after();
                    const uint32_t st = smem_base + (uint32_t)slot * G8P_STAGE;
                    const uint64_t da = umma_desc_sw128(st), db = umma_desc_sw128(st + HALF_BYTES);
#pragma unroll
                    for (int j = 0; j < G8_BK / 32; ++j)
                        umma_i8_pair(tacc, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc,
                                     (kb > 0 || j > 0) ? 1u : 0u);
                    umma_commit_pair(bar_empty + slot * 8);
                    umma_commit_pair(peer_empty + slot * 8);
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                }
                if (!alive) break;
                umma_commit_pair(bar_tfull + abuf * 8);
                umma_commit_pair(peer_tfull + abuf * 8);
                if (++abuf == 2) { abuf = 0; aphase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): warps 2..5 own TMEM lanes 32*(warp%4).. ----------------
        const int q = warp & 3;
        uint32_t *xpose = xpose_all + q * 32 * G8_XP_PITCH;
        int abuf = 0;
        uint32_t aphase = 0;
        bool alive = true;
        const uint32_t leader_tempty = map_to_cta(bar_tempty, 0);
        for (int t = pair; t < tiles && alive; t += n_pairs) {
            const int mb = t % p.m_blocks, nb = t / p.m_blocks;
            alive = mbar_wait(bar_tfull + abuf * 8, aphase, status);
            if (!alive) break;
            tc_fence_after();
            const int row = mb * 256 + (int)rank * G8_BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)abuf * BN;
            epilogue_row<BN>(p, colsum, out, row, taddr, nb, xpose);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(leader_tempty + abuf * 8);
            if (++abuf == 2) { abuf = 0; aphase ^= 1u; }
        }
    }

    // ---------------- common exit ----------------
    // Neither CTA may leave (or give its TMEM back) while the other can still read its shared
    // memory or arrive on its barriers.
    tc_fence_before();
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * BN));
    }
}

// ---------------------------------------------------------------------------
// B prepack: [K][N] row-major -> B^T [N][Kp] (zero padded) + column sums
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(256)
pack_i8_b_kernel(const int8_t *__restrict__ b, int8_t *__restrict__ bt, int32_t *__restrict__ colsum,
                 int K, int N, int Kp) {
    // one warp per output row n: lanes stride over k
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (n >= N) return;
    int s = 0;
    for (int k = lane; k < Kp; k += 32) {
        const int8_t v = (k < K) ? b[(size_t)k * N + n] : (int8_t)0;
        bt[(size_t)n * Kp + k] = v;
        s += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) colsum[n] = s;
}

// row sums of A over k (one warp per row), the bytes read as u8 or i8
__global__ void __launch_bounds__(256)
rowsum_a_kernel(const uint8_t *__restrict__ a, int32_t *__restrict__ rowsum, int M, int K, int is_unsigned) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= M) return;
    const uint8_t *r = a + (size_t)row * K;
    int s = 0;
    for (int k = lane; k < K; k += 32) s += is_unsigned ? (int)r[k] : (int)(int8_t)r[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) rowsum[row] = s;
}

// pads A [M][K] to [M][Kp] when K is not a multiple of 16 (TMA row pitch)
__global__ void pad_rows_kernel(const uint8_t *__restrict__ a, uint8_t *__restrict__ ap, int M, int K,
                                int Kp) {
    const size_t total = (size_t)M * Kp;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(i % Kp);
        const size_t m = i / Kp;
        ap[i] = (k < K) ? a[m * K + k] : (uint8_t)0;
    }
}

int pack_i8_b(yscv_cuda_ctx *ctx, const int8_t *d_b, size_t k, size_t n, int8_t *d_bt,
              int32_t *d_colsum, size_t kp) {
    const int blocks = (int)((n + 7) / 8);
    pack_i8_b_kernel<<<blocks, 256, 0, ctx->stream>>>(d_b, d_bt, d_colsum, (int)k, (int)n, (int)kp);
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    return YSCV_CUDA_OK;
}

template <int BN>
static int launch_g8(yscv_cuda_ctx *ctx, const void *d_a, size_t lda, const yscv_cuda_i8b *b, size_t m,
                     void *d_out, const G8Params &proto) {
    G8Params p = proto;
    p.M = (int)m;
    p.N = (int)b->n;
    p.K = (int)b->kp;
    p.m_blocks = (p.M + G8_BM - 1) / G8_BM;
    p.n_blocks = (p.N + BN - 1) / BN;
    p.k_blocks = (p.K + G8_BK - 1) / G8_BK;
    const int stage_bytes = G8_BM * G8_BK + BN * G8_BK;
    p.stages = (227 * 1024 - 1024 - G8_XP_BYTES) / stage_bytes;
    if (p.stages > 8) p.stages = 8;
    const int smem = p.stages * stage_bytes + 256 + G8_XP_BYTES;
    CUtensorMap tm_a, tm_b;
    int rc = encode_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d_a, m, b->kp, lda, G8_BM, G8_BK,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = encode_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b->d_bt, b->n, b->kp, b->kp, BN, G8_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    auto kern = int8_gemm_tc_kernel<BN>;
    rc = ensure_dynamic_smem(reinterpret_cast<const void *>(kern), ctx->device, 227 * 1024);
    if (rc) return rc;
    const int tiles = p.m_blocks * p.n_blocks;
    const int sms = ctx->sm_count;
    int grid = tiles < sms ? tiles : sms;
    p.tail_first = tiles;
    p.tail_units = 0;
    // Fewer tiles than half the SMs and a long K loop: cut the K loops into equal runs over all
    // CTAs (see G8Params). The owners' fix-up costs about 4 us at the end of the kernel, which
    // only K >= 8192 on a mostly idle machine pays back (64 x 11008 x 4096: 30.8 -> 22.6 us);
    // with full waves of tiles the extra L2 traffic of the partial sums made every shape tried
    // slower (config 3: 34.9 -> 41.1 us), so those keep whole tiles per CTA.
    const int tail = tiles % sms;
    const long long tail_blocks = (long long)tail * p.k_blocks;
    if (ctx->int8_tail_split && tiles < sms && tail * 2 <= sms && p.k_blocks >= 64) {
        int units = (int)((tail_blocks + sms - 1) / sms);
        if (units < 4) units = 4;  // at most k_blocks / 4 + 1 parts per tile
        const int ctas = (int)((tail_blocks + units - 1) / units);
        rc = ctx->gemm_ws.reserve((size_t)sms * G8_BM * 256 * sizeof(int32_t));
        if (rc) return rc;
        if (!ctx->gemm_flags.ptr) {
            rc = ctx->gemm_flags.reserve((size_t)sms * 4 * sizeof(int));
            if (rc) return rc;
            YSCV_CUDA_TRY(cudaMemsetAsync(ctx->gemm_flags.ptr, 0, (size_t)sms * 4 * sizeof(int), ctx->stream));
        }
        p.tail_first = tiles - tail;
        p.tail_units = units;
        p.ws = reinterpret_cast<int32_t *>(ctx->gemm_ws.ptr);
        p.ws_flag = reinterpret_cast<int *>(ctx->gemm_flags.ptr);
        p.epoch = ++ctx->gemm_epoch;
        grid = p.tail_first > 0 ? sms : ctas;
    }
    snprintf(ctx->report_int8, sizeof(ctx->report_int8),
             "int8_gemm_tc m=%d n=%d k=%d: tcgen05 kind::i8, CTA tile %dx%d, %d stages of %d KB, %d tiles on %d CTAs"
             "%s, %s",
             p.M, p.N, p.K, G8_BM, BN, p.stages, stage_bytes / 1024, tiles, grid,
             p.tail_units ? " (tail split along K)" : "", p.mode == 0 ? "int32 out" : "requantised bytes out");
    ctx->prof_begin();
    YSCV_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(G8_THREADS), (size_t)smem, ctx->stream, tm_a, tm_b,
                             (const int32_t *)b->d_colsum, d_out, p, ctx->d_status));
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    return YSCV_CUDA_OK;
}

static int launch_g8_pair(yscv_cuda_ctx *ctx, const void *d_a, size_t lda, const yscv_cuda_i8b *b, size_t m,
                          void *d_out, const G8Params &proto) {
    G8Params p = proto;
    p.M = (int)m;
    p.N = (int)b->n;
    p.K = (int)b->kp;
    p.m_blocks = (p.M + 255) / 256;
    p.n_blocks = (p.N + G8P_BN - 1) / G8P_BN;
    p.k_blocks = (p.K + G8_BK - 1) / G8_BK;
    p.stages = (227 * 1024 - 1024 - G8_XP_BYTES) / G8P_STAGE;
    if (p.stages > 8) p.stages = 8;
    const int smem = p.stages * G8P_STAGE + 256 + G8_XP_BYTES;
    CUtensorMap tm_a, tm_b;
    int rc = encode_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, d_a, m, b->kp, lda, G8_BM, G8_BK,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = encode_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, b->d_bt, b->n, b->kp, b->kp, G8_BM, G8_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = ensure_dynamic_smem(reinterpret_cast<const void *>(int8_gemm_pair_kernel), ctx->device, 227 * 1024);
    if (rc) return rc;
    const int tiles = p.m_blocks * p.n_blocks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->sm_count / 2 * 2);
    cfg.blockDim = dim3(G8_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    // The kernel is persistent with a static walk over the tiles, so every pair of the grid must
    // be resident at once: a GPC with an odd number of usable SMs leaves one SM without a
    // partner, and a pair that only starts when another has finished would do all its tiles
    // after everybody else's.
    if (ctx->max_pairs == 0) {
        int n = 0;
        YSCV_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, int8_gemm_pair_kernel, &cfg));
        ctx->max_pairs = n > 0 ? n : 1;
    }
    const int pairs = tiles < ctx->max_pairs ? tiles : ctx->max_pairs;
    cfg.gridDim = dim3(2 * pairs);
    snprintf(ctx->report_int8, sizeof(ctx->report_int8),
             "int8_gemm_pair m=%d n=%d k=%d: tcgen05 kind::i8 cta_group::2, pair tile 256x%d, %d stages of %d KB per CTA, "
             "%d tiles on %d CTA pairs (%d can be resident), %s",
             p.M, p.N, p.K, G8P_BN, p.stages, G8P_STAGE / 1024, tiles, pairs, ctx->max_pairs,
             p.mode == 0 ? "int32 out" : "requantised bytes out");
    ctx->prof_begin();
    YSCV_CUDA_TRY(cudaLaunchKernelEx(&cfg, int8_gemm_pair_kernel, tm_a, tm_b, (const int32_t *)b->d_colsum, d_out, p,
                                     ctx->d_status));
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    return YSCV_CUDA_OK;
}

// d_a: [m][k] bytes (i8, or u8 when a_unsigned). mode 0: d_out int32 [m][n]; mode 1: bytes [m][n].
int int8_gemm(yscv_cuda_ctx *ctx, const void *d_a, const yscv_cuda_i8b *b, size_t m, void *d_out,
              int a_unsigned, int a_zp, int mode, float composite, float y_zp, int qmin, int qmax,
              int round_mode, const int32_t *d_corr, const float *d_comp_pc, int relu) {
    G8Params p = {};
    p.corr = d_corr;
    p.comp_pc = d_comp_pc;
    p.relu = relu;
    p.a_unsigned = a_unsigned;
    p.a_zp = a_zp;
    p.mode = mode;
    p.composite = composite;
    p.y_zp = y_zp;
    p.qmin = qmin;
    p.qmax = qmax;
    p.round_mode = round_mode;
    p.ldc = (long long)b->n;
    p.b_zp = b->b_zp;
    p.k_true = (int)b->k;
    if (b->b_zp != 0) {
        int rc = ctx->rowsum.reserve(m * sizeof(int32_t));
        if (rc) return rc;
        rowsum_a_kernel<<<(unsigned)((m + 7) / 8), 256, 0, ctx->stream>>>(
            reinterpret_cast<const uint8_t *>(d_a), reinterpret_cast<int32_t *>(ctx->rowsum.ptr), (int)m,
            (int)b->k, a_unsigned);
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
        p.rowsum = reinterpret_cast<const int32_t *>(ctx->rowsum.ptr);
    }
    const void *a = d_a;
    size_t lda = b->k;
    if (b->k != b->kp || (reinterpret_cast<uintptr_t>(d_a) & 15)) {
        // TMA needs a 16-byte aligned base and row pitch: stage A into a padded copy
        int rc = ctx->scratch.reserve(m * b->kp);
        if (rc) return rc;
        const size_t total = m * b->kp;
        const int blocks = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
        pad_rows_kernel<<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const uint8_t *>(d_a),
                                                         reinterpret_cast<uint8_t *>(ctx->scratch.ptr),
                                                         (int)m, (int)b->k, (int)b->kp);
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
        a = ctx->scratch.ptr;
        lda = b->kp;
    }
    // wide tiles when there are enough of them to fill the machine, else narrower ones
    const size_t tiles256 = ((m + G8_BM - 1) / G8_BM) * ((b->n + 255) / 256);
    // CTA pairs (256 x 256 per pair) once there are enough pair tiles to occupy most pairs
    const size_t pair_tiles = ((m + 255) / 256) * ((b->n + 255) / 256);
    const size_t pairs = (size_t)(ctx->sm_count / 2);
    const bool pair_ok = b->n >= 256 && m >= 256 && pair_tiles * 10 >= pairs * 8;
    // Where the pair kernel measured faster: int32 output (the rows written are four times the
    // bytes, and halving the operand traffic leaves them room) from three rounds of pair tiles
    // on, and a single round of the one-CTA kernel on more than half of the SMs, which the
    // L2 -> SM traffic bounds (1024 x 4096 x 4096: 27.2 -> 22.7 us).
    // Neither holds for K < 2048 (the pair's longer fill shows) or when the 256-row blocks leave
    // the pairs more rounds than the one-CTA kernel has (300 rows: two blocks, the second nearly empty).
    const bool pair_wins = b->kp >= 2048 &&
                           ((mode == 0 && pair_tiles >= 3 * pairs) ||
                            (tiles256 <= (size_t)ctx->sm_count && tiles256 * 2 > (size_t)ctx->sm_count &&
                             pair_tiles <= pairs));
    if (pair_ok && (ctx->int8_pairs > 0 || (ctx->int8_pairs < 0 && pair_wins))) {
        ctx->last_kernel = "int8_gemm_pair(tcgen05,cta_group::2,256x256)";
        return launch_g8_pair(ctx, a, lda, b, m, d_out, p);
    }
    if (b->n >= 256 && tiles256 >= (size_t)ctx->sm_count) {
        ctx->last_kernel = "int8_gemm_tc(tcgen05,128x256)";
        return launch_g8<256>(ctx, a, lda, b, m, d_out, p);
    }
    if (b->n > 64) {
        ctx->last_kernel = "int8_gemm_tc(tcgen05,128x128)";
        return launch_g8<128>(ctx, a, lda, b, m, d_out, p);
    }
    ctx->last_kernel = "int8_gemm_tc(tcgen05,128x64)";
    return launch_g8<64>(ctx, a, lda, b, m, d_out, p);
}

}  // namespace yscv
