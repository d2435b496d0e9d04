// Prefill-shaped (M > 16) packed-int4 x fp32 matmul on the 5th-generation tensor
// cores: weights are dequantised to bf16 in shared memory and multiplied with bf16
// activations by tcgen05.mma.kind::f16 with fp32 accumulators in TMEM.
//
// Replaces packed_int4_gemm_dispatch for large M
// (crates/yscv-kernels/src/ops/int4_matmul.rs:387-435, 548-605) with the same operands:
// weights [N][K/2] nibbles + scales [N][K/32], activations [M][K] f32, output [M][N] f32.
// Accuracy contract: bf16 rounding of q*scale and of the activations, fp32 accumulate;
// relative Frobenius error ~3e-3 against the fp32 scalar kernel (bound 2e-2).
//
// Orientation: the weight rows are the MMA's M side (128 output channels per MMA, one or
// two such tiles per CTA tile), the tokens its N side (a tile of BT tokens, NT tiles per
// pass), so a short prefill still fills the instruction and every weight tile is
// dequantised once per NT*BT tokens.
//
// Kernel: persistent, 448 threads:
//   warp 0      TMA producer: per 64-k block the packed nibbles [128 rows][32 B] and the
//               bf16 activation tile [BT tokens][64 k] (128-byte swizzle)
//   warp 1      allocates TMEM, issues the MMAs (4 per block, N = BT up to 256), commits
//               stages, A buffers and finished accumulators
//   warps 2-9   dequantise: two threads per weight row of the tile, one per 32-k group
//               (consecutive lanes read consecutive 16-byte pieces of the packed tile: no bank
//               conflicts); 8 nibbles become four bf16x2 with 3 shifts + 4 lop3
//               (0x4300 | nibble^8 = 136 + q exactly), then subtract 136 and multiply by the
//               group scale, which was fetched one k block ahead; one 16-byte store per word
//               into the swizzled A tile (double-buffered)
//   warps 10-13 epilogue: tcgen05.ld, coalesced fp32 stores out[token][n]
// The nibble pairs come out as k = (0,4),(1,5),(2,6),(3,7) of each group of 8; the
// activation pre-pass writes its bf16 copy in the same order, so no permutation is
// needed in the loop. All mbarrier waits are bounded.
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.cuh"
#include "tma.cuh"

namespace yscv {

constexpr int PG_BM = 128;      // weight rows per tile
constexpr int PG_BK = 64;       // k per block: 64 bf16 = one 128-byte swizzle row
constexpr int PG_THREADS = 448;
constexpr int PG_DEQ_WARPS = 8;

struct PGParams {
    int M, N, K;
    int BT, NT;          // tokens per MMA tile (multiple of 16, <= 256), tiles per pass
    int n_tiles, t_chunks, k_blocks;
    int stages, stage_bytes;
    int acc_bufs;        // accumulator buffers in TMEM: 2, or 1 when one buffer takes all 512 columns
    // K split (few tiles, e.g. a decode batch of 64 against 8192 weight rows): work item
    // (tile, slice) covers k blocks [slice * kb_per, ...) and writes its fp32 partial sums into
    // slice `slice` of a workspace [ksplit][M][N]; a second kernel adds the slices in order.
    int ksplit, kb_per;
    // k sub-blocks of 64 per ring stage and hand-over (1 or 2). With narrow token tiles a block's
    // MMAs are short and a hand-over (dequantised tile -> MMA -> buffer back) costs ~1000 cycles
    // whatever the work: two sub-blocks per hand-over halve their number. k_blocks, kb_per count stages.
    int ksub;
};

__device__ __forceinline__ void pg_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void pg_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ uint64_t pg_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void pg_mma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void pg_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}

__device__ __forceinline__ void pg_tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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

// fp32 activations -> bf16, k order inside every group of 8 permuted to 0,4,1,5,2,6,3,7
__global__ void act_to_bf16_kernel(const float *__restrict__ act, __nv_bfloat16 *__restrict__ out,
                                   size_t groups8) {
    pdl_wait();      // the activations come from the predecessor, which may also still read `out`
    pdl_trigger();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < groups8;
         i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(act) + 2 * i);
        const float4 b = __ldg(reinterpret_cast<const float4 *>(act) + 2 * i + 1);
        __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, b.x);  // k 0,4
        __nv_bfloat162 p1 = __floats2bfloat162_rn(a.y, b.y);  // k 1,5
        __nv_bfloat162 p2 = __floats2bfloat162_rn(a.z, b.z);  // k 2,6
        __nv_bfloat162 p3 = __floats2bfloat162_rn(a.w, b.w);  // k 3,7
        uint4 v;
        v.x = *reinterpret_cast<uint32_t *>(&p0);
        v.y = *reinterpret_cast<uint32_t *>(&p1);
        v.z = *reinterpret_cast<uint32_t *>(&p2);
        v.w = *reinterpret_cast<uint32_t *>(&p3);
        reinterpret_cast<uint4 *>(out)[i] = v;
    }
}

// NA = 128-row weight tiles per CTA tile (1 or 2). With two, the activation tile of a k block is
// fetched once for 256 weight rows: the kernel is bound by what the SMs pull through the crossbar
// from L2 (with the dequantisation switched off and three quarters of the MMAs left out it still
// takes 0.8 of its time), and the activation tile is nine tenths of that.
// KSUB = 64-k sub-blocks per ring stage and hand-over (1 or 2; PGParams::ksub); SPLITK: the tiles'
// K loops may be cut into slices (PGParams::ksplit > 1), else every tile walks all of K
template <int NA, int KSUB, bool SPLITK>
__global__ void __launch_bounds__(PG_THREADS, 1)
int4_prefill_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                         const float *__restrict__ scales, float *__restrict__ out, PGParams p,
                         int *__restrict__ status) {
    constexpr int W_BYTES = NA * PG_BM * 32;       // packed nibbles of one k block: 4 KB per 128 rows
    constexpr int A_TILE = PG_BM * PG_BK * 2;      // dequantised bf16 tile of 128 rows: 16 KB
    constexpr int A_BUF = KSUB * NA * A_TILE;      // one buffer of dequantised tiles: [sub-block][weight tile]
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = smem_u32(smem);
    // [A buffer 0][A buffer 1][stages x {act tiles NT*BT*128 B | packed nibbles}][barriers][tmem slot]
    const uint32_t a_tiles = smem_base;
    const uint32_t ring = smem_base + 2 * A_BUF;
    const int act_bytes = p.NT * p.BT * 128;       // activation tile of one sub-block; a stage holds
                                                   // [ksub activation tiles][ksub packed tiles]
    const uint32_t bars = ring + (uint32_t)p.stages * p.stage_bytes;
    const uint32_t bar_full = bars, bar_empty = bars + 64, bar_afull = bars + 128, bar_aempty = bars + 144;
    const uint32_t bar_tfull = bars + 160, bar_tempty = bars + 176;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 2 * A_BUF + (size_t)p.stages * p.stage_bytes + 192);
    const int tiles = p.n_tiles * p.t_chunks * (SPLITK ? p.ksplit : 1);
    const int acc_cols = p.NT * p.BT;              // tokens per pass; NA * acc_cols TMEM columns per accumulator buffer (<= 256)

    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(bar_full + i * 8, 1);
            mbar_init(bar_empty + i * 8, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_afull + i * 8, PG_DEQ_WARPS);  // one arrival per dequant warp
            mbar_init(bar_aempty + i * 8, 1);
            mbar_init(bar_tfull + i * 8, 1);
            mbar_init(bar_tempty + i * 8, 4);   // one arrival per epilogue warp
        }
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    pg_fence_before();
    __syncthreads();
    pg_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // programmatic dependent launch: the set-up above may overlap the tail of the predecessor (the
    // activation pre-pass); everything below reads what it wrote or writes what it may still read
    pdl_wait();
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
                const int ksplit = SPLITK ? p.ksplit : 1;
                const int nt_i = t % p.n_tiles, ks = SPLITK ? (t / p.n_tiles) % ksplit : 0, tc = t / (p.n_tiles * ksplit);
                const int kb0 = SPLITK ? ks * p.kb_per : 0, kb1 = SPLITK ? min(p.k_blocks, kb0 + p.kb_per) : p.k_blocks;
                for (int kb = kb0; kb < kb1; ++kb) {
                    alive = mbar_wait(bar_empty + slot * 8, phase ^ 1u, status);
                    if (!alive) break;
                    const uint32_t st = ring + (uint32_t)slot * p.stage_bytes;
                    const uint32_t full = bar_full + slot * 8;
                    mbar_expect_tx(full, (uint32_t)(KSUB * (act_bytes + W_BYTES)));
                    #pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        const int kx = kb * KSUB + sub;   // 64-k block
                        for (int j = 0; j < p.NT; ++j)
                            tma_load_2d(st + sub * act_bytes + j * (p.BT * 128), &tm_a, kx * PG_BK, tc * acc_cols + j * p.BT, full);
                        tma_load_2d(st + KSUB * act_bytes + sub * W_BYTES, &tm_w, kx * 32, nt_i * (NA * PG_BM), full);
                    }
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // D fp32, A and B bf16, both K-major, N = BT, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.BT >> 3) << 17) |
                                   ((uint32_t)(PG_BM >> 4) << 24);
            int slot = 0, abuf = 0, tbuf = 0;
            uint32_t phase = 0, aphase = 0, tphase = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
                alive = mbar_wait(bar_tempty + tbuf * 8, tphase ^ 1u, status);
                if (!alive) break;
                pg_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)tbuf * 256;
                const int kb0 = SPLITK ? ((t / p.n_tiles) % p.ksplit) * p.kb_per : 0;
                const int kb1 = SPLITK ? min(p.k_blocks, kb0 + p.kb_per) : p.k_blocks;
                for (int kb = kb0; kb < kb1; ++kb) {
                    alive = mbar_wait(bar_full + slot * 8, phase, status) &&
                            mbar_wait(bar_afull + abuf * 8, aphase, status);
                    if (!alive) break;
                    pg_fence_after();
                    const uint32_t st = ring + (uint32_t)slot * p.stage_bytes;
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
#pragma unroll
                        for (int a = 0; a < NA; ++a) {
                            const uint64_t da = pg_desc_sw128(a_tiles + abuf * A_BUF + (sub * NA + a) * A_TILE);
                            for (int j = 0; j < p.NT; ++j) {
                                const uint64_t db = pg_desc_sw128(st + sub * act_bytes + j * (p.BT * 128));
#pragma unroll
                                for (int kk = 0; kk < PG_BK / 16; ++kk)  // K = 16 per instruction: +32 bytes
                                    pg_mma_bf16(tacc + a * acc_cols + j * p.BT, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2),
                                                idesc, (kb > kb0 || sub > 0 || kk > 0) ? 1u : 0u);
                            }
                        }
                    }
                    pg_commit(bar_empty + slot * 8);
                    pg_commit(bar_aempty + abuf * 8);
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                    if (++abuf == 2) { abuf = 0; aphase ^= 1u; }
                }
                if (!alive) break;
                pg_commit(bar_tfull + tbuf * 8);
                if (++tbuf == p.acc_bufs) { tbuf = 0; tphase ^= 1u; }
            }
        }
    } else if (warp < 2 + PG_DEQ_WARPS) {
        // ------- dequantise: lanes 2i, 2i+1 share weight row (warp - 2) * 16 + i, one group each -------
        const int r = (warp - 2) * 16 + (lane >> 1), half = lane & 1;
        const int groups = p.K / 32;
        int slot = 0, abuf = 0;
        uint32_t phase = 0, aphase = 0;
        bool alive = true;
        const __nv_bfloat162 bias = __float2bfloat162_rn(136.0f);
        for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
            const int nt_i = t % p.n_tiles;
            const int kb0 = SPLITK ? ((t / p.n_tiles) % p.ksplit) * p.kb_per : 0;
            const int kb1 = SPLITK ? min(p.k_blocks, kb0 + p.kb_per) : p.k_blocks;
            // this thread's weight row in each of the NA tiles, its scale pointer, the scale of the first block
            const float *srow[NA];
            bool live_row[NA];
            float sc_next[KSUB][NA];   // [sub-block][weight tile]
#pragma unroll
            for (int a = 0; a < NA; ++a) {
                const int row = nt_i * (NA * PG_BM) + a * PG_BM + r;
                live_row[a] = row < p.N;
                srow[a] = scales + (size_t)(live_row[a] ? row : 0) * groups + half;
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub)
                    sc_next[sub][a] = live_row[a] ? __ldg(srow[a] + (kb0 * KSUB + sub) * 2) : 0.0f;
            }
            for (int kb = kb0; kb < kb1; ++kb) {
                float sc[KSUB][NA];
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub) {
#pragma unroll
                    for (int a = 0; a < NA; ++a) {
                        sc[sub][a] = sc_next[sub][a];
                        // the next stage's scales travel while this one is converted
                        if (kb + 1 < kb1 && live_row[a])
                            sc_next[sub][a] = __ldg(srow[a] + ((kb + 1) * KSUB + sub) * 2);
                    }
                }
                alive = mbar_wait(bar_full + slot * 8, phase, status) &&
                        mbar_wait(bar_aempty + abuf * 8, aphase ^ 1u, status);
                if (!alive) break;
                const unsigned char *st = smem + 2 * A_BUF + (size_t)slot * p.stage_bytes + KSUB * act_bytes;
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub) {
                    {
#pragma unroll
                        for (int a = 0; a < NA; ++a) {
                            const uint4 w4 = *reinterpret_cast<const uint4 *>(st + sub * W_BYTES + (a * PG_BM + r) * 32 + half * 16);
                            const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
                            const __nv_bfloat162 s2 = __float2bfloat162_rn(sc[sub][a]);
                            unsigned char *arow = smem + (size_t)abuf * A_BUF + (size_t)(sub * NA + a) * A_TILE + (size_t)r * 128;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t w = words[i];
                                uint32_t x[4];
                                // 0x4300 | (nibble ^ 8) is the bf16 value 136 + q, exactly
                                asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[0]) : "r"(w));
                                asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[1]) : "r"(w >> 4));
                                asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[2]) : "r"(w >> 8));
                                asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[3]) : "r"(w >> 12));
                                uint4 o;
                                uint32_t *ov = &o.x;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162 *>(&x[j]);
                                    v = __hmul2(__hsub2(v, bias), s2);
                                    ov[j] = *reinterpret_cast<uint32_t *>(&v);
                                }
                                // 16-byte chunk c of row r sits at chunk c ^ (r & 7) (128-byte swizzle)
                                *reinterpret_cast<uint4 *>(arow + (((half * 4 + i) ^ (r & 7)) << 4)) = o;
                            }
                        }
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
        // ---------------- epilogue: warps 10..13 own TMEM lanes 32*(warp%4).. ----------------
        const int q = warp & 3;
        int tbuf = 0;
        uint32_t tphase = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < tiles && alive; t += gridDim.x) {
            const int ksplit = SPLITK ? p.ksplit : 1;
            const int nt_i = t % p.n_tiles, ks = SPLITK ? (t / p.n_tiles) % ksplit : 0, tc = t / (p.n_tiles * ksplit);
            float *const o_base = SPLITK ? out + (size_t)ks * p.M * p.N : out;   // (ksplit > 1: `out` is the workspace)
            alive = mbar_wait(bar_tfull + tbuf * 8, tphase, status);
            if (!alive) break;
            pg_fence_after();
#pragma unroll 1
            for (int a = 0; a < NA; ++a) {
                const int n = nt_i * (NA * PG_BM) + a * PG_BM + q * 32 + lane;   // output channel of this lane
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)tbuf * 256 + (uint32_t)(a * acc_cols);
#pragma unroll 1
                for (int c0 = 0; c0 < acc_cols; c0 += 32) {
                    uint32_t rr[32];
                    pg_tmem_ld32(taddr + c0, rr);
                    const int tok0 = tc * acc_cols + c0;
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (tok0 + j < p.M) o_base[(size_t)(tok0 + j) * p.N + n] = __uint_as_float(rr[j]);
                    }
                }
            }
            pg_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + tbuf * 8);
            if (++tbuf == p.acc_bufs) { tbuf = 0; tphase ^= 1u; }
        }
    }

    pg_fence_before();
    __syncthreads();
    if (warp == 1) {
        pg_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

// ---------------------------------------------------------------------------
// CTA-pair form for large prefills: tcgen05.mma.cta_group::2
// ---------------------------------------------------------------------------
//
// Two CTAs on the two SMs of a TPC (a cluster of 2) share a tile of 512 weight rows x 256 tokens.
// Each CTA dequantises its own 256 weight rows (two 128-row tiles, as the NA = 2 form above) and
// stages HALF of the activation tile of a k block (128 tokens); the leader (cluster rank 0) issues
// MMAs of M = 256, N = 256 that read both CTAs' shared memory and leave rows 0..127 in its own
// TMEM and rows 128..255 in the peer's. Per k block an SM then pulls 8 KB of nibbles + 16 KB of
// activations from L2 instead of 8 + 32 KB, and its tensor core reads half the activation bytes
// from shared memory per flop: the two limits of the one-CTA form.
//
// Signals (no multicast form; every signal is raised by the unit that finishes the work):
//   full_w[s]    each CTA: its own nibble tile of stage s landed (its dequantising warps wait)
//   full_act[s]  leader: BOTH CTAs' activation halves landed (the peer's load is the
//                .cta_group::2 form of the TMA load, completing its bytes on the leader's barrier)
//   afull[b]     leader, 16 arrivals: the eight dequantising warps of both CTAs filled A buffer b
//                (the peer's warps arrive remotely, after fence.proxy.async)
//   empty[s], aempty[b], tfull   each CTA its own: the leader commits its MMAs to both CTAs' barriers
//   tempty       leader, 8 arrivals: the epilogue warps of both CTAs drained the accumulators
// All waits are bounded; a wait that runs out sets the status word and the roles fall through to the
// cluster barrier at the end.
constexpr int PP_ACT = 128 * 128;              // 128 tokens x 64 k bf16: this CTA's half of the activation tile
constexpr int PP_W = 2 * PG_BM * 32;           // nibbles of this CTA's 256 rows for one k block
constexpr int PP_A_TILE = PG_BM * PG_BK * 2;   // 16 KB
// KSUB 64-k sub-blocks per ring stage and hand-over, as in the one-CTA kernel: a stage holds
// [KSUB activation halves][KSUB nibble tiles], an A buffer [sub-block][weight tile]
template <int KSUB> struct PPGeom {
    static constexpr int STAGE = KSUB * (PP_ACT + PP_W);     // 24 KB per sub-block
    static constexpr int A_BUF = KSUB * 2 * PP_A_TILE;
    static constexpr int ABUFS = KSUB == 1 ? 3 : 2;           // buffers of dequantised tiles
};

__device__ __forceinline__ void pp_mma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// commit to a barrier of either CTA of the pair (shared::cluster address)
__device__ __forceinline__ void pp_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
                 : "memory");
}

template <int KSUB>
__global__ void __launch_bounds__(PG_THREADS, 1)
int4_prefill_pair_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_a,
                         const float *__restrict__ scales, float *__restrict__ out, PGParams p,
                         int *__restrict__ status) {
    constexpr int PP_STAGE = PPGeom<KSUB>::STAGE, PP_A_BUF = PPGeom<KSUB>::A_BUF, PP_ABUFS = PPGeom<KSUB>::ABUFS;
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t smem_base = smem_u32(smem);
    // [A buffers][stages x {activation half | packed nibbles}][barriers][tmem slot]
    const uint32_t a_tiles = smem_base;
    const uint32_t ring = smem_base + PP_ABUFS * PP_A_BUF;
    const uint32_t bars = ring + (uint32_t)p.stages * PP_STAGE;
    const uint32_t bar_full_w = bars, bar_full_act = bars + 64, bar_empty = bars + 128;
    const uint32_t bar_afull = bars + 192, bar_aempty = bars + 224, bar_tfull = bars + 256, bar_tempty = bars + 264;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + PP_ABUFS * PP_A_BUF + (size_t)p.stages * PP_STAGE + 272);
    const int tiles = p.n_tiles * p.t_chunks;   // pair tiles: 512 weight rows x 256 tokens

    if (tid == 0) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(bar_full_w + i * 8, 1);
            mbar_init(bar_full_act + i * 8, 1);
            mbar_init(bar_empty + i * 8, 1);
        }
        for (int i = 0; i < PP_ABUFS; ++i) {
            mbar_init(bar_afull + i * 8, 2 * PG_DEQ_WARPS);
            mbar_init(bar_aempty + i * 8, 1);
        }
        mbar_init(bar_tfull, 1);
        mbar_init(bar_tempty, 8);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                     "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
    }
    pg_fence_before();
    cluster_sync_all();   // both CTAs' barriers exist before anyone arrives on a remote one
    pg_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();      // as in the one-CTA kernel
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_w));
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_a));
            int slot = 0;
            uint32_t phase = 0;
            bool alive = true;
            const uint32_t leader_full_act = map_to_cta(bar_full_act, 0);
            for (int t = pair; t < tiles && alive; t += n_pairs) {
                const int nt_i = t % p.n_tiles, tc = t / p.n_tiles;
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    alive = mbar_wait(bar_empty + slot * 8, phase ^ 1u, status);
                    if (!alive) break;
                    const uint32_t st = ring + (uint32_t)slot * PP_STAGE;
                    if (rank == 0) mbar_expect_tx(bar_full_act + slot * 8, 2 * KSUB * PP_ACT);
                    mbar_expect_tx(bar_full_w + slot * 8, KSUB * PP_W);
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        const int kx = kb * KSUB + sub;   // 64-k block
                        tma_load_2d_pair(st + sub * PP_ACT, &tm_a, kx * PG_BK, tc * 256 + (int)rank * 128, leader_full_act + slot * 8);
                        tma_load_2d(st + KSUB * PP_ACT + sub * PP_W, &tm_w, kx * 32, nt_i * 512 + (int)rank * 256, bar_full_w + slot * 8);
                    }
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader only) ----------------
        if (lane == 0 && rank == 0) {
            // D fp32, A and B bf16, both K-major, N = 256, M = 256 over the pair
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) |
                                   ((uint32_t)(256 >> 4) << 24);
            int slot = 0, abuf = 0;
            uint32_t phase = 0, aphase = 0, tphase = 0;
            bool alive = true;
            const uint32_t peer_empty = map_to_cta(bar_empty, 1), peer_aempty = map_to_cta(bar_aempty, 1);
            const uint32_t peer_tfull = map_to_cta(bar_tfull, 1);
            for (int t = pair; t < tiles && alive; t += n_pairs) {
                alive = mbar_spin_cluster(bar_tempty, tphase ^ 1u, status);
                if (!alive) break;
                pg_fence_after();
                for (int kb = 0; kb < p.k_blocks; ++kb) {
                    alive = mbar_wait_cluster(bar_full_act + slot * 8, phase, status) &&
                            mbar_spin_cluster(bar_afull + abuf * 8, aphase, status);
                    if (!alive) break;
                    pg_fence_after();
#pragma unroll
                    for (int sub = 0; sub < KSUB; ++sub) {
                        const uint64_t db = pg_desc_sw128(ring + (uint32_t)slot * PP_STAGE + sub * PP_ACT);
#pragma unroll
                        for (int a = 0; a < 2; ++a) {
                            const uint64_t da = pg_desc_sw128(a_tiles + abuf * PP_A_BUF + (sub * 2 + a) * PP_A_TILE);
#pragma unroll
                            for (int kk = 0; kk < PG_BK / 16; ++kk)  // K = 16 per instruction: +32 bytes
                                pp_mma_bf16(tmem_base + a * 256, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc,
                                            (kb > 0 || sub > 0 || kk > 0) ? 1u : 0u);
                        }
                    }
                    pp_commit(bar_empty + slot * 8);
                    pp_commit(peer_empty + slot * 8);
                    pp_commit(bar_aempty + abuf * 8);
                    pp_commit(peer_aempty + abuf * 8);
                    if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                    if (++abuf == PP_ABUFS) { abuf = 0; aphase ^= 1u; }
                }
                if (!alive) break;
                pp_commit(bar_tfull);
                pp_commit(peer_tfull);
                tphase ^= 1u;
            }
        }
    } else if (warp < 2 + PG_DEQ_WARPS) {
        // ------- dequantise (both CTAs): lanes 2i, 2i+1 share weight row (warp - 2) * 16 + i of each 128-row tile -------
        const int r = (warp - 2) * 16 + (lane >> 1), half = lane & 1;
        const int groups = p.K / 32;
        int slot = 0, abuf = 0;
        uint32_t phase = 0, aphase = 0;
        bool alive = true;
        const __nv_bfloat162 bias = __float2bfloat162_rn(136.0f);
        const uint32_t leader_afull = map_to_cta(bar_afull, 0);
        for (int t = pair; t < tiles && alive; t += n_pairs) {
            const int nt_i = t % p.n_tiles;
            const float *srow[2];
            bool live_row[2];
            float sc_next[KSUB][2];
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                const int row = nt_i * 512 + (int)rank * 256 + a * PG_BM + r;
                live_row[a] = row < p.N;
                srow[a] = scales + (size_t)(live_row[a] ? row : 0) * groups + half;
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub) sc_next[sub][a] = live_row[a] ? __ldg(srow[a] + sub * 2) : 0.0f;
            }
            for (int kb = 0; kb < p.k_blocks; ++kb) {
                float sc[KSUB][2];
#pragma unroll
                for (int sub = 0; sub < KSUB; ++sub) {
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
                        sc[sub][a] = sc_next[sub][a];
                        // the next stage's scales travel while this one is converted
                        if (kb + 1 < p.k_blocks && live_row[a]) sc_next[sub][a] = __ldg(srow[a] + ((kb + 1) * KSUB + sub) * 2);
                    }
                }
                alive = mbar_wait(bar_full_w + slot * 8, phase, status) &&
                        mbar_wait(bar_aempty + abuf * 8, aphase ^ 1u, status);
                if (!alive) break;
                const unsigned char *st = smem + PP_ABUFS * PP_A_BUF + (size_t)slot * PP_STAGE + KSUB * PP_ACT;
#pragma unroll
                for (int sa = 0; sa < KSUB * 2; ++sa) {
                    const int sub = sa >> 1, a = sa & 1;
                    const uint4 w4 = *reinterpret_cast<const uint4 *>(st + sub * PP_W + (a * PG_BM + r) * 32 + half * 16);
                    const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
                    const __nv_bfloat162 s2 = __float2bfloat162_rn(sc[sub][a]);
                    unsigned char *arow = smem + (size_t)abuf * PP_A_BUF + (size_t)sa * PP_A_TILE + (size_t)r * 128;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t w = words[i];
                        uint32_t x[4];
                        // 0x4300 | (nibble ^ 8) is the bf16 value 136 + q, exactly
                        asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[0]) : "r"(w));
                        asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[1]) : "r"(w >> 4));
                        asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[2]) : "r"(w >> 8));
                        asm("lop3.b32 %0, %1, 0x000f000f, 0x43084308, 0x6a;\n" : "=r"(x[3]) : "r"(w >> 12));
                        uint4 o;
                        uint32_t *ov = &o.x;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162 *>(&x[j]);
                            v = __hmul2(__hsub2(v, bias), s2);
                            ov[j] = *reinterpret_cast<uint32_t *>(&v);
                        }
                        // 16-byte chunk c of row r sits at chunk c ^ (r & 7) (128-byte swizzle)
                        *reinterpret_cast<uint4 *>(arow + (((half * 4 + i) ^ (r & 7)) << 4)) = o;
                    }
                }
                // make the generic-proxy writes visible to the async proxy: each CTA's tensor core reads
                // the A tile of its own shared memory
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(leader_afull + abuf * 8);
                if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                if (++abuf == PP_ABUFS) { abuf = 0; aphase ^= 1u; }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): warps 10..13 own TMEM lanes 32*(warp%4).. ----------------
        const int q = warp & 3;
        uint32_t tphase = 0;
        bool alive = true;
        const uint32_t leader_tempty = map_to_cta(bar_tempty, 0);
        for (int t = pair; t < tiles && alive; t += n_pairs) {
            const int nt_i = t % p.n_tiles, tc = t / p.n_tiles;
            alive = mbar_wait(bar_tfull, tphase, status);
            if (!alive) break;
            pg_fence_after();
#pragma unroll 1
            for (int a = 0; a < 2; ++a) {
                const int n = nt_i * 512 + (int)rank * 256 + a * PG_BM + q * 32 + lane;   // output channel of this lane
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * 256);
#pragma unroll 1
                for (int c0 = 0; c0 < 256; c0 += 32) {
                    uint32_t rr[32];
                    pg_tmem_ld32(taddr + c0, rr);
                    const int tok0 = tc * 256 + c0;
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (tok0 + j < p.M) out[(size_t)(tok0 + j) * p.N + n] = __uint_as_float(rr[j]);
                    }
                }
            }
            pg_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(leader_tempty);
            tphase ^= 1u;
        }
    }

    // neither CTA may leave (or give its TMEM back) while the other can still read its shared
    // memory or arrive on its barriers
    pg_fence_before();
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        pg_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512));
    }
}

// out = slice 0 + slice 1 + ... of the K-split workspace, in that order
__global__ void __launch_bounds__(256) add_kslices_kernel(const float4 *__restrict__ ws, float4 *__restrict__ out,
                                                          size_t n4, int slices) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        float4 a = ws[i];
        for (int s = 1; s < slices; ++s) {
            const float4 b = ws[(size_t)s * n4 + i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        out[i] = a;
    }
}

size_t int4_prefill_scratch_bytes(size_t m, size_t k) { return m * k * 2 + 256; }

bool int4_prefill_supported(size_t m, size_t n, size_t k, size_t gs) {
    return tensor_map_encoder() != nullptr && gs == 32 && k % 64 == 0 && m > 16 && n >= 1 &&
           m < (1u << 30) && n < (1u << 30) && k < (1u << 30);
}

template <int KSUB>
static int launch_prefill_pairs(yscv_cuda_ctx *ctx, const CUtensorMap &tm_w, const CUtensorMap &tm_a,
                                const float *scales, float *out, PGParams p) {
    using G = PPGeom<KSUB>;
    p.n_tiles = (p.N + 511) / 512;
    p.t_chunks = (p.M + 255) / 256;
    p.ksub = KSUB;
    p.k_blocks = p.K / (PG_BK * KSUB);
    p.ksplit = 1;
    p.acc_bufs = 1;
    p.stage_bytes = G::STAGE;
    p.stages = (227 * 1024 - G::ABUFS * G::A_BUF - 1024) / G::STAGE;
    if (p.stages > 8) p.stages = 8;
    const int smem = G::ABUFS * G::A_BUF + p.stages * G::STAGE + 512;
    auto kern = int4_prefill_pair_kernel<KSUB>;
    int rc = ensure_dynamic_smem(reinterpret_cast<const void *>(kern), ctx->device, 227 * 1024);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->sm_count / 2 * 2);
    cfg.blockDim = dim3(PG_THREADS);
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
    // persistent kernel with a static walk over the tiles: every pair of the grid must be resident
    if (ctx->max_prefill_pairs == 0) {
        int nres = 0;
        YSCV_CUDA_TRY(cudaOccupancyMaxActiveClusters(&nres, kern, &cfg));
        ctx->max_prefill_pairs = nres > 0 ? nres : 1;
    }
    const int tiles = p.n_tiles * p.t_chunks;
    const int pairs = tiles < ctx->max_prefill_pairs ? tiles : ctx->max_prefill_pairs;
    cfg.gridDim = dim3(2 * pairs);
    ctx->prof_begin();
    YSCV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tm_w, tm_a, scales, out, p, ctx->d_status));
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    snprintf(ctx->report_int4, sizeof(ctx->report_int4),
             "int4_prefill_gemm m=%d n=%d k=%d: tcgen05 bf16 cta_group::2, pair tile 512 rows x 256 tokens, %d k per stage, "
             "%d stages of %d KB per CTA, %d tiles on %d CTA pairs", p.M, p.N, p.K, KSUB * PG_BK, p.stages, G::STAGE / 1024, tiles, pairs);
    ctx->last_kernel = "int4_prefill_gemm(tcgen05,bf16,cta_group::2)";
    return YSCV_CUDA_OK;
}

// act_bf16 != nullptr: the activations are already bf16 in the GEMM's k order (what the pre-pass
// below writes; the decoder's norm and SwiGLU kernels can emit it): `act` and `scratch` are not used.
int int4_prefill_gemm(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales, const float *act,
                      float *out, size_t m, size_t n, size_t k, void *scratch, const void *act_bf16) {
    PGParams p = {};
    int rc_ws = 0;
    p.M = (int)m;
    p.N = (int)n;
    p.K = (int)k;
    // Two 128-row weight tiles per CTA tile (256 rows x up to 256 tokens, the two accumulators
    // filling all 512 TMEM columns, so the epilogue no longer overlaps the next tile) when that
    // still gives every SM a tile: the activation tile, nine tenths of the L2 -> SM traffic, is
    // then fetched once per 256 weight rows (2048 x 8192 x 8192: 918 -> 1121 TFLOP/s; 256 rows x
    // 128 tokens with double-buffered accumulators measured 664: N = 128 MMAs read a third more
    // shared memory per flop). Otherwise one weight tile x up to 256 tokens, accumulators
    // double-buffered. One MMA tile per pass (N = BT, a multiple of 16).
    const int m16 = (int)((m + 15) / 16 * 16);
    const size_t tiles2 = ((n + 2 * PG_BM - 1) / (2 * PG_BM)) * ((m + 255) / 256);
    const int NA = (m16 > 128 && tiles2 >= (size_t)ctx->sm_count) ? 2 : 1;
    const int bt_max = 256;
    p.BT = m16 <= bt_max ? m16 : bt_max;
    p.NT = 1;
    const int acc_cols = p.BT * p.NT;
    p.acc_bufs = NA * acc_cols > 256 ? 1 : 2;
    p.n_tiles = (p.N + NA * PG_BM - 1) / (NA * PG_BM);
    p.t_chunks = (p.M + acc_cols - 1) / acc_cols;
    // narrow token tiles: two 64-k sub-blocks per stage and hand-over (see PGParams)
    p.ksub = (NA == 1 && p.BT <= 128 && p.K % (2 * PG_BK) == 0) ? 2 : 1;
    p.k_blocks = p.K / (PG_BK * p.ksub);
    p.stage_bytes = ((p.ksub * (p.NT * p.BT * 128 + NA * PG_BM * 32) + 1023) / 1024) * 1024;
    p.stages = (227 * 1024 - 2 * p.ksub * NA * PG_BM * PG_BK * 2 - 1024) / p.stage_bytes;
    if (p.stages > 8) p.stages = 8;
    const int smem = 2 * p.ksub * NA * PG_BM * PG_BK * 2 + p.stages * p.stage_bytes + 256;
    // A decode batch (one narrow token tile): cut K into slices so that the work items fill whole
    // rounds of CTAs. Among 1..8 slices take the count with the shortest makespan
    // (rounds of items / slices), as long as a slice keeps at least 512 k and the fp32 partial sums
    // (written and read once per slice) stay below the bytes of the weights.
    p.ksplit = 1;
    {
        const int base_tiles = p.n_tiles * p.t_chunks;
        if (NA == 1 && p.t_chunks == 1 && p.BT <= 128 && (m * n) % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
            const int sms = ctx->sm_count;
            double best = (double)((base_tiles + sms - 1) / sms);
            for (int sl = 2; sl <= 8; ++sl) {
                if (p.k_blocks / sl < 8 / p.ksub) break;
                if (16.0 * sl * (double)m > (double)k) break;
                const double cost = (double)((base_tiles * sl + sms - 1) / sms) / sl + 0.02 * sl;
                if (cost < best - 1e-9) { best = cost; p.ksplit = sl; }
            }
        }
    }
    p.kb_per = (p.k_blocks + p.ksplit - 1) / p.ksplit;
    p.ksplit = (p.k_blocks + p.kb_per - 1) / p.kb_per;   // no empty slice (33 blocks in 8 slices of 5: seven slices)
    float *kernel_out = out;
    if (p.ksplit > 1) {
        rc_ws = ctx->gemm_ws.reserve((size_t)p.ksplit * m * n * sizeof(float));
        if (rc_ws) return rc_ws;
        kernel_out = reinterpret_cast<float *>(ctx->gemm_ws.ptr);
    }

    // CTA pairs (512 weight rows x 256 tokens per pair) when every pair still gets a tile
    const size_t pair_tiles = ((n + 511) / 512) * ((m + 255) / 256);
    const bool use_pairs = ctx->prefill_pairs && NA == 2 && pair_tiles >= (size_t)(ctx->sm_count / 2);

    const __nv_bfloat16 *abf = reinterpret_cast<const __nv_bfloat16 *>(act_bf16);
    if (!abf) {
        __nv_bfloat16 *mine = reinterpret_cast<__nv_bfloat16 *>(scratch);
        const size_t groups8 = m * k / 8;
        const unsigned cb = (unsigned)((groups8 + 255) / 256 < 8192 ? (groups8 + 255) / 256 : 8192);
        YSCV_CUDA_TRY(launch_pdl(act_to_bf16_kernel, dim3(cb), dim3(256), 0, ctx->stream, act, mine, groups8));
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
        abf = mine;
    }

    CUtensorMap tm_w, tm_a;
    int rc = encode_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, n, k / 2, k / 2, (uint32_t)(NA * PG_BM), 32,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    rc = encode_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, abf, m, k, k * 2, use_pairs ? 128u : (uint32_t)p.BT, PG_BK,
                   CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (use_pairs) {
        // two 64-k sub-blocks per stage and hand-over whenever K allows: 243 -> 232 us on 2048 x 8192 x 8192
        const bool two = p.K % (2 * PG_BK) == 0;
        return two ? launch_prefill_pairs<2>(ctx, tm_w, tm_a, scales, out, p) : launch_prefill_pairs<1>(ctx, tm_w, tm_a, scales, out, p);
    }
    auto kern = NA == 2 ? int4_prefill_gemm_kernel<2, 1, false>
                        : p.ksub == 2 ? (p.ksplit > 1 ? int4_prefill_gemm_kernel<1, 2, true> : int4_prefill_gemm_kernel<1, 2, false>)
                                      : (p.ksplit > 1 ? int4_prefill_gemm_kernel<1, 1, true> : int4_prefill_gemm_kernel<1, 1, false>);
    {
        const int arc = ensure_dynamic_smem(reinterpret_cast<const void *>(kern), ctx->device, 227 * 1024);
        if (arc) return arc;
    }
    const int tiles = p.n_tiles * p.t_chunks * p.ksplit;
    const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    ctx->prof_begin();
    YSCV_CUDA_TRY(launch_pdl(kern, dim3(grid), dim3(PG_THREADS), (size_t)smem, ctx->stream, tm_w, tm_a, scales, kernel_out, p,
                             ctx->d_status));
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    if (p.ksplit > 1) {
        const size_t n4 = m * n / 4;
        const unsigned blocks = (unsigned)((n4 + 255) / 256 < 1184 ? (n4 + 255) / 256 : 1184);
        YSCV_CUDA_TRY(launch_pdl(add_kslices_kernel, dim3(blocks), dim3(256), 0, ctx->stream,
                                 reinterpret_cast<const float4 *>(kernel_out), reinterpret_cast<float4 *>(out), n4, p.ksplit));
        ctx->launches++;
    }
    snprintf(ctx->report_int4, sizeof(ctx->report_int4),
             "int4_prefill_gemm m=%zu n=%zu k=%zu: tcgen05 bf16, CTA tile %d rows x %d tokens, %d k per stage, %d stages, "
             "%d K slice(s), %d tiles on %d CTAs", m, n, k, NA * PG_BM, p.BT, p.ksub * PG_BK, p.stages, p.ksplit, tiles, grid);
    ctx->last_kernel = "int4_prefill_gemm(tcgen05,bf16)";
    return YSCV_CUDA_OK;
}

}  // namespace yscv
