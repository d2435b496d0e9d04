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
//    the per-(row,group) scale is applied in fp32. Weights, scales and digit
//    planes are staged through shared memory by TMA (one producer thread per
//    CTA issues three or four bulk copies per stage into an mbarrier-guarded
//    ring; no register or issue-slot cost for bytes in flight), read back
//    conflict-free through the hardware XOR swizzle, and turned into MMA
//    fragments with 3 logic ops per 8 nibbles. One persistent CTA per SM owns a
//    contiguous row range; inside the CTA the K range of a stage is split
//    across warps and the partial sums are combined in a fixed order
//    (deterministic, no atomics). Every mbarrier wait is bounded.
#include "common.cuh"
#include "int4_digits.cuh"
#include "kernels.cuh"
#include "tma.cuh"

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

__global__ void __launch_bounds__(128)
act_quant_kernel(const float *__restrict__ act, unsigned char *__restrict__ blobs, int M, int K,
                 QuantLayout q) {
    // programmatic dependent launch: the activations come from the predecessor, and the main kernel of
    // the previous call may still read the blobs
    pdl_wait();
    pdl_trigger();
    const int slots = quant_slots(q);
    const int total = (K / 32) * slots;
    const int t = threadIdx.x & 3;
    const int quads = (gridDim.x * blockDim.x) >> 2;
    const int rounds = (total + quads - 1) / quads;  // same trip count for every lane
    for (int r = 0; r < rounds; ++r) {
        const int item = r * quads + ((blockIdx.x * blockDim.x + threadIdx.x) >> 2);
        const bool valid = item < total;
        const int Gabs = valid ? item % (K / 32) : 0, m = valid ? item / (K / 32) : 0;
        quantize_group(m < M ? act + (size_t)m * K + Gabs * 32 + 8 * t : nullptr, blobs, q, Gabs, m,
                       t, valid);
    }
}

// ---------------------------------------------------------------------------
// Fast kernel
// ---------------------------------------------------------------------------


struct FastGeom {
    int tiles;        // 16-row tiles per row block (1..TP2)
    int stages;       // ring depth
    int w_bytes, s_bytes, stage_bytes;
    int act_bytes;    // > 0: the producer stages the activations [M][K] in shared memory first
    QuantLayout q;
};

constexpr int FAST_CONSUMER_WARPS = 16;
constexpr int FAST_THREADS = (FAST_CONSUMER_WARPS + 1) * 32;  // + one producer warp

// MP  = padded M (1,2,4,8,16)
// GS  = groups of 32 k per stage: 16 (512 k) or 8 (256 k)
// TP2 = warps along the rows of a row block (2 or 8); the other 16/TP2 warps of
//       a tile split the stage's groups between them
//
// Shared memory: `stages` x { weights [GS/8 atoms][rows][128 B] (TMA 128B swizzle),
// scales [rows][GS] f32 (TMA 64B / 32B swizzle), digit blob }, then the reduction
// buffer, then the full[] / empty[] mbarriers.
//
// FUSEQ: the CTA quantises the activations itself into a shared-memory copy of the
// digit blobs (all K stages resident) while the first weight stages are in flight;
// otherwise the blobs come from global memory (act_quant_kernel ran before) and each
// stage brings its own.
template <int MP, int GS, int TP2, bool FUSEQ>
__global__ void __launch_bounds__(FAST_THREADS, 1)
int4_gemv_fast_kernel(const __grid_constant__ CUtensorMap tm_w,
                      const __grid_constant__ CUtensorMap tm_s,
                      const unsigned char *__restrict__ blobs, const float *__restrict__ act,
                      float *__restrict__ out, int M, int N, int K, FastGeom g,
                      int *__restrict__ status) {
    constexpr bool COLS = (MP <= 2);           // digit planes in MMA columns
    constexpr int NT = (MP > 8) ? 2 : 1;       // 8-wide activation tiles (planes form)
    constexpr int NACC = COLS ? 2 : NT * 4;
    constexpr int KSL = (16 / TP2 < GS) ? 16 / TP2 : GS;  // K slices per tile
    constexpr int GPW = GS / KSL;              // groups per warp per stage
    constexpr int ATOMS = GS / 8;              // 128-byte swizzle atoms per weight row per stage
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t = lane & 3;
    // let the next kernel of the stream be scheduled as soon as SMs free up
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // N * gridDim.x < 2^31 is checked on the host: 32-bit division is enough
    const int r0 = (int)(((unsigned)N * blockIdx.x) / gridDim.x);
    const int r1 = (int)(((unsigned)N * (blockIdx.x + 1)) / gridDim.x);
    if (r0 >= r1) return;
    const int rb_rows = g.tiles * 16;
    const int n_rb = (r1 - r0 + rb_rows - 1) / rb_rows;
    const int k_stages = K / (GS * 32);
    const int total = n_rb * k_stages;
    const uint32_t ring_bytes = (uint32_t)g.stages * g.stage_bytes;
    float *red = reinterpret_cast<float *>(smem + ring_bytes);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_base + ring_bytes + 16 * 8 * 32 * 4;
    const uint32_t bar_empty = bar_full + 8 * 8;
    const uint32_t bar_act = bar_empty + 8 * 8;
    unsigned char *dig = smem + ring_bytes + 16 * 8 * 32 * 4 + 2 * 8 * 8 + 16;  // FUSEQ: resident blobs
    float *act_s = reinterpret_cast<float *>(dig + (size_t)(K / (32 * GS)) * g.q.blob_bytes);
    // byte offset of the digit blob relative to the stage base (per-stage copy) or to `dig`
    const uint32_t b_off = FUSEQ ? 0u : (uint32_t)(g.w_bytes + g.s_bytes);

    // ---------------- producer: one thread drives the TMA ring ----------------
    // With the activations staged by TMA (act_bytes > 0) they are the first copy in the
    // queue and the first ring of weight stages follows immediately, before the block-wide
    // sync. Without that staging the ring is issued after the sync on purpose: ~200 KB of
    // weight traffic per SM in front of the consumers' own activation loads delays the
    // quantisation prologue by about 2 us.
    const bool is_producer = (warp == FAST_CONSUMER_WARPS) && (lane == 0);
    const uint32_t tx = (uint32_t)(g.w_bytes + g.s_bytes + (FUSEQ ? 0 : g.q.blob_bytes));
    int p_slot = 0, p_ks = 0, p_rb = 0;
    uint32_t p_phase = 0;
    auto issue_stage = [&]() {
        const uint32_t st = smem_base + (uint32_t)p_slot * g.stage_bytes;
        const uint32_t full = bar_full + p_slot * 8;
        const int row0 = r0 + p_rb * rb_rows;
        mbar_expect_tx(full, tx);
#pragma unroll
        for (int a = 0; a < ATOMS; ++a)
            tma_load_2d(st + a * (rb_rows * 128), &tm_w, p_ks * (GS * 16) + a * 128, row0, full);
        tma_load_2d(st + g.w_bytes, &tm_s, p_ks * GS, row0, full);
        if constexpr (!FUSEQ)
            bulk_load(st + b_off, blobs + (size_t)p_ks * g.q.blob_bytes, g.q.blob_bytes, full);
        if (++p_slot == g.stages) { p_slot = 0; p_phase ^= 1u; }
        if (++p_ks == k_stages) { p_ks = 0; ++p_rb; }
    };
    const int first_wave = total < g.stages ? total : g.stages;
    if (is_producer) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_w));
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tm_s));
        for (int i = 0; i < g.stages; ++i) {
            mbar_init(bar_full + i * 8, 1);
            mbar_init(bar_empty + i * 8, FAST_CONSUMER_WARPS);
        }
        mbar_init(bar_act, 1);
        mbar_fence_init();
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        if (FUSEQ && g.act_bytes > 0) {
            asm volatile("griddepcontrol.wait;\n" ::: "memory");  // activations come from a predecessor
            mbar_expect_tx(bar_act, (uint32_t)g.act_bytes);
            bulk_load(smem_u32(act_s), act, (uint32_t)g.act_bytes, bar_act);
            for (int it = 0; it < first_wave; ++it) issue_stage();
        }
    }
    __syncthreads();
    // everything below reads a predecessor's output (activations / digit blobs) or writes
    // memory a predecessor may still be reading (the output)
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    if (warp == FAST_CONSUMER_WARPS) {
        if (lane == 0) {
            if (!(FUSEQ && g.act_bytes > 0))
                for (int it = 0; it < first_wave; ++it) issue_stage();
            bool alive = true;
            for (int it = first_wave; it < total && alive; ++it) {
                alive = mbar_wait(bar_empty + p_slot * 8, p_phase ^ 1u, status);
                if (alive) issue_stage();
            }
            // A consumer that gave up leaves copies unobserved: wait (bounded) for every
            // stage this thread armed before the CTA may exit.
            if (!alive) {
                for (int i = 0; i < g.stages; ++i) mbar_wait(bar_full + i * 8, 0, nullptr);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    if constexpr (FUSEQ) {
        // quantise the activations while the first weight stages are in flight
        const int slots = quant_slots(g.q);
        const int items = (K / 32) * slots;
        constexpr int QUADS = FAST_CONSUMER_WARPS * 8;
        const int rounds = (items + QUADS - 1) / QUADS;
        const bool staged = g.act_bytes > 0;
        bool act_ok = true;
        if (staged) act_ok = mbar_wait(bar_act, 0, status);
        for (int r = 0; r < rounds; ++r) {
            const int item = r * QUADS + (tid >> 2);
            const bool valid = item < items;
            const int Gabs = valid ? item % (K / 32) : 0, m = valid ? item / (K / 32) : 0;
            const size_t off = (size_t)m * K + Gabs * 32 + 8 * t;
            if (staged)
                quantize_group<true>(m < M && act_ok ? act_s + off : nullptr, dig, g.q, Gabs, m, t, valid);
            else
                quantize_group<false>(m < M ? act + off : nullptr, dig, g.q, Gabs, m, t, valid);
        }
        named_bar_sync(1, FAST_CONSUMER_WARPS * 32);
    }
    const int tile = warp % TP2;
    const int kslice = warp / TP2;
    const bool active = (tile < g.tiles) && (kslice < KSL);
    const int G0 = kslice * GPW;  // first group of this warp inside a stage
    const int rowA = tile * 16 + gq;  // the second row (rowA + 8) has the same swizzle phases

    // offsets relative to the stage base, constant for the whole kernel
    uint32_t w_off[GPW];
#pragma unroll
    for (int gi = 0; gi < GPW; ++gi) {
        const int G = G0 + gi;
        w_off[gi] = (uint32_t)(G >> 3) * (rb_rows * 128) + (uint32_t)rowA * 128 +
                    ((((uint32_t)G & 7u) ^ (uint32_t)(rowA & 7)) << 4) + t * 4;
    }
    // scale tile: 16-byte chunk j of a row sits at chunk j ^ phase (TMA 64B / 32B swizzle)
    const uint32_t s_phase = (GS == 16) ? ((rowA >> 1) & 3) : ((rowA >> 2) & 1);
    const uint32_t s_row = g.w_bytes + (uint32_t)rowA * (GS * 4);
    // the digit-blob layout is a pure function of (MP, GS): keep it in compile-time constants
    // so that every per-group offset below folds into an immediate (see quant_layout())
    constexpr int Q_MS = COLS ? (MP == 1 ? 4 : 8) : (MP < 8 ? MP + 1 : MP);
    constexpr int Q_MC = COLS ? 4 : (MP <= 8 ? 8 : 16);
    constexpr int Q_OFF_H1 = COLS ? 0 : GS * Q_MS * 4 * 16;
    constexpr int Q_OFF_META = COLS ? 0 : Q_OFF_H1 + GS * Q_MS * 4 * 8;
    constexpr int fc = COLS ? Q_MS : 1;  // columns stored per group (columns form)
    const int mslot = (MP < 8) ? min(gq, Q_MS - 1) : gq;
    const uint32_t f_off = COLS ? b_off + (uint32_t)((G0 * fc + (gq & (fc - 1))) * 4 + t) * 16
                                : b_off + (uint32_t)((G0 * Q_MS + mslot) * 4 + t) * 16;
    const uint32_t h1_off = b_off + Q_OFF_H1 + (uint32_t)((G0 * Q_MS + mslot) * 4 + t) * 8;
    const uint32_t mt_off = b_off + Q_OFF_META + (uint32_t)(G0 * Q_MC + 2 * t) * 8;
    constexpr uint32_t f_step = COLS ? fc * 4 * 16 : Q_MS * 4 * 16;  // bytes per group
    constexpr uint32_t h1_step = Q_MS * 4 * 8, mt_step = Q_MC * 8;
    // 16-byte chunk offsets of this thread's scale groups (four groups per chunk)
    uint32_t s_ch[(GPW + 3) / 4];
#pragma unroll
    for (int c = 0; c < (GPW + 3) / 4; ++c)
        s_ch[c] = s_row + (((((uint32_t)(G0 + 4 * c)) >> 2) ^ s_phase) << 4);
    const int mul_hi = (t & 1) ? 1 : 65536;  // columns form: plane weight of this thread's c0

    float acc[NACC];
#pragma unroll
    for (int j = 0; j < NACC; ++j) acc[j] = 0.0f;

    int c_slot = 0, c_ks = 0, c_rb = 0;
    uint32_t c_phase = 0;
    bool dead = false;  // a wait ran out: keep walking the loop (the named barriers below
                        // still need this warp) but stop waiting and computing
    for (int it = 0; it < total; ++it) {
        if (!dead) dead = !mbar_wait(bar_full + c_slot * 8, c_phase, status);
        if (active && !dead) {
            const unsigned char *st = smem + (size_t)c_slot * g.stage_bytes;
            // digit blob of this K stage: inside the stage, or in the resident copy
            const unsigned char *db = FUSEQ ? dig + (size_t)c_ks * g.q.blob_bytes : st;
            float sA[GPW], sB[GPW];
            if constexpr (GPW % 4 == 0) {
#pragma unroll
                for (int gi = 0; gi < GPW; gi += 4) {
                    const uint4 x = lds128(st, s_ch[gi / 4]);
                    const uint4 y = lds128(st, s_ch[gi / 4] + 8 * (GS * 4));
                    sA[gi] = __uint_as_float(x.x); sA[gi + 1] = __uint_as_float(x.y);
                    sA[gi + 2] = __uint_as_float(x.z); sA[gi + 3] = __uint_as_float(x.w);
                    sB[gi] = __uint_as_float(y.x); sB[gi + 1] = __uint_as_float(y.y);
                    sB[gi + 2] = __uint_as_float(y.z); sB[gi + 3] = __uint_as_float(y.w);
                }
            } else {
#pragma unroll
                for (int gi = 0; gi < GPW; ++gi) {
                    const uint32_t G = (uint32_t)(G0 + gi);
                    const uint32_t o = (((G >> 2) ^ s_phase) << 4) + (G & 3u) * 4;
                    sA[gi] = lds_f32(st, s_row + o);
                    sB[gi] = lds_f32(st, s_row + 8 * (GS * 4) + o);
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
                    const uint4 f = lds128(db, f_off + gi * f_step);
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
                        const uint4 h0 = lds128(db, f_off + gi * f_step + n * (8 * 4 * 16));
                        const uint2 h1 = lds64(db, h1_off + gi * h1_step + n * (8 * 4 * 8));
                        const uint4 mt = lds128(db, mt_off + gi * mt_step + n * (8 * 8));
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
        // this warp is done reading the stage: hand the slot back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + c_slot * 8);
        if (++c_slot == g.stages) { c_slot = 0; c_phase ^= 1u; }
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
            named_bar_sync(1, FAST_CONSUMER_WARPS * 32);
            const int row0 = r0 + c_rb * rb_rows;
            if constexpr (COLS) {
                // element (tile, half, gq, m): sum over K slices and the thread pair t=2m,2m+1
                const int items = g.tiles * 2 * 8 * MP;
                for (int i = tid; i < items; i += FAST_CONSUMER_WARPS * 32) {
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
                for (int i = tid; i < items; i += FAST_CONSUMER_WARPS * 32) {
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
            if (c_rb < n_rb) named_bar_sync(1, FAST_CONSUMER_WARPS * 32);  // `red` is reused
        }
    }
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
    return tensor_map_encoder() != nullptr && gs == 32 && k % 256 == 0 && k >= 256 && m >= 1 &&
           m <= 16 && n >= 1 && n < (1u << 22) && k < (1u << 24);
}

// Largest resident digit copy the fused-quantisation variant keeps in shared memory.
constexpr int FUSEQ_MAX_DIGIT_BYTES = 72 * 1024;

template <int MP, int GS, int TP2, bool FUSEQ>
static int launch_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                       const unsigned char *blobs, const float *act, float *out, int M, int N,
                       int K, const QuantLayout &q) {
    const int grid = ctx->sm_count;
    const int rows_per_cta = (N + grid - 1) / grid;
    FastGeom g;
    g.q = q;
    g.tiles = min(TP2, (rows_per_cta + 15) / 16);
    const int rb_rows = g.tiles * 16;
    g.w_bytes = rb_rows * GS * 16;
    g.s_bytes = rb_rows * GS * 4;
    const int digit_bytes = FUSEQ ? (K / (32 * GS)) * q.blob_bytes : 0;
    // stage the activations through TMA when they are small (M <= 2) and 16-byte aligned
    g.act_bytes = (FUSEQ && MP <= 2 && (size_t)M * K * 4 <= 32 * 1024 &&
                   (reinterpret_cast<uintptr_t>(act) & 15) == 0) ? M * K * 4 : 0;
    g.stage_bytes = ((g.w_bytes + g.s_bytes + (FUSEQ ? 0 : q.blob_bytes) + 1023) / 1024) * 1024;
    const int red_bytes = 16 * 8 * 32 * 4;
    const int bar_bytes = 2 * 8 * 8 + 16;
    const int budget = 227 * 1024 - red_bytes - bar_bytes - digit_bytes - g.act_bytes - 1024;
    g.stages = max(2, min(8, budget / g.stage_bytes));
    const int smem = g.stages * g.stage_bytes + red_bytes + bar_bytes + digit_bytes + g.act_bytes;
    // tensor maps: weights as bytes [N][K/2], box [rb_rows][128] with the 128-byte swizzle;
    // scales as f32 [N][K/32], box [rb_rows][GS] with the swizzle that matches its width
    // (a decode loop calls with the same few weight matrices over and over: the encoded maps of the
    // last calls are kept in the context; a map depends only on the addresses and the shape)
    static_assert(sizeof(CUtensorMap) == sizeof(ctx->tm_cache[0].w), "tensor map size");
    int rc;
    yscv_cuda_ctx::TmCacheEntry *ce = nullptr;
    for (auto &e : ctx->tm_cache)
        if (e.a == wq && e.b == scales && e.n == N && e.k == K && e.rows == rb_rows && e.gs == GS) ce = &e;
    if (!ce) {
        ce = &ctx->tm_cache[ctx->tm_next];
        ctx->tm_next = (ctx->tm_next + 1) % (int)(sizeof(ctx->tm_cache) / sizeof(ctx->tm_cache[0]));
        ce->a = nullptr;
        rc = encode_2d(reinterpret_cast<CUtensorMap *>(ce->w), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, wq, (uint64_t)N,
                       (uint64_t)K / 2, (uint64_t)K / 2, (uint32_t)rb_rows, 128, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        rc = encode_2d(reinterpret_cast<CUtensorMap *>(ce->s), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, scales, (uint64_t)N,
                       (uint64_t)K / 32, (uint64_t)K / 8, (uint32_t)rb_rows, GS,
                       GS == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
        if (rc) return rc;
        ce->a = wq; ce->b = scales; ce->n = N; ce->k = K; ce->rows = rb_rows; ce->gs = GS;
    }
    const CUtensorMap &tm_w = *reinterpret_cast<const CUtensorMap *>(ce->w), &tm_s = *reinterpret_cast<const CUtensorMap *>(ce->s);
    auto kern = int4_gemv_fast_kernel<MP, GS, TP2, FUSEQ>;
    rc = ensure_dynamic_smem(reinterpret_cast<const void *>(kern), ctx->device, 227 * 1024);
    if (rc) return rc;
    snprintf(ctx->report_int4, sizeof(ctx->report_int4),
             "int4_gemv_fast m=%d(pad %d) n=%d k=%d: %d-row blocks, %d groups/stage, %d stages, %s, grid %d",
             M, MP, N, K, rb_rows, GS, g.stages, FUSEQ ? "activations quantised in the kernel" : "digit planes from scratch",
             grid);
    ctx->prof_begin();
    // Programmatic dependent launch: this grid may be scheduled while the previous kernel of
    // the stream drains; it touches nothing a predecessor may have written (activations,
    // digit blobs) or may still read (the output) before griddepcontrol.wait.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(FAST_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    YSCV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tm_w, tm_s, blobs, act, out, M, N, K, g, ctx->d_status));
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    return YSCV_CUDA_OK;
}

template <int MP, int GS>
static int launch_fast_tp(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                          const float *act, float *out, int M, int N, int K, void *scratch) {
    const QuantLayout q = quant_layout(MP, GS);
    const int rows_per_cta = (N + ctx->sm_count - 1) / ctx->sm_count;
    const bool small = rows_per_cta <= 32;
    if constexpr (MP <= 4) {
        // few activation rows: every CTA quantises them itself, no separate launch
        if ((K / (32 * GS)) * q.blob_bytes <= FUSEQ_MAX_DIGIT_BYTES) {
            ctx->last_kernel = "int4_gemv_fast(imma,tma,fused-quant)";
            return small ? launch_fast<MP, GS, 2, true>(ctx, wq, scales, nullptr, act, out, M, N, K, q)
                         : launch_fast<MP, GS, 8, true>(ctx, wq, scales, nullptr, act, out, M, N, K, q);
        }
    }
    unsigned char *blobs = reinterpret_cast<unsigned char *>(scratch);
    const int items = (K / 32) * quant_slots(q);
    YSCV_CUDA_TRY(launch_pdl(act_quant_kernel, dim3((items * 4 + 127) / 128), dim3(128), 0, ctx->stream, act, blobs, M, K, q));
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    ctx->last_kernel = "int4_gemv_fast(imma,tma)";
    return small ? launch_fast<MP, GS, 2, false>(ctx, wq, scales, blobs, act, out, M, N, K, q)
                 : launch_fast<MP, GS, 8, false>(ctx, wq, scales, blobs, act, out, M, N, K, q);
}

int int4_gemv_fast(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales, const float *act,
                   float *out, size_t m, size_t n, size_t k, void *scratch) {
    const int M = (int)m, N = (int)n, K = (int)k;
    const int MP = padded_m(M);
    const int GS = stage_groups(MP, K);
    switch (MP) {
        case 1: return GS == 16 ? launch_fast_tp<1, 16>(ctx, wq, scales, act, out, M, N, K, scratch)
                                : launch_fast_tp<1, 8>(ctx, wq, scales, act, out, M, N, K, scratch);
        case 2: return GS == 16 ? launch_fast_tp<2, 16>(ctx, wq, scales, act, out, M, N, K, scratch)
                                : launch_fast_tp<2, 8>(ctx, wq, scales, act, out, M, N, K, scratch);
        case 4: return GS == 16 ? launch_fast_tp<4, 16>(ctx, wq, scales, act, out, M, N, K, scratch)
                                : launch_fast_tp<4, 8>(ctx, wq, scales, act, out, M, N, K, scratch);
        case 8: return launch_fast_tp<8, 8>(ctx, wq, scales, act, out, M, N, K, scratch);
        default: return launch_fast_tp<16, 8>(ctx, wq, scales, act, out, M, N, K, scratch);
    }
}

// ---------------------------------------------------------------------------
// Entry point for callers that must not allocate
// ---------------------------------------------------------------------------

// Scratch of the allocation-free entry point: the digit planes of up to 16 activation
// rows of length up to YSCV_STATIC_SCRATCH_MAX_K. Every GPU that loads this library
// holds these ~1.7 MB until the process exits.
constexpr size_t YSCV_STATIC_SCRATCH_MAX_K = 32768;
constexpr size_t YSCV_STATIC_SCRATCH_BYTES = (YSCV_STATIC_SCRATCH_MAX_K / 256) * 13312 + 256;
static __device__ __align__(256) unsigned char g_static_scratch[YSCV_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a stand-in for the device array, never an
// address a kernel may be given; the real address is looked up once per device.
static void *g_static_scratch_ptr[64] = {nullptr};
static std::mutex g_static_scratch_mutex;

// the scratch-using variant only: digit planes are always produced by act_quant_kernel
template <int MP, int GS>
static int launch_scratch_variant(yscv_cuda_ctx *ctx, const uint8_t *wq, const float *scales,
                                  const float *act, float *out, int M, int N, int K,
                                  unsigned char *blobs) {
    const QuantLayout q = quant_layout(MP, GS);
    const int rows_per_cta = (N + ctx->sm_count - 1) / ctx->sm_count;
    const int items = (K / 32) * quant_slots(q);
    YSCV_CUDA_TRY(launch_pdl(act_quant_kernel, dim3((items * 4 + 127) / 128), dim3(128), 0, ctx->stream, act, blobs, M, K, q));
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    ctx->last_kernel = "int4_gemv_fast(imma,tma,static-scratch)";
    return rows_per_cta <= 32
               ? launch_fast<MP, GS, 2, false>(ctx, wq, scales, blobs, act, out, M, N, K, q)
               : launch_fast<MP, GS, 8, false>(ctx, wq, scales, blobs, act, out, M, N, K, q);
}

}  // namespace yscv

extern "C" int yscv_cuda_int4_matmul_dev_static(yscv_cuda_ctx *ctx, const uint8_t *d_packed,
                                                const float *d_scales, size_t n, size_t k,
                                                size_t group_size, const float *d_activation,
                                                float *d_output, size_t m) {
    using namespace yscv;
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (!d_packed || !d_scales || !d_activation || !d_output)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (m == 0) return YSCV_CUDA_OK;
    if (m > 16)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED,
                    "the allocation-free entry point takes at most 16 activation rows, got %zu", m);
    if (k > YSCV_STATIC_SCRATCH_MAX_K)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED,
                    "k=%zu exceeds the %zu the built-in scratch array was sized for", k,
                    (size_t)YSCV_STATIC_SCRATCH_MAX_K);
    const bool aligned = ((reinterpret_cast<uintptr_t>(d_packed) | reinterpret_cast<uintptr_t>(d_scales) |
                           reinterpret_cast<uintptr_t>(d_activation)) & 15) == 0;
    if (!aligned || !int4_gemv_fast_supported(m, n, k, group_size))
        return fail(YSCV_CUDA_ERR_UNSUPPORTED,
                    "the allocation-free entry point needs group_size 32, k %% 256 == 0 and 16-byte "
                    "aligned operands (n=%zu k=%zu group=%zu)", n, k, group_size);
    if (int4_gemv_scratch_bytes(m, k) > YSCV_STATIC_SCRATCH_BYTES)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "scratch need exceeds the built-in array");
    if (ctx->device < 0 || ctx->device >= 64) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "device index");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    unsigned char *blobs = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (!g_static_scratch_ptr[ctx->device]) {
            // first call on this device: resolve the device address of the array
            void *ptr = nullptr;
            YSCV_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
            g_static_scratch_ptr[ctx->device] = ptr;
        }
        blobs = reinterpret_cast<unsigned char *>(g_static_scratch_ptr[ctx->device]);
    }
    const int M = (int)m, N = (int)n, K = (int)k;
    const int MP = padded_m(M);
    const int GS = stage_groups(MP, K);
    switch (MP) {
        case 1: return GS == 16 ? launch_scratch_variant<1, 16>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs)
                                : launch_scratch_variant<1, 8>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs);
        case 2: return GS == 16 ? launch_scratch_variant<2, 16>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs)
                                : launch_scratch_variant<2, 8>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs);
        case 4: return GS == 16 ? launch_scratch_variant<4, 16>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs)
                                : launch_scratch_variant<4, 8>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs);
        case 8: return launch_scratch_variant<8, 8>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs);
        default: return launch_scratch_variant<16, 8>(ctx, d_packed, d_scales, d_activation, d_output, M, N, K, blobs);
    }
}

namespace yscv {

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
