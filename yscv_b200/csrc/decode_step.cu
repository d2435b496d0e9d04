// One launch = one single-token decode step (batch 1) through every layer of a Llama-shaped
// int4 decoder.
//
// The reference runs a decode step as a chain of ONNX nodes (apps/llm-bench/src/main.rs:491-561
// drives crates/yscv-onnx/src/runner: the packed-int4 MatMul of linear.rs:223-278, RMSNorm
// norm.rs:1497-1518, rotate-half RoPE rope.rs:24-117, the KV-cache append kv_cache.rs:118-254,
// grouped-query attention linear.rs:552-646, SiLU activation.rs:1000-1005). At batch 1 every
// linear moves a few MB, so on this GPU a chain of separate launches spends its time between
// kernels, not in them. Here the whole stack is one persistent cooperative kernel, one CTA per
// SM:
//
//   * one producer thread per CTA walks the layers' four weight matrices (qkv, output, gate+up,
//     down) in order and streams this CTA's rows of each through a TMA ring; the weights are
//     constants, so the ring keeps filling across operator boundaries and never waits for an
//     activation;
//   * 16 consumer warps run the operators: residual add + RMSNorm (or SwiGLU) fused into the
//     staging of the activation vector, its conversion to block-fixed-point digit planes, the
//     integer-MMA dot products of the M = 1 decode GEMV (same arithmetic as int4_gemv.cu), the
//     residual add fused into the store of the output and down projections, and RoPE + cache
//     append + attention with one CTA per query head;
//   * operators that need another CTA's output are separated by a grid-wide barrier (a counter
//     in global memory, bounded spin, abort flag), five per layer.
//
// A CTA's rows of a matrix are walked in row blocks of at most 8 tiles of 16 rows; the digit
// planes of at most 8192 activations are resident at a time, so a longer down projection is
// walked in K chunks (stage a chunk, consume its stages, keep the accumulators).
//
// Limits (checked when the plan is built): group size 32, K % 512 == 0, hidden and
// n_q * head_dim <= 8192, head_dim <= 128.
//
// decode_step_batch.cuh (included below) is the form for 2..8 sequences per step.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "int4_digits.cuh"
#include "kernels.cuh"
#include "tma.cuh"

namespace yscv {

constexpr int DS_CONSUMER_WARPS = 16;
constexpr int DS_CONSUMERS = DS_CONSUMER_WARPS * 32;
constexpr int DS_THREADS = DS_CONSUMERS + 32;  // + the producer warp
constexpr int DS_GS = 16;                      // groups of 32 k per stage
constexpr int DS_RED_BYTES = 4096;             // K slices x tiles x 2 accumulators x 32 lanes, f32
constexpr int DS_BAR_BYTES = 256;
constexpr int DS_MAX_STAGES = 8;
constexpr int DS_BLOB_BYTES = DS_GS * 4 * 4 * 16;  // digit blob of one stage (M = 1, columns form)
constexpr int DS_SPIN_LIMIT = 1 << 21;
constexpr int DS_DEFAULT_VARIANT = 7;  // pairing, sixteen slices, merge table; the relaxed poll measured slower

// One int4 linear as the kernel sees it (array in global memory).
struct alignas(64) StepMat {
    CUtensorMap tm_w;  // weights as bytes [n][k/2], box [tiles*16][128], 128-byte swizzle
    CUtensorMap tm_s;  // scales as f32 [n][k/32], box [tiles*16][16], 64-byte swizzle
    int n, k, tiles, k_stages;
    int pad[12];
};

struct StepParams {
    const StepMat *mats;      // [layers][4]: qkv, output, gate+up, down
    const float *gamma;       // [layers][2][hidden]
    float *const *kcache;     // [layers] -> [max_seq][n_kv][d_head] (f32, or int8 when kv_int8), then
    float *const *vcache;     // (int8 only) [layers] -> [max_seq] f32 row scales
    int kv_int8;
    const float *embedding;   // [vocab][hidden]
    const int32_t *token;
    const int32_t *pos;
    float *x;                 // [hidden] residual stream, result of the step
    float *qkv, *attn, *gu;   // scratch between operators; attn = [n_q][splits][d_head + 2]
    int splits;               // CTAs per query head in the attention phase
    // grouped attention (long contexts): one CTA per (KV head, key chunk) serves all the query
    // heads of the group from one pass over the chunk's keys and values; a short second phase
    // merges the g_splits chunks of every head into attn_out [n_q][d_head]
    int attn_grouped, g_splits, g_chunk_cap;
    float *attn_out;
    // optional tail (tail != 0): final RMSNorm, fp32 LM head [vocab][hidden] -> logits [vocab],
    // greedy argmax (last index among equal maxima) into *token_out, *pos_out = position + 1
    int tail;
    const float *final_gamma, *lm_head;
    float *logits;
    float *best_val;          // [gridDim.x] per-CTA maxima
    int *best_idx;
    int32_t *token_out, *pos_out;
    unsigned int *sync;       // [0] barrier arrivals, [1] CTAs that left, [2] abort flag
    int *status;
    int layers, hidden, inter, n_q, n_kv, d_head, max_seq, vocab;
    float eps, theta;
    int stages, slot_bytes, dig_bytes, act_floats;
    // shape of the four matrices of a layer (the same in every layer): rows, 16-row tiles per
    // CTA, K stages; kept here so that no thread waits on global memory to learn them
    int mat_n[4], mat_tiles[4], mat_ks[4];
    int mat_kps[4];  // K stages per ring slot: a matrix with few rows per CTA packs several
    int mat_nrb[4];  // row blocks a CTA walks per matrix (each of mat_tiles tiles)
    int kc_stages;   // K stages whose digit planes fit the digit area at once (a K chunk); only
                     // the down projection may be longer than one chunk
    // gate/up pairing: a CTA owns the intermediate indices [i0, i1) and streams gate rows
    // [i0, i1) and up rows [inter + i0, inter + i1) as the two halves of its slab, so that
    // silu(gate) * up is formed in the store of that GEMV (gu then holds [inter] values)
    int pair_gu;     // 0: gate_up rows split like any matrix, SwiGLU while staging the down GEMV
    int gu_half_tiles;
    int one_tile_16;  // 1: a one-tile slab is split over 16 K slices (all warps) instead of 8
    int merge_table;  // 1: the split-merge weights go through a shared-memory table
    int relaxed_poll; // 1: the barrier polls with relaxed loads and fences once
    int spin_limit;   // probes after which a waiting CTA gives up (grid barrier, peer slots)
    // tensor parallelism (tp_size > 1): this launch is one rank of tp_size identical launches on
    // tp_size GPUs. The weights handed to the plan are this rank's shards (n_q, n_kv, inter are
    // the local counts); the output and down projections then produce partial sums over K, which
    // the ranks exchange through tp_peer[r], rank r's exchange region mapped into this process
    // (peer memory over NVLink; tp_peer[tp_rank] is the local one):
    //   slot word (parity, source rank, row) = {f32 partial sum, 32-bit tag} as one 64-bit store,
    //   written into every peer's region by the thread that owns the row, who then polls its own
    //   region until all tp_size - 1 words carry this exchange's tag and adds them in rank order.
    // No multicast, no atomics, no collective library inside the step.
    int tp_rank, tp_size, tp_cap;          // tp_cap: rows per (parity, source) slot array
    unsigned long long *tp_peer[8];
    unsigned int *tp_seq;                  // steps this plan has run (device word, local)
    int lm_row0, lm_rows;                  // this rank's rows of the LM head (all of them when tp_size == 1)
    // batch form (decode_step_batch_kernel): sequences per step, all at the same position. x, qkv,
    // attn, gu, logits, best_val / best_idx and the token arrays then hold `batch` rows; the caches
    // are [batch][max_seq][n_kv][d_head]
    int batch, red_bytes;
};


// ---- consumer-side helpers (the 512 consumer threads only; named barrier 1) ---------------

__device__ __forceinline__ void cons_sync() { named_bar_sync(1, DS_CONSUMERS); }

__device__ __forceinline__ float cons_sum(float v, float *misc) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    cons_sync();  // misc may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) misc[threadIdx.x >> 5] = v;
    cons_sync();
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < DS_CONSUMER_WARPS; ++i) t += misc[i];
    return t;
}

__device__ __forceinline__ float cons_max(float v, float *misc) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    cons_sync();
    if ((threadIdx.x & 31) == 0) misc[threadIdx.x >> 5] = v;
    cons_sync();
    float t = -INFINITY;
#pragma unroll
    for (int i = 0; i < DS_CONSUMER_WARPS; ++i) t = fmaxf(t, misc[i]);
    return t;
}

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned int ld_relaxed_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_sys_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;\n" ::"l"(p), "l"(v) : "memory");
}

// Slot index of exchange word (parity, source rank, row); slots past the row arrays hold the
// greedy-token exchange: (parity, source rank, {value, index}).
__device__ __forceinline__ size_t tp_slot(const StepParams &p, int parity, int src, int row) {
    return ((size_t)(parity * p.tp_size + src)) * p.tp_cap + row;
}
__device__ __forceinline__ size_t tp_arg_slot(const StepParams &p, int parity, int src, int which) {
    return (size_t)2 * p.tp_size * p.tp_cap + (size_t)((parity * p.tp_size + src) * 2 + which);
}

// Polls one word of the local exchange region until it carries `tag`. Bounded: after
// p.spin_limit probes the abort flag and the status word are set and whatever is there is
// returned; a raised abort flag ends the wait early.
__device__ __forceinline__ unsigned int tp_wait_word(const StepParams &p, const unsigned long long *src,
                                                     unsigned int tag) {
    unsigned long long w = ld_relaxed_sys_u64(src);
    int spins = 0;
    while ((unsigned int)(w >> 32) != tag) {
        ++spins;
        if ((spins & 63) == 0 && ld_acquire_u32(&p.sync[2]) != 0u) {
            *p.status = YSCV_DEV_FLAG_TIMEOUT;
            break;
        }
        if (spins > p.spin_limit) {
            atomicExch(&p.sync[2], 1u);
            *p.status = YSCV_DEV_FLAG_TIMEOUT;
            break;
        }
        w = ld_relaxed_sys_u64(src);
    }
    return (unsigned int)w;
}

// All-reduce of one element of a row-parallel GEMV across the ranks, by the thread that owns
// the row: publish this rank's partial sum in every peer's region, then add the ranks'
// partials in rank order (the same order, hence the same bits, on every rank).
__device__ __forceinline__ float tp_reduce_row(const StepParams &p, int row, float v, unsigned int tag,
                                               int parity) {
    const unsigned long long word = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    const size_t mine = tp_slot(p, parity, p.tp_rank, row);
    for (int r = 0; r < p.tp_size; ++r)
        if (r != p.tp_rank) st_relaxed_sys_u64(p.tp_peer[r] + mine, word);
    const unsigned long long *local = p.tp_peer[p.tp_rank];
    // Every pending peer's word is probed in the same round (the loads of a round are in flight
    // together: one trip to L2 per round instead of one per peer). Bounded like tp_wait_word:
    // after p.spin_limit rounds, or when another CTA has raised the abort flag, the status word
    // is set and whatever is there is summed.
    unsigned long long w[8];
    unsigned int pending = 0u;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        w[r] = 0ull;
        if (r < p.tp_size && r != p.tp_rank) pending |= 1u << r;
    }
    for (int spins = 0; pending != 0u; ++spins) {
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if ((pending >> r) & 1u) w[r] = ld_relaxed_sys_u64(local + tp_slot(p, parity, r, row));
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (((pending >> r) & 1u) && (unsigned int)(w[r] >> 32) == tag) pending &= ~(1u << r);
        if (pending == 0u) break;
        if ((spins & 63) == 63 && ld_acquire_u32(&p.sync[2]) != 0u) {
            *p.status = YSCV_DEV_FLAG_TIMEOUT;
            break;
        }
        if (spins > p.spin_limit) {
            atomicExch(&p.sync[2], 1u);
            *p.status = YSCV_DEV_FLAG_TIMEOUT;
            break;
        }
    }
    float sum = 0.0f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if (r < p.tp_size) {
            const float part = r == p.tp_rank ? v : __uint_as_float((unsigned int)w[r]);
            sum = r == 0 ? part : sum + part;
        }
    }
    return sum;
}

// Grid-wide barrier of the consumers. `epoch` counts the barriers of this launch (the same in
// every thread). A CTA that waits longer than the limit raises the abort flag; from then on
// every barrier of every CTA falls through, the kernel runs to its end and the host finds the
// status word set.
__device__ __forceinline__ void grid_barrier(const StepParams &p, unsigned int &epoch) {
    ++epoch;
    cons_sync();
    if (threadIdx.x == 0) {
        // release: the CTA's writes (ordered before this thread by the bar.sync above) become
        // visible before the arrival; the acquire load that sees the last arrival orders
        // everything after the barrier behind all CTAs' writes
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;\n" ::"l"(p.sync) : "memory");
        const unsigned int target = epoch * gridDim.x;
        int spins = 0;
        while ((p.relaxed_poll ? ld_relaxed_u32(&p.sync[0]) : ld_acquire_u32(&p.sync[0])) < target) {
            ++spins;
            if ((spins & 63) == 0 && ld_acquire_u32(&p.sync[2]) != 0u) {
                // another CTA gave up (in this launch or an earlier one of the same plan): the
                // step's result is void, say so again in case the status word was read and cleared
                *p.status = YSCV_DEV_FLAG_TIMEOUT;
                break;
            }
            if (spins > p.spin_limit) {
                atomicExch(&p.sync[2], 1u);
                *p.status = YSCV_DEV_FLAG_TIMEOUT;
                break;
            }
        }
        if (p.relaxed_poll) asm volatile("fence.acq_rel.gpu;\n" ::: "memory");
    }
    cons_sync();
}

// The activation vector is in act_s: turn it into the digit planes of every K stage.
// The all-zero padding row of the columns form (`pad`) never changes: it is written once per
// launch, for the longest K, and nothing else touches the digit area afterwards.
__device__ __forceinline__ void quantize_activation(const float *act_s, unsigned char *dig, int K, bool pad) {
    const QuantLayout q = quant_layout(1, DS_GS);
    const int tid = threadIdx.x, t = tid & 3;
    const int items = (K / 32) * (pad ? 2 : 1);
    const int rounds = (items + DS_CONSUMERS / 4 - 1) / (DS_CONSUMERS / 4);
    for (int r = 0; r < rounds; ++r) {
        const int item = r * (DS_CONSUMERS / 4) + (tid >> 2);
        const bool valid = item < items;
        const int Gabs = valid ? item % (K / 32) : 0, m = valid ? item / (K / 32) : 0;
        quantize_group<true>(m < 1 ? act_s + Gabs * 32 + 8 * t : nullptr, dig, q, Gabs, m, t, valid);
    }
    cons_sync();
}

struct RingPos {
    int slot;
    uint32_t phase;
};

// The M = 1 GEMV of one row block of a matrix: consume_stages walks K stages [ks_begin, ks_end)
// of the block in the ring and adds into the two accumulators of the thread; finish_rows
// combines the K slices in a fixed order and stores. Same fragment arithmetic as
// int4_gemv_fast_kernel<1, 16, TP2, true>. `dig_stage0` is the K stage whose digit planes sit
// at the start of the digit area (the first stage of the current K chunk).
template <int TP2>
__device__ __forceinline__ void consume_stages(const StepParams &p, const unsigned char *smem,
                                               uint32_t bar_full, uint32_t bar_empty,
                                               const unsigned char *dig, RingPos &c, int tiles,
                                               int ks_begin, int ks_end, int kps, int dig_stage0,
                                               float (&acc)[2], bool &dead) {
    constexpr int GS = DS_GS;
    constexpr int KSL = (16 / TP2 < GS) ? 16 / TP2 : GS;
    constexpr int GPW = GS / KSL;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, t = lane & 3;
    const int rb_rows = tiles * 16;
    const uint32_t w_bytes = (uint32_t)rb_rows * GS * 16;
    const int tile = warp % TP2, kslice = warp / TP2;
    const bool active = (tile < tiles) && (kslice < KSL);
    const int G0 = kslice * GPW;
    const int rowA = tile * 16 + gq;
    uint32_t w_off[GPW];
#pragma unroll
    for (int gi = 0; gi < GPW; ++gi) {
        const int G = G0 + gi;
        w_off[gi] = (uint32_t)(G >> 3) * (rb_rows * 128) + (uint32_t)rowA * 128 +
                    ((((uint32_t)G & 7u) ^ (uint32_t)(rowA & 7)) << 4) + t * 4;
    }
    const uint32_t s_phase = (rowA >> 1) & 3;
    const uint32_t s_row = w_bytes + (uint32_t)rowA * (GS * 4);
    const uint32_t f_off = (uint32_t)((G0 * 4 + (gq & 3)) * 4 + t) * 16;
    constexpr uint32_t f_step = 4 * 4 * 16;
    uint32_t s_ch[(GPW + 3) / 4];
#pragma unroll
    for (int cc = 0; cc < (GPW + 3) / 4; ++cc)
        s_ch[cc] = s_row + (((((uint32_t)(G0 + 4 * cc)) >> 2) ^ s_phase) << 4);
    const int mul_hi = (t & 1) ? 1 : 65536;

    const uint32_t sub_bytes = (uint32_t)rb_rows * (GS * 16 + GS * 4);  // one K stage inside a slot
    for (int ks0 = ks_begin; ks0 < ks_end; ks0 += kps) {
        if (!dead) dead = !mbar_wait(bar_full + c.slot * 8, c.phase, p.status);
        const int nsub = min(kps, ks_end - ks0);
        if (active && !dead) {
            for (int j = 0; j < nsub; ++j) {
                const unsigned char *st = smem + (size_t)c.slot * p.slot_bytes + (size_t)j * sub_bytes;
                const unsigned char *db = dig + (size_t)(ks0 + j - dig_stage0) * DS_BLOB_BYTES;
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
                    const uint4 f = lds128(db, f_off + gi * f_step);
                    int cfrag[4];
                    mma_u8s8(cfrag, a, f.x, f.y, 0, 0, 0, 0);
                    const int vA = cfrag[0] * mul_hi + (cfrag[1] * 256 + (int)f.w);
                    const int vB = cfrag[2] * mul_hi + (cfrag[3] * 256 + (int)f.w);
                    const float as = __uint_as_float(f.z);
                    acc[0] = fmaf(sA[gi] * as, (float)vA, acc[0]);
                    acc[1] = fmaf(sB[gi] * as, (float)vB, acc[1]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + c.slot * 8);
        if (++c.slot == p.stages) { c.slot = 0; c.phase ^= 1u; }
    }
}

// store: 0 out[row] = v; 1 out[row] = resid + v (resid fetched by the caller before the K loop);
// 2 the block is gate tiles then up tiles of intermediate indices: out[i] = silu(gate_i) * up_i.
// Rows (indices) of the block start at row_base; nothing at or past r1 is written.
template <int TP2>
__device__ __forceinline__ void finish_rows(const StepParams &p, float *red, int tiles, int row_base, int r1,
                                            float *out, int store, const float (&acc)[2], float resid,
                                            unsigned int tp_tag, int tp_parity) {
    constexpr int GS = DS_GS;
    constexpr int KSL = (16 / TP2 < GS) ? 16 / TP2 : GS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = warp % TP2, kslice = warp / TP2;
    const bool active = (tile < tiles) && (kslice < KSL);
    if (active) {
        red[((kslice * tiles + tile) * 2 + 0) * 32 + lane] = acc[0];
        red[((kslice * tiles + tile) * 2 + 1) * 32 + lane] = acc[1];
    }
    cons_sync();
    const int my_row = row_base + (tid >> 4) * 16 + (tid & 7) + ((tid >> 3) & 1) * 8;
    // element (tile, half, gq): sum over the K slices and the thread pair t = 0, 1
    if (store == 2) {
        const int th = tiles / 2;
        if (tid < th * 16) {
            const int q8 = tid & 7, half = (tid >> 3) & 1, tl = tid >> 4;
            float g = 0.0f, u = 0.0f;
            for (int ks = 0; ks < KSL; ++ks) {
                const float *pg = red + ((ks * tiles + tl) * 2 + half) * 32 + q8 * 4;
                const float *pu = red + ((ks * tiles + tl + th) * 2 + half) * 32 + q8 * 4;
                g += pg[0] + pg[1];
                u += pu[0] + pu[1];
            }
            const float sg = 1.0f / (1.0f + expf(-g));
            if (my_row < r1) out[my_row] = (g * sg) * u;
        }
    } else if (tid < tiles * 16) {   // tiles <= 8: at most 128 rows, one per thread
        const int q8 = tid & 7, half = (tid >> 3) & 1, tl = tid >> 4;
        float v = 0.0f;
        for (int ks = 0; ks < KSL; ++ks) {
            const float *pp = red + ((ks * tiles + tl) * 2 + half) * 32 + q8 * 4;
            v += pp[0] + pp[1];
        }
        // store 1 under tensor parallelism: v is this rank's partial sum over its K slice
        if (my_row < r1) {
            if (store == 1 && p.tp_size > 1) v = tp_reduce_row(p, my_row, v, tp_tag, tp_parity);
            out[my_row] = store == 1 ? resid + v : v;
        }
    }
    cons_sync();  // `red` is reused by the next block
}

// Grouped attention, phase 1. CTA (kvh, split): RoPE of the group's queries and of the new key,
// cache append (the split that holds the new position), scores of all the group's query heads
// against this split's keys (the key row quarter a thread holds serves every head), a local
// softmax per head, the unnormalised weighted value sums. Leaves {acc[d], max, exp-sum} per
// (query head, split) in p.attn. Scratch: q [grp][d], new k and v [d] each, partial sums
// [parts][grp][d], 32 floats, scores [grp][chunk_cap].
__device__ __forceinline__ void attention_group(const StepParams &p, int kvh, int split, int pos,
                                                float *kc, float *vc, const float *rope_cs,
                                                float *scratch, const float *qkv_base = nullptr,
                                                float *attn_base = nullptr) {
    // (batch form: the sequence's own q|k|v row, partial-result block and cache slices)
    const float *const qkv_in = qkv_base ? qkv_base : p.qkv;
    float *const attn_o = attn_base ? attn_base : p.attn;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int d = p.d_head, half = d / 2;
    const int grp = p.n_q / p.n_kv, S = p.g_splits, cap = p.g_chunk_cap;
    const int vecs = d / 4, parts = DS_CONSUMERS / (grp * vecs);
    float *qs = scratch, *kcur = qs + grp * d, *vcur = kcur + d, *partial = vcur + d;
    float *wred = partial + parts * grp * d, *scores = wred + 32;
    const size_t kv_stride = (size_t)p.n_kv * d;
    const float *kbase = kc + (size_t)kvh * d, *vbase = vc + (size_t)kvh * d;
    const int limit = pos + 1;
    const int chunk = (limit + S - 1) / S;
    const int k0 = split * chunk, k1 = min(limit, k0 + chunk);
    const int h0 = kvh * grp;   // first query head of the group
    if (k0 >= k1) {  // nothing for this split yet: the neutral element of the merge
        for (int i = tid; i < grp * (d + 2); i += DS_CONSUMERS) {
            const int hh = i / (d + 2), j = i - hh * (d + 2);
            attn_o[((size_t)(h0 + hh) * S + split) * (d + 2) + j] = j == d ? -INFINITY : 0.0f;
        }
        return;
    }
    const int nk = k1 - k0;
    const bool has_new = pos >= k0 && pos < k1;

    // ---- loads: the first 128 key rows of the chunk (a quarter row per thread), q, new k, v ----
    constexpr int KQ = 8;
    const int kq = tid >> 2, sub = tid & 3, q4n = d / 16;
    float4 kreg[KQ];
#pragma unroll
    for (int j = 0; j < KQ; ++j)
        kreg[j] = (j < q4n && k0 + kq < p.max_seq)
                      ? __ldg(reinterpret_cast<const float4 *>(kbase + (size_t)(k0 + kq) * kv_stride + sub * (d / 4)) + j)
                      : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    // one rotary pair per thread: the group's queries (grp * d/2 pairs), then the new key
    for (int i = tid; i < (grp + 1) * half; i += DS_CONSUMERS) {
        const int hh = i / half, ri = i - hh * half;
        const bool is_k = hh == grp;
        const float *src = qkv_in + (size_t)(is_k ? p.n_q + kvh : h0 + hh) * d;
        const float x0 = __ldcg(src + ri), x1 = __ldcg(src + ri + half);
        const float cs = rope_cs[2 * ri], sn = rope_cs[2 * ri + 1];
        const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
        float *dst = is_k ? kcur : qs + hh * d;
        dst[ri] = y0;
        dst[ri + half] = y1;
        if (is_k && has_new) {
            float *cd = kc + ((size_t)pos * p.n_kv + kvh) * d;
            cd[ri] = y0;
            cd[ri + half] = y1;
        }
    }
    for (int i = tid; i < d; i += DS_CONSUMERS) {
        const float v = __ldcg(qkv_in + (size_t)(p.n_q + p.n_kv + kvh) * d + i);
        vcur[i] = v;
        if (has_new) vc[((size_t)pos * p.n_kv + kvh) * d + i] = v;
    }
    cons_sync();

    // ---- scores: four threads per key; the quarter row in registers serves every query head ----
    const float scale = 1.0f / sqrtf((float)d);
    if (k0 + kq == pos) {
        const float4 *kcur4 = reinterpret_cast<const float4 *>(kcur + sub * (d / 4));
#pragma unroll
        for (int j = 0; j < KQ; ++j) kreg[j] = j < q4n ? kcur4[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    for (int kk = kq, pass = 0; kk < ((nk + 127) & ~127); kk += DS_CONSUMERS / 4, ++pass) {
        const int key = k0 + kk;
        if (pass > 0 && kk < nk) {
            const float4 *krow = key == pos ? reinterpret_cast<const float4 *>(kcur + sub * (d / 4))
                                            : reinterpret_cast<const float4 *>(kbase + (size_t)key * kv_stride + sub * (d / 4));
#pragma unroll
            for (int j = 0; j < KQ; ++j) kreg[j] = j < q4n ? krow[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        for (int hh = 0; hh < grp; ++hh) {
            const float4 *q4 = reinterpret_cast<const float4 *>(qs + hh * d + sub * (d / 4));
            float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
            for (int j = 0; j < KQ; ++j) {
                if (j < q4n) {
                    const float4 qv = q4[j];
                    d0 = fmaf(qv.x, kreg[j].x, d0);
                    d1 = fmaf(qv.y, kreg[j].y, d1);
                    d2 = fmaf(qv.z, kreg[j].z, d2);
                    d3 = fmaf(qv.w, kreg[j].w, d3);
                }
            }
            float dot = (d0 + d1) + (d2 + d3);
            // every lane takes part in the shuffles (the loop bound is a multiple of 128 keys)
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (kk < nk && sub == 0) scores[hh * cap + kk] = dot * scale;
        }
    }
    cons_sync();

    // ---- softmax per head: 16 / grp warps per head ----
    const int wph = DS_CONSUMER_WARPS / grp, hh_w = warp / wph, wi = warp - hh_w * wph;
    float *sc = scores + hh_w * cap;
    float mx = -INFINITY;
    for (int kk = wi * 32 + lane; kk < nk; kk += wph * 32) mx = fmaxf(mx, sc[kk]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) wred[warp] = mx;
    cons_sync();
    mx = -INFINITY;
    for (int i = 0; i < wph; ++i) mx = fmaxf(mx, wred[hh_w * wph + i]);
    cons_sync();
    float se = 0.0f;
    for (int kk = wi * 32 + lane; kk < nk; kk += wph * 32) {
        const float e = expf(sc[kk] - mx);
        sc[kk] = e;
        se += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    if (lane == 0) wred[warp] = se;
    cons_sync();  // (also publishes the exponentials)
    if (wi == 0 && lane == 0) {
        float t = 0.0f;
        for (int i = 0; i < wph; ++i) t += wred[hh_w * wph + i];
        float *po = attn_o + ((size_t)(h0 + hh_w) * S + split) * (d + 2);
        po[d] = mx;
        po[d + 1] = t;
    }

    // ---- weighted values: thread (part, head, float4 column); the group's heads re-read the
    // same value rows, which the L1 serves ----
    const int c4 = tid % vecs, hv = (tid / vecs) % grp, part = tid / (vecs * grp);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (part < parts) {
        const float *w = scores + hv * cap;
        const float4 vcur4 = *(reinterpret_cast<const float4 *>(vcur) + c4);
        for (int kb = part; kb < nk; kb += 8 * parts) {
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int kk = kb + j * parts;
                v[j] = (kk < nk && k0 + kk != pos)
                           ? __ldg(reinterpret_cast<const float4 *>(vbase + (size_t)(k0 + kk) * kv_stride) + c4)
                           : vcur4;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int kk = kb + j * parts;
                const float ww = kk < nk ? w[kk] : 0.0f;
                acc.x = fmaf(ww, v[j].x, acc.x);
                acc.y = fmaf(ww, v[j].y, acc.y);
                acc.z = fmaf(ww, v[j].z, acc.z);
                acc.w = fmaf(ww, v[j].w, acc.w);
            }
        }
        *(reinterpret_cast<float4 *>(partial + ((size_t)part * grp + hv) * d) + c4) = acc;
    }
    cons_sync();
    for (int i = tid; i < grp * d; i += DS_CONSUMERS) {
        const int hh = i / d, dd = i - hh * d;
        float v = 0.0f;
        for (int pt = 0; pt < parts; ++pt) v += partial[((size_t)pt * grp + hh) * d + dd];
        attn_o[((size_t)(h0 + hh) * S + split) * (d + 2) + dd] = v;
    }
    cons_sync();  // scratch is reused
}

// Grouped attention, phase 2: CTA h merges the g_splits (<= 32) partial results of query head h
// (the usual max-rescaling of a split softmax) into attn_out[h][d_head]. The 512 threads form
// 512 / d_head groups that take the splits round-robin, every load of a thread in flight at once.
__device__ __forceinline__ void attention_merge(const StepParams &p, int h, float *scratch, float *misc) {
    const int tid = threadIdx.x, d = p.d_head, S = p.g_splits;
    const int G = DS_CONSUMERS / d, g = tid / d, dd = tid - g * d;   // d divides 512
    const float *pp = p.attn + (size_t)h * S * (d + 2);
    float m[8], e[8], a[8];   // ceil(32 / G) <= 8 for d_head <= 128
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int sp = g + j * G;
        const bool on = sp < S;
        m[j] = on ? __ldcg(pp + (size_t)sp * (d + 2) + d) : -INFINITY;
        e[j] = on ? __ldcg(pp + (size_t)sp * (d + 2) + d + 1) : 0.0f;
        a[j] = on ? __ldcg(pp + (size_t)sp * (d + 2) + dd) : 0.0f;
    }
    float M = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) M = fmaxf(M, m[j]);
    M = cons_max(M, misc);
    float L = 0.0f, v = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float w = m[j] > -INFINITY ? expf(m[j] - M) : 0.0f;
        L = fmaf(w, e[j], L);
        v = fmaf(w, a[j], v);
    }
    // scratch: [G][d] partial sums, then [G] partial exp-sums
    scratch[g * d + dd] = v;
    if (dd == 0) scratch[G * d + g] = L;
    cons_sync();
    if (tid < d) {
        float vs = 0.0f, Ls = 0.0f;
        for (int i = 0; i < G; ++i) {
            vs += scratch[i * d + tid];
            Ls += scratch[G * d + i];
        }
        p.attn_out[(size_t)h * d + tid] = Ls > 0.0f ? vs / Ls : 0.0f;
    }
    cons_sync();  // scratch is reused
}

// Attention of the one query of head h over positions 0 .. pos, the keys dealt in contiguous
// chunks to p.splits CTAs per head: RoPE of the head's q and of its KV head's new k, cache
// append (one CTA per KV head), then this CTA's chunk of scores, a local softmax and the
// unnormalised weighted V sum. It leaves {acc[d], max, exp-sum}; the output projection
// merges the splits while it stages its activations. The phase is a chain of short steps
// that each wait on global memory, so every load that does not depend on an earlier step
// (the head's q/k/v, up to 128 cached key rows, the value rows) is issued before anything
// else; rows past the current position are fetched speculatively (the cache holds max_seq
// rows) and never used.
template <int VB>   // value rows whose loads are in flight together past the prefetched ones
__device__ __forceinline__ void attention_head(const StepParams &p, int layer, int h, int split, int pos,
                                               float *kc, float *vc, const float *rope_cs,
                                               float *scratch, float *misc, const float *qkv_base = nullptr,
                                               float *attn_base = nullptr) {
    // (batch form: the sequence's own q|k|v row, partial-result block and cache slices)
    const float *const qkv_in = qkv_base ? qkv_base : p.qkv;
    float *const attn_o = attn_base ? attn_base : p.attn;
    const int tid = threadIdx.x;
    const int d = p.d_head, half = d / 2;
    const int grp = p.n_q / p.n_kv, kvh = h / grp;
    float *qs = scratch, *kcur = qs + d, *vcur = kcur + d, *partial = vcur + d;  // partial: [512/(d/4)][d]
    float *scores = partial + 4 * DS_CONSUMERS;                                  // [max_seq]
    const size_t kv_stride = (size_t)p.n_kv * d;
    const float *kbase = kc + (size_t)kvh * d, *vbase = vc + (size_t)kvh * d;
    const int limit = pos + 1;
    const int chunk = (limit + p.splits - 1) / p.splits;
    const int k0 = split * chunk, k1 = min(limit, k0 + chunk);   // this CTA's keys
    float *po = attn_o + ((size_t)h * p.splits + split) * (d + 2);
    if (k0 >= k1) {  // nothing for this split yet: the neutral element of the merge
        for (int i = tid; i < d; i += DS_CONSUMERS) po[i] = 0.0f;
        if (tid == 0) { po[d] = -INFINITY; po[d + 1] = 0.0f; }
        return;
    }
    const bool has_new = (pos >= k0 && pos < k1);          // the split that sees the new position
    const bool owner = has_new && (h % grp) == 0;          // ... of the first head of the group appends

    // ---- loads ----
    constexpr int KQ = 8;   // float4 per thread of a key row: d/16 <= 8
    constexpr int NV = 4;   // value rows prefetched per thread
    const int kq = tid >> 2, sub = tid & 3, q4n = d / 16;       // 4 threads per key row
    const int vec = d / 4, nparts = DS_CONSUMERS / vec, part = tid / vec, c4 = tid % vec;
    float4 kreg[KQ], vreg[NV];
#pragma unroll
    for (int j = 0; j < KQ; ++j)
        kreg[j] = (j < q4n && k0 + kq < p.max_seq)
                      ? __ldg(reinterpret_cast<const float4 *>(kbase + (size_t)(k0 + kq) * kv_stride + sub * (d / 4)) + j)
                      : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int key = k0 + part + j * nparts;
        vreg[j] = key < p.max_seq ? __ldg(reinterpret_cast<const float4 *>(vbase + (size_t)key * kv_stride) + c4)
                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float x0 = 0.0f, x1 = 0.0f;
    const bool is_k = tid >= half;
    const int ri = is_k ? tid - half : tid;
    if (tid < d) {
        const float *src = qkv_in + (size_t)(is_k ? p.n_q + kvh : h) * d;
        x0 = __ldcg(src + ri);
        x1 = __ldcg(src + ri + half);
    } else if (tid < 2 * d) {
        x0 = __ldcg(qkv_in + (size_t)(p.n_q + p.n_kv + kvh) * d + (tid - d));
    }

    // ---- RoPE, append ----
    if (tid < d) {
        const float cs = rope_cs[2 * ri], sn = rope_cs[2 * ri + 1];  // the same for every layer
        const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
        float *dst = is_k ? kcur : qs;
        dst[ri] = y0;
        dst[ri + half] = y1;
        if (is_k && owner) {
            float *cd = kc + ((size_t)pos * p.n_kv + kvh) * d;
            cd[ri] = y0;
            cd[ri + half] = y1;
        }
    } else if (tid < 2 * d) {
        vcur[tid - d] = x0;
        if (owner) vc[((size_t)pos * p.n_kv + kvh) * d + (tid - d)] = x0;
    }
    cons_sync();

    // ---- scores: four threads per key, a quarter of the row each ----
    const float scale = 1.0f / sqrtf((float)d);
    const int nk = k1 - k0;
    const float4 *q4 = reinterpret_cast<const float4 *>(qs + sub * (d / 4));
    float mx = -INFINITY;
    auto quarter_dot = [&](const float4 (&kv)[KQ]) {
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int j = 0; j < KQ; ++j) {
            if (j < q4n) {
                const float4 qv = q4[j];
                d0 = fmaf(qv.x, kv[j].x, d0);
                d1 = fmaf(qv.y, kv[j].y, d1);
                d2 = fmaf(qv.z, kv[j].z, d2);
                d3 = fmaf(qv.w, kv[j].w, d3);
            }
        }
        return (d0 + d1) + (d2 + d3);
    };
    // the new position's key comes from shared memory: patch it into the prefetched registers
    // or load it in its pass
    if (k0 + kq == pos) {
        const float4 *kcur4 = reinterpret_cast<const float4 *>(kcur + sub * (d / 4));
#pragma unroll
        for (int j = 0; j < KQ; ++j) kreg[j] = j < q4n ? kcur4[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    for (int kk = kq, pass = 0; kk < ((nk + 127) & ~127); kk += DS_CONSUMERS / 4, ++pass) {
        const int key = k0 + kk;
        float dot = 0.0f;
        if (kk < nk) {
            if (pass == 0) {
                dot = quarter_dot(kreg);
            } else {
                // all of the row quarter's loads first, then the arithmetic
                const float4 *krow = key == pos ? reinterpret_cast<const float4 *>(kcur + sub * (d / 4))
                                                : reinterpret_cast<const float4 *>(kbase + (size_t)key * kv_stride + sub * (d / 4));
                float4 kv[KQ];
#pragma unroll
                for (int j = 0; j < KQ; ++j) kv[j] = j < q4n ? krow[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                dot = quarter_dot(kv);
            }
        }
        // every lane takes part in the shuffles (the loop bound is a multiple of 128 keys)
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        if (kk < nk) {
            const float sc = dot * scale;
            if (sub == 0) scores[kk] = sc;
            mx = fmaxf(mx, sc);
        }
    }
    mx = cons_max(mx, misc);
    float se = 0.0f;
    for (int kk = tid; kk < nk; kk += DS_CONSUMERS) {
        const float e = expf(scores[kk] - mx);
        scores[kk] = e;
        se += e;
    }
    se = cons_sum(se, misc);  // (its barriers also publish `scores`)

    // ---- weighted V: d/4 threads per key row, the keys dealt round-robin to 512/(d/4) parts ----
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float4 vcur4 = *(reinterpret_cast<const float4 *>(vcur) + c4);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int kk = part + j * nparts;
        if (kk < nk) {
            const float4 v = k0 + kk == pos ? vcur4 : vreg[j];
            const float w = scores[kk];
            acc.x = fmaf(w, v.x, acc.x);
            acc.y = fmaf(w, v.y, acc.y);
            acc.z = fmaf(w, v.z, acc.z);
            acc.w = fmaf(w, v.w, acc.w);
        }
    }
    // the rest of the part's keys, VB rows' loads in flight at a time
    for (int kb = part + NV * nparts; kb < nk; kb += VB * nparts) {
        float4 v[VB];
#pragma unroll
        for (int j = 0; j < VB; ++j) {
            const int kk = kb + j * nparts;
            v[j] = (kk < nk && k0 + kk != pos)
                       ? __ldg(reinterpret_cast<const float4 *>(vbase + (size_t)(k0 + kk) * kv_stride) + c4)
                       : vcur4;
        }
#pragma unroll
        for (int j = 0; j < VB; ++j) {
            const int kk = kb + j * nparts;
            const float w = kk < nk ? scores[kk] : 0.0f;
            acc.x = fmaf(w, v[j].x, acc.x);
            acc.y = fmaf(w, v[j].y, acc.y);
            acc.z = fmaf(w, v[j].z, acc.z);
            acc.w = fmaf(w, v[j].w, acc.w);
        }
    }
    *(reinterpret_cast<float4 *>(partial + (size_t)part * d) + c4) = acc;
    cons_sync();
    if (tid < d) {
        float v = 0.0f;
        for (int pt = 0; pt < nparts; ++pt) v += partial[pt * d + tid];
        po[tid] = v;
    }
    if (tid == 0) { po[d] = mx; po[d + 1] = se; }
    cons_sync();  // scratch is reused
}

// ---- int8 KV cache (KvDtype::I8 of the reference, crates/yscv-onnx/src/runner/kv_cache.rs:44-90) ----
//
// A cached row is one token's n_kv * d_head keys (or values) of one layer as int8 with ONE f32
// scale: scale = abs_max / 127 (1.0 when abs_max <= f32::EPSILON), q = clamp(round_half_away(v *
// (1 / scale)), -127, 127), read back as (float)q * scale: the arithmetic of
// rope_kv_append_kernel<int8_t>. The scale spans every KV head, so a CTA that needs the new
// position's key or value rotates / fetches the whole row, whichever head it works on.

__device__ __forceinline__ float4 s8x4_to_f4(uint32_t w) {
    return make_float4((float)(int8_t)(w & 255u), (float)(int8_t)((w >> 8) & 255u),
                       (float)(int8_t)((w >> 16) & 255u), (float)(int8_t)(w >> 24));
}

// Quantises `tmp[0 .. W)` (shared memory) as one cache row. Leaves the dequantised values of KV
// head kvh in cur[d]; write == true also stores the row at position pos and its scale.
__device__ __forceinline__ void quantise_row_i8(const StepParams &p, const float *tmp, float amax, int kvh, int pos,
                                                int8_t *cache, float *scales, float *cur, bool write, float *misc) {
    const int tid = threadIdx.x, d = p.d_head, W = p.n_kv * d;
    amax = cons_max(amax, misc);   // (its barriers also publish tmp)
    const float scale = (amax <= 1.1920929e-07f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    for (int i = tid; i < W; i += DS_CONSUMERS) {
        const float x = __fmul_rn(tmp[i], inv);
        // NaN -> 0, as Rust's saturating float-to-int cast does
        const int q = (x != x) ? 0 : (int)fminf(fmaxf(roundf(x), -127.0f), 127.0f);
        if (write) cache[(size_t)pos * W + i] = (int8_t)q;
        if (i / d == kvh) cur[i - kvh * d] = (float)q * scale;
    }
    if (write && tid == 0) scales[pos] = scale;
    cons_sync();   // tmp is reused, cur is complete
}

// The new position's key and value rows: RoPE of every KV head's key, both rows quantised;
// kcur / vcur receive what a reader of the cache would see for KV head kvh.
__device__ __forceinline__ void append_rows_i8(const StepParams &p, int kvh, int pos, int8_t *kc8, float *ksc,
                                               int8_t *vc8, float *vsc, const float *rope_cs, float *tmp,
                                               float *misc, float *kcur, float *vcur, bool write) {
    const int tid = threadIdx.x, d = p.d_head, half = d / 2, W = p.n_kv * d;
    float amax = 0.0f;
    for (int i = tid; i < p.n_kv * half; i += DS_CONSUMERS) {
        const int hh = i / half, ri = i - hh * half;
        const float *src = p.qkv + (size_t)(p.n_q + hh) * d;
        const float x0 = __ldcg(src + ri), x1 = __ldcg(src + ri + half);
        const float cs = rope_cs[2 * ri], sn = rope_cs[2 * ri + 1];
        const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
        tmp[hh * d + ri] = y0;
        tmp[hh * d + ri + half] = y1;
        amax = fmaxf(amax, fmaxf(fabsf(y0), fabsf(y1)));
    }
    quantise_row_i8(p, tmp, amax, kvh, pos, kc8, ksc, kcur, write, misc);
    amax = 0.0f;
    for (int i = tid; i < W; i += DS_CONSUMERS) {
        const float v = __ldcg(p.qkv + (size_t)(p.n_q + p.n_kv) * d + i);
        tmp[i] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    quantise_row_i8(p, tmp, amax, kvh, pos, vc8, vsc, vcur, write, misc);
}

// attention_head over an int8 cache. d_head is 64 or 128 (a quarter row is 16 or 32 bytes).
template <int VB>
__device__ __forceinline__ void attention_head_i8(const StepParams &p, int h, int split, int pos, int8_t *kc8,
                                                  float *ksc, int8_t *vc8, float *vsc, const float *rope_cs,
                                                  float *scratch, float *misc) {
    const int tid = threadIdx.x;
    const int d = p.d_head, half = d / 2;
    const int grp = p.n_q / p.n_kv, kvh = h / grp;
    float *qs = scratch, *kcur = qs + d, *vcur = kcur + d, *partial = vcur + d;  // partial: [512/(d/4)][d]
    float *scores = partial + 4 * DS_CONSUMERS;                                  // [max_seq]
    const size_t kv_stride = (size_t)p.n_kv * d;   // bytes per cached row
    const int8_t *kbase = kc8 + (size_t)kvh * d, *vbase = vc8 + (size_t)kvh * d;
    const int limit = pos + 1;
    const int chunk = (limit + p.splits - 1) / p.splits;
    const int k0 = split * chunk, k1 = min(limit, k0 + chunk);
    float *po = p.attn + ((size_t)h * p.splits + split) * (d + 2);
    if (k0 >= k1) {
        for (int i = tid; i < d; i += DS_CONSUMERS) po[i] = 0.0f;
        if (tid == 0) { po[d] = -INFINITY; po[d + 1] = 0.0f; }
        return;
    }
    const bool has_new = (pos >= k0 && pos < k1);
    const int nk = k1 - k0;
    const int kq = tid >> 2, sub = tid & 3, n16 = d / 64;   // 4 threads per key row, 16-byte pieces per quarter
    const int vec = d / 4, nparts = DS_CONSUMERS / vec, part = tid / vec, c4 = tid % vec;
    // first pass of keys: loads in flight before anything else
    uint4 k8[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    float kscl = 0.0f;
    if (kq < nk && k0 + kq != pos) {
        const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)(k0 + kq) * kv_stride + sub * (d / 4));
        k8[0] = __ldg(kr);
        if (n16 > 1) k8[1] = __ldg(kr + 1);
        kscl = __ldg(ksc + k0 + kq);
    }
    // the head's query, rotated
    if (tid < half) {
        const float *src = p.qkv + (size_t)h * d;
        const float x0 = __ldcg(src + tid), x1 = __ldcg(src + tid + half);
        const float cs = rope_cs[2 * tid], sn = rope_cs[2 * tid + 1];
        qs[tid] = x0 * cs - x1 * sn;
        qs[tid + half] = x0 * sn + x1 * cs;
    }
    if (has_new)   // (the same for every thread of the CTA) the first head's CTA stores the rows
        append_rows_i8(p, kvh, pos, kc8, ksc, vc8, vsc, rope_cs, partial, misc, kcur, vcur, h == 0);
    else
        cons_sync();

    // ---- scores ----
    const float scale = 1.0f / sqrtf((float)d);
    const float4 *q4 = reinterpret_cast<const float4 *>(qs + sub * (d / 4));
    auto quarter_dot8 = [&](const uint4 (&kv)[2], float rs) {
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (j < n16) {
                const uint32_t w[4] = {kv[j].x, kv[j].y, kv[j].z, kv[j].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 kf = s8x4_to_f4(w[i]), qv = q4[j * 4 + i];
                    d0 = fmaf(qv.x, kf.x, d0);
                    d1 = fmaf(qv.y, kf.y, d1);
                    d2 = fmaf(qv.z, kf.z, d2);
                    d3 = fmaf(qv.w, kf.w, d3);
                }
            }
        }
        return ((d0 + d1) + (d2 + d3)) * rs;
    };
    float mx = -INFINITY;
    for (int kk = kq, pass = 0; kk < ((nk + 127) & ~127); kk += DS_CONSUMERS / 4, ++pass) {
        const int key = k0 + kk;
        float dot = 0.0f;
        if (kk < nk) {
            if (key == pos) {
                const float4 *kc4 = reinterpret_cast<const float4 *>(kcur + sub * (d / 4));
                float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
                for (int j = 0; j < d / 16; ++j) {
                    const float4 qv = q4[j], kf = kc4[j];
                    d0 = fmaf(qv.x, kf.x, d0);
                    d1 = fmaf(qv.y, kf.y, d1);
                    d2 = fmaf(qv.z, kf.z, d2);
                    d3 = fmaf(qv.w, kf.w, d3);
                }
                dot = (d0 + d1) + (d2 + d3);
            } else {
                if (pass > 0) {
                    const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)key * kv_stride + sub * (d / 4));
                    k8[0] = __ldg(kr);
                    if (n16 > 1) k8[1] = __ldg(kr + 1);
                    kscl = __ldg(ksc + key);
                }
                dot = quarter_dot8(k8, kscl);
            }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        if (kk < nk) {
            const float sc = dot * scale;
            if (sub == 0) scores[kk] = sc;
            mx = fmaxf(mx, sc);
        }
    }
    mx = cons_max(mx, misc);
    float se = 0.0f;
    for (int kk = tid; kk < nk; kk += DS_CONSUMERS) {
        const float e = expf(scores[kk] - mx);
        scores[kk] = e;
        se += e;
    }
    se = cons_sum(se, misc);  // (its barriers also publish `scores`)

    // ---- weighted V: d/4 threads per key row (4 bytes each), keys dealt round-robin to the parts ----
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    const float4 vcur4 = *(reinterpret_cast<const float4 *>(vcur) + c4);
    for (int kb = part; kb < nk; kb += VB * nparts) {
        uint32_t v[VB];
        float vs[VB];
#pragma unroll
        for (int j = 0; j < VB; ++j) {
            const int kk = kb + j * nparts;
            const bool on = kk < nk && k0 + kk != pos;
            v[j] = on ? __ldg(reinterpret_cast<const uint32_t *>(vbase + (size_t)(k0 + kk) * kv_stride) + c4) : 0u;
            vs[j] = on ? __ldg(vsc + k0 + kk) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < VB; ++j) {
            const int kk = kb + j * nparts;
            if (kk < nk) {
                const bool is_new = k0 + kk == pos;
                const float4 vf = is_new ? vcur4 : s8x4_to_f4(v[j]);
                const float w = scores[kk] * (is_new ? 1.0f : vs[j]);
                acc.x = fmaf(w, vf.x, acc.x);
                acc.y = fmaf(w, vf.y, acc.y);
                acc.z = fmaf(w, vf.z, acc.z);
                acc.w = fmaf(w, vf.w, acc.w);
            }
        }
    }
    *(reinterpret_cast<float4 *>(partial + (size_t)part * d) + c4) = acc;
    cons_sync();
    if (tid < d) {
        float v = 0.0f;
        for (int pt = 0; pt < nparts; ++pt) v += partial[pt * d + tid];
        po[tid] = v;
    }
    if (tid == 0) { po[d] = mx; po[d + 1] = se; }
    cons_sync();  // scratch is reused
}

// attention_group (phase 1 of the grouped form) over an int8 cache.
__device__ __forceinline__ void attention_group_i8(const StepParams &p, int kvh, int split, int pos, int8_t *kc8,
                                                   float *ksc, int8_t *vc8, float *vsc, const float *rope_cs,
                                                   float *scratch, float *misc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int d = p.d_head, half = d / 2;
    const int grp = p.n_q / p.n_kv, S = p.g_splits, cap = p.g_chunk_cap;
    const int vecs = d / 4, parts = DS_CONSUMERS / (grp * vecs);
    float *qs = scratch, *kcur = qs + grp * d, *vcur = kcur + d, *partial = vcur + d;
    float *wred = partial + parts * grp * d, *scores = wred + 32;
    const size_t kv_stride = (size_t)p.n_kv * d;
    const int8_t *kbase = kc8 + (size_t)kvh * d, *vbase = vc8 + (size_t)kvh * d;
    const int limit = pos + 1;
    const int chunk = (limit + S - 1) / S;
    const int k0 = split * chunk, k1 = min(limit, k0 + chunk);
    const int h0 = kvh * grp;
    if (k0 >= k1) {
        for (int i = tid; i < grp * (d + 2); i += DS_CONSUMERS) {
            const int hh = i / (d + 2), j = i - hh * (d + 2);
            p.attn[((size_t)(h0 + hh) * S + split) * (d + 2) + j] = j == d ? -INFINITY : 0.0f;
        }
        return;
    }
    const int nk = k1 - k0;
    const bool has_new = pos >= k0 && pos < k1;
    const int kq = tid >> 2, sub = tid & 3, n16 = d / 64;
    uint4 k8[2] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};
    float kscl = 0.0f;
    if (kq < nk && k0 + kq != pos) {
        const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)(k0 + kq) * kv_stride + sub * (d / 4));
        k8[0] = __ldg(kr);
        if (n16 > 1) k8[1] = __ldg(kr + 1);
        kscl = __ldg(ksc + k0 + kq);
    }
    // the group's queries, rotated
    for (int i = tid; i < grp * half; i += DS_CONSUMERS) {
        const int hh = i / half, ri = i - hh * half;
        const float *src = p.qkv + (size_t)(h0 + hh) * d;
        const float x0 = __ldcg(src + ri), x1 = __ldcg(src + ri + half);
        const float cs = rope_cs[2 * ri], sn = rope_cs[2 * ri + 1];
        qs[hh * d + ri] = x0 * cs - x1 * sn;
        qs[hh * d + ri + half] = x0 * sn + x1 * cs;
    }
    if (has_new)   // the first KV head's CTA stores the rows
        append_rows_i8(p, kvh, pos, kc8, ksc, vc8, vsc, rope_cs, partial, misc, kcur, vcur, kvh == 0);
    else
        cons_sync();

    // ---- scores: four threads per key; the quarter row in registers serves every query head ----
    const float scale = 1.0f / sqrtf((float)d);
    for (int kk = kq, pass = 0; kk < ((nk + 127) & ~127); kk += DS_CONSUMERS / 4, ++pass) {
        const int key = k0 + kk;
        const bool is_new = key == pos;
        float4 kf[8];   // the quarter row as floats (d/16 <= 8 float4)
        float rs = 1.0f;
        if (kk < nk) {
            if (is_new) {
                const float4 *kc4 = reinterpret_cast<const float4 *>(kcur + sub * (d / 4));
#pragma unroll
                for (int j = 0; j < 8; ++j) kf[j] = j < d / 16 ? kc4[j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            } else {
                if (pass > 0) {
                    const uint4 *kr = reinterpret_cast<const uint4 *>(kbase + (size_t)key * kv_stride + sub * (d / 4));
                    k8[0] = __ldg(kr);
                    if (n16 > 1) k8[1] = __ldg(kr + 1);
                    kscl = __ldg(ksc + key);
                }
                rs = kscl;
                const uint32_t w[8] = {k8[0].x, k8[0].y, k8[0].z, k8[0].w, k8[1].x, k8[1].y, k8[1].z, k8[1].w};
#pragma unroll
                for (int j = 0; j < 8; ++j) kf[j] = s8x4_to_f4(w[j]);   // (zeros past the quarter)
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) kf[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        for (int hh = 0; hh < grp; ++hh) {
            const float4 *q4 = reinterpret_cast<const float4 *>(qs + hh * d + sub * (d / 4));
            float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < d / 16) {
                    const float4 qv = q4[j];
                    d0 = fmaf(qv.x, kf[j].x, d0);
                    d1 = fmaf(qv.y, kf[j].y, d1);
                    d2 = fmaf(qv.z, kf[j].z, d2);
                    d3 = fmaf(qv.w, kf[j].w, d3);
                }
            }
            float dot = ((d0 + d1) + (d2 + d3)) * rs;
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (kk < nk && sub == 0) scores[hh * cap + kk] = dot * scale;
        }
    }
    cons_sync();

    // ---- softmax per head: 16 / grp warps per head ----
    const int wph = DS_CONSUMER_WARPS / grp, hh_w = warp / wph, wi = warp - hh_w * wph;
    float *sc = scores + hh_w * cap;
    float mx = -INFINITY;
    for (int kk = wi * 32 + lane; kk < nk; kk += wph * 32) mx = fmaxf(mx, sc[kk]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) wred[warp] = mx;
    cons_sync();
    mx = -INFINITY;
    for (int i = 0; i < wph; ++i) mx = fmaxf(mx, wred[hh_w * wph + i]);
    cons_sync();
    float se = 0.0f;
    for (int kk = wi * 32 + lane; kk < nk; kk += wph * 32) {
        const float e = expf(sc[kk] - mx);
        sc[kk] = e;
        se += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    if (lane == 0) wred[warp] = se;
    cons_sync();
    if (wi == 0 && lane == 0) {
        float t = 0.0f;
        for (int i = 0; i < wph; ++i) t += wred[hh_w * wph + i];
        float *po = p.attn + ((size_t)(h0 + hh_w) * S + split) * (d + 2);
        po[d] = mx;
        po[d + 1] = t;
    }

    // ---- weighted values: thread (part, head, 4 columns) ----
    const int c4 = tid % vecs, hv = (tid / vecs) % grp, part = tid / (vecs * grp);
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (part < parts) {
        const float *w = scores + hv * cap;
        const float4 vcur4 = *(reinterpret_cast<const float4 *>(vcur) + c4);
        for (int kb = part; kb < nk; kb += 8 * parts) {
            uint32_t v[8];
            float vs[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int kk = kb + j * parts;
                const bool on = kk < nk && k0 + kk != pos;
                v[j] = on ? __ldg(reinterpret_cast<const uint32_t *>(vbase + (size_t)(k0 + kk) * kv_stride) + c4) : 0u;
                vs[j] = on ? __ldg(vsc + k0 + kk) : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int kk = kb + j * parts;
                if (kk < nk) {
                    const bool is_new = k0 + kk == pos;
                    const float4 vf = is_new ? vcur4 : s8x4_to_f4(v[j]);
                    const float ww = w[kk] * (is_new ? 1.0f : vs[j]);
                    acc.x = fmaf(ww, vf.x, acc.x);
                    acc.y = fmaf(ww, vf.y, acc.y);
                    acc.z = fmaf(ww, vf.z, acc.z);
                    acc.w = fmaf(ww, vf.w, acc.w);
                }
            }
        }
        *(reinterpret_cast<float4 *>(partial + ((size_t)part * grp + hv) * d) + c4) = acc;
    }
    cons_sync();
    for (int i = tid; i < grp * d; i += DS_CONSUMERS) {
        const int hh = i / d, dd = i - hh * d;
        float v = 0.0f;
        for (int pt = 0; pt < parts; ++pt) v += partial[((size_t)pt * grp + hh) * d + dd];
        p.attn[((size_t)(h0 + hh) * S + split) * (d + 2) + dd] = v;
    }
    cons_sync();  // scratch is reused
}

// SIMPLE: every matrix is one row block and one K chunk per CTA and attention runs per query
// head (small models, short contexts); the loops over blocks and chunks then fold away at
// compile time, which is worth 7 % of a TinyLlama step.
template <bool SIMPLE>
__global__ void __launch_bounds__(DS_THREADS, 1) decode_step_kernel(const StepParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ring_bytes = (uint32_t)p.stages * p.slot_bytes;
    float *red = reinterpret_cast<float *>(smem + ring_bytes);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_base + ring_bytes + DS_RED_BYTES;
    const uint32_t bar_empty = bar_full + 8 * DS_MAX_STAGES;
    unsigned char *dig = smem + ring_bytes + DS_RED_BYTES + DS_BAR_BYTES;
    float *act_s = reinterpret_cast<float *>(dig + p.dig_bytes);
    float *misc = act_s + p.act_floats;  // 32 floats
    float *rope_cs = misc + 32;          // [d_head/2] x {cos, sin} of this step's position
    float **cache_ptr = reinterpret_cast<float **>(rope_cs + p.d_head);  // [layers] x {k, v}
    float *wtab = reinterpret_cast<float *>(cache_ptr + 2 * p.layers);   // [n_q][4 or 16] split-merge weights
    const int nmat = p.layers * 4;

    // A position outside the cache: nothing is appended, nothing is computed, the status word
    // says so (every thread of every CTA takes the same way out, before any barrier).
    {
        const int pos_in = *p.pos;
        if (pos_in < 0 || pos_in >= p.max_seq) {
            if (blockIdx.x == 0 && tid == 0) *p.status = YSCV_DEV_POS_OVERFLOW;
            return;
        }
    }

    if (tid == DS_CONSUMERS) {
        for (int i = 0; i < p.stages; ++i) {
            mbar_init(bar_full + i * 8, 1);
            mbar_init(bar_empty + i * 8, DS_CONSUMER_WARPS);
        }
        mbar_fence_init();
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    __syncthreads();

    // ---------------- producer: the weight stream of every layer, in order ----------------
    if (warp == DS_CONSUMER_WARPS) {
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            bool alive = true;
            for (int mi = 0; mi < nmat && alive; ++mi) {
                const StepMat *m = p.mats + mi;
                const int j = mi & 3;
                const bool paired = j == 2 && p.pair_gu;
                const int n = paired ? p.inter : p.mat_n[j];
                const int tiles = p.mat_tiles[j], k_stages = p.mat_ks[j], n_rb = p.mat_nrb[j];
                const int r0 = (int)(((unsigned)n * blockIdx.x) / gridDim.x);
                const int rb_rows = tiles * 16;
                const int block_rows = (paired ? tiles / 2 : tiles) * 16;
                const int kps = p.mat_kps[j];
                const uint32_t sub_bytes = (uint32_t)rb_rows * (DS_GS * 16 + DS_GS * 4);
                // the consumers' order: K chunk, row block, K stage
                for (int cs = 0; cs < k_stages && alive; cs += p.kc_stages) {
                    const int ce = min(k_stages, cs + p.kc_stages);
                    for (int rb = 0; rb < n_rb && alive; ++rb) {
                        const int row0 = r0 + rb * block_rows;
                        for (int ks0 = cs; ks0 < ce && alive; ks0 += kps) {
                            // a fresh barrier passes the wait on the opposite parity at once
                            alive = mbar_wait(bar_empty + slot * 8, phase ^ 1u, p.status);
                            if (!alive) break;
                            const int nsub = min(kps, ce - ks0);
                            const uint32_t full = bar_full + slot * 8;
                            mbar_expect_tx(full, (uint32_t)nsub * sub_bytes);
                            for (int q = 0; q < nsub; ++q) {
                                const uint32_t st = smem_base + (uint32_t)slot * p.slot_bytes + (uint32_t)q * sub_bytes;
                                const int ks = ks0 + q;
                                if (paired) {
                                    // two boxes of half the block each: gate rows, then the matching up rows
                                    for (int h = 0; h < 2; ++h) {
                                        const int row = h * p.inter + row0;
                                        tma_load_2d(st + h * block_rows * 128, &m->tm_w, ks * (DS_GS * 16), row, full);
                                        tma_load_2d(st + rb_rows * 128 + h * block_rows * 128, &m->tm_w,
                                                    ks * (DS_GS * 16) + 128, row, full);
                                        tma_load_2d(st + rb_rows * 256 + h * block_rows * (DS_GS * 4), &m->tm_s,
                                                    ks * DS_GS, row, full);
                                    }
                                } else {
                                    tma_load_2d(st, &m->tm_w, ks * (DS_GS * 16), row0, full);
                                    tma_load_2d(st + rb_rows * 128, &m->tm_w, ks * (DS_GS * 16) + 128, row0, full);
                                    tma_load_2d(st + rb_rows * 256, &m->tm_s, ks * DS_GS, row0, full);
                                }
                            }
                            if (++slot == p.stages) { slot = 0; phase ^= 1u; }
                        }
                    }
                }
            }
            // a consumer that gave up leaves copies unobserved: wait (bounded) for every slot
            if (!alive)
                for (int i = 0; i < p.stages; ++i) mbar_wait(bar_full + i * 8, 0, nullptr);
        }
        return;
    }

    // ---------------- consumers ----------------
    unsigned int epoch = 0;
    RingPos c = {0, 0u};
    bool dead = false;
    const int H = p.hidden, I = p.inter;
    // exchanges of this launch are tagged tp_tag_base + 1 ... + 2 * layers (the row-parallel
    // GEMVs) and + 2 * layers + 1 (the greedy token)
    const unsigned int tp_seq = p.tp_size > 1 ? *p.tp_seq : 0u;
    const unsigned int tp_tag_base = tp_seq * (unsigned int)(2 * p.layers + 1);
    int tp_ar = 0;

    // One matrix: for every K chunk, `stage_chunk(k0, klen)` leaves the activations of that
    // chunk in act_s and their digit planes in `dig`; then every row block of the CTA walks the
    // chunk's stages. (More than one chunk only with a single row block: the accumulators then
    // live across the chunks.)
    auto gemv = [&](int mi, float *out, int store, auto &&stage_chunk) {
        const int j = mi & 3;
        const int tiles = p.mat_tiles[j], k_stages = p.mat_ks[j], kps = p.mat_kps[j];
        const int n_rb = SIMPLE ? 1 : p.mat_nrb[j];
        const int kc = SIMPLE ? k_stages : p.kc_stages;
        // rows of the matrix, or (paired gate/up) intermediate indices
        const unsigned n = (j == 2 && p.pair_gu) ? (unsigned)p.inter : (unsigned)p.mat_n[j];
        const int r0 = (int)((n * blockIdx.x) / gridDim.x);
        const int r1 = (int)((n * (blockIdx.x + 1)) / gridDim.x);
        const int block_rows = (store == 2 ? tiles / 2 : tiles) * 16;
        // row-parallel GEMV under tensor parallelism: the tag of this exchange (never 0, the
        // value of untouched slots) and its slot parity (two exchanges per layer: consecutive
        // ones alternate, also across launches)
        const unsigned int tp_tag = tp_tag_base + (unsigned int)tp_ar + 1u;
        float acc[2] = {0.0f, 0.0f};
        for (int cs = 0; cs < k_stages; cs += kc) {
            const int ce = min(k_stages, cs + kc);
            stage_chunk(cs * (DS_GS * 32), (ce - cs) * (DS_GS * 32));
            for (int rb = 0; rb < n_rb; ++rb) {
                const int row_base = r0 + rb * block_rows;
                const bool last = ce == k_stages;
                // the thread that will store a row fetches its residual value before the K loop
                float resid = 0.0f;
                if (store == 1 && last && tid < tiles * 16) {
                    const int my_row = row_base + (tid >> 4) * 16 + (tid & 7) + ((tid >> 3) & 1) * 8;
                    if (my_row < r1) resid = __ldcg(out + my_row);
                }
                if (n_rb > 1) { acc[0] = 0.0f; acc[1] = 0.0f; }
                if (tiles == 1 && p.one_tile_16) {
                    consume_stages<1>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) finish_rows<1>(p, red, tiles, row_base, r1, out, store, acc, resid, tp_tag, tp_ar & 1);
                } else if (tiles <= 2) {
                    consume_stages<2>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) finish_rows<2>(p, red, tiles, row_base, r1, out, store, acc, resid, tp_tag, tp_ar & 1);
                } else if (!SIMPLE && tiles <= 4) {   // (small models have no 3- or 4-tile slab)
                    consume_stages<4>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) finish_rows<4>(p, red, tiles, row_base, r1, out, store, acc, resid, tp_tag, tp_ar & 1);
                } else {
                    consume_stages<8>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) finish_rows<8>(p, red, tiles, row_base, r1, out, store, acc, resid, tp_tag, tp_ar & 1);
                }
            }
        }
        if (store == 1) ++tp_ar;
    };
    // act_s = RMSNorm(x) * gamma
    auto stage_norm = [&](const float *gamma) {
        // hidden <= 8192: a thread's (up to 16) elements and gammas stay in registers across the
        // reduction
        constexpr int NE = SIMPLE ? 8 : 16;
        float xv[NE], gv[NE];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < NE; ++j) {
            const int i = tid + j * DS_CONSUMERS;
            xv[j] = i < H ? __ldcg(p.x + i) : 0.0f;
            gv[j] = i < H ? __ldg(gamma + i) : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < NE; ++j) ss = fmaf(xv[j], xv[j], ss);
        for (int i = tid + NE * DS_CONSUMERS; i < H; i += DS_CONSUMERS) {
            const float v = __ldcg(p.x + i);
            ss = fmaf(v, v, ss);
        }
        const float total = cons_sum(ss, misc);
        const float inv = 1.0f / sqrtf(total / (float)H + p.eps);
#pragma unroll
        for (int j = 0; j < NE; ++j) {
            const int i = tid + j * DS_CONSUMERS;
            if (i < H) act_s[i] = (xv[j] * inv) * gv[j];
        }
        for (int i = tid + NE * DS_CONSUMERS; i < H; i += DS_CONSUMERS) act_s[i] = (__ldcg(p.x + i) * inv) * gamma[i];
        cons_sync();
    };

    // per-launch constants: the position, its rotary factors, the cache pointers; the padding
    // row of the digit planes
    const int pos = *p.pos;   // inside [0, max_seq): checked at the top
    if (tid < p.d_head / 2) {
        const float inv_freq = 1.0f / powf(p.theta, 2.0f * (float)tid / (float)p.d_head);
        sincosf(inv_freq * (float)pos, &rope_cs[2 * tid + 1], &rope_cs[2 * tid]);
    }
    for (int i = tid; i < 2 * p.layers; i += DS_CONSUMERS)
        cache_ptr[i] = (i & 1) ? p.vcache[i >> 1] : p.kcache[i >> 1];
    {
        const QuantLayout q = quant_layout(1, DS_GS);
        const int groups = p.dig_bytes / (4 * 4 * 16);
        for (int item = tid >> 2; item < groups; item += DS_CONSUMERS / 4)
            quantize_group<true>(nullptr, dig, q, item, 1, tid & 3, true);
    }
    // x = embedding[token]
    {
        int tok = *p.token;
        tok = tok < 0 ? 0 : (tok >= p.vocab ? p.vocab - 1 : tok);
        const int i0 = (int)(((unsigned)H * blockIdx.x) / gridDim.x);
        const int i1 = (int)(((unsigned)H * (blockIdx.x + 1)) / gridDim.x);
        for (int i = i0 + tid; i < i1; i += DS_CONSUMERS) p.x[i] = p.embedding[(size_t)tok * H + i];
    }
    grid_barrier(p, epoch);

    // activation staging of the three kinds of GEMV input (each ends with the digit planes)
    auto stage_normed = [&](const float *gamma) {
        stage_norm(gamma);
        quantize_activation(act_s, dig, H, false);
    };
    // merge of the attention splits (the usual max-rescaling of a split softmax)
    auto stage_attention = [&]() {
        const int AW = p.n_q * p.d_head;
        if (!SIMPLE && p.attn_grouped) {
#pragma unroll 4
            for (int i = tid; i < AW; i += DS_CONSUMERS) act_s[i] = __ldcg(p.attn_out + i);
        } else if (p.splits > 4) {
            // many key chunks per head (few heads on this GPU, long context): per (head, chunk)
            // the weight exp(m - M) / L once, through the shared-memory table [n_q][16]
            if (tid < p.n_q) {
                const float *pp = p.attn + (size_t)tid * p.splits * (p.d_head + 2) + p.d_head;
                float M = -INFINITY;
                for (int sp = 0; sp < p.splits; ++sp) M = fmaxf(M, __ldcg(pp + (size_t)sp * (p.d_head + 2)));
                float L = 0.0f;
                for (int sp = 0; sp < p.splits; ++sp) {
                    const float m = __ldcg(pp + (size_t)sp * (p.d_head + 2));
                    const float w = m > -INFINITY ? expf(m - M) : 0.0f;
                    L = fmaf(w, __ldcg(pp + (size_t)sp * (p.d_head + 2) + 1), L);
                    wtab[tid * 16 + sp] = w;
                }
                const float invL = L > 0.0f ? 1.0f / L : 0.0f;
                for (int sp = 0; sp < p.splits; ++sp) wtab[tid * 16 + sp] *= invL;
            }
            cons_sync();
            for (int i = tid; i < AW; i += DS_CONSUMERS) {
                const int hh = i / p.d_head, dd = i - hh * p.d_head;
                const float *pp = p.attn + (size_t)hh * p.splits * (p.d_head + 2) + dd;
                const float *w = wtab + hh * 16;
                float acc = 0.0f;
#pragma unroll 4
                for (int sp = 0; sp < p.splits; ++sp) acc = fmaf(w[sp], __ldcg(pp + (size_t)sp * (p.d_head + 2)), acc);
                act_s[i] = acc;
            }
        } else if (p.merge_table) {
            // per (head, split): weight exp(m - M) / L once, through shared memory
            if (tid < p.n_q) {
                const float *pp = p.attn + (size_t)tid * p.splits * (p.d_head + 2) + p.d_head;
                float m[4], e[4];
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    const bool on = sp < p.splits;
                    m[sp] = on ? __ldcg(pp + (size_t)sp * (p.d_head + 2)) : -INFINITY;
                    e[sp] = on ? __ldcg(pp + (size_t)sp * (p.d_head + 2) + 1) : 0.0f;
                }
                float M = -INFINITY, L = 0.0f, w[4];
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) M = fmaxf(M, m[sp]);
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    w[sp] = m[sp] > -INFINITY ? expf(m[sp] - M) : 0.0f;
                    L = fmaf(w[sp], e[sp], L);
                }
                const float invL = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) wtab[tid * 4 + sp] = w[sp] * invL;
            }
            // 4 x 512 elements per pass, their partial sums in registers across the barrier
            for (int base = 0; base < AW; base += 4 * DS_CONSUMERS) {
                float a[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base + tid + j * DS_CONSUMERS;
                    const int hh = i / p.d_head, dd = i - hh * p.d_head;
                    const float *pp = p.attn + (size_t)hh * p.splits * (p.d_head + 2) + dd;
#pragma unroll
                    for (int sp = 0; sp < 4; ++sp)
                        a[j][sp] = (i < AW && sp < p.splits) ? __ldcg(pp + (size_t)sp * (p.d_head + 2)) : 0.0f;
                }
                if (base == 0) cons_sync();  // the weight table is complete
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base + tid + j * DS_CONSUMERS;
                    if (i < AW) {
                        const float *w = wtab + (i / p.d_head) * 4;
                        act_s[i] = fmaf(w[3], a[j][3], fmaf(w[2], a[j][2], fmaf(w[1], a[j][1], w[0] * a[j][0])));
                    }
                }
            }
        } else {
#pragma unroll 4
            for (int i = tid; i < AW; i += DS_CONSUMERS) {
                const int hh = i / p.d_head, dd = i - hh * p.d_head;
                const float *pp = p.attn + (size_t)hh * p.splits * (p.d_head + 2);
                float a[4], m[4], e[4];  // splits <= 4
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    const bool on = sp < p.splits;
                    a[sp] = on ? __ldcg(pp + (size_t)sp * (p.d_head + 2) + dd) : 0.0f;
                    m[sp] = on ? __ldcg(pp + (size_t)sp * (p.d_head + 2) + p.d_head) : -INFINITY;
                    e[sp] = on ? __ldcg(pp + (size_t)sp * (p.d_head + 2) + p.d_head + 1) : 0.0f;
                }
                float M = -INFINITY;
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) M = fmaxf(M, m[sp]);
                float L = 0.0f, v = 0.0f;
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    const float w = m[sp] > -INFINITY ? expf(m[sp] - M) : 0.0f;
                    L = fmaf(w, e[sp], L);
                    v = fmaf(w, a[sp], v);
                }
                act_s[i] = L > 0.0f ? v / L : 0.0f;
            }
        }
        cons_sync();
        quantize_activation(act_s, dig, AW, false);
    };
    // the MLP activations [k0, k0 + klen): already silu(gate) * up (paired), or formed here
    auto stage_mlp = [&](int k0, int klen) {
        if (k0 > 0) cons_sync();  // every warp is done with the previous chunk's act_s and planes
        if (p.pair_gu) {
#pragma unroll 4
            for (int i = tid; i < klen; i += DS_CONSUMERS) act_s[i] = __ldcg(p.gu + k0 + i);
        } else {
            for (int i0 = tid; i0 < klen; i0 += 12 * DS_CONSUMERS) {
                float g[12], u[12];
#pragma unroll
                for (int j = 0; j < 12; ++j) {  // up to 24 loads in flight per thread
                    const int i = i0 + j * DS_CONSUMERS;
                    g[j] = i < klen ? __ldcg(p.gu + k0 + i) : 0.0f;
                    u[j] = i < klen ? __ldcg(p.gu + I + k0 + i) : 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 12; ++j) {
                    const int i = i0 + j * DS_CONSUMERS;
                    const float sg = 1.0f / (1.0f + expf(-g[j]));
                    if (i < klen) act_s[i] = (g[j] * sg) * u[j];
                }
            }
        }
        cons_sync();
        quantize_activation(act_s, dig, klen, false);
    };

    for (int l = 0; l < p.layers; ++l) {
        const float *g1 = p.gamma + (size_t)(2 * l) * H, *g2 = g1 + H;
        // attention block: norm -> qkv
        gemv(4 * l + 0, p.qkv, 0, [&](int, int) { stage_normed(g1); });
        grid_barrier(p, epoch);
        // RoPE, cache append, attention: a few CTAs per query head, or (long contexts) one CTA
        // per KV head and key chunk followed by a merge phase
        if (!SIMPLE && p.attn_grouped) {
            if ((int)blockIdx.x < p.n_kv * p.g_splits) {
                if (p.kv_int8)
                    attention_group_i8(p, blockIdx.x / p.g_splits, blockIdx.x % p.g_splits, pos,
                                       reinterpret_cast<int8_t *>(cache_ptr[2 * l]), p.kcache[p.layers + l],
                                       reinterpret_cast<int8_t *>(cache_ptr[2 * l + 1]), p.vcache[p.layers + l],
                                       rope_cs, act_s, misc);
                else
                    attention_group(p, blockIdx.x / p.g_splits, blockIdx.x % p.g_splits, pos, cache_ptr[2 * l],
                                    cache_ptr[2 * l + 1], rope_cs, act_s);
            }
            grid_barrier(p, epoch);
            if ((int)blockIdx.x < p.n_q) attention_merge(p, blockIdx.x, act_s, misc);
        } else if ((int)blockIdx.x < p.n_q * p.splits) {
            if (p.kv_int8)
                attention_head_i8<SIMPLE ? 4 : 8>(p, blockIdx.x / p.splits, blockIdx.x % p.splits, pos,
                                                  reinterpret_cast<int8_t *>(cache_ptr[2 * l]), p.kcache[p.layers + l],
                                                  reinterpret_cast<int8_t *>(cache_ptr[2 * l + 1]), p.vcache[p.layers + l],
                                                  rope_cs, act_s, misc);
            else
                attention_head<SIMPLE ? 4 : 8>(p, l, blockIdx.x / p.splits, blockIdx.x % p.splits, pos, cache_ptr[2 * l],
                                               cache_ptr[2 * l + 1], rope_cs, act_s, misc);
        }
        grid_barrier(p, epoch);
        // output projection, residual add in the store
        gemv(4 * l + 1, p.x, 1, [&](int, int) { stage_attention(); });
        grid_barrier(p, epoch);
        // MLP: norm -> gate+up -> SwiGLU -> down, residual add in the store
        gemv(4 * l + 2, p.gu, p.pair_gu ? 2 : 0, [&](int, int) { stage_normed(g2); });
        grid_barrier(p, epoch);
        gemv(4 * l + 3, p.x, 1, stage_mlp);
        grid_barrier(p, epoch);
    }

    // ---- optional tail: final norm, LM head, greedy token ----
    if (p.tail) {
        stage_norm(p.final_gamma);   // act_s = the normalised last hidden state
        // this rank's rows of the LM head (all of them on one GPU); tokens are global indices
        const int v0 = p.lm_row0 + (int)(((unsigned long long)p.lm_rows * blockIdx.x) / gridDim.x);
        const int v1 = p.lm_row0 + (int)(((unsigned long long)p.lm_rows * (blockIdx.x + 1)) / gridDim.x);
        // one warp per vocabulary row, the same summation order as f32_matmul_kernel
        float best = -INFINITY;
        int besti = -1;
        const float4 *x4 = reinterpret_cast<const float4 *>(act_s);
        for (int row = v0 + warp; row < v1; row += DS_CONSUMER_WARPS) {
            const float4 *wr = reinterpret_cast<const float4 *>(p.lm_head + (size_t)(row - p.lm_row0) * H);
            float acc = 0.0f;
            // eight 16-byte loads in flight per lane (64 KB per SM): the row streams at the HBM
            // rate; the additions keep their order
#pragma unroll 8
            for (int cidx = lane; cidx < H / 4; cidx += 32) {
                const float4 wv = __ldg(wr + cidx), xv = x4[cidx];
                acc = fmaf(wv.x, xv.x, acc);
                acc = fmaf(wv.y, xv.y, acc);
                acc = fmaf(wv.z, xv.z, acc);
                acc = fmaf(wv.w, xv.w, acc);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) p.logits[row] = acc;
            if (besti < 0 || !(acc < best)) { best = acc; besti = row; }  // later index wins ties
        }
        // CTA maximum: rows ascend within a warp, warps interleave rows -> compare (value, index)
        float *bv = misc;
        int *bi = reinterpret_cast<int *>(misc + 16);
        cons_sync();
        if (lane == 0) { bv[warp] = best; bi[warp] = besti; }
        cons_sync();
        if (tid == 0) {
            float b = -INFINITY;
            int ib = -1;
            for (int i = 0; i < DS_CONSUMER_WARPS; ++i)
                if (bi[i] >= 0 && (ib < 0 || bv[i] > b || (bv[i] == b && bi[i] > ib))) { b = bv[i]; ib = bi[i]; }
            p.best_val[blockIdx.x] = b;
            p.best_idx[blockIdx.x] = ib;
        }
        grid_barrier(p, epoch);
        if (blockIdx.x == 0 && warp == 0) {
            float b = -INFINITY;
            int ib = -1;
            for (int i = lane; i < (int)gridDim.x; i += 32) {
                const float v = __ldcg(p.best_val + i);
                const int iv = __ldcg(p.best_idx + i);
                if (iv >= 0 && (ib < 0 || v > b || (v == b && iv > ib))) { b = v; ib = iv; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float v = __shfl_xor_sync(0xffffffffu, b, o);
                const int iv = __shfl_xor_sync(0xffffffffu, ib, o);
                if (iv >= 0 && (ib < 0 || v > b || (v == b && iv > ib))) { b = v; ib = iv; }
            }
            if (lane == 0) {
                if (p.tp_size > 1) {
                    // exchange the ranks' best (value, index): same slots-and-tags scheme as the
                    // row-parallel GEMVs, parity by step; every rank reduces in rank order with
                    // the same tie rule (the larger index wins), so every rank picks the same token
                    const unsigned int tag = tp_tag_base + (unsigned int)(2 * p.layers) + 1u;
                    const int par = (int)(tp_seq & 1u);
                    const unsigned long long wv = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(b);
                    const unsigned long long wi = ((unsigned long long)tag << 32) | (unsigned long long)(unsigned int)ib;
                    for (int r = 0; r < p.tp_size; ++r) {
                        if (r == p.tp_rank) continue;
                        st_relaxed_sys_u64(p.tp_peer[r] + tp_arg_slot(p, par, p.tp_rank, 0), wv);
                        st_relaxed_sys_u64(p.tp_peer[r] + tp_arg_slot(p, par, p.tp_rank, 1), wi);
                    }
                    const unsigned long long *local = p.tp_peer[p.tp_rank];
                    float gb = -INFINITY;
                    int gi = -1;
                    for (int r = 0; r < p.tp_size; ++r) {
                        float v = b;
                        int iv = ib;
                        if (r != p.tp_rank) {
                            v = __uint_as_float(tp_wait_word(p, local + tp_arg_slot(p, par, r, 0), tag));
                            iv = (int)tp_wait_word(p, local + tp_arg_slot(p, par, r, 1), tag);
                        }
                        if (iv >= 0 && (gi < 0 || v > gb || (v == gb && iv > gi))) { gb = v; gi = iv; }
                    }
                    ib = gi;
                }
                *p.token_out = ib < 0 ? 0 : ib;
                *p.pos_out = pos + 1;
            }
        }
    }

    // the last CTA to leave resets the barrier words for the next launch
    if (tid == 0) {
        __threadfence();
        const unsigned int prev = atomicAdd(&p.sync[1], 1u);
        if (prev == gridDim.x - 1) {
            p.sync[0] = 0u;
            p.sync[1] = 0u;
            if (p.tp_size > 1) *p.tp_seq = tp_seq + 1u;  // the next launch's exchanges get fresh tags
            __threadfence();
        }
    }
}

#include "decode_step_batch.cuh"

}  // namespace yscv

// ---------------------------------------------------------------------------
// Host side: the plan and its C ABI
// ---------------------------------------------------------------------------

struct yscv_cuda_decode_plan {
    int device = 0;
    yscv::StepParams params = {};
    int smem = 0;
    bool simple = false;
    void *d_mats = nullptr, *d_gamma = nullptr, *d_kptr = nullptr, *d_vptr = nullptr;
    void *d_scratch = nullptr, *d_sync = nullptr;
    bool poisoned = false;   // a bounded wait ran out in a step of this plan (yscv_cuda_decode_plan_check)
    int tp_rank = 0, tp_size = 1;
    int batch = 1;           // > 1: decode_step_batch_kernel
};

extern "C" void yscv_cuda_decode_plan_free(yscv_cuda_decode_plan *plan) {
    if (!plan) return;
    cudaSetDevice(plan->device);
    cudaFree(plan->d_mats);
    cudaFree(plan->d_gamma);
    cudaFree(plan->d_kptr);
    cudaFree(plan->d_vptr);
    cudaFree(plan->d_scratch);
    cudaFree(plan->d_sync);
    delete plan;
}

extern "C" int yscv_cuda_decode_plan_create(yscv_cuda_ctx *ctx, const yscv_cuda_decode_layer *layers,
                                            size_t n_layers, size_t hidden, size_t inter, size_t n_q,
                                            size_t n_kv, size_t d_head, size_t max_seq, float eps,
                                            float rope_theta, yscv_cuda_decode_plan **out) {
    return yscv_cuda_decode_plan_create_ex(ctx, layers, n_layers, hidden, inter, n_q, n_kv, d_head, max_seq, eps,
                                           rope_theta, nullptr, out);
}

extern "C" int yscv_cuda_decode_plan_create_ex(yscv_cuda_ctx *ctx, const yscv_cuda_decode_layer *layers,
                                               size_t n_layers, size_t hidden, size_t inter, size_t n_q,
                                               size_t n_kv, size_t d_head, size_t max_seq, float eps,
                                               float rope_theta, const yscv_cuda_decode_options *opt,
                                               yscv_cuda_decode_plan **out) {
    using namespace yscv;
    if (!ctx || !layers || !out || n_layers == 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (tensor_map_encoder() == nullptr) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "no tensor-map encoder in this driver");
    const int grid = ctx->sm_count;
    if (n_kv == 0 || n_q % n_kv != 0 || d_head == 0 || d_head % 16 != 0 || d_head > 128 ||
        DS_CONSUMERS % d_head != 0 || n_q > (size_t)grid)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: n_q=%zu n_kv=%zu d_head=%zu not supported on %d SMs",
                    n_q, n_kv, d_head, grid);
    const size_t qkv_rows = (n_q + 2 * n_kv) * d_head, attn_w = n_q * d_head;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    auto *plan = new yscv_cuda_decode_plan();
    plan->device = ctx->device;
    auto bail = [&](int rc) {
        yscv_cuda_decode_plan_free(plan);
        return rc;
    };
    // kernel variants (options: a bit mask): 1 gate/up pairing, 2 sixteen K slices for one-tile
    // slabs, 4 merge-weight table, 8 relaxed barrier polling
    // batch form: 2..8 sequences per step (always with paired gate/up rows)
    const int batch = (opt && opt->batch > 1) ? opt->batch : 1;
    const int variant = ((opt && opt->variant >= 0) ? opt->variant : DS_DEFAULT_VARIANT) | (batch > 1 ? 1 : 0);
    // geometry limits, overridable so that small test shapes reach the row-block and K-chunk
    // paths: tiles per row block (2..8, even), k per chunk (a multiple of 512)
    int max_tiles = (opt && opt->max_tiles > 0) ? opt->max_tiles : 8;
    max_tiles = max_tiles < 2 ? 2 : (max_tiles > 8 ? 8 : max_tiles & ~1);
    int kc_limit = (opt && opt->k_chunk > 0) ? opt->k_chunk / 512 : 16;   // 16 stages = 8192 k = 64 KB of digit planes
    kc_limit = kc_limit < 1 ? 1 : (kc_limit > 16 ? 16 : kc_limit);
    if (batch > 1 && kc_limit > 4) kc_limit = 4;   // 32 activations per staging thread: chunks of 2048 k
    const yscv_cuda_tp_comm *tp = opt ? opt->tp : nullptr;
    const bool kv_int8 = opt && opt->kv_int8 != 0;
    if (batch > DSB_ROWS)
        return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: at most %d sequences per step, got %d", DSB_ROWS, batch));
    if (batch > 1 && (tp || kv_int8))
        return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: the batch form runs on one GPU with f32 caches"));
    if (batch > 1 && (hidden > 2048 || n_q * d_head > 2048 || d_head % 8 != 0))
        return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED,
                         "decode plan: the batch form needs hidden and n_q * d_head <= 2048 (hidden=%zu, n_q*d_head=%zu)",
                         hidden, n_q * d_head));
    if (tp && (tp->device != ctx->device || !tp->connected))
        return bail(fail(YSCV_CUDA_ERR_BAD_ARG, "decode plan: the exchange region is not connected on device %d", ctx->device));
    if (tp && tp->cap_rows < hidden)
        return bail(fail(YSCV_CUDA_ERR_BAD_ARG, "decode plan: the exchange region holds %zu rows, hidden is %zu", tp->cap_rows, hidden));
    if (kv_int8 && d_head != 64 && d_head != 128)
        return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: int8 caches need d_head 64 or 128, got %zu", d_head));
    if (kv_int8 && n_kv * d_head > 2048)
        return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: int8 caches need n_kv * d_head <= 2048, got %zu", n_kv * d_head));
    // rows (or paired indices) per CTA -> row blocks of at most `cap` tiles, balanced. (Taking
    // more, smaller blocks where that wastes fewer padding rows, 5 x 5 tiles instead of 4 x 7 for
    // 388 rows, measured 4 % slower on the 70B shape: every stage has a fixed cost per warp.)
    auto blocks_of = [&](size_t per_cta, int cap, int *tiles_out) {
        const int n_rb = (int)((per_cta + (size_t)cap * 16 - 1) / ((size_t)cap * 16));
        const size_t per_block = (per_cta + n_rb - 1) / n_rb;
        *tiles_out = (int)((per_block + 15) / 16);
        return n_rb;
    };
    const bool pair_gu = (variant & 1) != 0;
    int nrb[4] = {1, 1, 1, 1}, tl[4] = {1, 1, 1, 1};
    // every matrix: shape, geometry, tensor maps
    std::vector<StepMat> mats(n_layers * 4);
    size_t k_max = 0;
    int slot_bytes = 0;
    for (size_t l = 0; l < n_layers; ++l) {
        const yscv_cuda_int4_weight *w[4] = {layers[l].qkv, layers[l].o, layers[l].gate_up, layers[l].down};
        const size_t want_n[4] = {qkv_rows, hidden, 2 * inter, hidden};
        const size_t want_k[4] = {hidden, attn_w, hidden, inter};
        if (!layers[l].d_gamma_attn || !layers[l].d_gamma_mlp || !layers[l].d_kcache || !layers[l].d_vcache ||
            (kv_int8 && (!layers[l].d_kscale || !layers[l].d_vscale)))
            return bail(fail(YSCV_CUDA_ERR_BAD_ARG, "decode plan: layer %zu has a null pointer", l));
        // key and value rows are read with 128-bit loads
        if ((reinterpret_cast<uintptr_t>(layers[l].d_kcache) | reinterpret_cast<uintptr_t>(layers[l].d_vcache)) & 15)
            return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: the caches of layer %zu must be 16-byte aligned", l));
        for (int j = 0; j < 4; ++j) {
            if (!w[j]) return bail(fail(YSCV_CUDA_ERR_BAD_ARG, "decode plan: layer %zu has a null weight", l));
            if (w[j]->m_w != want_n[j] || w[j]->k != want_k[j])
                return bail(fail(YSCV_CUDA_ERR_BAD_ARG,
                                 "decode plan: layer %zu matrix %d is [%zu][%zu], expected [%zu][%zu]",
                                 l, j, w[j]->m_w, w[j]->k, want_n[j], want_k[j]));
            if (w[j]->group_size != 32)
                return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: group size %zu (only 32)",
                                 w[j]->group_size));
            const size_t n = w[j]->m_w, k = w[j]->k;
            if (k % 512 != 0 || n < (size_t)grid ||
                ((reinterpret_cast<uintptr_t>(w[j]->d_packed) | reinterpret_cast<uintptr_t>(w[j]->d_scales)) & 15))
                return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED,
                                 "decode plan: matrix [%zu][%zu] needs k %% 512 == 0, n >= %d and 16-byte alignment",
                                 n, k, grid));
            StepMat &m = mats[l * 4 + j];
            memset(&m, 0, sizeof(m));
            m.n = (int)n;
            m.k = (int)k;
            m.k_stages = (int)(k / 512);
            uint32_t box_rows;
            if (j == 2 && pair_gu) {
                // gate rows and the matching up rows: two boxes of half the block each
                int half = 1;
                nrb[j] = blocks_of((inter + grid - 1) / grid, max_tiles / 2, &half);
                m.tiles = 2 * half;
                box_rows = (uint32_t)half * 16;
            } else {
                nrb[j] = blocks_of((n + grid - 1) / grid, max_tiles, &m.tiles);
                box_rows = (uint32_t)m.tiles * 16;
            }
            tl[j] = m.tiles;
            int rc = encode_2d(&m.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w[j]->d_packed, n, k / 2, k / 2, box_rows,
                               128, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return bail(rc);
            rc = encode_2d(&m.tm_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, w[j]->d_scales, n, k / 32, k / 8, box_rows,
                           DS_GS, CU_TENSOR_MAP_SWIZZLE_64B);
            if (rc) return bail(rc);
            const uint32_t rb_rows = (uint32_t)m.tiles * 16;
            k_max = k > k_max ? k : k_max;
            const int sb = (int)rb_rows * (DS_GS * 16 + DS_GS * 4);
            slot_bytes = sb > slot_bytes ? sb : slot_bytes;
        }
    }
    slot_bytes = ((slot_bytes + 1023) / 1024) * 1024;
    StepParams &p = plan->params;
    // K chunk: the digit planes and activations of one chunk are resident at a time; only the
    // down projection may span several chunks, and then with a single row block
    const int kc_stages = std::min<int>((int)(k_max / 512), kc_limit);
    if (hidden / 512 > (size_t)kc_stages || attn_w / 512 > (size_t)kc_stages ||
        (inter / 512 > (size_t)kc_stages && nrb[3] != 1))
        return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED,
                         "decode plan: hidden=%zu / n_q*d_head=%zu exceed one K chunk of %d, or the down projection "
                         "needs both several chunks and several row blocks", hidden, attn_w, kc_stages * 512));
    p.kc_stages = kc_stages;
    p.dig_bytes = kc_stages * (batch > 1 ? DSB_BLOB_BYTES : DS_BLOB_BYTES);
    p.batch = batch;
    p.red_bytes = batch > 1 ? 2 * DS_RED_BYTES : DS_RED_BYTES;
    // attention form: per query head with up to 4 key chunks, or (long contexts, or
    // YSCV_CUDA_STEP_ATTN=1) per KV head with up to 32 key chunks and a merge phase
    // key chunks (CTAs) per query head: up to 4, or up to 16 when this GPU has so few heads that
    // 4 would leave most SMs idle (tensor-parallel shards)
    const int splits = batch > 1 ? (int)std::max<size_t>(1, std::min<size_t>(4, (size_t)grid / (n_q * batch)))
                                 : (int)std::min<size_t>(n_q * 4 * 2 <= (size_t)grid ? 16 : 4, (size_t)grid / n_q);
    const size_t grp = n_q / n_kv;
    const bool group_ok = (grp & (grp - 1)) == 0 && grp <= 16 && grp * d_head <= 2048 &&
                          DS_CONSUMERS % (grp * d_head / 4) == 0;
    const int attn_form = opt ? opt->attention_form : -1;
    // batch form: per (sequence, query head, key chunk) by default; per KV head and key chunk
    // (one pass over a chunk's rows serves every query head of the group; the chunks are merged
    // while the output projection stages its input, no merge phase) only on request: at the
    // TinyLlama shape with 128-256 cached positions it measured 10 % slower per step
    const bool grouped = batch > 1 ? (group_ok && attn_form == 1)
                                   : group_ok && (attn_form >= 0 ? attn_form != 0 : (max_seq + splits - 1) / splits > 256);
    const int g_splits = batch > 1 ? (int)std::max<size_t>(1, std::min<size_t>(4, (size_t)grid / (n_kv * batch)))
                                   : (int)std::max<size_t>(1, std::min<size_t>(32, (size_t)grid / n_kv));
    const int g_cap = (int)(((max_seq + g_splits - 1) / g_splits + 3) / 4 * 4);
    // the attention scratch lives in the activation area between the GEMVs: widen that area if
    // it needs more
    const size_t g_parts = DS_CONSUMERS / (grp * d_head / 4 ? grp * d_head / 4 : 1);
    const size_t attn_scratch =
        grouped ? (grp * d_head + 2 * d_head + g_parts * grp * d_head + 32 + grp * (size_t)g_cap) * sizeof(float)
                : (3 * d_head + 4 * DS_CONSUMERS + max_seq) * sizeof(float);
    size_t act_floats = (size_t)kc_stages * 512;
    if (attn_scratch > act_floats * 4) act_floats = (attn_scratch + 3) / 4;
    if (batch > 1) {
        // the tail keeps the normalised rows [8][hidden] in the digit area and the scratch behind
        // it, then the per-warp maxima [8][16] x {value, index} at the start of the scratch
        const size_t rows_bytes = (size_t)DSB_ROWS * hidden * sizeof(float);
        const size_t need = rows_bytes > (size_t)p.dig_bytes ? (rows_bytes - p.dig_bytes) / 4 : 0;
        act_floats = std::max<size_t>(std::max<size_t>(act_floats, need), 2 * DSB_ROWS * DS_CONSUMER_WARPS);
    }
    act_floats = (act_floats + 3) / 4 * 4;
    if (act_floats * 4 > 96 * 1024)
        return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: max_seq=%zu does not fit one CTA per head", max_seq));
    p.act_floats = (int)act_floats;
    // misc, rotary factors, cache pointers, split-merge weights
    const int tables = 128 + (int)d_head * 4 + (int)n_layers * 2 * 8 + (int)n_q * 16 * (splits > 4 ? 4 : 1) + 16;
    const int fixed = p.red_bytes + DS_BAR_BYTES + p.dig_bytes + p.act_floats * 4 + tables;
    const int budget = 227 * 1024 - fixed - 1024;
    p.stages = budget / slot_bytes;
    if (p.stages > DS_MAX_STAGES) p.stages = DS_MAX_STAGES;
    if (p.stages < 2) return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: k=%zu leaves no room for the weight ring", k_max));
    p.slot_bytes = slot_bytes;
    plan->smem = p.stages * slot_bytes + fixed;

    // device copies: matrices, gammas, cache pointers, scratch, barrier words
    // cache pointers, then (int8 caches) the row-scale tables
    std::vector<float *> kptr(2 * n_layers, nullptr), vptr(2 * n_layers, nullptr);
    for (size_t l = 0; l < n_layers; ++l) {
        kptr[l] = reinterpret_cast<float *>(layers[l].d_kcache);
        vptr[l] = reinterpret_cast<float *>(layers[l].d_vcache);
        kptr[n_layers + l] = layers[l].d_kscale;
        vptr[n_layers + l] = layers[l].d_vscale;
    }
    const size_t attn_floats = (size_t)batch * n_q * (size_t)(grouped ? g_splits : splits) * (d_head + 2);
    const size_t scratch_floats = (size_t)batch * (qkv_rows + 2 * inter + attn_w + 2 * (size_t)grid) + attn_floats;
#define PLAN_TRY(expr)                                                                       \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            return bail(fail(YSCV_CUDA_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e))); \
    } while (0)
    PLAN_TRY(cudaMalloc(&plan->d_mats, mats.size() * sizeof(StepMat)));
    PLAN_TRY(cudaMalloc(&plan->d_gamma, n_layers * 2 * hidden * sizeof(float)));
    PLAN_TRY(cudaMalloc(&plan->d_kptr, 2 * n_layers * sizeof(float *)));
    PLAN_TRY(cudaMalloc(&plan->d_vptr, 2 * n_layers * sizeof(float *)));
    PLAN_TRY(cudaMalloc(&plan->d_scratch, scratch_floats * sizeof(float)));
    PLAN_TRY(cudaMalloc(&plan->d_sync, 4 * sizeof(unsigned int)));
    PLAN_TRY(cudaMemcpyAsync(plan->d_mats, mats.data(), mats.size() * sizeof(StepMat), cudaMemcpyHostToDevice, ctx->stream));
    PLAN_TRY(cudaMemcpyAsync(plan->d_kptr, kptr.data(), 2 * n_layers * sizeof(float *), cudaMemcpyHostToDevice, ctx->stream));
    PLAN_TRY(cudaMemcpyAsync(plan->d_vptr, vptr.data(), 2 * n_layers * sizeof(float *), cudaMemcpyHostToDevice, ctx->stream));
    PLAN_TRY(cudaMemsetAsync(plan->d_sync, 0, 4 * sizeof(unsigned int), ctx->stream));
    for (size_t l = 0; l < n_layers; ++l) {
        float *g = reinterpret_cast<float *>(plan->d_gamma) + l * 2 * hidden;
        PLAN_TRY(cudaMemcpyAsync(g, layers[l].d_gamma_attn, hidden * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
        PLAN_TRY(cudaMemcpyAsync(g + hidden, layers[l].d_gamma_mlp, hidden * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    }
    PLAN_TRY(cudaStreamSynchronize(ctx->stream));  // the host vectors go out of scope
    plan->simple = batch == 1 && nrb[0] == 1 && nrb[1] == 1 && nrb[2] == 1 && nrb[3] == 1 &&
                   (int)(k_max / 512) <= kc_stages && !grouped;
    plan->batch = batch;
    auto kern = batch > 1 ? decode_step_batch_kernel : (plan->simple ? decode_step_kernel<true> : decode_step_kernel<false>);
    PLAN_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan->smem));
    int per_sm = 0;
    PLAN_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, DS_THREADS, plan->smem));
    if (per_sm < 1) return bail(fail(YSCV_CUDA_ERR_UNSUPPORTED, "decode plan: the step kernel does not fit an SM"));
#undef PLAN_TRY
    p.mats = reinterpret_cast<const StepMat *>(plan->d_mats);
    p.gamma = reinterpret_cast<const float *>(plan->d_gamma);
    p.kcache = reinterpret_cast<float *const *>(plan->d_kptr);
    p.vcache = reinterpret_cast<float *const *>(plan->d_vptr);
    p.kv_int8 = kv_int8 ? 1 : 0;
    float *s = reinterpret_cast<float *>(plan->d_scratch);
    p.qkv = s;
    p.attn = s + (size_t)batch * qkv_rows;
    p.gu = p.attn + attn_floats;
    p.attn_out = p.gu + (size_t)batch * 2 * inter;
    p.best_val = p.attn_out + (size_t)batch * attn_w;
    p.best_idx = reinterpret_cast<int *>(p.best_val + (size_t)batch * grid);
    p.splits = (batch > 1 && grouped) ? g_splits : splits;   // (batch form: chunks per head in p.attn)
    p.attn_grouped = grouped ? 1 : 0;
    p.g_splits = g_splits;
    p.g_chunk_cap = g_cap;
    p.sync = reinterpret_cast<unsigned int *>(plan->d_sync);
    p.status = ctx->d_status;
    p.layers = (int)n_layers;
    p.hidden = (int)hidden;
    p.inter = (int)inter;
    p.n_q = (int)n_q;
    p.n_kv = (int)n_kv;
    p.d_head = (int)d_head;
    p.max_seq = (int)max_seq;
    p.eps = eps;
    p.theta = rope_theta;
    p.pair_gu = pair_gu ? 1 : 0;
    p.gu_half_tiles = tl[2] / 2;
    p.one_tile_16 = (variant & 2) ? 1 : 0;
    p.merge_table = (variant & 4) ? 1 : 0;
    p.relaxed_poll = (variant & 8) ? 1 : 0;
    p.spin_limit = (opt && opt->spin_limit > 0) ? opt->spin_limit : DS_SPIN_LIMIT;
    p.tp_rank = 0;
    p.tp_size = 1;
    if (tp) {
        p.tp_rank = tp->rank;
        p.tp_size = tp->world;
        p.tp_cap = (int)tp->cap_rows;
        for (int r = 0; r < tp->world; ++r) p.tp_peer[r] = reinterpret_cast<unsigned long long *>(tp->peer[r]);
        p.tp_seq = tp->d_seq;
        plan->tp_rank = tp->rank;
        plan->tp_size = tp->world;
    }
    for (int j = 0; j < 4; ++j) {
        p.mat_n[j] = mats[j].n;
        p.mat_tiles[j] = mats[j].tiles;
        p.mat_ks[j] = mats[j].k_stages;
        const int sub = mats[j].tiles * 16 * (DS_GS * 16 + DS_GS * 4);
        p.mat_kps[j] = std::max(1, std::min(slot_bytes / sub, 8));
        p.mat_nrb[j] = nrb[j];
    }
    *out = plan;
    return YSCV_CUDA_OK;
}

static int launch_step(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan, yscv::StepParams &p) {
    using namespace yscv;
    p.status = ctx->d_status;
    // the CTAs wait on one another: cooperative launch, one CTA per SM
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->sm_count);
    cfg.blockDim = dim3(DS_THREADS);
    cfg.dynamicSmemBytes = plan->smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ctx->prof_begin();
    if (plan->batch > 1)
        YSCV_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_step_batch_kernel, p));
    else if (plan->simple)
        YSCV_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_step_kernel<true>, p));
    else
        YSCV_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_step_kernel<false>, p));
    ctx->prof_end();
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    ctx->last_kernel = plan->batch > 1 ? (p.tail ? "decode_step_batch(persistent,tma,imma,+lm_head)" : "decode_step_batch(persistent,tma,imma)")
                                       : (p.tail ? "decode_step(persistent,tma,imma,+lm_head)" : "decode_step(persistent,tma,imma)");
    return YSCV_CUDA_OK;
}

extern "C" int yscv_cuda_decode_plan_check(yscv_cuda_ctx *ctx, yscv_cuda_decode_plan *plan) {
    using namespace yscv;
    if (!ctx || !plan) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (plan->poisoned) return fail(YSCV_CUDA_ERR_TIMEOUT, "a bounded wait ran out in an earlier step of this plan: rebuild it");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    unsigned int words[4] = {0, 0, 0, 0};
    YSCV_CUDA_TRY(cudaMemcpyAsync(words, plan->d_sync, sizeof(words), cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (words[2] != 0u) {
        plan->poisoned = true;
        return fail(YSCV_CUDA_ERR_TIMEOUT, "a bounded wait ran out in a step of this plan: its results are void, rebuild it");
    }
    return YSCV_CUDA_OK;
}

static int step_common(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan, const float *d_embedding, size_t vocab,
                       const int32_t *d_token, const int32_t *d_pos, float *d_x, yscv::StepParams &p) {
    using namespace yscv;
    if (!ctx || !plan || !d_embedding || !d_token || !d_pos || !d_x || vocab == 0)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (plan->device != ctx->device) return fail(YSCV_CUDA_ERR_BAD_ARG, "plan belongs to device %d", plan->device);
    if (plan->poisoned)
        return fail(YSCV_CUDA_ERR_TIMEOUT, "a bounded wait ran out in an earlier step of this plan: rebuild it");
    if (vocab >= (1u << 30)) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "vocabulary too large");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    p = plan->params;
    p.embedding = d_embedding;
    p.vocab = (int)vocab;
    p.token = d_token;
    p.pos = d_pos;
    p.x = d_x;
    p.tail = 0;
    p.lm_row0 = 0;
    p.lm_rows = (int)vocab;
    op_counters().decode_step_calls++;
    return YSCV_CUDA_OK;
}

extern "C" int yscv_cuda_decode_plan_step_dev(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan,
                                              const float *d_embedding, size_t vocab, const int32_t *d_token,
                                              const int32_t *d_pos, float *d_x) {
    yscv::StepParams p;
    int rc = step_common(ctx, plan, d_embedding, vocab, d_token, d_pos, d_x, p);
    if (rc) return rc;
    return launch_step(ctx, plan, p);
}

extern "C" int yscv_cuda_decode_plan_step_token_shard_dev(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan,
                                                          const float *d_embedding, size_t vocab, int32_t *d_token,
                                                          int32_t *d_pos, const float *d_final_gamma,
                                                          const float *d_lm_head_rows, size_t lm_row0,
                                                          size_t lm_rows, float *d_x, float *d_logits) {
    using namespace yscv;
    if (!d_final_gamma || !d_lm_head_rows || !d_logits) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (lm_rows == 0 || lm_row0 + lm_rows > vocab)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "LM head rows [%zu, %zu) are not inside the vocabulary of %zu", lm_row0,
                    lm_row0 + lm_rows, vocab);
    if ((reinterpret_cast<uintptr_t>(d_lm_head_rows) & 15) != 0)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "the LM head must be 16-byte aligned");
    StepParams p;
    int rc = step_common(ctx, plan, d_embedding, vocab, d_token, d_pos, d_x, p);
    if (rc) return rc;
    if (p.tp_size == 1 && lm_rows != vocab)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "a plan for one GPU needs every row of the LM head");
    p.tail = 1;
    p.final_gamma = d_final_gamma;
    p.lm_head = d_lm_head_rows;
    p.lm_row0 = (int)lm_row0;
    p.lm_rows = (int)lm_rows;
    p.logits = d_logits;
    p.token_out = d_token;
    p.pos_out = d_pos;
    return launch_step(ctx, plan, p);
}

extern "C" int yscv_cuda_decode_plan_step_token_dev(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan,
                                                    const float *d_embedding, size_t vocab, int32_t *d_token,
                                                    int32_t *d_pos, const float *d_final_gamma,
                                                    const float *d_lm_head, float *d_x, float *d_logits) {
    return yscv_cuda_decode_plan_step_token_shard_dev(ctx, plan, d_embedding, vocab, d_token, d_pos, d_final_gamma,
                                                      d_lm_head, 0, vocab, d_x, d_logits);
}
