// One launch = one decode step of a small batch (2..8 sequences at the same position) through
// every layer: the batch form of decode_step_kernel, included by decode_step.cu (it uses that
// file's StepParams, barriers, ring bookkeeping and per-head attention).
//
// The reference decodes a batch as the same ONNX node chain with M = batch rows in every MatMul
// (apps/llm-bench/src/main.rs:491-561, crates/yscv-onnx/src/runner/linear.rs:223-278). Here the
// batch rows ride through the one-launch step:
//   * the weight stream, the ring and the grid barriers are those of the batch-1 kernel: every
//     weight byte is still read once per step, whatever the batch;
//   * the GEMVs become M = 8 small matmuls on the integer MMA path: the activations of all batch
//     rows are turned into the three-digit-plane form of int4_gemv.cu (8 rows = the 8 columns of
//     one mma.m16n8k32 per plane), rows past the batch are zero;
//   * the staging of every phase works on all rows at once (64 threads per row): RMSNorm,
//     the merge of the attention splits, SwiGLU products, each straight from registers into the
//     digit planes;
//   * attention runs per (sequence, query head, key chunk) work item over the CTAs (or, on
//     request, per (sequence, KV head, key chunk) serving the whole group of query heads);
//   * the tail does the final norm of every row, the LM head with one pass over the weights
//     for all rows, and one greedy token per row.
// Limits (checked when the plan is built): hidden, n_q * head_dim <= 2048 and K chunks of 2048
// (32 activations per thread in registers), f32 caches, at most four key chunks per head, one GPU.

constexpr int DSB_ROWS = 8;                               // activation rows of the MMA (batch padded)
constexpr int DSB_TPR = DS_CONSUMERS / DSB_ROWS;          // 64 threads stage one row
constexpr int DSB_EPT = 32;                               // activations per thread and staging pass
constexpr int DSB_BLOB_BYTES = DS_GS * (DSB_ROWS * 4 * 16 + DSB_ROWS * 4 * 8 + DSB_ROWS * 8);  // planes form, one K stage

// Threads (row = tid / 64, quad = (tid % 64) / 4, t = tid % 4) hold v[j][0..7] = activations
// k = (j * 16 + quad) * 32 + 8 t .. + 7 of their row, j < passes: write their digit planes.
// Rows at or past `batch` pass zeros (their planes were cleared once per launch, nothing is written).
__device__ __forceinline__ void dsb_quantize_rows(const float (&v)[DSB_EPT / 8][8], unsigned char *dig, int klen, int batch) {
    const QuantLayout q = quant_layout(DSB_ROWS, DS_GS);
    const int tid = threadIdx.x, row = tid / DSB_TPR, quad = (tid % DSB_TPR) >> 2, t = tid & 3;
    const int groups = klen / 32;
#pragma unroll
    for (int j = 0; j < DSB_EPT / 8; ++j) {
        const int G = j * (DSB_TPR / 4) + quad;
        // (a warp stages one row: rows past the batch skip the arithmetic as a whole)
        if (row < batch) quantize_group_values(v[j], dig, q, G < groups ? G : 0, row, t, G < groups);
    }
    cons_sync();
}

// M = 8 form of consume_stages: K stages [ks_begin, ks_end) of one row block, three integer MMAs
// per group (digit planes 2, 1, 0 of all eight activation rows), four accumulators per thread:
// rows gq / gq + 8 of the tile x activation rows 2t / 2t + 1. Same arithmetic as
// int4_gemv_fast_kernel<8, ...>.
template <int TP2>
__device__ __forceinline__ void dsb_consume_stages(const StepParams &p, const unsigned char *smem, uint32_t bar_full,
                                                   uint32_t bar_empty, const unsigned char *dig, RingPos &c, int tiles,
                                                   int ks_begin, int ks_end, int kps, int dig_stage0, float (&acc)[4],
                                                   bool &dead) {
    constexpr int GS = DS_GS;
    constexpr int KSL = (16 / TP2 < GS) ? 16 / TP2 : GS;
    constexpr int GPW = GS / KSL;
    constexpr int MS = DSB_ROWS, MC = DSB_ROWS;
    constexpr int OFF_H1 = GS * MS * 4 * 16, OFF_META = OFF_H1 + GS * MS * 4 * 8;
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
    const uint32_t f_off = (uint32_t)((G0 * MS + gq) * 4 + t) * 16;
    const uint32_t h1_off = OFF_H1 + (uint32_t)((G0 * MS + gq) * 4 + t) * 8;
    const uint32_t mt_off = OFF_META + (uint32_t)(G0 * MC + 2 * t) * 8;
    constexpr uint32_t f_step = MS * 4 * 16, h1_step = MS * 4 * 8, mt_step = MC * 8;

    const uint32_t sub_bytes = (uint32_t)rb_rows * (GS * 16 + GS * 4);  // one K stage inside a slot
    for (int ks0 = ks_begin; ks0 < ks_end; ks0 += kps) {
        if (!dead) dead = !mbar_wait(bar_full + c.slot * 8, c.phase, p.status);
        const int nsub = min(kps, ks_end - ks0);
        if (active && !dead) {
            for (int j = 0; j < nsub; ++j) {
                const unsigned char *st = smem + (size_t)c.slot * p.slot_bytes + (size_t)j * sub_bytes;
                const unsigned char *db = dig + (size_t)(ks0 + j - dig_stage0) * DSB_BLOB_BYTES;
#pragma unroll
                for (int gi = 0; gi < GPW; ++gi) {
                    const uint32_t G = (uint32_t)(G0 + gi);
                    const uint32_t so = (((G >> 2) ^ s_phase) << 4) + (G & 3u) * 4;
                    const float sA = lds_f32(st, s_row + so), sB = lds_f32(st, s_row + 8 * (GS * 4) + so);
                    const uint32_t wA = lds32(st, w_off[gi]), wB = lds32(st, w_off[gi] + 1024);
                    uint32_t a[4];
                    a[0] = nib_u8(wA);
                    a[1] = nib_u8(wB);
                    a[2] = nib_u8(wA >> 4);
                    a[3] = nib_u8(wB >> 4);
                    const uint4 h0 = lds128(db, f_off + gi * f_step);
                    const uint2 h1 = lds64(db, h1_off + gi * h1_step);
                    const uint4 mt = lds128(db, mt_off + gi * mt_step);
                    int c2[4], c1[4], c0[4];
                    mma_u8s8(c2, a, h0.x, h0.y, 0, 0, 0, 0);
                    mma_u8s8(c1, a, h0.z, h0.w, 0, 0, 0, 0);
                    mma_u8s8(c0, a, h1.x, h1.y, (int)mt.y, (int)mt.w, (int)mt.y, (int)mt.w);
                    const float as0 = __uint_as_float(mt.x), as1 = __uint_as_float(mt.z);
                    const int v0 = c2[0] * 65536 + (c1[0] * 256 + c0[0]);
                    const int v1 = c2[1] * 65536 + (c1[1] * 256 + c0[1]);
                    const int v2 = c2[2] * 65536 + (c1[2] * 256 + c0[2]);
                    const int v3 = c2[3] * 65536 + (c1[3] * 256 + c0[3]);
                    acc[0] = fmaf(sA * as0, (float)v0, acc[0]);
                    acc[1] = fmaf(sA * as1, (float)v1, acc[1]);
                    acc[2] = fmaf(sB * as0, (float)v2, acc[2]);
                    acc[3] = fmaf(sB * as1, (float)v3, acc[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + c.slot * 8);
        if (++c.slot == p.stages) { c.slot = 0; c.phase ^= 1u; }
    }
}

// Combines the K slices of a row block in a fixed order and stores the batch rows:
// store 0: out[m * ld + row] = v; 1: out[m * ld + row] += v (the residual stream);
// 2: the block is gate tiles then up tiles of intermediate indices: out[m * ld + i] = silu(gate) * up.
template <int TP2>
__device__ __forceinline__ void dsb_finish_rows(float *red, int tiles, int row_base, int r1, float *out, int ld,
                                                int store, int batch, const float (&acc)[4]) {
    constexpr int GS = DS_GS;
    constexpr int KSL = (16 / TP2 < GS) ? 16 / TP2 : GS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = warp % TP2, kslice = warp / TP2;
    if ((tile < tiles) && (kslice < KSL)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) red[((kslice * tiles + tile) * 4 + j) * 32 + lane] = acc[j];
    }
    cons_sync();
    // element (tile, row-in-tile r16, batch row m) sits in accumulator j = (r16 >= 8 ? 2 : 0) + (m & 1)
    // of lane (r16 & 7) * 4 + (m >> 1)
    auto total = [&](int tl, int r16, int m) {
        const int j = ((r16 >> 3) << 1) + (m & 1), ln = (r16 & 7) * 4 + (m >> 1);
        float v = 0.0f;
        for (int ks = 0; ks < KSL; ++ks) v += red[((ks * tiles + tl) * 4 + j) * 32 + ln];
        return v;
    };
    if (store == 2) {
        const int th = tiles / 2;
        for (int i = tid; i < th * 16 * DSB_ROWS; i += DS_CONSUMERS) {
            const int r16 = i & 15, tl = (i >> 4) % th, m = i / (16 * th);
            const int idx = row_base + tl * 16 + r16;
            if (m < batch && idx < r1) {
                const float g = total(tl, r16, m), u = total(tl + th, r16, m);
                const float sg = 1.0f / (1.0f + expf(-g));
                out[(size_t)m * ld + idx] = (g * sg) * u;
            }
        }
    } else {
        for (int i = tid; i < tiles * 16 * DSB_ROWS; i += DS_CONSUMERS) {
            const int r16 = i & 15, tl = (i >> 4) % tiles, m = i / (16 * tiles);
            const int row = row_base + tl * 16 + r16;
            if (m < batch && row < r1) {
                const float v = total(tl, r16, m);
                float *o = out + (size_t)m * ld + row;
                *o = store == 1 ? __ldcg(o) + v : v;
            }
        }
    }
    cons_sync();  // `red` is reused by the next block
}

__global__ void __launch_bounds__(DS_THREADS, 1) decode_step_batch_kernel(const StepParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ring_bytes = (uint32_t)p.stages * p.slot_bytes;
    float *red = reinterpret_cast<float *>(smem + ring_bytes);
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_full = smem_base + ring_bytes + p.red_bytes;
    const uint32_t bar_empty = bar_full + 8 * DS_MAX_STAGES;
    unsigned char *dig = smem + ring_bytes + p.red_bytes + DS_BAR_BYTES;
    float *act_s = reinterpret_cast<float *>(dig + p.dig_bytes);   // attention scratch / tail rows
    float *misc = act_s + p.act_floats;  // 32 floats
    float *rope_cs = misc + 32;          // [d_head/2] x {cos, sin} of this step's position
    float **cache_ptr = reinterpret_cast<float **>(rope_cs + p.d_head);  // [layers] x {k, v}
    const int nmat = p.layers * 4;
    const int B = p.batch;

    {
        const int pos0 = *p.pos;
        if (pos0 < 0 || pos0 >= p.max_seq) {
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
    // (the same walk as decode_step_kernel: K chunk, row block, K stage; gate/up always paired)
    if (warp == DS_CONSUMER_WARPS) {
        if (lane == 0) {
            int slot = 0;
            uint32_t phase = 0;
            bool alive = true;
            for (int mi = 0; mi < nmat && alive; ++mi) {
                const StepMat *m = p.mats + mi;
                const int j = mi & 3;
                const bool paired = j == 2;
                const int n = paired ? p.inter : p.mat_n[j];
                const int tiles = p.mat_tiles[j], k_stages = p.mat_ks[j], n_rb = p.mat_nrb[j];
                const int r0 = (int)(((unsigned)n * blockIdx.x) / gridDim.x);
                const int rb_rows = tiles * 16;
                const int block_rows = (paired ? tiles / 2 : tiles) * 16;
                const int kps = p.mat_kps[j];
                const uint32_t sub_bytes = (uint32_t)rb_rows * (DS_GS * 16 + DS_GS * 4);
                for (int cs = 0; cs < k_stages && alive; cs += p.kc_stages) {
                    const int ce = min(k_stages, cs + p.kc_stages);
                    for (int rb = 0; rb < n_rb && alive; ++rb) {
                        const int row0 = r0 + rb * block_rows;
                        for (int ks0 = cs; ks0 < ce && alive; ks0 += kps) {
                            alive = mbar_wait(bar_empty + slot * 8, phase ^ 1u, p.status);
                            if (!alive) break;
                            const int nsub = min(kps, ce - ks0);
                            const uint32_t full = bar_full + slot * 8;
                            mbar_expect_tx(full, (uint32_t)nsub * sub_bytes);
                            for (int q = 0; q < nsub; ++q) {
                                const uint32_t st = smem_base + (uint32_t)slot * p.slot_bytes + (uint32_t)q * sub_bytes;
                                const int ks = ks0 + q;
                                if (paired) {
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
    const int qkv_w = (p.n_q + 2 * p.n_kv) * p.d_head, AW = p.n_q * p.d_head;
    const int srow = tid / DSB_TPR, sl = tid % DSB_TPR;   // staging: this thread's batch row, its place in it

    // One matrix for all batch rows; `stage_chunk(k0, klen)` leaves the digit planes of the
    // activations [k0, k0 + klen) of every row in `dig`.
    auto gemv = [&](int mi, float *out, int ld, int store, auto &&stage_chunk) {
        const int j = mi & 3;
        const int tiles = p.mat_tiles[j], k_stages = p.mat_ks[j], kps = p.mat_kps[j];
        const int n_rb = p.mat_nrb[j], kc = p.kc_stages;
        const unsigned n = (j == 2) ? (unsigned)p.inter : (unsigned)p.mat_n[j];
        const int r0 = (int)((n * blockIdx.x) / gridDim.x);
        const int r1 = (int)((n * (blockIdx.x + 1)) / gridDim.x);
        const int block_rows = (store == 2 ? tiles / 2 : tiles) * 16;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int cs = 0; cs < k_stages; cs += kc) {
            const int ce = min(k_stages, cs + kc);
            stage_chunk(cs * (DS_GS * 32), (ce - cs) * (DS_GS * 32));
            for (int rb = 0; rb < n_rb; ++rb) {
                const int row_base = r0 + rb * block_rows;
                const bool last = ce == k_stages;
                if (n_rb > 1) { acc[0] = acc[1] = acc[2] = acc[3] = 0.0f; }
                if (tiles == 1) {
                    dsb_consume_stages<1>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) dsb_finish_rows<1>(red, tiles, row_base, r1, out, ld, store, B, acc);
                } else if (tiles <= 2) {
                    dsb_consume_stages<2>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) dsb_finish_rows<2>(red, tiles, row_base, r1, out, ld, store, B, acc);
                } else if (tiles <= 4) {
                    dsb_consume_stages<4>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) dsb_finish_rows<4>(red, tiles, row_base, r1, out, ld, store, B, acc);
                } else {
                    dsb_consume_stages<8>(p, smem, bar_full, bar_empty, dig, c, tiles, cs, ce, kps, cs, acc, dead);
                    if (last) dsb_finish_rows<8>(red, tiles, row_base, r1, out, ld, store, B, acc);
                }
            }
        }
    };

    // per-launch constants
    const int pos = *p.pos;
    if (tid < p.d_head / 2) {
        const float inv_freq = 1.0f / powf(p.theta, 2.0f * (float)tid / (float)p.d_head);
        sincosf(inv_freq * (float)pos, &rope_cs[2 * tid + 1], &rope_cs[2 * tid]);
    }
    for (int i = tid; i < 2 * p.layers; i += DS_CONSUMERS)
        cache_ptr[i] = (i & 1) ? p.vcache[i >> 1] : p.kcache[i >> 1];
    {
        // rows past the batch: zero planes for every group of a chunk, once per launch
        const QuantLayout q = quant_layout(DSB_ROWS, DS_GS);
        const int groups = p.kc_stages * DS_GS;
        for (int item = tid >> 2; item < groups * (DSB_ROWS - B); item += DS_CONSUMERS / 4)
            quantize_group<true>(nullptr, dig, q, item % groups, B + item / groups, tid & 3, true);
    }
    // x[b] = embedding[token[b]]
    for (int b = 0; b < B; ++b) {
        int tok = p.token[b];
        tok = tok < 0 ? 0 : (tok >= p.vocab ? p.vocab - 1 : tok);
        const int i0 = (int)(((unsigned)H * blockIdx.x) / gridDim.x);
        const int i1 = (int)(((unsigned)H * (blockIdx.x + 1)) / gridDim.x);
        for (int i = i0 + tid; i < i1; i += DS_CONSUMERS) p.x[(size_t)b * H + i] = p.embedding[(size_t)tok * H + i];
    }
    grid_barrier(p, epoch);

    // RMSNorm of every row (hidden <= 2048: a thread's 32 values stay in registers), then planes
    auto stage_normed = [&](const float *gamma) {
        float v[DSB_EPT / 8][8];
        float ss = 0.0f;
        const float *xr = p.x + (size_t)srow * H;
#pragma unroll
        for (int j = 0; j < DSB_EPT / 8; ++j) {
            const int k = (j * (DSB_TPR / 4) + (sl >> 2)) * 32 + 8 * (sl & 3);
            const bool on = srow < B && k < H;
            const float4 a = on ? __ldcg(reinterpret_cast<const float4 *>(xr + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 b4 = on ? __ldcg(reinterpret_cast<const float4 *>(xr + k) + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
            v[j][4] = b4.x; v[j][5] = b4.y; v[j][6] = b4.z; v[j][7] = b4.w;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(v[j][i], v[j][i], ss);
        }
        // sum over the row's two warps
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        cons_sync();
        if (lane == 0) misc[warp] = ss;
        cons_sync();
        const float total = misc[2 * srow] + misc[2 * srow + 1];
        const float inv = 1.0f / sqrtf(total / (float)H + p.eps);
#pragma unroll
        for (int j = 0; j < DSB_EPT / 8; ++j) {
            const int k = (j * (DSB_TPR / 4) + (sl >> 2)) * 32 + 8 * (sl & 3);
            if (k < H) {
                const float4 g0 = __ldg(reinterpret_cast<const float4 *>(gamma + k));
                const float4 g1 = __ldg(reinterpret_cast<const float4 *>(gamma + k) + 1);
                v[j][0] = (v[j][0] * inv) * g0.x; v[j][1] = (v[j][1] * inv) * g0.y;
                v[j][2] = (v[j][2] * inv) * g0.z; v[j][3] = (v[j][3] * inv) * g0.w;
                v[j][4] = (v[j][4] * inv) * g1.x; v[j][5] = (v[j][5] * inv) * g1.y;
                v[j][6] = (v[j][6] * inv) * g1.z; v[j][7] = (v[j][7] * inv) * g1.w;
            }
        }
        dsb_quantize_rows(v, dig, H, B);
    };
    // merge of the attention splits of every row (at most 4 chunks per head), then planes
    auto stage_attention = [&]() {
        float v[DSB_EPT / 8][8];
        const int d = p.d_head, S = p.splits;
        const float *ab = p.attn + (size_t)srow * p.n_q * S * (d + 2);
#pragma unroll
        for (int j = 0; j < DSB_EPT / 8; ++j) {
            const int k = (j * (DSB_TPR / 4) + (sl >> 2)) * 32 + 8 * (sl & 3);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = 0.0f;
            if (srow < B && k < AW) {
                const int hh = k / d, dd = k - hh * d;   // 8 consecutive values stay inside one head
                const float *pp = ab + (size_t)hh * S * (d + 2);
                float m[4], w[4], M = -INFINITY, L = 0.0f;
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    m[sp] = sp < S ? __ldcg(pp + (size_t)sp * (d + 2) + d) : -INFINITY;
                    M = fmaxf(M, m[sp]);
                }
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    w[sp] = m[sp] > -INFINITY ? expf(m[sp] - M) : 0.0f;
                    L = fmaf(w[sp], sp < S ? __ldcg(pp + (size_t)sp * (d + 2) + d + 1) : 0.0f, L);
                }
                const float invL = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
                for (int sp = 0; sp < 4; ++sp) {
                    if (sp < S) {
                        const float *ap = pp + (size_t)sp * (d + 2) + dd;   // (rows of d + 2 floats: scalar loads)
                        const float ws = w[sp] * invL;
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[j][i] = fmaf(ws, __ldcg(ap + i), v[j][i]);
                    }
                }
            }
        }
        dsb_quantize_rows(v, dig, AW, B);
    };
    // the MLP activations [k0, k0 + klen) of every row: silu(gate) * up was formed in the gate/up store
    auto stage_mlp = [&](int k0, int klen) {
        if (k0 > 0) cons_sync();  // every warp is done with the previous chunk's planes
        float v[DSB_EPT / 8][8];
        const float *gr = p.gu + (size_t)srow * I + k0;
#pragma unroll
        for (int j = 0; j < DSB_EPT / 8; ++j) {
            const int k = (j * (DSB_TPR / 4) + (sl >> 2)) * 32 + 8 * (sl & 3);
            const bool on = srow < B && k < klen;
            const float4 a = on ? __ldcg(reinterpret_cast<const float4 *>(gr + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 b4 = on ? __ldcg(reinterpret_cast<const float4 *>(gr + k) + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[j][0] = a.x; v[j][1] = a.y; v[j][2] = a.z; v[j][3] = a.w;
            v[j][4] = b4.x; v[j][5] = b4.y; v[j][6] = b4.z; v[j][7] = b4.w;
        }
        dsb_quantize_rows(v, dig, klen, B);
    };

    // attention work items over the CTAs: (sequence, KV head, key chunk) serving the whole group of
    // query heads, or (sequence, query head, key chunk) where the group shape does not allow that
    const int per_seq = (p.attn_grouped ? p.n_kv : p.n_q) * p.splits;
    const int att_items = B * per_seq;
    for (int l = 0; l < p.layers; ++l) {
        const float *g1 = p.gamma + (size_t)(2 * l) * H, *g2 = g1 + H;
        gemv(4 * l + 0, p.qkv, qkv_w, 0, [&](int, int) { stage_normed(g1); });
        grid_barrier(p, epoch);
        // RoPE, cache append, attention
        for (int it = blockIdx.x; it < att_items; it += gridDim.x) {
            const int b = it / per_seq, hs = it - b * per_seq;
            const size_t cache_off = (size_t)b * p.max_seq * p.n_kv * p.d_head;
            const float *qkv_b = p.qkv + (size_t)b * qkv_w;
            float *attn_b = p.attn + (size_t)b * p.n_q * p.splits * (p.d_head + 2);
            if (p.attn_grouped)
                attention_group(p, hs / p.splits, hs % p.splits, pos, cache_ptr[2 * l] + cache_off,
                                cache_ptr[2 * l + 1] + cache_off, rope_cs, act_s, qkv_b, attn_b);
            else
                attention_head<4>(p, l, hs / p.splits, hs % p.splits, pos, cache_ptr[2 * l] + cache_off,
                                  cache_ptr[2 * l + 1] + cache_off, rope_cs, act_s, misc, qkv_b, attn_b);
        }
        grid_barrier(p, epoch);
        gemv(4 * l + 1, p.x, H, 1, [&](int, int) { stage_attention(); });
        grid_barrier(p, epoch);
        gemv(4 * l + 2, p.gu, I, 2, [&](int, int) { stage_normed(g2); });
        grid_barrier(p, epoch);
        gemv(4 * l + 3, p.x, H, 1, stage_mlp);
        grid_barrier(p, epoch);
    }

    // ---- optional tail: final norm of every row, LM head, one greedy token per row ----
    if (p.tail) {
        // the normalised rows [B][H] take the digit area and the scratch behind it
        float *xn = reinterpret_cast<float *>(dig);
        {
            float ss = 0.0f;
            const float *xr = p.x + (size_t)srow * H;
            if (srow < B)
                for (int i = sl; i < H; i += DSB_TPR) { const float t = __ldcg(xr + i); ss = fmaf(t, t, ss); }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            cons_sync();
            if (lane == 0) misc[warp] = ss;
            cons_sync();
            const float inv = 1.0f / sqrtf((misc[2 * srow] + misc[2 * srow + 1]) / (float)H + p.eps);
            if (srow < B)
                for (int i = sl; i < H; i += DSB_TPR) xn[(size_t)srow * H + i] = (__ldcg(xr + i) * inv) * p.final_gamma[i];
            cons_sync();
        }
        const int v0 = (int)(((unsigned long long)p.vocab * blockIdx.x) / gridDim.x);
        const int v1 = (int)(((unsigned long long)p.vocab * (blockIdx.x + 1)) / gridDim.x);
        float best[DSB_ROWS];
        int besti[DSB_ROWS];
#pragma unroll
        for (int b = 0; b < DSB_ROWS; ++b) { best[b] = -INFINITY; besti[b] = -1; }
        // one warp per vocabulary row; the row's weights are read once for all batch rows; per
        // (row, batch row) the same summation order as f32_matmul_kernel
        for (int row = v0 + warp; row < v1; row += DS_CONSUMER_WARPS) {
            const float4 *wr = reinterpret_cast<const float4 *>(p.lm_head + (size_t)row * H);
            float acc[DSB_ROWS];
#pragma unroll
            for (int b = 0; b < DSB_ROWS; ++b) acc[b] = 0.0f;
#pragma unroll 4
            for (int cidx = lane; cidx < H / 4; cidx += 32) {
                const float4 wv = __ldg(wr + cidx);
#pragma unroll
                for (int b = 0; b < DSB_ROWS; ++b) {
                    if (b < B) {
                        const float4 xv = reinterpret_cast<const float4 *>(xn + (size_t)b * H)[cidx];
                        acc[b] = fmaf(wv.x, xv.x, acc[b]);
                        acc[b] = fmaf(wv.y, xv.y, acc[b]);
                        acc[b] = fmaf(wv.z, xv.z, acc[b]);
                        acc[b] = fmaf(wv.w, xv.w, acc[b]);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < DSB_ROWS; ++b) {
                if (b < B) {
                    float a = acc[b];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                    if (lane == 0) p.logits[(size_t)b * p.vocab + row] = a;
                    if (besti[b] < 0 || !(a < best[b])) { best[b] = a; besti[b] = row; }  // later index wins ties
                }
            }
        }
        // CTA maxima per batch row: (value, index) pairs through shared memory
        float *bv = act_s;                                          // [rows][warps]
        int *bi = reinterpret_cast<int *>(act_s + DSB_ROWS * DS_CONSUMER_WARPS);
        cons_sync();
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < DSB_ROWS; ++b) { bv[b * DS_CONSUMER_WARPS + warp] = best[b]; bi[b * DS_CONSUMER_WARPS + warp] = besti[b]; }
        }
        cons_sync();
        if (tid < B) {
            float bb = -INFINITY;
            int ib = -1;
            for (int i = 0; i < DS_CONSUMER_WARPS; ++i) {
                const float v = bv[tid * DS_CONSUMER_WARPS + i];
                const int iv = bi[tid * DS_CONSUMER_WARPS + i];
                if (iv >= 0 && (ib < 0 || v > bb || (v == bb && iv > ib))) { bb = v; ib = iv; }
            }
            p.best_val[(size_t)tid * gridDim.x + blockIdx.x] = bb;
            p.best_idx[(size_t)tid * gridDim.x + blockIdx.x] = ib;
        }
        grid_barrier(p, epoch);
        if ((int)blockIdx.x < B && warp == 0) {
            const int b = blockIdx.x;
            float bb = -INFINITY;
            int ib = -1;
            for (int i = lane; i < (int)gridDim.x; i += 32) {
                const float v = __ldcg(p.best_val + (size_t)b * gridDim.x + i);
                const int iv = __ldcg(p.best_idx + (size_t)b * gridDim.x + i);
                if (iv >= 0 && (ib < 0 || v > bb || (v == bb && iv > ib))) { bb = v; ib = iv; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float v = __shfl_xor_sync(0xffffffffu, bb, o);
                const int iv = __shfl_xor_sync(0xffffffffu, ib, o);
                if (iv >= 0 && (ib < 0 || v > bb || (v == bb && iv > ib))) { bb = v; ib = iv; }
            }
            if (lane == 0) {
                p.token_out[b] = ib < 0 ? 0 : ib;
                if (b == 0) *p.pos_out = pos + 1;
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
            __threadfence();
        }
    }
}
