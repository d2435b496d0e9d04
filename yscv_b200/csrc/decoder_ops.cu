// The fp32 operators that sit between the quantized linears of a Llama-shape
// decoder step: embedding gather, RMSNorm (with the residual add fused in front),
// rotate-half RoPE fused with the KV-cache append, GQA attention over the cache,
// SwiGLU, the fp32 LM-head matmul and the greedy argmax.
//
// Semantics follow the reference's CPU operators
//   RMSNorm   crates/yscv-kernels/src/ops/norm.rs:1497-1518
//   RoPE      crates/yscv-kernels/src/ops/rope.rs:24-117 (rotate-half, pairs (i, i+d/2))
//   GQA       crates/yscv-onnx/src/runner/linear.rs:552-646 (kv head = q head / group,
//             max-subtracted softmax; causality is added here because the exported
//             graphs the reference runs carry it in their mask)
//   SiLU      crates/yscv-kernels/src/ops/simd/activation.rs:1000-1005
//   embedding crates/yscv-kernels/src/ops/embedding.rs:12
//   argmax    apps/llm-bench/src/main.rs:538-543 (LAST index among equal maxima)
//   KV cache  crates/yscv-onnx/src/runner/kv_cache.rs:118-254 (f32 storage)
// All of them are bandwidth-trivial next to the weight streams; they exist so that a
// whole decode step stays on the device and can be replayed as one CUDA graph: the
// sequence position and the token ids are read from device memory, never passed as
// kernel arguments.
#include <cuda_fp16.h>

#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.cuh"

namespace yscv {

__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float block_max(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[w] = v;
    __syncthreads();
    float t = -INFINITY;
    for (int i = 0; i < nw; ++i) t = fmaxf(t, red[i]);
    return t;
}

__global__ void embedding_kernel(const float *__restrict__ w, const int32_t *__restrict__ tokens,
                                 float *__restrict__ out, int vocab, int dim) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    int tok = tokens[row];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const float4 *src = reinterpret_cast<const float4 *>(w + (size_t)tok * dim);
    float4 *dst = reinterpret_cast<float4 *>(out + (size_t)row * dim);
    for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) dst[i] = src[i];
}

// x_out = x + delta (delta may be null); normed = x_out * (1/sqrt(mean(x_out^2)+eps)) * gamma
__global__ void __launch_bounds__(256)
add_rms_norm_kernel(const float *x, const float *__restrict__ delta,
                    const float *__restrict__ gamma, float eps, int hidden,
                    float *x_out, float *__restrict__ normed) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = x[base + i];
        if (delta) v += delta[base + i];
        if (x_out) x_out[base + i] = v;
        ss = fmaf(v, v, ss);
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    // x_out may alias x (in-place residual update): read the sum back instead of adding twice;
    // every thread re-reads exactly the elements it wrote
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v;
        if (x_out) {
            v = x_out[base + i];
        } else {
            v = x[base + i];
            if (delta) v += delta[base + i];
        }
        normed[base + i] = (v * inv) * gamma[i];
    }
}

// Eight fp32 values -> bf16 in the order the packed-int4 prefill GEMM consumes its activations:
// k = 0,4,1,5,2,6,3,7 of every group of 8 (what its nibble unpack produces), round to nearest even;
// the same bits as its own activation pre-pass writes.
__device__ __forceinline__ uint4 pack_bf16_gemm_order(const float (&v)[8]) {
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[4]);
    __nv_bfloat162 p1 = __floats2bfloat162_rn(v[1], v[5]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[2], v[6]);
    __nv_bfloat162 p3 = __floats2bfloat162_rn(v[3], v[7]);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t *>(&p0);
    o.y = *reinterpret_cast<uint32_t *>(&p1);
    o.z = *reinterpret_cast<uint32_t *>(&p2);
    o.w = *reinterpret_cast<uint32_t *>(&p3);
    return o;
}

// add_rms_norm_kernel with the normalised rows written as bf16 activations of the next prefill-shaped
// linear (hidden % 8 == 0); the same arithmetic, so the bf16 values equal those the linear's own
// pre-pass would make of the fp32 rows.
__global__ void __launch_bounds__(256)
add_rms_norm_act_kernel(const float *x, const float *__restrict__ delta, const float *__restrict__ gamma, float eps,
                        int hidden, float *x_out, uint4 *__restrict__ normed_act) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red[8];
    const size_t base = (size_t)blockIdx.x * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = x[base + i];
        if (delta) v += delta[base + i];
        if (x_out) x_out[base + i] = v;
        ss = fmaf(v, v, ss);
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)hidden + eps);
    if (x_out) __syncthreads();   // the second pass reads elements other threads wrote
    for (int g8 = threadIdx.x; g8 < hidden / 8; g8 += blockDim.x) {
        float n[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int i = g8 * 8 + j;
            float v;
            if (x_out) {
                v = x_out[base + i];
            } else {
                v = x[base + i];
                if (delta) v += delta[base + i];
            }
            n[j] = (v * inv) * gamma[i];
        }
        normed_act[base / 8 + g8] = pack_bf16_gemm_order(n);
    }
}

// swiglu_kernel with the result written as bf16 activations of the next prefill-shaped linear (inter % 8 == 0)
__global__ void swiglu_act_kernel(const float *__restrict__ gu, uint4 *__restrict__ out_act, size_t rows, int inter) {
    pdl_wait();
    pdl_trigger();
    const size_t total8 = rows * (size_t)(inter / 8);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total8; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / (inter / 8);
        const int c = (int)(i % (inter / 8)) * 8;
        float n[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float g = gu[r * 2 * inter + c + j], u = gu[r * 2 * inter + inter + c + j];
            const float sg = 1.0f / (1.0f + expf(-g));
            n[j] = (g * sg) * u;
        }
        out_act[i] = pack_bf16_gemm_order(n);
    }
}

// Element access to a KV cache row: f32 storage, or per-row symmetric int8 with one f32
// scale per row (KvDtype::I8 of crates/yscv-onnx/src/runner/kv_cache.rs:8-90; a row is one
// token's n_kv*d values of one layer). Reads dequantise on the fly: (float)q * scale.
template <typename KV>
__device__ __forceinline__ float kv_get(const KV *row, int i, float scale);
template <>
__device__ __forceinline__ float kv_get<float>(const float *row, int i, float) { return row[i]; }
template <>
__device__ __forceinline__ float kv_get<int8_t>(const int8_t *row, int i, float scale) {
    return __fmul_rn((float)row[i], scale);
}

// LayerStorage::append for KvDtype::I8 (kv_cache.rs:44-60) on one row held in `src` (global or
// shared memory): scale = abs_max / 127 (1.0 when abs_max <= f32::EPSILON), inv = 1 / scale,
// q = clamp(round_half_away(v * inv), -127, 127). Every thread of the block calls it.
__device__ __forceinline__ void kv_quantize_row(const float *src, int len, int8_t *dst, float *scale_out,
                                                float *red) {
    float amax = 0.0f;
    for (int i = threadIdx.x; i < len; i += blockDim.x) amax = fmaxf(amax, fabsf(src[i]));
    amax = block_max(amax, red);
    const float scale = (amax <= 1.1920929e-07f) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float inv = __fdiv_rn(1.0f, scale);
    if (threadIdx.x == 0) *scale_out = scale;
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
        const float x = __fmul_rn(src[i], inv);
        // NaN -> 0, as Rust's saturating float-to-int cast does
        dst[i] = (x != x) ? (int8_t)0 : (int8_t)(int)fminf(fmaxf(roundf(x), -127.0f), 127.0f);
    }
    __syncthreads();  // `red` and `src` may be reused by the caller
}

// qkv rows: [q (n_q*d) | k (n_kv*d) | v (n_kv*d)], row r = b*seq + s at position *pos + s.
// Rotates q in place, writes rotated k and v into the cache at [b][position][head][d]
// (f32), or quantised per row with their scales at [b][position] (int8). A position outside
// [0, max_seq) appends nothing and raises YSCV_DEV_POS_OVERFLOW in the status word.
// Dynamic shared memory: d floats of rotary factors (+ n_kv*d floats of rotated keys, int8).
template <typename KV>
__global__ void rope_kv_append_kernel(float *__restrict__ qkv, int seq, int n_q, int n_kv, int d,
                                      float theta, const int32_t *__restrict__ pos,
                                      KV *__restrict__ kc, KV *__restrict__ vc,
                                      float *__restrict__ kscale, float *__restrict__ vscale,
                                      int max_seq, int *__restrict__ status) {
    pdl_wait();
    pdl_trigger();
    constexpr bool I8 = sizeof(KV) == 1;
    extern __shared__ float rsm[];
    __shared__ float red[8];
    const int half = d / 2;
    float *cs_tab = rsm, *sn_tab = rsm + half, *krow = rsm + d;
    const int row = blockIdx.x, b = row / seq, s = row % seq;
    const int p = *pos + s;
    const bool in_range = p >= 0 && p < max_seq;
    if (!in_range && threadIdx.x == 0) *status = YSCV_DEV_POS_OVERFLOW;
    const int row_w = (n_q + 2 * n_kv) * d;
    float *r = qkv + (size_t)row * row_w;
    const float fp = (float)p;
    // the angle of pair i is the same for every head: one table per row
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float inv_freq = 1.0f / powf(theta, 2.0f * (float)i / (float)d);
        sincosf(inv_freq * fp, &sn_tab[i], &cs_tab[i]);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < (n_q + n_kv) * half; idx += blockDim.x) {
        const int h = idx / half, i = idx % half;
        const float cs = cs_tab[i], sn = sn_tab[i];
        float *v = r + (size_t)h * d;
        const float x0 = v[i], x1 = v[i + half];
        const float y0 = x0 * cs - x1 * sn, y1 = x0 * sn + x1 * cs;
        if (h < n_q) {
            v[i] = y0;
            v[i + half] = y1;
        } else if constexpr (I8) {
            krow[(h - n_q) * d + i] = y0;
            krow[(h - n_q) * d + i + half] = y1;
        } else if (in_range) {
            float *dst = reinterpret_cast<float *>(kc) + (((size_t)b * max_seq + p) * n_kv + (h - n_q)) * d;
            dst[i] = y0;
            dst[i + half] = y1;
        }
    }
    const float *vsrc = r + (size_t)(n_q + n_kv) * d;
    if constexpr (I8) {
        __syncthreads();
        if (in_range) {  // (uniform across the block)
            const size_t slot = (size_t)b * max_seq + p;
            kv_quantize_row(krow, n_kv * d, reinterpret_cast<int8_t *>(kc) + slot * n_kv * d, kscale + slot, red);
            kv_quantize_row(vsrc, n_kv * d, reinterpret_cast<int8_t *>(vc) + slot * n_kv * d, vscale + slot, red);
        }
    } else if (in_range) {
        float *vdst = reinterpret_cast<float *>(vc) + ((size_t)b * max_seq + p) * n_kv * d;
        for (int i = threadIdx.x; i < n_kv * d; i += blockDim.x) vdst[i] = vsrc[i];
    }
}

// One block per (b, q head, sq). Keys 0 .. *pos + sq (causal) or *pos + seq_q - 1.
template <typename KV>
__global__ void __launch_bounds__(128)
gqa_attention_kernel(const float *__restrict__ q, int q_stride, int seq_q, int n_q, int n_kv, int d,
                     const KV *__restrict__ kc, const KV *__restrict__ vc,
                     const float *__restrict__ kscale, const float *__restrict__ vscale, int max_seq,
                     const int32_t *__restrict__ pos, int causal, float *__restrict__ out) {
    pdl_wait();
    pdl_trigger();
    constexpr bool I8 = sizeof(KV) == 1;
    extern __shared__ float sm[];
    float *scores = sm;           // max_seq
    float *qs = sm + max_seq;     // d
    __shared__ float red[4];
    const int sq = blockIdx.x, qh = blockIdx.y, b = blockIdx.z;
    const int kv_h = qh / (n_q / n_kv);
    int limit = *pos + (causal ? sq + 1 : seq_q);
    limit = limit > max_seq ? max_seq : (limit < 0 ? 0 : limit);
    const float scale = 1.0f / sqrtf((float)d);
    const float *qrow = q + ((size_t)b * seq_q + sq) * q_stride + (size_t)qh * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) qs[i] = qrow[i];
    __syncthreads();
    const KV *kb = kc + (size_t)b * max_seq * n_kv * d + (size_t)kv_h * d;
    const KV *vb = vc + (size_t)b * max_seq * n_kv * d + (size_t)kv_h * d;
    const float *ksc = I8 ? kscale + (size_t)b * max_seq : nullptr;
    const float *vsc = I8 ? vscale + (size_t)b * max_seq : nullptr;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float mx = -INFINITY;
    // a warp per key: lanes stride over d (coalesced), shuffle-reduce
    for (int sk = warp; sk < limit; sk += 4) {
        const KV *kr = kb + (size_t)sk * n_kv * d;
        const float rs = I8 ? ksc[sk] : 1.0f;
        float dot = 0.0f;
        for (int i = lane; i < d; i += 32) dot = fmaf(qs[i], kv_get<KV>(kr, i, rs), dot);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float sc = dot * scale;
        if (lane == 0) scores[sk] = sc;
        mx = fmaxf(mx, sc);
    }
    mx = block_max(mx, red);
    float se = 0.0f;
    for (int sk = threadIdx.x; sk < limit; sk += blockDim.x) {
        const float e = expf(scores[sk] - mx);
        scores[sk] = e;
        se += e;
    }
    se = block_sum(se, red);
    const float inv = se > 0.0f ? 1.0f / se : 0.0f;
    float *orow = out + ((size_t)b * seq_q + sq) * (size_t)n_q * d + (size_t)qh * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.0f;
        for (int sk = 0; sk < limit; ++sk)
            acc = fmaf(scores[sk] * inv, kv_get<KV>(vb + (size_t)sk * n_kv * d, i, I8 ? vsc[sk] : 1.0f), acc);
        orow[i] = acc;
    }
}

// Prompt-pass attention (many query positions per sequence): the kernel above reads every key and
// value row of a sequence once per (query position, query head), from L2: 137 GB per layer for a
// 2048-token prompt at the 70B shape. Here a block takes QB consecutive query positions x all the
// query heads of ONE KV head, 64 (position, head) pairs, four per warp, and walks the keys in chunks
// of 64 rows staged in shared memory (dequantised on the way in for int8 caches), so a row is read
// from L2 once per block. Scores: a lane per key (its row read 16 bytes at a time, the four query
// rows broadcast from shared memory: every key value read feeds four FMAs). Weighted value sum: a
// lane owns four consecutive elements of the head (with D = 64 the half warps take alternate keys),
// every value read again feeds four FMAs. Each pair keeps a running maximum, exp-sum and
// unnormalised output (the usual max-rescaling of a chunked softmax).
// D = head size (64 or 128); dynamic shared memory: keys [64][D + 4], values [64][D], weights
// [pairs][64], query rows [pairs][D].
constexpr int PF_KT = 64;      // keys per chunk
constexpr int PF_QH = 4;       // (position, head) pairs per warp
template <typename KV, int D>
__global__ void __launch_bounds__(512, 1)
gqa_prefill_tiled_kernel(const float *__restrict__ q, int q_stride, int seq_q, int n_q, int n_kv,
                         const KV *__restrict__ kc, const KV *__restrict__ vc,
                         const float *__restrict__ kscale, const float *__restrict__ vscale, int max_seq,
                         const int32_t *__restrict__ pos, int causal, float *__restrict__ out, int QB) {
    pdl_wait();
    pdl_trigger();
    constexpr bool I8 = sizeof(KV) == 1;
    constexpr int KP = D + 4;   // key row pitch: a lane per key reads its row 16 bytes at a time without bank conflicts
    constexpr int KPAR = 32 / (D / 4);
    extern __shared__ __align__(16) float pf_sm[];
    const int n_pairs = (blockDim.x >> 5) * PF_QH;
    float *ks = pf_sm, *vs = pf_sm + PF_KT * KP, *sc_all = vs + PF_KT * D;
    float *qs_all = sc_all + n_pairs * PF_KT;
    const int G = n_q / n_kv;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kv_h = blockIdx.y, b = blockIdx.z;
    const int p0 = *pos;
    auto limit_of = [&](int s) {
        const int l = p0 + (causal ? s + 1 : seq_q);
        return l > max_seq ? max_seq : (l < 0 ? 0 : l);
    };
    // this warp's pairs: index warp * 4 + j -> head idx % G of the group, position idx / G of the tile
    int sq[PF_QH], qh[PF_QH], lim[PF_QH];
    bool live[PF_QH];
    int warp_limit = 0;
#pragma unroll
    for (int j = 0; j < PF_QH; ++j) {
        const int idx = warp * PF_QH + j;
        sq[j] = blockIdx.x * QB + idx / G;
        qh[j] = kv_h * G + idx % G;
        live[j] = idx < G * QB && sq[j] < seq_q;
        lim[j] = live[j] ? limit_of(sq[j]) : 0;
        warp_limit = max(warp_limit, lim[j]);
    }
    const int last_sq = min(seq_q, ((int)blockIdx.x + 1) * QB) - 1;
    const int block_limit = limit_of(last_sq);   // limits do not decrease with the position
    const float scale = 1.0f / sqrtf((float)D);
    const int e4 = (lane % (D / 4)) * 4, kpar = lane / (D / 4);
    float4 acc[PF_QH];
    float m[PF_QH], l[PF_QH];
    float *sc = sc_all + warp * PF_QH * PF_KT, *qs = qs_all + warp * PF_QH * D;
#pragma unroll
    for (int j = 0; j < PF_QH; ++j) {
        acc[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        m[j] = -INFINITY;
        l[j] = 0.0f;
        for (int i = lane; i < D; i += 32)
            qs[j * D + i] = live[j] ? q[((size_t)b * seq_q + sq[j]) * q_stride + (size_t)qh[j] * D + i] : 0.0f;
    }
    __syncwarp();
    const size_t row_elems = (size_t)n_kv * D;
    const KV *kb = kc + (size_t)b * max_seq * row_elems + (size_t)kv_h * D;
    const KV *vb = vc + (size_t)b * max_seq * row_elems + (size_t)kv_h * D;
    for (int c0 = 0; c0 < block_limit; c0 += PF_KT) {
        const int rows = min(PF_KT, block_limit - c0);
        // stage the chunk: 4 values per thread and step
        for (int idx = threadIdx.x; idx < rows * (D / 4); idx += blockDim.x) {
            const int r = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
            const size_t off = (size_t)(c0 + r) * row_elems + c4;
            float4 kv4, vv4;
            if constexpr (I8) {
                const float rk = kscale[(size_t)b * max_seq + c0 + r], rv = vscale[(size_t)b * max_seq + c0 + r];
                const char4 k4 = *reinterpret_cast<const char4 *>(kb + off), v4 = *reinterpret_cast<const char4 *>(vb + off);
                kv4 = make_float4(__fmul_rn((float)k4.x, rk), __fmul_rn((float)k4.y, rk), __fmul_rn((float)k4.z, rk), __fmul_rn((float)k4.w, rk));
                vv4 = make_float4(__fmul_rn((float)v4.x, rv), __fmul_rn((float)v4.y, rv), __fmul_rn((float)v4.z, rv), __fmul_rn((float)v4.w, rv));
            } else {
                kv4 = *reinterpret_cast<const float4 *>(kb + off);
                vv4 = *reinterpret_cast<const float4 *>(vb + off);
            }
            *reinterpret_cast<float4 *>(ks + r * KP + c4) = kv4;
            *reinterpret_cast<float4 *>(vs + r * D + c4) = vv4;
        }
        __syncthreads();
        const int nkw = min(rows, warp_limit - c0);   // keys of this chunk any of the warp's pairs attends to
        if (nkw > 0) {
            // scores: a lane per key (keys lane and lane + 32 of the chunk); a query piece read once for both keys
            float sv[2][PF_QH];
            {
                float dot[2][PF_QH];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < PF_QH; ++j) dot[h][j] = 0.0f;
                const float4 *kr0 = reinterpret_cast<const float4 *>(ks + lane * KP);
                const float4 *kr1 = reinterpret_cast<const float4 *>(ks + (lane + 32) * KP);
                if (nkw > 32) {   // the same for the whole warp
#pragma unroll 2
                    for (int i = 0; i < D / 4; ++i) {
                        const float4 k0 = kr0[i], k1 = kr1[i];
#pragma unroll
                        for (int j = 0; j < PF_QH; ++j) {
                            const float4 a = reinterpret_cast<const float4 *>(qs + j * D)[i];
                            dot[0][j] = fmaf(a.x, k0.x, dot[0][j]);
                            dot[0][j] = fmaf(a.y, k0.y, dot[0][j]);
                            dot[0][j] = fmaf(a.z, k0.z, dot[0][j]);
                            dot[0][j] = fmaf(a.w, k0.w, dot[0][j]);
                            dot[1][j] = fmaf(a.x, k1.x, dot[1][j]);
                            dot[1][j] = fmaf(a.y, k1.y, dot[1][j]);
                            dot[1][j] = fmaf(a.z, k1.z, dot[1][j]);
                            dot[1][j] = fmaf(a.w, k1.w, dot[1][j]);
                        }
                    }
                } else {
#pragma unroll 4
                    for (int i = 0; i < D / 4; ++i) {
                        const float4 k0 = kr0[i];
#pragma unroll
                        for (int j = 0; j < PF_QH; ++j) {
                            const float4 a = reinterpret_cast<const float4 *>(qs + j * D)[i];
                            dot[0][j] = fmaf(a.x, k0.x, dot[0][j]);
                            dot[0][j] = fmaf(a.y, k0.y, dot[0][j]);
                            dot[0][j] = fmaf(a.z, k0.z, dot[0][j]);
                            dot[0][j] = fmaf(a.w, k0.w, dot[0][j]);
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int k = lane + 32 * h;
#pragma unroll
                    for (int j = 0; j < PF_QH; ++j)
                        sv[h][j] = k < lim[j] - c0 && k < rows ? dot[h][j] * scale : -INFINITY;   // rows past the limit hold stale values
                }
            }
#pragma unroll
            for (int j = 0; j < PF_QH; ++j) {
                float cm = fmaxf(sv[0][j], sv[1][j]);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, o));
                const float m_new = fmaxf(m[j], cm);
                // a pair whose limit lies before this chunk keeps its state (m_new == m, nothing added)
                const float alpha = m_new == -INFINITY ? 1.0f : expf(m[j] - m_new);   // 0 for a pair's first chunk
                float ps = 0.0f;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float e = sv[h][j] == -INFINITY ? 0.0f : expf(sv[h][j] - m_new);
                    sc[j * PF_KT + lane + 32 * h] = e;
                    ps += e;
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
                l[j] = l[j] * alpha + ps;
                acc[j].x *= alpha; acc[j].y *= alpha; acc[j].z *= alpha; acc[j].w *= alpha;
                m[j] = m_new;
            }
            __syncwarp();
            // weighted value sum: the weights of four consecutive keys of a pair come with one 16-byte read
            // (weights past nkw are 0 or belong to rows that are not read)
            for (int k4 = 0; k4 < nkw; k4 += 4 * KPAR) {
                const int kq = k4 + 4 * kpar;   // this half warp's four keys
                float4 pj[PF_QH];
#pragma unroll
                for (int j = 0; j < PF_QH; ++j) pj[j] = *reinterpret_cast<const float4 *>(sc + j * PF_KT + kq);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (kq + u < nkw) {
                        const float4 v4 = *reinterpret_cast<const float4 *>(vs + (kq + u) * D + e4);
#pragma unroll
                        for (int j = 0; j < PF_QH; ++j) {
                            const float pk = u == 0 ? pj[j].x : u == 1 ? pj[j].y : u == 2 ? pj[j].z : pj[j].w;
                            acc[j].x = fmaf(pk, v4.x, acc[j].x);
                            acc[j].y = fmaf(pk, v4.y, acc[j].y);
                            acc[j].z = fmaf(pk, v4.z, acc[j].z);
                            acc[j].w = fmaf(pk, v4.w, acc[j].w);
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < PF_QH; ++j) {
        if constexpr (KPAR == 2) {
            acc[j].x += __shfl_xor_sync(0xffffffffu, acc[j].x, 16);
            acc[j].y += __shfl_xor_sync(0xffffffffu, acc[j].y, 16);
            acc[j].z += __shfl_xor_sync(0xffffffffu, acc[j].z, 16);
            acc[j].w += __shfl_xor_sync(0xffffffffu, acc[j].w, 16);
        }
        if (live[j] && kpar == 0) {
            const float inv = l[j] > 0.0f ? 1.0f / l[j] : 0.0f;
            float *orow = out + ((size_t)b * seq_q + sq[j]) * (size_t)n_q * D + (size_t)qh[j] * D;
            *reinterpret_cast<float4 *>(orow + e4) = make_float4(acc[j].x * inv, acc[j].y * inv, acc[j].z * inv, acc[j].w * inv);
        }
    }
}

// Decode-shaped attention (one query position per sequence) with the keys split across
// blocks so that a long cache fills the machine: block (split, kv head, b) handles keys
// [split*chunk, ...) for ALL the query heads of its KV head's group from one pass over the
// chunk's key and value rows (a row is read once per group, not once per query head), leaves
// per query head an unnormalised partial output, its running max and its exp-sum in `part`;
// attention_combine_kernel merges the splits (the usual max-rescaling of a split softmax).
// Query heads are taken eight at a time. d % 16 == 0, d <= 128, blockDim.x == chunk == 128.
// Dynamic shared memory: q [8][d], weights [8][chunk], partial sums [128 / (d/4)][8][d].
template <typename KV>
__global__ void __launch_bounds__(128)
gqa_decode_split_kernel(const float *__restrict__ q, int q_stride, int n_q, int n_kv, int d,
                        const KV *__restrict__ kc, const KV *__restrict__ vc,
                        const float *__restrict__ kscale, const float *__restrict__ vscale, int max_seq,
                        const int32_t *__restrict__ pos, int chunk, float *__restrict__ part) {
    pdl_wait();
    pdl_trigger();
    constexpr bool I8 = sizeof(KV) == 1;
    constexpr int HB = 8;   // query heads per pass
    extern __shared__ float sm[];
    float *qs = sm;                    // [HB][d]
    float *wts = qs + HB * d;          // [HB][chunk]
    float *psum = wts + HB * chunk;    // [key groups][HB][d]
    __shared__ float red[4];
    const int tid = threadIdx.x;
    const int split = blockIdx.x, kv_h = blockIdx.y, b = blockIdx.z, n_splits = gridDim.x;
    const int grp = n_q / n_kv;
    int limit = *pos + 1;
    limit = limit > max_seq ? max_seq : (limit < 0 ? 0 : limit);
    const int k0 = split * chunk, k1 = min(limit, k0 + chunk);
    const int nk = k1 - k0;
    const float scale = 1.0f / sqrtf((float)d);
    const KV *kb = kc + (size_t)b * max_seq * n_kv * d + (size_t)kv_h * d;
    const KV *vb = vc + (size_t)b * max_seq * n_kv * d + (size_t)kv_h * d;
    const float *ksc = I8 ? kscale + (size_t)b * max_seq : nullptr;
    const float *vsc = I8 ? vscale + (size_t)b * max_seq : nullptr;
    const int quads = d / 4, kgroups = blockDim.x / quads;      // V phase: thread = (key group, 4 dims)
    const int vq = tid % quads, vg = tid / quads;
    for (int h0 = 0; h0 < grp; h0 += HB) {
        const int nh = min(HB, grp - h0);
        const int qh0 = kv_h * grp + h0;
        if (nk <= 0) {  // nothing for this split yet: the neutral element of the merge
            for (int i = tid; i < nh * (d + 2); i += blockDim.x) {
                const int hh = i / (d + 2), j = i - hh * (d + 2);
                part[(((size_t)b * n_q + qh0 + hh) * n_splits + split) * (d + 2) + j] = j == d ? -INFINITY : 0.0f;
            }
            continue;
        }
        __syncthreads();   // the previous pass is done with the shared arrays
        for (int i = tid; i < nh * d; i += blockDim.x)
            qs[i] = q[(size_t)b * q_stride + (size_t)(qh0 + i / d) * d + (i % d)];
        __syncthreads();
        // ---- scores: thread j owns key k0 + j, walks its row once, 16 elements at a time ----
        float dot[HB];
#pragma unroll
        for (int h = 0; h < HB; ++h) dot[h] = 0.0f;
        if (tid < nk) {
            const KV *kr = kb + (size_t)(k0 + tid) * n_kv * d;
            const float rs = I8 ? ksc[k0 + tid] : 1.0f;
            for (int c = 0; c < d; c += 16) {
                float kv[16];
                if constexpr (I8) {
                    const int4 w = __ldg(reinterpret_cast<const int4 *>(kr + c));
                    const int ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int t = 0; t < 16; ++t)
                        kv[t] = __fmul_rn((float)(int8_t)((ww[t >> 2] >> (8 * (t & 3))) & 255), rs);
                } else {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const float4 f = __ldg(reinterpret_cast<const float4 *>(kr + c) + t);
                        kv[4 * t] = f.x; kv[4 * t + 1] = f.y; kv[4 * t + 2] = f.z; kv[4 * t + 3] = f.w;
                    }
                }
#pragma unroll
                for (int h = 0; h < HB; ++h) {
                    if (h < nh) {
                        const float *qh = qs + h * d + c;
#pragma unroll
                        for (int t = 0; t < 16; ++t) dot[h] = fmaf(qh[t], kv[t], dot[h]);
                    }
                }
            }
        }
        // ---- per head: local softmax over the chunk; the weights go to shared memory ----
        for (int h = 0; h < nh; ++h) {
            const float sc = tid < nk ? dot[h] * scale : -INFINITY;
            const float mx = block_max(sc, red);
            float e = tid < nk ? expf(sc - mx) : 0.0f;
            const float se = block_sum(e, red);
            // int8 values: fold the row scale of the value row into its weight once
            if (I8 && tid < nk) e = e * vsc[k0 + tid];
            wts[h * chunk + tid] = e;
            if (tid == 0) {
                float *po = part + (((size_t)b * n_q + qh0 + h) * n_splits + split) * (d + 2);
                po[d] = mx;
                po[d + 1] = se;
            }
        }
        __syncthreads();
        // ---- weighted values: thread (key group vg, dims 4*vq..): a value row quad serves every head ----
        float acc[HB][4];
#pragma unroll
        for (int h = 0; h < HB; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.0f;
        if (vg < kgroups) {
            // four value rows' loads in flight per thread, then the arithmetic
            for (int j0 = vg; j0 < nk; j0 += 4 * kgroups) {
                float v4[4][4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + u * kgroups;
                    const KV *vr = vb + (size_t)(k0 + (j < nk ? j : j0)) * n_kv * d;
                    if constexpr (I8) {
                        const int w = __ldg(reinterpret_cast<const int *>(vr) + vq);
                        v4[u][0] = (float)(int8_t)(w & 255); v4[u][1] = (float)(int8_t)((w >> 8) & 255);
                        v4[u][2] = (float)(int8_t)((w >> 16) & 255); v4[u][3] = (float)(int8_t)((w >> 24) & 255);
                    } else {
                        const float4 f = __ldg(reinterpret_cast<const float4 *>(vr) + vq);
                        v4[u][0] = f.x; v4[u][1] = f.y; v4[u][2] = f.z; v4[u][3] = f.w;
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = j0 + u * kgroups;
                    if (j >= nk) break;
#pragma unroll
                    for (int h = 0; h < HB; ++h) {
                        if (h < nh) {
                            const float w = wts[h * chunk + j];
                            acc[h][0] = fmaf(w, v4[u][0], acc[h][0]);
                            acc[h][1] = fmaf(w, v4[u][1], acc[h][1]);
                            acc[h][2] = fmaf(w, v4[u][2], acc[h][2]);
                            acc[h][3] = fmaf(w, v4[u][3], acc[h][3]);
                        }
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < HB; ++h)
                if (h < nh)
                    *reinterpret_cast<float4 *>(psum + ((size_t)vg * HB + h) * d + 4 * vq) =
                        make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
        }
        __syncthreads();
        for (int i = tid; i < nh * d; i += blockDim.x) {
            const int h = i / d, dd = i - h * d;
            float v = 0.0f;
            for (int g = 0; g < kgroups; ++g) v += psum[((size_t)g * HB + h) * d + dd];
            part[(((size_t)b * n_q + qh0 + h) * n_splits + split) * (d + 2) + dd] = v;
        }
    }
}

// ---- decode attention over an int8 cache on the tensor cores ------------------------------
//
// Same work split and the same `part` records as gqa_decode_split_kernel (one block per key chunk
// of 128, KV head and sequence, eight query heads of the group per pass), but both contractions
// run as mma.sync.m16n8k16 on fp16 operands with fp32 accumulators: an int8 cache entry is exact
// in fp16 (0x6400 | (q ^ 0x80) is 1024 + q + 128, minus 1152), the rotated query and the softmax
// weights are split into two fp16 terms (hi + lo, error below 2^-21 relative), so the result
// differs from the fp32 loop only in summation order.
//   scores^T [16 keys x 8 heads] = K tile [16 keys x d] (A, straight from the staged rows) x
//                                  Q^T [d x 8 heads] (B, two terms)
//   out [8 heads x d]            = P [8 (of 16 rows) x 128 keys] (A, two terms) x V [128 keys x d]
//                                  (B, read from a transposed copy of the chunk's value rows)
// The k order inside an MMA is free as long as both operands agree: a thread takes 4 consecutive
// d (or keys) for the four k slots it owns, so its K bytes are one 16-byte read per 64 d and its V
// bytes one 32-bit read per 16 keys. d is 64 or 128.
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// four int8 -> two fp16 pairs {x0, x1}, {x2, x3}, exact
__device__ __forceinline__ void s8x4_to_h2x2(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t x = w ^ 0x80808080u;
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    uint32_t p0 = __byte_perm(x, 0x64646464u, 0x4140), p1 = __byte_perm(x, 0x64646464u, 0x4342);
    __half2 h0 = __hsub2(*reinterpret_cast<__half2 *>(&p0), bias), h1 = __hsub2(*reinterpret_cast<__half2 *>(&p1), bias);
    lo = *reinterpret_cast<uint32_t *>(&h0);
    hi = *reinterpret_cast<uint32_t *>(&h1);
}
// two floats -> fp16 pair of their leading terms and fp16 pair of the remainders
__device__ __forceinline__ void split_h2(float a, float b, uint32_t &hi, uint32_t &lo) {
    const __half ha = __float2half_rn(a), hb = __float2half_rn(b);
    const __half la = __float2half_rn(a - __half2float(ha)), lb = __float2half_rn(b - __half2float(hb));
    const __half2 h = __halves2half2(ha, hb), l = __halves2half2(la, lb);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

__global__ void __launch_bounds__(128)
gqa_decode_split_tc_kernel(const float *__restrict__ q, int q_stride, int n_q, int n_kv, int d,
                           const int8_t *__restrict__ kc, const int8_t *__restrict__ vc,
                           const float *__restrict__ kscale, const float *__restrict__ vscale, int max_seq,
                           const int32_t *__restrict__ pos, float *__restrict__ part) {
    pdl_wait();
    pdl_trigger();
    constexpr int CH = 128, HB = 8;
    constexpr int SP = CH + 4;            // scores row pitch (floats)
    constexpr int PP = CH + 8;            // weight row pitch (halves)
    extern __shared__ __align__(16) unsigned char tsm[];
    const int kp = d;                     // key row pitch (bytes); for d = 128 the 16-byte piece c of row r sits
    const int ksw = d == 128 ? 4 : 0;     // at piece c ^ ((r & 1) * 4): the eight lanes of a read phase (two
                                          // rows x four pieces) then touch eight different bank groups
    const int vp = CH + 16;               // transposed value row pitch (bytes): conflict-free 32-bit reads
    unsigned char *Ks = tsm;                                         // [CH][d]
    unsigned char *Vt = Ks + CH * kp;                                // [d][CH + 16]
    float *Ssm = reinterpret_cast<float *>(Vt + d * vp);             // [HB][SP]
    __half *Ph = reinterpret_cast<__half *>(Ssm + HB * SP);          // [HB][PP] leading terms
    __half *Pl = Ph + HB * PP;                                       // [HB][PP] remainders
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kv_h = blockIdx.y, b = blockIdx.z, n_splits = gridDim.x;
    const int grp = n_q / n_kv;
    int limit = *pos + 1;
    limit = limit > max_seq ? max_seq : (limit < 0 ? 0 : limit);
    const int k0 = split * CH, k1 = min(limit, k0 + CH);
    const int nk = k1 - k0;
    if (nk <= 0) {  // nothing for this split yet: the neutral element of the merge
        for (int i = tid; i < grp * (d + 2); i += blockDim.x) {
            const int hh = i / (d + 2), j = i - hh * (d + 2);
            part[(((size_t)b * n_q + kv_h * grp + hh) * n_splits + split) * (d + 2) + j] = j == d ? -INFINITY : 0.0f;
        }
        return;
    }
    const float scale = 1.0f / sqrtf((float)d);
    const int8_t *kb = kc + (size_t)b * max_seq * n_kv * d + (size_t)kv_h * d;
    const int8_t *vb = vc + (size_t)b * max_seq * n_kv * d + (size_t)kv_h * d;
    const float *ksc = kscale + (size_t)b * max_seq, *vsc = vscale + (size_t)b * max_seq;

    // ---- stage the chunk: key rows as they are, value rows transposed; rows past nk are zeros ----
    {
        const int pieces = d / 16;        // 16-byte pieces per row
        uint4 kw[8], vw[8];               // every load in flight before the first store
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = tid + u * 128, row = i / pieces, pc = i - row * pieces;
            kw[u] = vw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (u < pieces && row < nk) {
                kw[u] = __ldg(reinterpret_cast<const uint4 *>(kb + (size_t)(k0 + row) * n_kv * d) + pc);
                vw[u] = __ldg(reinterpret_cast<const uint4 *>(vb + (size_t)(k0 + row) * n_kv * d) + pc);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = tid + u * 128, row = i / pieces, pc = i - row * pieces;
            if (u < pieces) {
                *reinterpret_cast<uint4 *>(Ks + row * kp + ((pc ^ ((row & 1) * ksw)) << 4)) = kw[u];
                const uint32_t w[4] = {vw[u].x, vw[u].y, vw[u].z, vw[u].w};
#pragma unroll
                // (value row d keeps key k at byte k ^ ((d >> 4) << 2): the eight lanes that hold the
                // eight pieces of one key row then store into eight different banks)
                for (int e = 0; e < 16; ++e)
                    Vt[(pc * 16 + e) * vp + (row ^ (pc << 2))] = (unsigned char)(w[e >> 2] >> (8 * (e & 3)));
            }
        }
    }
    __syncthreads();

    for (int h0 = 0; h0 < grp; h0 += HB) {
        const int nh = min(HB, grp - h0);
        const int qh0 = kv_h * grp + h0;
        // ---- this thread's query operands: head g, for the k step (64-block B, quarter s4) the
        // four d = 64 B + 16 t + 4 s4 .. + 3, as leading terms and remainders ----
        uint32_t qh[8][2], ql[8][2];      // [k step][b0, b1]
        {
            const float *qr = q + (size_t)b * q_stride + (size_t)(qh0 + (g < nh ? g : 0)) * d;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (ks * 16 < d && g < nh) v = __ldg(reinterpret_cast<const float4 *>(qr + (ks >> 2) * 64 + 16 * t + 4 * (ks & 3)));
                split_h2(v.x, v.y, qh[ks][0], ql[ks][0]);
                split_h2(v.z, v.w, qh[ks][1], ql[ks][1]);
            }
        }
        // ---- scores^T: warp w takes keys 32 w .. 32 w + 31 as two tiles of 16 ----
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const int keyA = warp * 32 + mt * 16 + g, keyB = keyA + 8;
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                if (blk * 64 < d) {
                    // (keyA and keyB = keyA + 8 have the same parity, hence the same swizzle)
                    const int pc = (blk * 4 + t) ^ ((keyA & 1) * ksw);
                    const uint4 wa = *reinterpret_cast<const uint4 *>(Ks + keyA * kp + (pc << 4));
                    const uint4 wb = *reinterpret_cast<const uint4 *>(Ks + keyB * kp + (pc << 4));
                    const uint32_t xa[4] = {wa.x, wa.y, wa.z, wa.w}, xb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                    for (int s4 = 0; s4 < 4; ++s4) {
                        uint32_t a0, a2, a1, a3;
                        s8x4_to_h2x2(xa[s4], a0, a2);
                        s8x4_to_h2x2(xb[s4], a1, a3);
                        const int ks = blk * 4 + s4;
                        mma_f16(c, a0, a1, a2, a3, ql[ks][0], ql[ks][1]);
                        mma_f16(c, a0, a1, a2, a3, qh[ks][0], qh[ks][1]);
                    }
                }
            }
            // c0, c1 = (keyA, heads 2t, 2t+1); c2, c3 = (keyB, same heads)
            const float sa = keyA < nk ? __ldg(ksc + k0 + keyA) * scale : 0.0f;
            const float sb = keyB < nk ? __ldg(ksc + k0 + keyB) * scale : 0.0f;
            Ssm[(2 * t) * SP + keyA] = keyA < nk ? c[0] * sa : -INFINITY;
            Ssm[(2 * t + 1) * SP + keyA] = keyA < nk ? c[1] * sa : -INFINITY;
            Ssm[(2 * t) * SP + keyB] = keyB < nk ? c[2] * sb : -INFINITY;
            Ssm[(2 * t + 1) * SP + keyB] = keyB < nk ? c[3] * sb : -INFINITY;
        }
        __syncthreads();
        // ---- softmax over the chunk: warp w takes heads 2 w and 2 w + 1, a lane four keys ----
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int h = 2 * warp + hh;
            const float4 sv = *reinterpret_cast<const float4 *>(Ssm + h * SP + 4 * lane);
            float mx = fmaxf(fmaxf(sv.x, sv.y), fmaxf(sv.z, sv.w));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const int key = 4 * lane;
            float e[4] = {sv.x, sv.y, sv.z, sv.w};
            float se = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                e[i] = (key + i < nk && h < nh) ? expf(e[i] - mx) : 0.0f;
                se += e[i];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
            if (lane == 0 && h < nh) {
                float *po = part + (((size_t)b * n_q + qh0 + h) * n_splits + split) * (d + 2);
                po[d] = mx;
                po[d + 1] = se;
            }
            // the value row's scale is folded into its weight; two fp16 terms per weight
            uint32_t hi01, lo01, hi23, lo23;
            const float4 vs = key < nk ? make_float4(__ldg(vsc + k0 + min(key, nk - 1)), __ldg(vsc + k0 + min(key + 1, nk - 1)),
                                                     __ldg(vsc + k0 + min(key + 2, nk - 1)), __ldg(vsc + k0 + min(key + 3, nk - 1)))
                                       : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            split_h2(e[0] * vs.x, e[1] * vs.y, hi01, lo01);
            split_h2(e[2] * vs.z, e[3] * vs.w, hi23, lo23);
            *reinterpret_cast<uint2 *>(Ph + h * PP + key) = make_uint2(hi01, hi23);
            *reinterpret_cast<uint2 *>(Pl + h * PP + key) = make_uint2(lo01, lo23);
        }
        __syncthreads();
        // ---- out = P x V: warp w takes d / 32 column tiles of 8; rows 8..15 of P are zero ----
        const int ntw = d / 32;           // column tiles per warp (2 or 4)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j < ntw) {
                const int col = (warp * ntw + j) * 8 + g;     // this thread's B column (a d index)
                float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int ks = 0; ks < CH / 16; ++ks) {
                    const int key0 = ks * 16 + 4 * t;
                    const uint2 ah = *reinterpret_cast<const uint2 *>(Ph + g * PP + key0);
                    const uint2 al = *reinterpret_cast<const uint2 *>(Pl + g * PP + key0);
                    uint32_t b0, b1;
                    s8x4_to_h2x2(*reinterpret_cast<const uint32_t *>(Vt + col * vp + (key0 ^ ((col >> 4) << 2))), b0, b1);
                    mma_f16(o, al.x, 0u, al.y, 0u, b0, b1);
                    mma_f16(o, ah.x, 0u, ah.y, 0u, b0, b1);
                }
                // o0, o1 = (head g, d = tile * 8 + 2t, + 1)
                if (g < nh) {
                    float *po = part + (((size_t)b * n_q + qh0 + g) * n_splits + split) * (d + 2) + (warp * ntw + j) * 8 + 2 * t;
                    po[0] = o[0];
                    po[1] = o[1];
                }
            }
        }
        __syncthreads();   // the score and weight arrays are reused by the next pass
    }
}

__global__ void attention_combine_kernel(const float *__restrict__ part, int n_splits, int d,
                                         float *__restrict__ out) {
    pdl_wait();
    pdl_trigger();
    // block per (q head, b); out row [b][n_q*d]
    const size_t hb = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
    const float *p = part + hb * n_splits * (d + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, p[(size_t)s * (d + 2) + d]);
    float L = 0.0f;
    for (int s = 0; s < n_splits; ++s) {
        const float m = p[(size_t)s * (d + 2) + d];
        if (m > -INFINITY) L += expf(m - M) * p[(size_t)s * (d + 2) + d + 1];
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < n_splits; ++s) {
            const float m = p[(size_t)s * (d + 2) + d];
            if (m > -INFINITY) acc = fmaf(expf(m - M), p[(size_t)s * (d + 2) + i], acc);
        }
        out[hb * d + i] = acc * inv;
    }
}

// gate_up rows: [gate (inter) | up (inter)] -> out = silu(gate) * up
__global__ void swiglu_kernel(const float *__restrict__ gu, float *__restrict__ out, size_t rows,
                              int inter) {
    pdl_wait();
    pdl_trigger();
    const size_t total = rows * (size_t)inter;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / inter;
        const int c = (int)(i % inter);
        const float g = gu[r * 2 * inter + c], u = gu[r * 2 * inter + inter + c];
        const float s = 1.0f / (1.0f + expf(-g));
        out[i] = (g * s) * u;
    }
}

// out[m][n] = sum_k x[m][k] * w[n][k]; one warp per weight row, up to 4 x rows per pass
template <int MT>
__global__ void __launch_bounds__(256)
f32_matmul_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
                  int m0, int M, int N, int K) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const int mt = min(MT, M - m0);
    for (int n = blockIdx.x * wpb + (threadIdx.x >> 5); n < N; n += gridDim.x * wpb) {
        const float4 *wr = reinterpret_cast<const float4 *>(w + (size_t)n * K);
        float acc[MT];
#pragma unroll
        for (int i = 0; i < MT; ++i) acc[i] = 0.0f;
#pragma unroll 4
        for (int c = lane; c < K / 4; c += 32) {
            const float4 wv = __ldg(wr + c);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                if (i < mt) {
                    const float4 xv = __ldg(reinterpret_cast<const float4 *>(x + (size_t)(m0 + i) * K) + c);
                    acc[i] = fmaf(wv.x, xv.x, acc[i]);
                    acc[i] = fmaf(wv.y, xv.y, acc[i]);
                    acc[i] = fmaf(wv.z, xv.z, acc[i]);
                    acc[i] = fmaf(wv.w, xv.w, acc[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < MT; ++i) {
            float v = acc[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && i < mt) out[(size_t)(m0 + i) * N + n] = v;
        }
    }
}

// The same product for a wide batch (m > 8): a shared-memory tiled SGEMM, 128 weight rows x 64
// activation rows per block, K walked 32 at a time, every thread an 8 x 4 block of outputs.
// The weights are read once from HBM per 64 activation rows.
constexpr int FM_BN = 128, FM_BM = 64, FM_BK = 32;
__global__ void __launch_bounds__(256)
f32_matmul_tiled_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
                        int M, int N, int K) {
    pdl_wait();
    pdl_trigger();
    __shared__ float ws[FM_BK][FM_BN + 4];
    __shared__ float xs[FM_BK][FM_BM + 4];
    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * FM_BN, m0 = blockIdx.y * FM_BM;
    const int tn = tid % 16, tm = tid / 16;      // outputs n0 + tn*8 .. +7, m0 + tm*4 .. +3
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += FM_BK) {
        // stage the tiles transposed: [k][row]; rows / k past the edge are zero
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256, r = idx / 8, c = (idx % 8) * 4;   // 128 rows x 8 float4
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (n0 + r < N && k0 + c < K) v = __ldg(reinterpret_cast<const float4 *>(w + (size_t)(n0 + r) * K + k0 + c));
            ws[c][r] = v.x; ws[c + 1][r] = v.y; ws[c + 2][r] = v.z; ws[c + 3][r] = v.w;
        }
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = tid + it * 256, r = idx / 8, c = (idx % 8) * 4;   // 64 rows x 8 float4
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (m0 + r < M && k0 + c < K) v = __ldg(reinterpret_cast<const float4 *>(x + (size_t)(m0 + r) * K + k0 + c));
            xs[c][r] = v.x; xs[c + 1][r] = v.y; xs[c + 2][r] = v.z; xs[c + 3][r] = v.w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < FM_BK; ++kk) {
            const float4 wa = *reinterpret_cast<const float4 *>(&ws[kk][tn * 8]);
            const float4 wb = *reinterpret_cast<const float4 *>(&ws[kk][tn * 8 + 4]);
            const float4 xa = *reinterpret_cast<const float4 *>(&xs[kk][tm * 4]);
            const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
            const float xv[4] = {xa.x, xa.y, xa.z, xa.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int n = n0 + tn * 8 + j;
            if (n < N) out[(size_t)m * N + n] = acc[i][j];
        }
    }
}

// greedy token per row: the LAST index among equal maxima (Iterator::max_by)
__global__ void __launch_bounds__(256)
argmax_last_kernel(const float *__restrict__ logits, int vocab, int32_t *__restrict__ out) {
    pdl_wait();
    pdl_trigger();
    __shared__ float bv[256];
    __shared__ int bi[256];
    const float *row = logits + (size_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int idx = -1;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (idx < 0 || !(v < best)) {  // v >= best (or NaN): later index wins ties
            best = v;
            idx = i;
        }
    }
    bv[threadIdx.x] = best;
    bi[threadIdx.x] = idx;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float a = bv[threadIdx.x], b = bv[threadIdx.x + s];
            const int ia = bi[threadIdx.x], ib = bi[threadIdx.x + s];
            const bool take_b = ib >= 0 && (ia < 0 || b > a || (b == a && ib > ia));
            if (take_b) {
                bv[threadIdx.x] = b;
                bi[threadIdx.x] = ib;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[blockIdx.x] = bi[0] < 0 ? 0 : bi[0];
}

// two-stage variant for wide vocabularies: 64 blocks per row leave (value, index) partials,
// the single-block kernel above then reduces those (indices carried along)
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float *__restrict__ logits, int vocab, float *__restrict__ pv,
                      int32_t *__restrict__ pi) {
    pdl_wait();
    pdl_trigger();
    __shared__ float bv[256];
    __shared__ int bi[256];
    const int row = blockIdx.y, nb = gridDim.x;
    const int per = (vocab + nb - 1) / nb;
    const int lo = blockIdx.x * per, hi = min(vocab, lo + per);
    const float *r = logits + (size_t)row * vocab;
    float best = -INFINITY;
    int idx = -1;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = r[i];
        if (idx < 0 || !(v < best)) { best = v; idx = i; }
    }
    bv[threadIdx.x] = best;
    bi[threadIdx.x] = idx;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float a = bv[threadIdx.x], b = bv[threadIdx.x + s];
            const int ia = bi[threadIdx.x], ib = bi[threadIdx.x + s];
            if (ib >= 0 && (ia < 0 || b > a || (b == a && ib > ia))) { bv[threadIdx.x] = b; bi[threadIdx.x] = ib; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) { pv[row * nb + blockIdx.x] = bv[0]; pi[row * nb + blockIdx.x] = bi[0]; }
}

__global__ void __launch_bounds__(64)
argmax_final_kernel(const float *__restrict__ pv, const int32_t *__restrict__ pi, int nb,
                    int32_t *__restrict__ out) {
    pdl_wait();
    pdl_trigger();
    // partials are in increasing index order: scan them in order, later wins ties
    if (threadIdx.x != 0) return;
    const int row = blockIdx.x;
    float best = -INFINITY;
    int idx = -1;
    for (int j = 0; j < nb; ++j) {
        const int i = pi[row * nb + j];
        const float v = pv[row * nb + j];
        if (i >= 0 && (idx < 0 || !(v < best))) { best = v; idx = i; }
    }
    out[row] = idx < 0 ? 0 : idx;
}

__global__ void advance_pos_kernel(int32_t *pos, int by) {
    pdl_wait();  // the predecessor may still read *pos, and its own predecessors must be covered
    pdl_trigger();
    *pos += by;
}

}  // namespace yscv

using namespace yscv;

#define DEC_PROLOGUE(ctx)                                                    \
    if (!(ctx)) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");           \
    YSCV_CUDA_TRY(cudaSetDevice((ctx)->device))
#define DEC_EPILOGUE(ctx, name)                  \
    YSCV_CUDA_TRY(cudaGetLastError());           \
    (ctx)->launches++;                           \
    (ctx)->last_kernel = name;                   \
    return YSCV_CUDA_OK

extern "C" {

int yscv_cuda_embedding_dev(yscv_cuda_ctx *ctx, const float *d_weight, size_t vocab, size_t dim,
                            const int32_t *d_tokens, size_t rows, float *d_out) {
    DEC_PROLOGUE(ctx);
    if (!d_weight || !d_tokens || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (dim % 4 != 0) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "embedding dim must be a multiple of 4");
    if ((reinterpret_cast<uintptr_t>(d_weight) | reinterpret_cast<uintptr_t>(d_out)) & 15)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "embedding table and output must be 16-byte aligned");
    if (rows == 0) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(launch_pdl(embedding_kernel, dim3((unsigned)rows), dim3(128), 0, ctx->stream, d_weight, d_tokens, d_out, (int)vocab, (int)dim));
    DEC_EPILOGUE(ctx, "embedding");
}

int yscv_cuda_add_rms_norm_dev(yscv_cuda_ctx *ctx, const float *d_x, const float *d_delta,
                               const float *d_gamma, float eps, size_t rows, size_t hidden,
                               float *d_x_out, float *d_normed) {
    DEC_PROLOGUE(ctx);
    if (!d_x || !d_gamma || !d_normed) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (rows == 0) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(launch_pdl(add_rms_norm_kernel, dim3((unsigned)rows), dim3(256), 0, ctx->stream, d_x, d_delta, d_gamma, eps, (int)hidden,
                                                                 d_x_out, d_normed));
    DEC_EPILOGUE(ctx, "add_rms_norm");
}

}  // extern "C"

template <typename KV>
static int rope_kv_append_impl(yscv_cuda_ctx *ctx, float *d_qkv, size_t batch, size_t seq, size_t n_q,
                               size_t n_kv, size_t d_head, float theta, const int32_t *d_pos,
                               KV *d_kcache, KV *d_vcache, float *d_kscale, float *d_vscale,
                               size_t max_seq) {
    DEC_PROLOGUE(ctx);
    if (!d_qkv || !d_pos || !d_kcache || !d_vcache) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (sizeof(KV) == 1 && (!d_kscale || !d_vscale)) return fail(YSCV_CUDA_ERR_BAD_ARG, "null scale table");
    if (d_head == 0 || d_head % 2 != 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "d_head must be even for RoPE");
    if (n_kv == 0 || max_seq == 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "n_kv and max_seq must be positive");
    if (batch * seq == 0) return YSCV_CUDA_OK;
    const size_t smem = (d_head + (sizeof(KV) == 1 ? n_kv * d_head : 0)) * sizeof(float);
    if (smem > 48 * 1024)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "RoPE tables for d_head=%zu, n_kv=%zu do not fit shared memory", d_head, n_kv);
    YSCV_CUDA_TRY(launch_pdl(rope_kv_append_kernel<KV>, dim3((unsigned)(batch * seq)), dim3(128), smem, ctx->stream,
                             d_qkv, (int)seq, (int)n_q, (int)n_kv, (int)d_head, theta, d_pos, d_kcache, d_vcache,
                             d_kscale, d_vscale, (int)max_seq, ctx->d_status));
    DEC_EPILOGUE(ctx, sizeof(KV) == 1 ? "rope_kv_append(int8 cache)" : "rope_kv_append");
}

template <typename KV>
static int gqa_attention_impl(yscv_cuda_ctx *ctx, const float *d_q, size_t q_stride, size_t batch,
                              size_t seq_q, size_t n_q, size_t n_kv, size_t d_head, const KV *d_kcache,
                              const KV *d_vcache, const float *d_kscale, const float *d_vscale,
                              size_t max_seq, const int32_t *d_pos, int causal, float *d_out);

extern "C" {

int yscv_cuda_rope_kv_append_dev(yscv_cuda_ctx *ctx, float *d_qkv, size_t batch, size_t seq, size_t n_q,
                                 size_t n_kv, size_t d_head, float theta, const int32_t *d_pos,
                                 float *d_kcache, float *d_vcache, size_t max_seq) {
    return rope_kv_append_impl<float>(ctx, d_qkv, batch, seq, n_q, n_kv, d_head, theta, d_pos, d_kcache, d_vcache,
                                      nullptr, nullptr, max_seq);
}

int yscv_cuda_rope_kv_append_i8_dev(yscv_cuda_ctx *ctx, float *d_qkv, size_t batch, size_t seq, size_t n_q,
                                    size_t n_kv, size_t d_head, float theta, const int32_t *d_pos,
                                    int8_t *d_kcache, float *d_kscale, int8_t *d_vcache, float *d_vscale,
                                    size_t max_seq) {
    return rope_kv_append_impl<int8_t>(ctx, d_qkv, batch, seq, n_q, n_kv, d_head, theta, d_pos, d_kcache, d_vcache,
                                       d_kscale, d_vscale, max_seq);
}

}  // extern "C"

template <typename KV>
static int gqa_attention_impl(yscv_cuda_ctx *ctx, const float *d_q, size_t q_stride, size_t batch,
                              size_t seq_q, size_t n_q, size_t n_kv, size_t d_head, const KV *d_kcache,
                              const KV *d_vcache, const float *d_kscale, const float *d_vscale,
                              size_t max_seq, const int32_t *d_pos, int causal, float *d_out) {
    DEC_PROLOGUE(ctx);
    if (!d_q || !d_kcache || !d_vcache || !d_pos || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (sizeof(KV) == 1 && (!d_kscale || !d_vscale)) return fail(YSCV_CUDA_ERR_BAD_ARG, "null scale table");
    if (n_kv == 0 || n_q % n_kv != 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "n_q must be a multiple of n_kv");
    if (batch * seq_q == 0) return YSCV_CUDA_OK;
    if (seq_q == 1 && causal && max_seq > 128) {
        // decode over a long cache: split the keys across blocks, then merge
        if (d_head % 16 != 0 || d_head > 128)
            return fail(YSCV_CUDA_ERR_UNSUPPORTED, "d_head %zu not supported by the decode attention", d_head);
        // key and value rows are read with 128-bit loads
        if (((reinterpret_cast<uintptr_t>(d_kcache) | reinterpret_cast<uintptr_t>(d_vcache)) & 15) != 0)
            return fail(YSCV_CUDA_ERR_UNSUPPORTED, "the key and value caches must be 16-byte aligned");
        const int chunk = 128;
        const int n_splits = (int)((max_seq + chunk - 1) / chunk);
        const size_t need = batch * n_q * (size_t)n_splits * (d_head + 2) * sizeof(float);
        int rc = ctx->scratch_attn.reserve(need);
        if (rc) return rc;
        float *part = reinterpret_cast<float *>(ctx->scratch_attn.ptr);
        // one block per (key chunk, KV head, sequence): it serves every query head of the group
        dim3 grid((unsigned)n_splits, (unsigned)n_kv, (unsigned)batch);
        const size_t kgroups = 128 / (d_head / 4);
        const size_t split_smem = (8 * d_head + 8 * chunk + kgroups * 8 * d_head) * sizeof(float);
        if constexpr (sizeof(KV) == 1) {
            // int8 caches with head sizes of 64 or 128: both contractions on the tensor cores
            if ((d_head == 64 || d_head == 128) && ctx->attn_tensor_cores) {
                const size_t tc_smem = 128 * d_head + d_head * (128 + 16) + 8 * (128 + 4) * sizeof(float) +
                                       2 * 8 * (128 + 8) * sizeof(uint16_t);
                YSCV_CUDA_TRY(launch_pdl(gqa_decode_split_tc_kernel, dim3(grid), dim3(128), tc_smem, ctx->stream, d_q,
                                         (int)q_stride, (int)n_q, (int)n_kv, (int)d_head,
                                         reinterpret_cast<const int8_t *>(d_kcache), reinterpret_cast<const int8_t *>(d_vcache),
                                         d_kscale, d_vscale, (int)max_seq, d_pos, part));
                YSCV_CUDA_TRY(cudaGetLastError());
                ctx->launches++;
                YSCV_CUDA_TRY(launch_pdl(attention_combine_kernel, dim3(dim3((unsigned)n_q, (unsigned)batch)), dim3(128), 0,
                                         ctx->stream, part, n_splits, (int)d_head, d_out));
                DEC_EPILOGUE(ctx, "gqa_attention(split-k,int8 cache,mma)");
            }
        }
        YSCV_CUDA_TRY(launch_pdl(gqa_decode_split_kernel<KV>, dim3(grid), dim3(128), split_smem,
                                 ctx->stream, d_q, (int)q_stride, (int)n_q, (int)n_kv, (int)d_head, d_kcache, d_vcache,
                                 d_kscale, d_vscale, (int)max_seq, d_pos, chunk, part));
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
        YSCV_CUDA_TRY(launch_pdl(attention_combine_kernel, dim3(dim3((unsigned)n_q, (unsigned)batch)), dim3(128), 0, ctx->stream, part, n_splits,
                                                                                               (int)d_head, d_out));
        DEC_EPILOGUE(ctx, sizeof(KV) == 1 ? "gqa_attention(split-k,int8 cache)" : "gqa_attention(split-k)");
    }
    // a prompt pass: query positions in tiles, keys and values staged once per tile
    const size_t group = n_q / n_kv;
    const bool rows_aligned = ((reinterpret_cast<uintptr_t>(d_kcache) | reinterpret_cast<uintptr_t>(d_vcache)) & 15) == 0;
    if (seq_q >= 16 && (d_head == 64 || d_head == 128) && group <= 64 && rows_aligned &&
        (reinterpret_cast<uintptr_t>(d_out) & 15) == 0) {
        // 64 (position, head) pairs per block where the group allows, four per warp
        const int QB = (int)(64 / group) > 0 ? (int)(64 / group) : 1;
        const int pairs = (int)group * QB;
        const int warps = (pairs + PF_QH - 1) / PF_QH;
        const size_t pf_smem = (PF_KT * (d_head + 4) + PF_KT * d_head + (size_t)warps * PF_QH * (PF_KT + d_head)) * sizeof(float);
        auto kern = d_head == 64 ? gqa_prefill_tiled_kernel<KV, 64> : gqa_prefill_tiled_kernel<KV, 128>;
        int arc = ensure_dynamic_smem(reinterpret_cast<const void *>(kern), ctx->device, 160 * 1024);
        if (arc) return arc;
        dim3 pgrid((unsigned)((seq_q + QB - 1) / QB), (unsigned)n_kv, (unsigned)batch);
        YSCV_CUDA_TRY(launch_pdl(kern, dim3(pgrid), dim3(32 * warps), pf_smem, ctx->stream, d_q, (int)q_stride, (int)seq_q,
                                 (int)n_q, (int)n_kv, d_kcache, d_vcache, d_kscale, d_vscale, (int)max_seq, d_pos, causal,
                                 d_out, QB));
        DEC_EPILOGUE(ctx, sizeof(KV) == 1 ? "gqa_attention(prompt tiles,int8 cache)" : "gqa_attention(prompt tiles)");
    }
    const size_t smem = (max_seq + d_head) * sizeof(float);
    if (smem > 200 * 1024) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "max_seq %zu too long for the attention kernel", max_seq);
    if (smem > 48 * 1024) {
        int arc = ensure_dynamic_smem(reinterpret_cast<const void *>(gqa_attention_kernel<KV>), ctx->device, 200 * 1024);
        if (arc) return arc;
    }
    dim3 grid((unsigned)seq_q, (unsigned)n_q, (unsigned)batch);
    YSCV_CUDA_TRY(launch_pdl(gqa_attention_kernel<KV>, dim3(grid), dim3(128), smem, ctx->stream, d_q, (int)q_stride, (int)seq_q,
                             (int)n_q, (int)n_kv, (int)d_head, d_kcache, d_vcache, d_kscale, d_vscale, (int)max_seq,
                             d_pos, causal, d_out));
    DEC_EPILOGUE(ctx, sizeof(KV) == 1 ? "gqa_attention(int8 cache)" : "gqa_attention");
}

extern "C" {

int yscv_cuda_gqa_attention_dev(yscv_cuda_ctx *ctx, const float *d_q, size_t q_stride, size_t batch,
                                size_t seq_q, size_t n_q, size_t n_kv, size_t d_head,
                                const float *d_kcache, const float *d_vcache, size_t max_seq,
                                const int32_t *d_pos, int causal, float *d_out) {
    return gqa_attention_impl<float>(ctx, d_q, q_stride, batch, seq_q, n_q, n_kv, d_head, d_kcache, d_vcache, nullptr,
                                     nullptr, max_seq, d_pos, causal, d_out);
}

int yscv_cuda_gqa_attention_i8_dev(yscv_cuda_ctx *ctx, const float *d_q, size_t q_stride, size_t batch,
                                   size_t seq_q, size_t n_q, size_t n_kv, size_t d_head,
                                   const int8_t *d_kcache, const float *d_kscale, const int8_t *d_vcache,
                                   const float *d_vscale, size_t max_seq, const int32_t *d_pos, int causal,
                                   float *d_out) {
    return gqa_attention_impl<int8_t>(ctx, d_q, q_stride, batch, seq_q, n_q, n_kv, d_head, d_kcache, d_vcache, d_kscale,
                                      d_vscale, max_seq, d_pos, causal, d_out);
}

int yscv_cuda_swiglu_dev(yscv_cuda_ctx *ctx, const float *d_gate_up, size_t rows, size_t inter,
                         float *d_out) {
    DEC_PROLOGUE(ctx);
    if (!d_gate_up || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (rows * inter == 0) return YSCV_CUDA_OK;
    const size_t total = rows * inter;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 65535 ? (total + 255) / 256 : 65535);
    YSCV_CUDA_TRY(launch_pdl(swiglu_kernel, dim3(blocks), dim3(256), 0, ctx->stream, d_gate_up, d_out, rows, (int)inter));
    DEC_EPILOGUE(ctx, "swiglu");
}

int yscv_cuda_add_rms_norm_act_dev(yscv_cuda_ctx *ctx, const float *d_x, const float *d_delta, const float *d_gamma,
                                   float eps, size_t rows, size_t hidden, float *d_x_out, void *d_normed_act) {
    DEC_PROLOGUE(ctx);
    if (!d_x || !d_gamma || !d_normed_act) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (hidden % 8 != 0 || (reinterpret_cast<uintptr_t>(d_normed_act) & 15))
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "hidden must be a multiple of 8 and the activation buffer 16-byte aligned");
    if (rows == 0) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(launch_pdl(add_rms_norm_act_kernel, dim3((unsigned)rows), dim3(256), 0, ctx->stream, d_x, d_delta, d_gamma, eps,
                             (int)hidden, d_x_out, reinterpret_cast<uint4 *>(d_normed_act)));
    DEC_EPILOGUE(ctx, "add_rms_norm(bf16 activations out)");
}

int yscv_cuda_swiglu_act_dev(yscv_cuda_ctx *ctx, const float *d_gate_up, size_t rows, size_t inter, void *d_out_act) {
    DEC_PROLOGUE(ctx);
    if (!d_gate_up || !d_out_act) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (inter % 8 != 0 || (reinterpret_cast<uintptr_t>(d_out_act) & 15))
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "inter must be a multiple of 8 and the activation buffer 16-byte aligned");
    if (rows * inter == 0) return YSCV_CUDA_OK;
    const size_t total8 = rows * (inter / 8);
    const unsigned blocks = (unsigned)((total8 + 255) / 256 < 65535 ? (total8 + 255) / 256 : 65535);
    YSCV_CUDA_TRY(launch_pdl(swiglu_act_kernel, dim3(blocks), dim3(256), 0, ctx->stream, d_gate_up,
                             reinterpret_cast<uint4 *>(d_out_act), rows, (int)inter));
    DEC_EPILOGUE(ctx, "swiglu(bf16 activations out)");
}

int yscv_cuda_f32_matmul_dev(yscv_cuda_ctx *ctx, const float *d_w, const float *d_x, size_t m, size_t n,
                             size_t k, float *d_out) {
    DEC_PROLOGUE(ctx);
    if (!d_w || !d_x || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (k % 4 != 0) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "k must be a multiple of 4");
    if ((reinterpret_cast<uintptr_t>(d_w) | reinterpret_cast<uintptr_t>(d_x)) & 15)
        return fail(YSCV_CUDA_ERR_UNSUPPORTED, "weights and activations must be 16-byte aligned");
    if (m * n == 0) return YSCV_CUDA_OK;
    const unsigned blocks = (unsigned)((n + 7) / 8 < (size_t)(16 * ctx->sm_count) ? (n + 7) / 8 : 16 * ctx->sm_count);
    if (m > 8 && ctx->f32_tensor_cores && f32_gemm_tc_supported(d_w, d_x, m, n, k)) {
        // wide batch: three TF32 products per fp32 product on the tensor cores, weights read once
        int rc = ctx->scratch.reserve(f32_gemm_tc_scratch_bytes(m, k));
        if (rc) return rc;
        rc = f32_gemm_tc(ctx, d_w, d_x, m, n, k, d_out, ctx->scratch.ptr);
        if (rc) return rc;
        ctx->last_kernel = "f32_matmul(tcgen05,3xtf32)";
        return YSCV_CUDA_OK;
    }
    if (m > 8) {
        // wide batch without the tensor-core form (k not a multiple of 32): tiled SGEMM, the weights
        // cross HBM once per 64 activation rows
        dim3 grid((unsigned)((n + FM_BN - 1) / FM_BN), (unsigned)((m + FM_BM - 1) / FM_BM));
        YSCV_CUDA_TRY(launch_pdl(f32_matmul_tiled_kernel, grid, dim3(256), 0, ctx->stream, d_w, d_x, d_out, (int)m, (int)n, (int)k));
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
        ctx->last_kernel = "f32_matmul(tiled)";
        return YSCV_CUDA_OK;
    }
    // one pass over the weights per 4 activation rows
    for (size_t m0 = 0; m0 < m; m0 += 4) {
        YSCV_CUDA_TRY(launch_pdl(f32_matmul_kernel<4>, dim3(blocks), dim3(256), 0, ctx->stream, d_w, d_x, d_out, (int)m0, (int)m, (int)n, (int)k));
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
    }
    ctx->last_kernel = "f32_matmul";
    return YSCV_CUDA_OK;
}

int yscv_cuda_argmax_last_dev(yscv_cuda_ctx *ctx, const float *d_logits, size_t rows, size_t vocab,
                              int32_t *d_out) {
    DEC_PROLOGUE(ctx);
    if (!d_logits || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (rows == 0) return YSCV_CUDA_OK;
    if (vocab == 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "empty vocabulary");
    if (vocab >= 8192) {
        const int nb = 64;
        int rc = ctx->scratch_attn.reserve(rows * nb * 8);
        if (rc) return rc;
        float *pv = reinterpret_cast<float *>(ctx->scratch_attn.ptr);
        int32_t *pi = reinterpret_cast<int32_t *>(pv + rows * nb);
        YSCV_CUDA_TRY(launch_pdl(argmax_partial_kernel, dim3(dim3(nb, (unsigned)rows)), dim3(256), 0, ctx->stream, d_logits, (int)vocab, pv, pi));
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
        YSCV_CUDA_TRY(launch_pdl(argmax_final_kernel, dim3((unsigned)rows), dim3(64), 0, ctx->stream, pv, pi, nb, d_out));
        DEC_EPILOGUE(ctx, "argmax_last(two-stage)");
    }
    YSCV_CUDA_TRY(launch_pdl(argmax_last_kernel, dim3((unsigned)rows), dim3(256), 0, ctx->stream, d_logits, (int)vocab, d_out));
    DEC_EPILOGUE(ctx, "argmax_last");
}

int yscv_cuda_advance_pos_dev(yscv_cuda_ctx *ctx, int32_t *d_pos, int by) {
    DEC_PROLOGUE(ctx);
    if (!d_pos) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    YSCV_CUDA_TRY(launch_pdl(advance_pos_kernel, dim3(1), dim3(1), 0, ctx->stream, d_pos, by));
    DEC_EPILOGUE(ctx, "advance_pos");
}

}  // extern "C"
