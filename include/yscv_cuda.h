/*
 * yscv_cuda.h -- C ABI of the B200 (sm_100a) quantized-matmul library.
 *
 * Drop-in boundary for the quantized-matmul hot path of enthropy7/YSCV: the
 * entry points below are what an FFI crate inside yscv-kernels / yscv-onnx
 * would bind in place of the CPU kernels it calls today. Each declaration
 * cites the reference interface it replaces (paths relative to the reference
 * project root).
 *
 * Conventions
 *  - Plain pointers and sizes only. Functions return 0 on success and a
 *    negative yscv_cuda_status otherwise; yscv_cuda_last_error() returns a
 *    thread-local message for the last failure on the calling thread.
 *  - "host" entry points take host pointers with the reference's exact slice
 *    layouts, copy in, run on the GPU, copy out and synchronise: they are the
 *    literal drop-ins for the reference's free functions.
 *  - "_dev" entry points take device pointers, enqueue on the context's stream
 *    and return without synchronising: weights stay resident in HBM, which is
 *    how a runner that uploads weights once at load time uses the library.
 *  - There is no CPU fallback anywhere. Shapes a kernel cannot take are
 *    rejected with YSCV_CUDA_ERR_UNSUPPORTED.
 *  - A context owns one CUDA stream (or borrows the caller's); calls on one
 *    context are serialised by the caller (the library takes no lock per call);
 *    different contexts may be used from different threads at the same time:
 *    the only process-wide state (per-kernel attributes set once, the operator
 *    counters, the table behind a yscv_cuda_registry) is guarded inside. Handles
 *    are immutable after creation and may be shared between contexts of the
 *    same device.
 *  - "_dev" entry points only enqueue work, with one exception: the first call
 *    for a shape larger than any seen before may grow the context's scratch
 *    buffers (a cudaFree and a cudaMalloc, which synchronise the device and are
 *    not allowed inside a stream capture). Run one call of every shape before
 *    capturing a CUDA graph.
 *  - Pointers given to "_dev" entry points must be aligned as the natural
 *    vector width of the operand asks (16 bytes for f32 rows read with 128-bit
 *    loads); a pointer that is not is rejected with YSCV_CUDA_ERR_UNSUPPORTED or
 *    takes a scalar path, it never faults.
 *
 * Layouts (identical to the reference's)
 *  - packed int4 weights: [N rows][K/2 bytes], one row per output channel,
 *    two's-complement nibbles, low nibble = even k
 *    (crates/yscv-kernels/src/ops/int4_matmul.rs:12-18, 29-40).
 *  - scales: [N][K/group_size] f32, no zero-point array (symmetric).
 *  - int8 GEMM: A [M,K] row-major i8, B [K,N] row-major i8, out [M,N] i32
 *    (crates/yscv-kernels/src/ops/int8_matmul.rs:195-208).
 */
#ifndef YSCV_CUDA_H
#define YSCV_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    YSCV_CUDA_OK = 0,
    YSCV_CUDA_ERR_BAD_ARG = -1,     /* the reference would debug_assert! */
    YSCV_CUDA_ERR_CUDA = -2,        /* a CUDA runtime / driver call failed */
    YSCV_CUDA_ERR_UNSUPPORTED = -3, /* no kernel for this shape; no CPU fallback */
    YSCV_CUDA_ERR_TIMEOUT = -4,     /* a bounded device-side wait ran out */
    YSCV_CUDA_ERR_NO_DEVICE = -5    /* no sm_100 device visible */
} yscv_cuda_status;

typedef struct yscv_cuda_ctx yscv_cuda_ctx;
typedef struct yscv_cuda_int4_weight yscv_cuda_int4_weight;
typedef struct yscv_cuda_i8b yscv_cuda_i8b;

/* ---- context ------------------------------------------------------------ */

/* Replaces the reference's CPU-feature probe (crates/yscv-cpu/src/lib.rs:74-154):
 * checks that `device` is an sm_100 part and creates a stream on it. */
int yscv_cuda_ctx_create(int device, yscv_cuda_ctx **out);
/* Same, but enqueues on a stream the caller owns (cudaStream_t passed as void*). */
int yscv_cuda_ctx_create_on_stream(int device, void *cuda_stream, yscv_cuda_ctx **out);
void yscv_cuda_ctx_destroy(yscv_cuda_ctx *ctx);
int yscv_cuda_ctx_synchronize(yscv_cuda_ctx *ctx);
/* Reads and clears the device-side status word (0 = none): 1 a bounded wait on a copy
 * barrier ran out, 2 a bounded wait on another CTA or another GPU ran out, 3 a sequence
 * position outside [0, max_seq) was given to a cache append (nothing was appended). */
int yscv_cuda_ctx_device_status(yscv_cuda_ctx *ctx, int *status);
const char *yscv_cuda_last_error(void);
/* Counterpart of runtime_dispatch_report() (crates/yscv-kernels/src/core.rs:30-137):
 * names the kernel variant the last call on this context dispatched to. */
const char *yscv_cuda_last_kernel(const yscv_cuda_ctx *ctx);
/* Number of kernels this library has launched on the context so far. */
uint64_t yscv_cuda_ctx_launch_count(const yscv_cuda_ctx *ctx);
/* runtime_dispatch_report() (crates/yscv-kernels/src/core.rs:111-137) for this context: the
 * device, and for the last int4 and the last int8 call the kernel variant with its tile
 * geometry and the shape it was chosen for. The string belongs to the calling thread and is
 * valid until its next call. */
const char *yscv_cuda_dispatch_report(const yscv_cuda_ctx *ctx);
/* Process-wide operator counters, the counterpart of QuantRuntimeStats
 * (crates/yscv-onnx/src/runner/quant_stats.rs:21-92): how many calls each kernel family
 * served since the last reset. cpu_fallbacks is always 0: this library has no CPU path. */
typedef struct {
    uint64_t int4_gemv_calls;      /* m <= 16 passes on the integer-MMA decode kernel */
    uint64_t int4_gemm_calls;      /* m > 16 calls on the tensor-core prefill GEMM */
    uint64_t int4_generic_calls;   /* passes on the warp-per-row kernel (odd group / k / alignment) */
    uint64_t int8_gemm_calls;      /* every int8 GEMM launch, whatever the epilogue */
    uint64_t qlinear_matmul_calls;
    uint64_t matmul_integer_calls;
    uint64_t requant_calls;        /* stand-alone requant passes */
    uint64_t decode_step_calls;    /* one-launch decode steps */
    uint64_t cpu_fallbacks;
} yscv_cuda_quant_stats;
void yscv_cuda_quant_stats_read(yscv_cuda_quant_stats *out);
void yscv_cuda_quant_stats_reset(void);
/* int4 matmuls with more than 16 activation rows run on the bf16 tensor-core path
 * (relative Frobenius error ~3e-3 against the fp32 kernel, bound 2e-2). exact != 0 keeps
 * the fp32-exact decode kernel for them, 16 rows per pass (slower, error ~1e-6): the
 * counterpart of choosing packed_int4_gemm_scalar over a SIMD variant
 * (crates/yscv-kernels/src/ops/int4_matmul.rs:548-605). */
int yscv_cuda_ctx_set_int4_prefill_exact(yscv_cuda_ctx *ctx, int exact);
/* Kernel-selection switch of the bf16 prefill GEMM: enable != 0 (the default) lets prefills
 * with at least one 512-row x 256-token tile per CTA pair run on CTA pairs (tcgen05
 * cta_group::2: each CTA dequantises 256 weight rows and stages half of the activation tile);
 * 0 keeps the one-CTA kernel. Same products, same summation order over k. */
int yscv_cuda_ctx_set_int4_prefill_cta_pairs(yscv_cuda_ctx *ctx, int enable);
/* Kernel-selection switch of the int8 GEMM, like the reference's environment gates on its
 * int8 paths (crates/yscv-onnx/src/runner/quant_stats.rs:68-71). The GEMM has a one-CTA kernel
 * and a CTA-pair kernel (tcgen05 cta_group::2: two SMs per 256 x 256 tile, each staging half of
 * both operands, so half the operand traffic from L2 per flop). mode < 0 (the default): the pair
 * kernel where it measured faster: int32 output with at least three rounds of pair tiles, and
 * any output when the one-CTA kernel would run a single round on more than half of the SMs;
 * mode == 0: the one-CTA kernel everywhere; mode > 0: the pair kernel on every shape it supports
 * (m, n >= 256 and pair tiles for at least 0.8 of the pairs). The results are identical
 * (integer arithmetic), only the speed differs. */
int yscv_cuda_ctx_set_int8_cta_pairs(yscv_cuda_ctx *ctx, int mode);
/* Second switch of the int8 GEMM, on by default: when the output tiles occupy at most half of
 * the SMs and K >= 8192, the K loops are cut into equal runs over all CTAs and the int32 partial
 * sums are added by the CTA that owns the tile (workspace of 128 KB per SM in the context,
 * allocated by the first call that needs it; the waits on the partial sums are bounded and report
 * status 2). Integer sums do not depend on the order, so the results are identical with the
 * switch off; 0 keeps whole tiles per CTA. */
int yscv_cuda_ctx_set_int8_tail_split(yscv_cuda_ctx *ctx, int enable);
/* Decode attention over int8 caches (yscv_cuda_gqa_attention_i8_dev with one query position and a
 * cache longer than 128, head size 64 or 128): on by default, both contractions run as fp16
 * tensor-core MMAs with fp32 accumulators (an int8 cache entry is exact in fp16, the query and the
 * softmax weights are split into two fp16 terms), which differs from the fp32 loop (0) only in
 * summation order. */
int yscv_cuda_ctx_set_attention_tensor_cores(yscv_cuda_ctx *ctx, int enable);
/* fp32 matmul of the decoder (yscv_cuda_f32_matmul_dev: the fp32 LM head) with more than 8
 * activation rows and k a multiple of 32: on by default, every fp32 product runs as three TF32
 * tensor-core products with fp32 accumulators (operands split into a TF32 part and a remainder;
 * relative error of a product ~2^-21), the weights cross HBM once; 0 keeps the tiled fp32 FMA
 * kernel. */
int yscv_cuda_ctx_set_f32_tensor_cores(yscv_cuda_ctx *ctx, int enable);
/* Per-kernel timing, the counterpart of YSCV_RUNNER_PROFILE
 * (crates/yscv-onnx/src/runner/profile.rs:1-120): while enabled, the dominant
 * kernel of every call is bracketed by CUDA events on the context's stream
 * (the first 4096 launches after a read; the events are created by _enable,
 * so that no launch path ever allocates).
 * _read synchronises, returns the number of bracketed launches and their summed
 * device time, and resets the counters. */
int yscv_cuda_ctx_profile_enable(yscv_cuda_ctx *ctx, int enable);
int yscv_cuda_ctx_profile_read(yscv_cuda_ctx *ctx, uint64_t *launches, double *total_ms);

/* ---- int4 block-quantized GEMV / GEMM: host drop-ins --------------------- */

/* packed_int4_gemv_dispatch (crates/yscv-kernels/src/ops/int4_matmul.rs:310-377).
 * Non-finite activations: the kernels for m <= 16 turn each group of 32 activations into
 * block-fixed-point integers first, so a group that holds a NaN or an infinity yields NaN for
 * every output row, where the reference's fp32 loop (int4_matmul.rs:61-80) yields NaN or, when
 * every weight that meets the infinity is non-zero and of one sign, an infinity of that sign.
 * Both are non-finite; finite inputs are unaffected. */
int yscv_cuda_packed_int4_gemv(yscv_cuda_ctx *ctx, const uint8_t *weight_packed,
                               const float *scales, const float *activation,
                               float *output, size_t m_w, size_t k, size_t group_size);

/* packed_int4_gemm_dispatch (crates/yscv-kernels/src/ops/int4_matmul.rs:548-605) */
int yscv_cuda_packed_int4_gemm(yscv_cuda_ctx *ctx, const uint8_t *weight_packed,
                               const float *scales, const float *activation,
                               float *output, size_t m, size_t n, size_t k,
                               size_t group_size);

/* pack_int4_symmetric_per_group (crates/yscv-kernels/src/ops/int4_matmul.rs:611-646).
 * `packed` (m_w*k/2 bytes) and `scales` (m_w*k/group_size floats) are caller-allocated. */
int yscv_cuda_pack_int4_symmetric_per_group(yscv_cuda_ctx *ctx, const float *weights,
                                            size_t m_w, size_t k, size_t group_size,
                                            uint8_t *packed, float *scales);

/* ---- int4: device-resident forms ---------------------------------------- */

/* PackedInt4Weight (crates/yscv-onnx/src/quantize/packed_int4.rs:28-39) resident in
 * HBM. _upload copies host slices; _wrap borrows device memory the caller keeps alive. */
int yscv_cuda_int4_weight_upload(yscv_cuda_ctx *ctx, const uint8_t *packed,
                                 const float *scales, size_t m_w, size_t k,
                                 size_t group_size, yscv_cuda_int4_weight **out);
int yscv_cuda_int4_weight_wrap(const uint8_t *d_packed, const float *d_scales, size_t m_w,
                               size_t k, size_t group_size, yscv_cuda_int4_weight **out);
void yscv_cuda_int4_weight_free(yscv_cuda_int4_weight *w);

/* The int4 branch of exec_matmul (crates/yscv-onnx/src/runner/linear.rs:223-278) on
 * device memory: d_activation [m,k] f32 -> d_output [m,n] f32. One pass over the
 * weights for any m (the reference re-reads them m times when m < 8). m <= 16 takes
 * the bandwidth-bound decode kernel, larger m the tensor-core prefill GEMM. */
int yscv_cuda_int4_matmul_dev(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w,
                              const float *d_activation, float *d_output, size_t m);

/* The fusion the reference's plan asks for (docs/int4-quant-pipeline-plan.md:45-51: the
 * activation conversion folded into the producing operator): yscv_cuda_int4_matmul_dev for
 * m > 16 whose activations the caller already holds as bf16 in the order the tensor-core GEMM
 * consumes (k = 0,4,1,5,2,6,3,7 of every group of 8, round to nearest even), as
 * yscv_cuda_add_rms_norm_act_dev and yscv_cuda_swiglu_act_dev write them: the GEMM's own
 * conversion pass is skipped, the result is the same bit for bit. Needs what the bf16 path of
 * yscv_cuda_int4_matmul_dev needs (group_size 32, k % 64 == 0, 16-byte aligned operands, the
 * fp32-exact prefill mode off); YSCV_CUDA_ERR_UNSUPPORTED otherwise. */
int yscv_cuda_int4_matmul_act_dev(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w,
                                  const void *d_activation_bf16, float *d_output, size_t m);

/* The same operator as a runner calls it: weights resident (uploaded once at load
 * time, like the reference's side-table built by quantize_matmul_weights_int4_packed,
 * crates/yscv-onnx/src/quantize/packed_int4.rs:50-128), activation and output in host
 * memory: copies activation [m,k] in, runs, copies output [m,n] out, synchronises. */
int yscv_cuda_int4_matmul(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w,
                          const float *activation, float *output, size_t m);

/* No counterpart in the reference. yscv_cuda_int4_matmul_dev for callers that are not
 * allowed to allocate device memory while they run: code inside a real-time or
 * latency-critical loop, a plugin whose host forbids cudaMalloc after start-up, a
 * process working under a fixed memory budget. The kernel's scratch (the digit planes
 * of the activations) lives in an array built into the library, about 1.7 MB on every
 * GPU that loads it, held until the process exits; this call performs no cudaMalloc,
 * cudaFree or other allocating call. Limits: m <= 16, k <= 32768, group_size 32,
 * k % 256 == 0, operands 16-byte aligned; anything else is rejected with
 * YSCV_CUDA_ERR_UNSUPPORTED. The first call on each device looks up the array's
 * device address; make that first call outside any stream capture. All calls on a
 * device share the one array (it keeps the last call's contents; every word a call
 * reads is rewritten by that call first, so nothing needs clearing), therefore two
 * calls that overlap on the GPU, e.g. from two contexts or streams, race: serialise
 * them. All pointers are device pointers; weights are passed directly, no handle. */
int yscv_cuda_int4_matmul_dev_static(yscv_cuda_ctx *ctx, const uint8_t *d_packed,
                                     const float *d_scales, size_t n, size_t k,
                                     size_t group_size, const float *d_activation,
                                     float *d_output, size_t m);

/* Weights exported as ONNX MatMulNBits (bits = 4, block_size = group) hold unsigned nibbles with
 * an implicit zero point of 8 in the same [N][K/2] layout, low nibble = even k; the reference
 * has no such import (its int4 weights live in a side-table, crates/yscv-onnx/src/quantize/
 * packed_int4.rs:28-39). byte ^ 0x88 turns them into this library's two's-complement nibbles;
 * scales are unchanged. src == dst is allowed. The host form is a load-time format conversion
 * and makes no CUDA call. */
int yscv_cuda_int4_from_matmulnbits(const uint8_t *src, uint8_t *dst, size_t bytes);
int yscv_cuda_int4_from_matmulnbits_dev(yscv_cuda_ctx *ctx, const uint8_t *d_src, uint8_t *d_dst,
                                        size_t bytes);

/* The inverse: this library's nibbles as MatMulNBits expects them (q + 8, zero point 8). The
 * same bit flip; named for the direction. */
int yscv_cuda_int4_to_matmulnbits(const uint8_t *src, uint8_t *dst, size_t bytes);

/* One weight of quantize_matmul_weights_int4_packed
 * (crates/yscv-onnx/src/quantize/packed_int4.rs:50-128): an fp32 initializer [dim0][dim1] in
 * the layout its node implies is transposed to [N][K] where needed, packed and kept resident.
 * The reference's rules hold: an odd or zero group_size is an error (YSCV_CUDA_ERR_BAD_ARG,
 * packed_int4.rs:54-58); a weight with k % group_size != 0 or k * n < 32 is silently skipped
 * (packed_int4.rs:102-104): the call returns 0 and leaves *out NULL, and the caller keeps
 * the fp32 weight. Unlike the reference's exec_gemm (runner/linear.rs:3-10), which never
 * consults the side table, handles made from Gemm weights are usable like any other. */
enum {
    YSCV_CUDA_WEIGHT_MATMUL_KN = 0, /* MatMul: [K][N] */
    YSCV_CUDA_WEIGHT_GEMM_NK = 1,   /* Gemm, transB = 1: [N][K], packed as it is */
    YSCV_CUDA_WEIGHT_GEMM_KN = 2    /* Gemm, transB = 0: [K][N] */
};
int yscv_cuda_int4_weight_from_f32(yscv_cuda_ctx *ctx, const float *weight, size_t dim0, size_t dim1,
                                   int layout, size_t group_size, yscv_cuda_int4_weight **out);
/* PackedInt4Weight's fields (packed_int4.rs:28-39) of a resident weight, and its bytes back
 * in host memory: packed [m_w * k / 2], scales [m_w * k / group_size]. */
size_t yscv_cuda_int4_weight_rows(const yscv_cuda_int4_weight *w);
size_t yscv_cuda_int4_weight_k(const yscv_cuda_int4_weight *w);
size_t yscv_cuda_int4_weight_group_size(const yscv_cuda_int4_weight *w);
int yscv_cuda_int4_weight_download(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w, uint8_t *packed,
                                   float *scales);

/* A byte container for one packed int4 weight. No counterpart in the reference, which keeps
 * packed int4 in memory only (packed_int4.rs:28-39) and re-quantises the fp32 model at every
 * start. Layout, little endian: 64-byte header {"YSCVINT4", u32 version = 1, u32 group_size,
 * u64 m_w, u64 k, u64 packed_bytes, u64 scale_count, 16 reserved bytes}, the packed bytes
 * padded with zeros to a multiple of 16, the f32 scales. _read validates the header and
 * returns views into `src`; host only, no CUDA call. */
size_t yscv_cuda_int4_container_size(size_t m_w, size_t k, size_t group_size);
int yscv_cuda_int4_container_write(const uint8_t *packed, const float *scales, size_t m_w, size_t k,
                                   size_t group_size, uint8_t *dst, size_t capacity, size_t *written);
int yscv_cuda_int4_container_read(const uint8_t *src, size_t len, size_t *m_w, size_t *k, size_t *group_size,
                                  const uint8_t **packed, const float **scales);
int yscv_cuda_int4_weight_from_container(yscv_cuda_ctx *ctx, const uint8_t *src, size_t len,
                                         yscv_cuda_int4_weight **out);

/* pack_int4_symmetric_per_group on device memory: d_weights [m_w,k] f32. */
int yscv_cuda_pack_int4_dev(yscv_cuda_ctx *ctx, const float *d_weights, size_t m_w,
                            size_t k, size_t group_size, uint8_t *d_packed,
                            float *d_scales);

/* ---- int8 GEMM: MatMulInteger / QLinearMatMul ------------------------------ */

/* int8_matmul_dispatch (crates/yscv-kernels/src/ops/int8_matmul.rs:2407-2413): host
 * a [m,k], b [k,n] row-major i8 -> host out [m,n] i32. B is transposed on the GPU on
 * every call, as the reference's non-prepacked entry point does on the CPU. */
int yscv_cuda_int8_matmul(yscv_cuda_ctx *ctx, const int8_t *a, const int8_t *b, size_t m,
                          size_t k, size_t n, int32_t *out);

/* pack_i8_b_for_matmul / PackedI8B (int8_matmul.rs:128-191): uploads b [k,n] once and
 * keeps B^T (K-major, the tensor-core operand layout) and its column sums in HBM.
 * _dev takes b already in device memory. */
int yscv_cuda_pack_i8_b_for_matmul(yscv_cuda_ctx *ctx, const int8_t *b, size_t k, size_t n,
                                   yscv_cuda_i8b **out);
int yscv_cuda_pack_i8_b_dev(yscv_cuda_ctx *ctx, const int8_t *d_b, size_t k, size_t n,
                            yscv_cuda_i8b **out);
void yscv_cuda_i8b_free(yscv_cuda_i8b *b);
/* Zero point of B (the b_zero_point input of MatMulInteger / QLinearMatMul, a scalar:
 * crates/yscv-onnx/src/runner/linear.rs:440-446, 651-660), default 0. The reference leaves
 * its integer path when any zero point is non-zero and computes in fp32 (linear.rs:701-735);
 * here the product stays exact: sum_k (a - a_zp)(b - b_zp) = acc - a_zp * colsum(B)[n]
 * - b_zp * rowsum(A)[m] + k * a_zp * b_zp in the epilogue (one extra pass over A). Weights
 * stored as uint8 with zero point z are given as int8 (byte ^ 0x80) with zero point z - 128. */
int yscv_cuda_i8b_set_zero_point(yscv_cuda_i8b *b, int32_t b_zero_point);
size_t yscv_cuda_i8b_k(const yscv_cuda_i8b *b); /* PackedI8B::k() */
size_t yscv_cuda_i8b_n(const yscv_cuda_i8b *b); /* PackedI8B::n() */

/* int8_matmul_prepacked_dispatch (int8_matmul.rs:2420-2425): host a [m,k] -> host out. */
int yscv_cuda_int8_matmul_prepacked(yscv_cuda_ctx *ctx, const int8_t *a, const yscv_cuda_i8b *b,
                                    size_t m, int32_t *out);
/* same on device memory, asynchronous on the context's stream */
int yscv_cuda_int8_matmul_prepacked_dev(yscv_cuda_ctx *ctx, const int8_t *d_a,
                                        const yscv_cuda_i8b *b, size_t m, int32_t *d_out);

/* Epilogue of QLinearMatMul: the requant_scalar contract
 * (crates/yscv-kernels/src/ops/int8_requant.rs:143-169): q = saturate(round((float)acc *
 * composite + y_zero_point)), separate multiply and add, to [qmin, qmax] ([-128,127] for
 * int8 output, [0,255] for uint8). round_mode 0 = ties to even (ONNX, the kernel-level
 * contract), 1 = half away from zero (what the runner's exec_qlinear_matmul does with
 * f32::round, crates/yscv-onnx/src/runner/linear.rs:481-485). */
typedef struct {
    int a_is_unsigned;    /* A holds uint8 instead of int8 */
    int32_t a_zero_point; /* exact: acc = sum_k (a - a_zp) * b, any value */
    float composite;      /* (a_scale * b_scale) / y_scale, computed in f32 by the caller */
    float y_zero_point;
    int32_t qmin, qmax;
    int round_mode;
} yscv_cuda_requant;

/* exec_qlinear_matmul (crates/yscv-onnx/src/runner/linear.rs:438-537) with b_zero_point 0:
 * a [m,k] bytes, prepacked b, out [m,n] one byte per element (uint8 or int8 per qmin/qmax).
 * Non-zero a_zero_point is computed exactly in integers (the reference falls back to an
 * fp32 GEMM there). */
int yscv_cuda_qlinear_matmul(yscv_cuda_ctx *ctx, const void *a, const yscv_cuda_i8b *b, size_t m,
                             const yscv_cuda_requant *rq, void *out);
int yscv_cuda_qlinear_matmul_dev(yscv_cuda_ctx *ctx, const void *d_a, const yscv_cuda_i8b *b,
                                 size_t m, const yscv_cuda_requant *rq, void *d_out);

/* exec_matmul_integer (crates/yscv-onnx/src/runner/linear.rs:648-737) with b_zero_point 0:
 * out [m,n] i32 = (a - a_zero_point) x b, exact. */
int yscv_cuda_matmul_integer(yscv_cuda_ctx *ctx, const void *a, int a_is_unsigned,
                             int32_t a_zero_point, const yscv_cuda_i8b *b, size_t m,
                             int32_t *out);
int yscv_cuda_matmul_integer_dev(yscv_cuda_ctx *ctx, const void *d_a, int a_is_unsigned,
                                 int32_t a_zero_point, const yscv_cuda_i8b *b, size_t m,
                                 int32_t *d_out);

/* requant_i32_row_to_i8_dispatch (crates/yscv-kernels/src/ops/int8_requant.rs:81-169) as a
 * pass of its own: acc [len] i32, len a multiple of the channel count c, optional bias [c]
 * (wrapping add), out[i] = clamp(round_ties_even((float)(acc[i] + bias[i % c]) * composite +
 * y_zero_point), -128, 127), ReLU after the saturation. The GEMM entry points above fuse the
 * same arithmetic behind the tensor cores; this one serves accumulators made elsewhere. */
int yscv_cuda_requant_i32_row_to_i8(yscv_cuda_ctx *ctx, const int32_t *acc, const int32_t *bias, float composite,
                                    float y_zero_point, int relu, int8_t *out, size_t len, size_t c);
int yscv_cuda_requant_i32_row_to_i8_dev(yscv_cuda_ctx *ctx, const int32_t *d_acc, const int32_t *d_bias,
                                        float composite, float y_zero_point, int relu, int8_t *d_out,
                                        size_t len, size_t c);

/* ---- resident weights keyed by initializer name ----------------------------------------
 * The runner's side tables: env.packed_int4_weights.get(&node.inputs[1])
 * (crates/yscv-onnx/src/runner/linear.rs:228) and prepacked_i8_weights / prepacked_i8_b(name)
 * (crates/yscv-onnx/src/plan/build.rs:1417-1454, crates/yscv-onnx/src/runner/tensor_env.rs:178-183),
 * filled once at load time. _put takes ownership of the handle (a second _put under the same
 * name frees the first, like HashMap::insert); _get returns NULL for a name that is absent;
 * _destroy frees every handle. Lookups may run concurrently from any thread. */
typedef struct yscv_cuda_registry yscv_cuda_registry;
int yscv_cuda_registry_create(yscv_cuda_registry **out);
void yscv_cuda_registry_destroy(yscv_cuda_registry *reg);
int yscv_cuda_registry_put_int4(yscv_cuda_registry *reg, const char *name, yscv_cuda_int4_weight *w);
int yscv_cuda_registry_put_i8b(yscv_cuda_registry *reg, const char *name, yscv_cuda_i8b *b);
const yscv_cuda_int4_weight *yscv_cuda_registry_get_int4(const yscv_cuda_registry *reg, const char *name);
const yscv_cuda_i8b *yscv_cuda_registry_get_i8b(const yscv_cuda_registry *reg, const char *name);
size_t yscv_cuda_registry_len(const yscv_cuda_registry *reg);
/* The load-time hooks in one call each: quantize_matmul_weights_int4_packed for one weight
 * (*packed = 0 when the reference's rules skip it) and the QLinearMatMul / MatMulInteger
 * prepack of build_runtime_index (*prepacked = 0 when should_prepack_i8_b says no). */
int yscv_cuda_registry_register_matmul_weight(yscv_cuda_ctx *ctx, yscv_cuda_registry *reg, const char *name,
                                              const float *weight, size_t dim0, size_t dim1, int layout,
                                              size_t group_size, int *packed);
int yscv_cuda_registry_register_i8_weight(yscv_cuda_ctx *ctx, yscv_cuda_registry *reg, const char *name,
                                          const int8_t *b, size_t k, size_t n, int *prepacked);
/* should_prepack_i8_b (crates/yscv-onnx/src/plan/build.rs:1371-1377) and
 * should_use_prepacked_i8_b (crates/yscv-onnx/src/runner/layout.rs:6-11), unchanged. */
int yscv_cuda_should_prepack_i8_b(size_t k, size_t n);
int yscv_cuda_should_use_prepacked_i8_b(size_t m, size_t k, size_t n);

/* ---- fp32 operators between the quantized linears of a decoder step ---------- */
/* All take device pointers and are asynchronous on the context's stream. The sequence
 * position (*d_pos) and the token ids live in device memory, so that a whole decode
 * step can be captured once in a CUDA graph and replayed. */

/* embedding_lookup (crates/yscv-kernels/src/ops/embedding.rs:12): out[r] = weight[tokens[r]] */
int yscv_cuda_embedding_dev(yscv_cuda_ctx *ctx, const float *d_weight, size_t vocab, size_t dim,
                            const int32_t *d_tokens, size_t rows, float *d_out);

/* rms_norm_last_dim_row (crates/yscv-kernels/src/ops/norm.rs:1497-1518) with the residual
 * add in front: x_out = x + delta (delta and x_out may be null), normed = rmsnorm(x_out)*gamma */
int yscv_cuda_add_rms_norm_dev(yscv_cuda_ctx *ctx, const float *d_x, const float *d_delta,
                               const float *d_gamma, float eps, size_t rows, size_t hidden,
                               float *d_x_out, float *d_normed);
/* The same with the normalised rows written as the bf16 activations of a following
 * yscv_cuda_int4_matmul_act_dev (hidden % 8 == 0, d_normed_act 16-byte aligned, rows x hidden bf16) */
int yscv_cuda_add_rms_norm_act_dev(yscv_cuda_ctx *ctx, const float *d_x, const float *d_delta,
                                   const float *d_gamma, float eps, size_t rows, size_t hidden,
                                   float *d_x_out, void *d_normed_act);

/* apply_rotary_embedding (crates/yscv-kernels/src/ops/rope.rs:24-117, rotate-half) on the
 * q and k parts of fused qkv rows [q | k | v] at positions *d_pos + s, fused with the
 * KvCache append (crates/yscv-onnx/src/runner/kv_cache.rs:118-254, f32 storage):
 * caches are [batch][max_seq][n_kv][d_head]. q is rotated in place. d_head even, d_head +
 * (int8 form) n_kv * d_head floats must fit 48 KB of shared memory. A position outside
 * [0, max_seq) appends nothing and sets the context's status word to 3. */
int yscv_cuda_rope_kv_append_dev(yscv_cuda_ctx *ctx, float *d_qkv, size_t batch, size_t seq,
                                 size_t n_q, size_t n_kv, size_t d_head, float theta,
                                 const int32_t *d_pos, float *d_kcache, float *d_vcache,
                                 size_t max_seq);

/* exec_grouped_query_attention (crates/yscv-onnx/src/runner/linear.rs:552-646) over the
 * cache: keys 0 .. *d_pos + seq_q - 1, or 0 .. *d_pos + sq when causal. q rows are
 * q_stride floats apart; out is [batch][seq_q][n_q*d_head]. */
int yscv_cuda_gqa_attention_dev(yscv_cuda_ctx *ctx, const float *d_q, size_t q_stride, size_t batch,
                                size_t seq_q, size_t n_q, size_t n_kv, size_t d_head,
                                const float *d_kcache, const float *d_vcache, size_t max_seq,
                                const int32_t *d_pos, int causal, float *d_out);

/* The same two operators over a cache stored as KvDtype::I8
 * (crates/yscv-onnx/src/runner/kv_cache.rs:8-90): every appended row (one token's
 * n_kv * d_head keys, or values, of one layer) is stored as int8 with one f32 scale,
 * scale = abs_max / 127 (1.0 when abs_max <= f32::EPSILON), q = clamp(round_half_away(v *
 * (1 / scale)), -127, 127); reads dequantise on the fly, (float)q * scale. Caches are int8
 * [batch][max_seq][n_kv][d_head], scale tables f32 [batch][max_seq]. */
int yscv_cuda_rope_kv_append_i8_dev(yscv_cuda_ctx *ctx, float *d_qkv, size_t batch, size_t seq, size_t n_q,
                                    size_t n_kv, size_t d_head, float theta, const int32_t *d_pos,
                                    int8_t *d_kcache, float *d_kscale, int8_t *d_vcache, float *d_vscale,
                                    size_t max_seq);
int yscv_cuda_gqa_attention_i8_dev(yscv_cuda_ctx *ctx, const float *d_q, size_t q_stride, size_t batch,
                                   size_t seq_q, size_t n_q, size_t n_kv, size_t d_head,
                                   const int8_t *d_kcache, const float *d_kscale, const int8_t *d_vcache,
                                   const float *d_vscale, size_t max_seq, const int32_t *d_pos, int causal,
                                   float *d_out);

/* SwiGLU on fused rows [gate | up] with the scalar SiLU of
 * crates/yscv-kernels/src/ops/simd/activation.rs:1000-1005: out = gate/(1+exp(-gate)) * up */
int yscv_cuda_swiglu_dev(yscv_cuda_ctx *ctx, const float *d_gate_up, size_t rows, size_t inter,
                         float *d_out);
/* The same with the result written as the bf16 activations of a following
 * yscv_cuda_int4_matmul_act_dev (inter % 8 == 0, d_out_act 16-byte aligned, rows x inter bf16) */
int yscv_cuda_swiglu_act_dev(yscv_cuda_ctx *ctx, const float *d_gate_up, size_t rows, size_t inter,
                             void *d_out_act);

/* fp32 matmul against a row-major [n,k] weight (the unquantized LM head):
 * out[m,n] = x[m,k] . w[n,k] */
int yscv_cuda_f32_matmul_dev(yscv_cuda_ctx *ctx, const float *d_w, const float *d_x, size_t m,
                             size_t n, size_t k, float *d_out);

/* greedy sampling as apps/llm-bench/src/main.rs:538-543 does it: per row the LAST index
 * among equal maxima */
int yscv_cuda_argmax_last_dev(yscv_cuda_ctx *ctx, const float *d_logits, size_t rows, size_t vocab,
                              int32_t *d_out);

/* *d_pos += by, on the stream (position_offset += 1, apps/llm-bench/src/main.rs:536) */
int yscv_cuda_advance_pos_dev(yscv_cuda_ctx *ctx, int32_t *d_pos, int by);

/* ---- int8 GEMM with the i8 requant epilogues of the quantized convolution path ----------
 * The pointwise (1x1) QLinearConv of the reference is an int8 GEMM over NHWC pixels,
 * A [m = pixels][k = c_in] i8, B [k][n = c_out] i8, followed by a requant pass
 * (crates/yscv-onnx/src/runner/conv/quantized.rs:340-500). Both are fused here.
 *
 * per-channel: int8_matmul_prepacked_dispatch + requant_i8_per_channel_dispatch
 * (crates/yscv-kernels/src/ops/int8_requant.rs:537-556):
 *   out[m,n] = clamp(round_ties_even((float)(acc[m,n] + corr[n]) * composite[n] + y_zp), -128, 127)
 * with the add wrapping as in the reference; corr[n] is what the caller folds together
 * there (bias[n] - x_zp * sum_k w[k,n]), composite[n] = x_scale * w_scale[n] / y_scale. */
int yscv_cuda_int8_matmul_requant_per_channel_dev(yscv_cuda_ctx *ctx, const int8_t *d_a,
                                                  const yscv_cuda_i8b *b, size_t m,
                                                  const int32_t *d_corr, const float *d_composite,
                                                  float y_zero_point, int8_t *d_out);
int yscv_cuda_int8_matmul_requant_per_channel(yscv_cuda_ctx *ctx, const int8_t *a,
                                              const yscv_cuda_i8b *b, size_t m, const int32_t *corr,
                                              const float *composite, float y_zero_point,
                                              int8_t *out);

/* per-tensor: int8_matmul_prepacked_dispatch + requant_i32_row_to_i8_dispatch
 * (int8_requant.rs:81-138, 143-169): optional bias[n] (wrapping add; may be NULL), scalar
 * composite, saturate to [-128,127], optional ReLU after the saturation. */
int yscv_cuda_int8_matmul_requant_i8_dev(yscv_cuda_ctx *ctx, const int8_t *d_a, const yscv_cuda_i8b *b,
                                         size_t m, const int32_t *d_bias, float composite,
                                         float y_zero_point, int relu, int8_t *d_out);
int yscv_cuda_int8_matmul_requant_i8(yscv_cuda_ctx *ctx, const int8_t *a, const yscv_cuda_i8b *b,
                                     size_t m, const int32_t *bias, float composite,
                                     float y_zero_point, int relu, int8_t *out);

/* ---- one decode step in one launch ---------------------------------------------------
 * No single counterpart in the reference: one iteration of the llm-bench decode loop
 * (apps/llm-bench/src/main.rs:491-561) runs the whole ONNX graph, i.e. per layer the
 * operators above in this order: RMSNorm, int4 MatMul (fused q|k|v rows), RoPE + KvCache
 * append, grouped-query attention (causal), int4 MatMul (output) + residual, RMSNorm,
 * int4 MatMul (gate|up rows), SiLU(gate)*up, int4 MatMul (down) + residual. A decode plan
 * runs that sequence for one sequence (or, with options.batch, 2..8 sequences at the same
 * position) as a single persistent cooperative kernel.
 * Requirements (else YSCV_CUDA_ERR_UNSUPPORTED): group size 32; every K a multiple of 512;
 * at least sm_count rows per matrix; hidden and n_q * d_head at most 8192; inter above 8192
 * only while the down projection has at most 128 rows per SM (hidden <= 128 * sm_count);
 * n_q <= sm_count; head_dim a multiple of 16 that divides 512, at most 128; max_seq small
 * enough for the scores of one head chunk in shared memory (about 2 * 10^4).
 * The plan borrows the weights and caches (they must outlive it) and copies the gammas. */
typedef struct yscv_cuda_decode_plan yscv_cuda_decode_plan;

typedef struct yscv_cuda_decode_layer {
    const yscv_cuda_int4_weight *qkv;      /* [(n_q + 2 n_kv) * d_head][hidden] */
    const yscv_cuda_int4_weight *o;        /* [hidden][n_q * d_head] */
    const yscv_cuda_int4_weight *gate_up;  /* [2 * inter][hidden]: gate rows, then up rows */
    const yscv_cuda_int4_weight *down;     /* [hidden][inter] */
    const float *d_gamma_attn;             /* [hidden] */
    const float *d_gamma_mlp;              /* [hidden] */
    void *d_kcache;                        /* [max_seq][n_kv][d_head]: f32, or int8 with options.kv_int8 */
    void *d_vcache;
    float *d_kscale;                       /* int8 caches only: [max_seq] f32, one scale per cached row */
    float *d_vscale;
} yscv_cuda_decode_layer;

int yscv_cuda_decode_plan_create(yscv_cuda_ctx *ctx, const yscv_cuda_decode_layer *layers,
                                 size_t n_layers, size_t hidden, size_t inter, size_t n_q,
                                 size_t n_kv, size_t d_head, size_t max_seq, float eps,
                                 float rope_theta, yscv_cuda_decode_plan **out);

/* Tensor-parallel decode steps. No counterpart in the reference (it has no multi-GPU
 * inference: crates/yscv-model/src/distributed.rs:27). One process per GPU; rank r of a group
 * of `world` (2..8) GPUs of one machine holds the column-parallel shard of qkv and gate|up
 * (its heads, its intermediate channels) and the row-parallel shard of the output and down
 * projections (its K slice), as yscv_b200/sharding.py cuts them. _create allocates this
 * rank's exchange region (2 * world * max_rows 8-byte words; max_rows >= hidden) and writes
 * its IPC handle; the host gathers every rank's handle (YSCV_CUDA_TP_HANDLE_BYTES each, in
 * rank order) and gives them to _connect, which maps the peers' regions. A plan built with
 * the connected group then exchanges the partial sums of the row-parallel GEMVs inside the
 * step kernel: plain 8-byte stores {f32 value, 32-bit tag} into every peer's region over
 * NVLink, a bounded poll of the own region, sums in rank order (identical bits on every
 * rank). Every rank must run the same sequence of steps; destroy the plan and the group on
 * every rank only after all of them have finished their last step. */
typedef struct yscv_cuda_tp_comm yscv_cuda_tp_comm;
#define YSCV_CUDA_TP_HANDLE_BYTES 64
int yscv_cuda_tp_comm_create(yscv_cuda_ctx *ctx, int rank, int world, size_t max_rows,
                             yscv_cuda_tp_comm **out, uint8_t handle_out[YSCV_CUDA_TP_HANDLE_BYTES]);
int yscv_cuda_tp_comm_connect(yscv_cuda_tp_comm *comm, const uint8_t *handles /* world x 64 bytes */);
void yscv_cuda_tp_comm_destroy(yscv_cuda_tp_comm *comm);
/* Test form of _connect: the peers' regions are stand-ins in this GPU's memory that nobody
 * ever writes, so every wait for a peer runs out. Used to exercise the give-up path of the
 * bounded waits on one GPU (with a short spin_limit below). */
int yscv_cuda_tp_comm_connect_unanswered(yscv_cuda_tp_comm *comm);

/* Optional settings of a plan; a NULL pointer or a zeroed struct with variant =
 * attention_form = -1 means the defaults. The geometry fields exist so that tests can push
 * small shapes down the paths large models take. */
typedef struct yscv_cuda_decode_options {
    int variant;        /* -1: default. Bit mask: 1 gate/up rows paired (SwiGLU in the store),
                           2 sixteen K slices for one-tile slabs, 4 split-merge weight table,
                           8 relaxed barrier polling */
    int max_tiles;      /* 0: default (8). 16-row tiles per row block, 2..8, even */
    int k_chunk;        /* 0: default (8192). k per resident chunk of digit planes, multiple of 512 */
    int attention_form; /* -1: chosen from max_seq. 0: CTAs per query head; 1: per KV head and key chunk */
    int spin_limit;     /* 0: default (2^21 probes, about a second). Probes after which a wait
                           for another CTA or another GPU gives up */
    const yscv_cuda_tp_comm *tp; /* NULL: one GPU. Else this rank's connected group; the layer
                                    weights and n_q, n_kv, inter are then the rank's shards */
    int kv_int8;        /* 0: f32 caches. 1: the caches are KvDtype::I8 as yscv_cuda_rope_kv_append_i8_dev
                           writes them (int8 rows of n_kv * d_head with one f32 scale per row in
                           d_kscale / d_vscale); d_head must be 64 or 128. Under tensor parallelism a
                           row is this rank's KV heads only, so its scale differs from the one-GPU one */
    int batch;          /* 0 or 1: one sequence per step. 2..8: that many sequences per step, all at the
                           same position (the batched decode of apps/llm-bench/src/main.rs:491-561):
                           d_token, d_x, d_logits then hold one entry / row per sequence
                           ([batch], [batch][hidden], [batch][vocab]) and the caches are
                           [batch][max_seq][n_kv][d_head]. One GPU, f32 caches, hidden and
                           n_q * d_head at most 2048 */
} yscv_cuda_decode_options;
int yscv_cuda_decode_plan_create_ex(yscv_cuda_ctx *ctx, const yscv_cuda_decode_layer *layers,
                                    size_t n_layers, size_t hidden, size_t inter, size_t n_q,
                                    size_t n_kv, size_t d_head, size_t max_seq, float eps,
                                    float rope_theta, const yscv_cuda_decode_options *opt,
                                    yscv_cuda_decode_plan **out);

/* Synchronises the stream and reports whether a bounded wait ran out in any step of this plan
 * so far: YSCV_CUDA_ERR_TIMEOUT if so. From then on the plan is poisoned: every later step
 * call returns YSCV_CUDA_ERR_TIMEOUT without launching (steps enqueued before the check still
 * fall through all their waits and set the context's status word to 2 again). Rebuild the
 * plan (and, for a tensor-parallel one, the group on every rank). */
int yscv_cuda_decode_plan_check(yscv_cuda_ctx *ctx, yscv_cuda_decode_plan *plan);

/* x = embedding[*d_token], then every layer at position *d_pos (appending to the caches at
 * that position); leaves the residual stream after the last layer, before the final norm,
 * in d_x [hidden]. Asynchronous on the context's stream. A device-side wait that runs out
 * sets the context's status word (yscv_cuda_ctx_device_status) and the plan must then be
 * rebuilt (yscv_cuda_decode_plan_check). A position outside [0, max_seq) computes and
 * appends nothing and sets the status word to 3. */
int yscv_cuda_decode_plan_step_dev(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan,
                                   const float *d_embedding, size_t vocab, const int32_t *d_token,
                                   const int32_t *d_pos, float *d_x);

/* The same step followed, in the same launch, by what llm-bench does after the graph
 * (apps/llm-bench/src/main.rs:536-543): the final RMSNorm (d_final_gamma [hidden]), the fp32 LM
 * head d_lm_head [vocab][hidden] -> d_logits [vocab], the greedy token (last index among equal
 * maxima) written to *d_token, and *d_pos += 1. d_x receives the residual stream as above. */
int yscv_cuda_decode_plan_step_token_dev(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan,
                                         const float *d_embedding, size_t vocab, int32_t *d_token,
                                         int32_t *d_pos, const float *d_final_gamma,
                                         const float *d_lm_head, float *d_x, float *d_logits);

/* The same with the LM head split by rows across the ranks of a tensor-parallel plan: this
 * rank holds rows [lm_row0, lm_row0 + lm_rows) of the LM head in d_lm_head_rows
 * [lm_rows][hidden] and writes only those entries of d_logits [vocab]; the ranks exchange
 * their best (value, index) inside the kernel and every rank writes the same greedy token.
 * (The plain entry point above, given a tensor-parallel plan, computes every row on every
 * rank.) */
int yscv_cuda_decode_plan_step_token_shard_dev(yscv_cuda_ctx *ctx, const yscv_cuda_decode_plan *plan,
                                               const float *d_embedding, size_t vocab, int32_t *d_token,
                                               int32_t *d_pos, const float *d_final_gamma,
                                               const float *d_lm_head_rows, size_t lm_row0, size_t lm_rows,
                                               float *d_x, float *d_logits);

void yscv_cuda_decode_plan_free(yscv_cuda_decode_plan *plan);

#ifdef __cplusplus
}
#endif
#endif
