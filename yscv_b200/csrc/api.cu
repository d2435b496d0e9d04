// C ABI of the library (see include/yscv_cuda.h): argument validation, host
// staging for the drop-in entry points, dispatch to the kernels.
#include <cstdlib>
#include <cstring>
#include <set>

#include "common.cuh"
#include "kernels.cuh"

namespace yscv {

std::string &last_error() {
    static thread_local std::string s;
    return s;
}

int fail(int status, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error() = buf;
    return status;
}

int ensure_dynamic_smem(const void *kernel, int device, int bytes) {
    static std::mutex mu;
    static std::set<std::pair<const void *, int>> done;
    std::lock_guard<std::mutex> lock(mu);
    if (done.count({kernel, device})) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done.insert({kernel, device});
    return YSCV_CUDA_OK;
}

OpCounters &op_counters() {
    static OpCounters c;
    return c;
}

int DeviceBuffer::reserve(size_t want) {
    if (want <= bytes && ptr) return YSCV_CUDA_OK;
    if (ptr) {
        YSCV_CUDA_TRY(cudaFree(ptr));
        ptr = nullptr;
        bytes = 0;
    }
    size_t sz = want < 256 ? 256 : want;
    YSCV_CUDA_TRY(cudaMalloc(&ptr, sz));
    bytes = sz;
    return YSCV_CUDA_OK;
}

void DeviceBuffer::release() {
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    bytes = 0;
}

static int check_int4_shape(size_t n, size_t k, size_t gs) {
    if (gs == 0 || (gs & 1)) return fail(YSCV_CUDA_ERR_BAD_ARG, "group_size must be even and > 0, got %zu", gs);
    if (k == 0 || k % gs != 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "k=%zu must be a positive multiple of group_size=%zu", k, gs);
    if (n == 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "weight has no rows");
    if (n >= (1u << 30) || k >= (1u << 30)) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "dimension too large");
    return YSCV_CUDA_OK;
}

// device-pointer int4 matmul, any m
static int int4_matmul_dev(yscv_cuda_ctx *ctx, const uint8_t *d_packed, const float *d_scales,
                           size_t n, size_t k, size_t gs, const float *d_act, float *d_out,
                           size_t m) {
    int rc = check_int4_shape(n, k, gs);
    if (rc) return rc;
    if (m == 0) return YSCV_CUDA_OK;
    // prefill shapes: dequantise to bf16 in shared memory, tcgen05 MMA, fp32 accumulate
    // (yscv_cuda_ctx_set_int4_prefill_exact keeps the fp32-exact kernel, 16 rows per pass)
    const bool exact_prefill = ctx->prefill_exact;
    const bool all_aligned = ((reinterpret_cast<uintptr_t>(d_packed) | reinterpret_cast<uintptr_t>(d_scales) |
                               reinterpret_cast<uintptr_t>(d_act)) & 15) == 0;
    if (!exact_prefill && all_aligned && int4_prefill_supported(m, n, k, gs)) {
        rc = ctx->scratch.reserve(int4_prefill_scratch_bytes(m, k));
        if (rc) return rc;
        op_counters().int4_gemm_calls++;
        return int4_prefill_gemm(ctx, d_packed, d_scales, d_act, d_out, m, n, k, ctx->scratch.ptr);
    }
    for (size_t m0 = 0; m0 < m; m0 += 16) {
        const size_t mc = m - m0 < 16 ? m - m0 : 16;
        const float *a = d_act + m0 * k;
        float *o = d_out + m0 * n;
        const bool aligned = ((reinterpret_cast<uintptr_t>(d_packed) | reinterpret_cast<uintptr_t>(d_scales) |
                               reinterpret_cast<uintptr_t>(a)) & 15) == 0;
        if (aligned && int4_gemv_fast_supported(mc, n, k, gs)) {
            rc = ctx->scratch.reserve(int4_gemv_scratch_bytes(16, k));
            if (rc) return rc;
            rc = int4_gemv_fast(ctx, d_packed, d_scales, a, o, mc, n, k, ctx->scratch.ptr);
            op_counters().int4_gemv_calls++;
        } else {
            rc = int4_gemv_generic(ctx, d_packed, d_scales, a, o, mc, n, k, gs);
            op_counters().int4_generic_calls++;
            snprintf(ctx->report_int4, sizeof(ctx->report_int4),
                     "int4_gemv_generic m=%zu n=%zu k=%zu group=%zu: warp per row, fp32 FMAs", mc, n, k, gs);
        }
        if (rc) return rc;
    }
    return YSCV_CUDA_OK;
}

}  // namespace yscv

// The event pairs are created by yscv_cuda_ctx_profile_enable, never here: a launch path
// must not allocate (launches past the pool are simply not bracketed).
void yscv_cuda_ctx::prof_begin() {
    if (!profiling || prof_used >= prof_events.size()) return;
    cudaEventRecord(prof_events[prof_used].first, stream);
}

void yscv_cuda_ctx::prof_end() {
    if (!profiling || prof_used >= prof_events.size()) return;
    cudaEventRecord(prof_events[prof_used].second, stream);
    prof_used++;
}

using namespace yscv;

extern "C" {

const char *yscv_cuda_last_error(void) { return last_error().c_str(); }

static int ctx_create_impl(int device, cudaStream_t stream, bool borrow, yscv_cuda_ctx **out) {
    if (!out) return fail(YSCV_CUDA_ERR_BAD_ARG, "out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(YSCV_CUDA_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(e));
    if (device < 0 || device >= count) return fail(YSCV_CUDA_ERR_BAD_ARG, "device %d out of range (%d visible)", device, count);
    cudaDeviceProp prop;
    YSCV_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(YSCV_CUDA_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only",
                    device, prop.major, prop.minor);
    YSCV_CUDA_TRY(cudaSetDevice(device));
    yscv_cuda_ctx *ctx = new yscv_cuda_ctx();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    if (borrow) {
        ctx->stream = stream;
        ctx->owns_stream = false;
    } else {
        cudaError_t se = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (se != cudaSuccess) {
            delete ctx;
            return fail(YSCV_CUDA_ERR_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(se));
        }
        ctx->owns_stream = true;
    }
    cudaError_t me = cudaMalloc(&ctx->d_status, sizeof(int));
    if (me == cudaSuccess) me = cudaMemset(ctx->d_status, 0, sizeof(int));
    if (me != cudaSuccess) {
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        return fail(YSCV_CUDA_ERR_CUDA, "status word: %s", cudaGetErrorString(me));
    }
    *out = ctx;
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_create(int device, yscv_cuda_ctx **out) {
    return ctx_create_impl(device, nullptr, false, out);
}

int yscv_cuda_ctx_create_on_stream(int device, void *cuda_stream, yscv_cuda_ctx **out) {
    return ctx_create_impl(device, reinterpret_cast<cudaStream_t>(cuda_stream), true, out);
}

void yscv_cuda_ctx_destroy(yscv_cuda_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    ctx->in0.release();
    ctx->in1.release();
    ctx->in2.release();
    ctx->out0.release();
    ctx->out1.release();
    ctx->scratch.release();
    ctx->scratch_attn.release();
    ctx->rowsum.release();
    ctx->tmp_bt.release();
    ctx->gemm_ws.release();
    ctx->gemm_flags.release();
    ctx->tmp_colsum.release();
    if (ctx->d_status) cudaFree(ctx->d_status);
    for (auto &ev : ctx->prof_events) {
        cudaEventDestroy(ev.first);
        cudaEventDestroy(ev.second);
    }
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int yscv_cuda_ctx_synchronize(yscv_cuda_ctx *ctx) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_device_status(yscv_cuda_ctx *ctx, int *status) {
    if (!ctx || !status) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    YSCV_CUDA_TRY(cudaMemcpyAsync(status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_profile_enable(yscv_cuda_ctx *ctx, int enable) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (enable) {
        YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
        while (ctx->prof_events.size() < 4096) {
            cudaEvent_t a, b;
            YSCV_CUDA_TRY(cudaEventCreate(&a));
            cudaError_t e = cudaEventCreate(&b);
            if (e != cudaSuccess) {
                cudaEventDestroy(a);
                return fail(YSCV_CUDA_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(e));
            }
            ctx->prof_events.emplace_back(a, b);
        }
    }
    ctx->profiling = enable != 0;
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_profile_read(yscv_cuda_ctx *ctx, uint64_t *launches, double *total_ms) {
    if (!ctx || !launches || !total_ms) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    double sum = 0.0;
    for (size_t i = 0; i < ctx->prof_used; ++i) {
        float ms = 0.0f;
        YSCV_CUDA_TRY(cudaEventElapsedTime(&ms, ctx->prof_events[i].first, ctx->prof_events[i].second));
        sum += ms;
    }
    *launches = ctx->prof_used;
    *total_ms = sum;
    ctx->prof_used = 0;
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_set_int4_prefill_exact(yscv_cuda_ctx *ctx, int exact) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    ctx->prefill_exact = exact != 0;
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_set_int4_prefill_cta_pairs(yscv_cuda_ctx *ctx, int enable) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    ctx->prefill_pairs = enable != 0;
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_set_int8_cta_pairs(yscv_cuda_ctx *ctx, int mode) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    ctx->int8_pairs = mode < 0 ? -1 : (mode > 0 ? 1 : 0);
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_set_int8_tail_split(yscv_cuda_ctx *ctx, int enable) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    ctx->int8_tail_split = enable != 0;
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_set_f32_tensor_cores(yscv_cuda_ctx *ctx, int enable) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    ctx->f32_tensor_cores = enable != 0;
    return YSCV_CUDA_OK;
}

int yscv_cuda_ctx_set_attention_tensor_cores(yscv_cuda_ctx *ctx, int enable) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    ctx->attn_tensor_cores = enable != 0;
    return YSCV_CUDA_OK;
}

const char *yscv_cuda_last_kernel(const yscv_cuda_ctx *ctx) { return ctx ? ctx->last_kernel : "none"; }

uint64_t yscv_cuda_ctx_launch_count(const yscv_cuda_ctx *ctx) { return ctx ? ctx->launches : 0; }

/* ---- int4 host drop-ins ---------------------------------------------------- */

int yscv_cuda_packed_int4_gemm(yscv_cuda_ctx *ctx, const uint8_t *weight_packed,
                               const float *scales, const float *activation, float *output,
                               size_t m, size_t n, size_t k, size_t group_size) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (!weight_packed || !scales || !activation || !output)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    int rc = check_int4_shape(n, k, group_size);
    if (rc) return rc;
    if (m == 0) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t wb = n * k / 2, sb = n * (k / group_size) * sizeof(float);
    const size_t ab = m * k * sizeof(float), ob = m * n * sizeof(float);
    if ((rc = ctx->in0.reserve(wb)) || (rc = ctx->in1.reserve(sb)) || (rc = ctx->in2.reserve(ab)) ||
        (rc = ctx->out0.reserve(ob)))
        return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in0.ptr, weight_packed, wb, cudaMemcpyHostToDevice, ctx->stream));
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in1.ptr, scales, sb, cudaMemcpyHostToDevice, ctx->stream));
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in2.ptr, activation, ab, cudaMemcpyHostToDevice, ctx->stream));
    rc = int4_matmul_dev(ctx, (const uint8_t *)ctx->in0.ptr, (const float *)ctx->in1.ptr, n, k,
                         group_size, (const float *)ctx->in2.ptr, (float *)ctx->out0.ptr, m);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(output, ctx->out0.ptr, ob, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

int yscv_cuda_packed_int4_gemv(yscv_cuda_ctx *ctx, const uint8_t *weight_packed,
                               const float *scales, const float *activation, float *output,
                               size_t m_w, size_t k, size_t group_size) {
    return yscv_cuda_packed_int4_gemm(ctx, weight_packed, scales, activation, output, 1, m_w, k,
                                      group_size);
}

int yscv_cuda_int4_from_matmulnbits_dev(yscv_cuda_ctx *ctx, const uint8_t *d_src, uint8_t *d_dst,
                                        size_t bytes) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (bytes && (!d_src || !d_dst)) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    return int4_from_matmulnbits(ctx, d_src, d_dst, bytes);
}

int yscv_cuda_int4_from_matmulnbits(const uint8_t *src, uint8_t *dst, size_t bytes) {
    if (bytes && (!src || !dst)) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    for (size_t i = 0; i < bytes; ++i) dst[i] = (uint8_t)(src[i] ^ 0x88u);
    return YSCV_CUDA_OK;
}

int yscv_cuda_pack_int4_dev(yscv_cuda_ctx *ctx, const float *d_weights, size_t m_w, size_t k,
                            size_t group_size, uint8_t *d_packed, float *d_scales) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (!d_weights || !d_packed || !d_scales) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    int rc = check_int4_shape(m_w, k, group_size);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    return pack_int4(ctx, d_weights, m_w, k, group_size, d_packed, d_scales);
}

int yscv_cuda_pack_int4_symmetric_per_group(yscv_cuda_ctx *ctx, const float *weights, size_t m_w,
                                            size_t k, size_t group_size, uint8_t *packed,
                                            float *scales) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (!weights || !packed || !scales) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    int rc = check_int4_shape(m_w, k, group_size);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t wb = m_w * k * sizeof(float), pb = m_w * k / 2;
    const size_t sb = m_w * (k / group_size) * sizeof(float);
    if ((rc = ctx->in0.reserve(wb)) || (rc = ctx->out0.reserve(pb)) || (rc = ctx->out1.reserve(sb)))
        return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in0.ptr, weights, wb, cudaMemcpyHostToDevice, ctx->stream));
    rc = pack_int4(ctx, (const float *)ctx->in0.ptr, m_w, k, group_size, (uint8_t *)ctx->out0.ptr,
                   (float *)ctx->out1.ptr);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(packed, ctx->out0.ptr, pb, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaMemcpyAsync(scales, ctx->out1.ptr, sb, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

/* ---- int4 device-resident forms -------------------------------------------- */

int yscv_cuda_int4_weight_upload(yscv_cuda_ctx *ctx, const uint8_t *packed, const float *scales,
                                 size_t m_w, size_t k, size_t group_size,
                                 yscv_cuda_int4_weight **out) {
    if (!ctx || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (!packed || !scales) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    int rc = check_int4_shape(m_w, k, group_size);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t wb = m_w * k / 2, sb = m_w * (k / group_size) * sizeof(float);
    void *dp = nullptr, *ds = nullptr;
    YSCV_CUDA_TRY(cudaMalloc(&dp, wb));
    cudaError_t e = cudaMalloc(&ds, sb);
    if (e == cudaSuccess) e = cudaMemcpyAsync(dp, packed, wb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(ds, scales, sb, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(dp);
        if (ds) cudaFree(ds);
        return fail(YSCV_CUDA_ERR_CUDA, "int4 weight upload: %s", cudaGetErrorString(e));
    }
    auto *w = new yscv_cuda_int4_weight();
    w->d_packed = (const uint8_t *)dp;
    w->d_scales = (const float *)ds;
    w->m_w = m_w;
    w->k = k;
    w->group_size = group_size;
    w->owns = true;
    w->device = ctx->device;
    *out = w;
    return YSCV_CUDA_OK;
}

int yscv_cuda_int4_weight_wrap(const uint8_t *d_packed, const float *d_scales, size_t m_w, size_t k,
                               size_t group_size, yscv_cuda_int4_weight **out) {
    if (!out) return fail(YSCV_CUDA_ERR_BAD_ARG, "out is null");
    *out = nullptr;
    if (!d_packed || !d_scales) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    int rc = check_int4_shape(m_w, k, group_size);
    if (rc) return rc;
    auto *w = new yscv_cuda_int4_weight();
    w->d_packed = d_packed;
    w->d_scales = d_scales;
    w->m_w = m_w;
    w->k = k;
    w->group_size = group_size;
    w->owns = false;
    w->device = -1;
    *out = w;
    return YSCV_CUDA_OK;
}

void yscv_cuda_int4_weight_free(yscv_cuda_int4_weight *w) {
    if (!w) return;
    if (w->owns) {
        cudaSetDevice(w->device);
        cudaFree(const_cast<uint8_t *>(w->d_packed));
        cudaFree(const_cast<float *>(w->d_scales));
    }
    delete w;
}

int yscv_cuda_int4_matmul_dev(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w,
                              const float *d_activation, float *d_output, size_t m) {
    if (!ctx || !w) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!d_activation || !d_output) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    return int4_matmul_dev(ctx, w->d_packed, w->d_scales, w->m_w, w->k, w->group_size, d_activation,
                           d_output, m);
}

int yscv_cuda_int4_matmul_act_dev(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w,
                                  const void *d_activation_bf16, float *d_output, size_t m) {
    if (!ctx || !w) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!d_activation_bf16 || !d_output) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    int rc = check_int4_shape(w->m_w, w->k, w->group_size);
    if (rc) return rc;
    if (m == 0) return YSCV_CUDA_OK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(w->d_packed) | reinterpret_cast<uintptr_t>(w->d_scales) |
                           reinterpret_cast<uintptr_t>(d_activation_bf16)) & 15) == 0;
    if (ctx->prefill_exact || !aligned || !int4_prefill_supported(m, w->m_w, w->k, w->group_size))
        return fail(YSCV_CUDA_ERR_UNSUPPORTED,
                    "bf16 activations need the tensor-core prefill path: m > 16, group 32, k %% 64 == 0, 16-byte "
                    "aligned operands, exact-prefill mode off (m=%zu n=%zu k=%zu)", m, w->m_w, w->k);
    op_counters().int4_gemm_calls++;
    return int4_prefill_gemm(ctx, w->d_packed, w->d_scales, nullptr, d_output, m, w->m_w, w->k, nullptr,
                             d_activation_bf16);
}

// Device alias of a host buffer the kernels may write directly (page-locked and mapped into the
// device's address space: cudaHostAlloc / cudaHostRegister memory under unified addressing),
// or null for pageable memory.
static void *mapped_alias(const void *host) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, host) != cudaSuccess) {
        cudaGetLastError();  // (older runtimes report pageable memory as an error)
        return nullptr;
    }
    return at.type == cudaMemoryTypeHost ? at.devicePointer : nullptr;
}

int yscv_cuda_int4_matmul(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w,
                          const float *activation, float *output, size_t m) {
    if (!ctx || !w) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!activation || !output) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (m == 0) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t ab = m * w->k * sizeof(float), ob = m * w->m_w * sizeof(float);
    int rc;
    if ((rc = ctx->in2.reserve(ab))) return rc;
    // A page-locked output buffer is written by the kernel itself (posted writes over PCIe, no
    // copy-engine pass behind the kernel); a pageable one goes through the staging buffer. The
    // activations are always copied in: every CTA reads all of them, which must not cross PCIe
    // 148 times.
    float *d_out = m <= 16 ? static_cast<float *>(mapped_alias(output)) : nullptr;
    const bool direct = d_out != nullptr && (reinterpret_cast<uintptr_t>(d_out) & 15) == 0;
    if (!direct) {
        if ((rc = ctx->out0.reserve(ob))) return rc;
        d_out = (float *)ctx->out0.ptr;
    }
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in2.ptr, activation, ab, cudaMemcpyHostToDevice, ctx->stream));
    rc = int4_matmul_dev(ctx, w->d_packed, w->d_scales, w->m_w, w->k, w->group_size,
                         (const float *)ctx->in2.ptr, d_out, m);
    if (rc) return rc;
    if (!direct) YSCV_CUDA_TRY(cudaMemcpyAsync(output, ctx->out0.ptr, ob, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

/* ---- int8 GEMM -------------------------------------------------------------- */

static int i8b_create(yscv_cuda_ctx *ctx, const int8_t *d_b, size_t k, size_t n, yscv_cuda_i8b **out) {
    const size_t kp = (k + 15) / 16 * 16;
    void *bt = nullptr, *cs = nullptr;
    YSCV_CUDA_TRY(cudaMalloc(&bt, n * kp));
    cudaError_t e = cudaMalloc(&cs, n * sizeof(int32_t));
    if (e != cudaSuccess) {
        cudaFree(bt);
        return fail(YSCV_CUDA_ERR_CUDA, "cudaMalloc(colsum): %s", cudaGetErrorString(e));
    }
    int rc = pack_i8_b(ctx, d_b, k, n, (int8_t *)bt, (int32_t *)cs, kp);
    if (rc) {
        cudaFree(bt);
        cudaFree(cs);
        return rc;
    }
    auto *h = new yscv_cuda_i8b();
    h->d_bt = (int8_t *)bt;
    h->d_colsum = (int32_t *)cs;
    h->k = k;
    h->n = n;
    h->kp = kp;
    h->device = ctx->device;
    *out = h;
    return YSCV_CUDA_OK;
}

static int check_i8_shape(size_t k, size_t n) {
    if (k == 0 || n == 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "int8 GEMM needs k > 0 and n > 0");
    if (k >= (1u << 30) || n >= (1u << 30)) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "dimension too large");
    return YSCV_CUDA_OK;
}

int yscv_cuda_pack_i8_b_dev(yscv_cuda_ctx *ctx, const int8_t *d_b, size_t k, size_t n,
                            yscv_cuda_i8b **out) {
    if (!ctx || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (!d_b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    int rc = check_i8_shape(k, n);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    return i8b_create(ctx, d_b, k, n, out);
}

int yscv_cuda_pack_i8_b_for_matmul(yscv_cuda_ctx *ctx, const int8_t *b, size_t k, size_t n,
                                   yscv_cuda_i8b **out) {
    if (!ctx || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (!b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    int rc = check_i8_shape(k, n);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    if ((rc = ctx->in1.reserve(k * n))) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in1.ptr, b, k * n, cudaMemcpyHostToDevice, ctx->stream));
    rc = i8b_create(ctx, (const int8_t *)ctx->in1.ptr, k, n, out);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

void yscv_cuda_i8b_free(yscv_cuda_i8b *b) {
    if (!b) return;
    cudaSetDevice(b->device);
    cudaFree(b->d_bt);
    cudaFree(b->d_colsum);
    delete b;
}

int yscv_cuda_i8b_set_zero_point(yscv_cuda_i8b *b, int32_t b_zero_point) {
    if (!b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null handle");
    if (b_zero_point < -128 || b_zero_point > 127)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "b_zero_point %d is not an int8 value", (int)b_zero_point);
    b->b_zp = (int)b_zero_point;
    return YSCV_CUDA_OK;
}

size_t yscv_cuda_i8b_k(const yscv_cuda_i8b *b) { return b ? b->k : 0; }
size_t yscv_cuda_i8b_n(const yscv_cuda_i8b *b) { return b ? b->n : 0; }

static int i8_gemm_dev(yscv_cuda_ctx *ctx, const void *d_a, const yscv_cuda_i8b *b, size_t m,
                       void *d_out, int a_unsigned, int a_zp, const yscv_cuda_requant *rq) {
    if (!ctx || !b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!d_a || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (m == 0) return YSCV_CUDA_OK;
    if (m >= (1u << 30)) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "dimension too large");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    op_counters().int8_gemm_calls++;
    if (rq) {
        op_counters().qlinear_matmul_calls++;
        if (rq->qmin > rq->qmax || rq->qmin < -128 || rq->qmax > 255 || rq->qmax - rq->qmin > 255)
            return fail(YSCV_CUDA_ERR_BAD_ARG, "requant range [%d,%d] does not fit one byte", rq->qmin, rq->qmax);
        return int8_gemm(ctx, d_a, b, m, d_out, rq->a_is_unsigned, rq->a_zero_point, 1, rq->composite,
                         rq->y_zero_point, rq->qmin, rq->qmax, rq->round_mode);
    }
    return int8_gemm(ctx, d_a, b, m, d_out, a_unsigned, a_zp, 0, 0.0f, 0.0f, 0, 0, 0);
}

// host A in, host output out (elem_bytes per output element)
static int i8_gemm_host(yscv_cuda_ctx *ctx, const void *a, const yscv_cuda_i8b *b, size_t m, void *out,
                        size_t elem_bytes, int a_unsigned, int a_zp, const yscv_cuda_requant *rq) {
    if (!ctx || !b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!a || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (m == 0) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t ab = m * b->k, ob = m * b->n * elem_bytes;
    int rc;
    if ((rc = ctx->in0.reserve(ab)) || (rc = ctx->out0.reserve(ob))) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in0.ptr, a, ab, cudaMemcpyHostToDevice, ctx->stream));
    rc = i8_gemm_dev(ctx, ctx->in0.ptr, b, m, ctx->out0.ptr, a_unsigned, a_zp, rq);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(out, ctx->out0.ptr, ob, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

int yscv_cuda_int8_matmul_prepacked_dev(yscv_cuda_ctx *ctx, const int8_t *d_a, const yscv_cuda_i8b *b,
                                        size_t m, int32_t *d_out) {
    return i8_gemm_dev(ctx, d_a, b, m, d_out, 0, 0, nullptr);
}

int yscv_cuda_int8_matmul_prepacked(yscv_cuda_ctx *ctx, const int8_t *a, const yscv_cuda_i8b *b,
                                    size_t m, int32_t *out) {
    return i8_gemm_host(ctx, a, b, m, out, sizeof(int32_t), 0, 0, nullptr);
}

int yscv_cuda_int8_matmul(yscv_cuda_ctx *ctx, const int8_t *a, const int8_t *b, size_t m, size_t k,
                          size_t n, int32_t *out) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (!a || !b || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (m == 0 || n == 0) return YSCV_CUDA_OK;
    if (k == 0) {
        memset(out, 0, m * n * sizeof(int32_t));
        return YSCV_CUDA_OK;
    }
    int rc = check_i8_shape(k, n);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    // B^T and its column sums live in buffers the context keeps (grow-only): no allocation
    // per call once the largest shape has been seen
    const size_t kp = (k + 15) / 16 * 16;
    if ((rc = ctx->in1.reserve(k * n)) || (rc = ctx->tmp_bt.reserve(n * kp)) ||
        (rc = ctx->tmp_colsum.reserve(n * sizeof(int32_t))))
        return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in1.ptr, b, k * n, cudaMemcpyHostToDevice, ctx->stream));
    rc = pack_i8_b(ctx, (const int8_t *)ctx->in1.ptr, k, n, (int8_t *)ctx->tmp_bt.ptr,
                   (int32_t *)ctx->tmp_colsum.ptr, kp);
    if (rc) return rc;
    yscv_cuda_i8b view;
    view.d_bt = (int8_t *)ctx->tmp_bt.ptr;
    view.d_colsum = (int32_t *)ctx->tmp_colsum.ptr;
    view.k = k;
    view.n = n;
    view.kp = kp;
    view.device = ctx->device;
    return yscv_cuda_int8_matmul_prepacked(ctx, a, &view, m, out);
}

int yscv_cuda_qlinear_matmul_dev(yscv_cuda_ctx *ctx, const void *d_a, const yscv_cuda_i8b *b, size_t m,
                                 const yscv_cuda_requant *rq, void *d_out) {
    if (!rq) return fail(YSCV_CUDA_ERR_BAD_ARG, "requant parameters are null");
    return i8_gemm_dev(ctx, d_a, b, m, d_out, 0, 0, rq);
}

int yscv_cuda_qlinear_matmul(yscv_cuda_ctx *ctx, const void *a, const yscv_cuda_i8b *b, size_t m,
                             const yscv_cuda_requant *rq, void *out) {
    if (!rq) return fail(YSCV_CUDA_ERR_BAD_ARG, "requant parameters are null");
    return i8_gemm_host(ctx, a, b, m, out, 1, 0, 0, rq);
}

// ---- int8 GEMM + the i8 requant epilogues of the convolution path ----

static int i8_requant_i8_dev(yscv_cuda_ctx *ctx, const int8_t *d_a, const yscv_cuda_i8b *b, size_t m,
                             const int32_t *d_corr, const float *d_comp_pc, float composite, float y_zp,
                             int relu, int8_t *d_out) {
    if (!ctx || !b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!d_a || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (m == 0) return YSCV_CUDA_OK;
    if (m >= (1u << 30)) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "dimension too large");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    op_counters().int8_gemm_calls++;
    return int8_gemm(ctx, d_a, b, m, d_out, 0, 0, 1, composite, y_zp, -128, 127, 0, d_corr, d_comp_pc, relu);
}

int yscv_cuda_int8_matmul_requant_per_channel_dev(yscv_cuda_ctx *ctx, const int8_t *d_a,
                                                  const yscv_cuda_i8b *b, size_t m, const int32_t *d_corr,
                                                  const float *d_composite, float y_zero_point,
                                                  int8_t *d_out) {
    if (!d_corr || !d_composite) return fail(YSCV_CUDA_ERR_BAD_ARG, "null per-channel vector");
    return i8_requant_i8_dev(ctx, d_a, b, m, d_corr, d_composite, 0.0f, y_zero_point, 0, d_out);
}

int yscv_cuda_int8_matmul_requant_i8_dev(yscv_cuda_ctx *ctx, const int8_t *d_a, const yscv_cuda_i8b *b,
                                         size_t m, const int32_t *d_bias, float composite,
                                         float y_zero_point, int relu, int8_t *d_out) {
    return i8_requant_i8_dev(ctx, d_a, b, m, d_bias, nullptr, composite, y_zero_point, relu, d_out);
}

// host operands: A, the per-channel vectors and the output are staged through the context
static int i8_requant_i8_host(yscv_cuda_ctx *ctx, const int8_t *a, const yscv_cuda_i8b *b, size_t m,
                              const int32_t *corr, const float *comp_pc, float composite, float y_zp,
                              int relu, int8_t *out) {
    if (!ctx || !b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!a || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (m == 0) return YSCV_CUDA_OK;
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t ab = m * b->k, ob = m * b->n, vb = b->n * 4;
    int rc;
    if ((rc = ctx->in0.reserve(ab)) || (rc = ctx->out0.reserve(ob)) || (rc = ctx->in1.reserve(vb)) ||
        (rc = ctx->in2.reserve(vb)))
        return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in0.ptr, a, ab, cudaMemcpyHostToDevice, ctx->stream));
    if (corr) YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in1.ptr, corr, vb, cudaMemcpyHostToDevice, ctx->stream));
    if (comp_pc) YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in2.ptr, comp_pc, vb, cudaMemcpyHostToDevice, ctx->stream));
    rc = i8_requant_i8_dev(ctx, (const int8_t *)ctx->in0.ptr, b, m, corr ? (const int32_t *)ctx->in1.ptr : nullptr,
                           comp_pc ? (const float *)ctx->in2.ptr : nullptr, composite, y_zp, relu,
                           (int8_t *)ctx->out0.ptr);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(out, ctx->out0.ptr, ob, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

int yscv_cuda_int8_matmul_requant_per_channel(yscv_cuda_ctx *ctx, const int8_t *a, const yscv_cuda_i8b *b,
                                              size_t m, const int32_t *corr, const float *composite,
                                              float y_zero_point, int8_t *out) {
    if (!corr || !composite) return fail(YSCV_CUDA_ERR_BAD_ARG, "null per-channel vector");
    return i8_requant_i8_host(ctx, a, b, m, corr, composite, 0.0f, y_zero_point, 0, out);
}

int yscv_cuda_int8_matmul_requant_i8(yscv_cuda_ctx *ctx, const int8_t *a, const yscv_cuda_i8b *b, size_t m,
                                     const int32_t *bias, float composite, float y_zero_point, int relu,
                                     int8_t *out) {
    return i8_requant_i8_host(ctx, a, b, m, bias, nullptr, composite, y_zero_point, relu, out);
}

int yscv_cuda_matmul_integer_dev(yscv_cuda_ctx *ctx, const void *d_a, int a_is_unsigned,
                                 int32_t a_zero_point, const yscv_cuda_i8b *b, size_t m,
                                 int32_t *d_out) {
    op_counters().matmul_integer_calls++;
    return i8_gemm_dev(ctx, d_a, b, m, d_out, a_is_unsigned, a_zero_point, nullptr);
}

int yscv_cuda_matmul_integer(yscv_cuda_ctx *ctx, const void *a, int a_is_unsigned, int32_t a_zero_point,
                             const yscv_cuda_i8b *b, size_t m, int32_t *out) {
    op_counters().matmul_integer_calls++;
    return i8_gemm_host(ctx, a, b, m, out, sizeof(int32_t), a_is_unsigned, a_zero_point, nullptr);
}

}  // extern "C"
