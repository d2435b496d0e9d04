// Load-time and bookkeeping side of the library: what the reference's runner does around the
// quantized kernels, restated for device-resident weights.
//
//   * the MatMul / Gemm weight path of quantize_matmul_weights_int4_packed
//     (crates/yscv-onnx/src/quantize/packed_int4.rs:50-128): transpose [K,N] -> [N,K], the
//     skip rules, pack, keep resident;
//   * a name-keyed table of resident weights, the counterpart of the side tables
//     `packed_int4_weights` and `prepacked_i8_weights` the handlers look up by initializer
//     name (crates/yscv-onnx/src/runner/linear.rs:228, crates/yscv-onnx/src/plan/build.rs:1417-1454,
//     crates/yscv-onnx/src/runner/tensor_env.rs:178-183), with the prepack gates of
//     plan/build.rs:1371-1377 and runner/layout.rs:6-11;
//   * requant_i32_row_to_i8_dispatch as a stand-alone pass
//     (crates/yscv-kernels/src/ops/int8_requant.rs:81-169);
//   * a byte container for a packed int4 weight (the reference keeps packed int4 in memory
//     only, packed_int4.rs:28-39) and the MatMulNBits nibble convention in both directions;
//   * operator counters and a dispatch report (crates/yscv-onnx/src/runner/quant_stats.rs:21-92,
//     crates/yscv-kernels/src/core.rs:111-137).
#include <cstring>
#include <map>
#include <shared_mutex>

#include "common.cuh"
#include "kernels.cuh"

namespace yscv {

// out[n][k] = in[k][n], 32x32 tiles through shared memory
__global__ void __launch_bounds__(256)
transpose_f32_kernel(const float *__restrict__ in, float *__restrict__ out, int K, int N) {
    __shared__ float tile[32][33];
    const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 32; j += 8) {
        const int k = k0 + j, n = n0 + tx;
        if (k < K && n < N) tile[j][tx] = in[(size_t)k * N + n];
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
        const int n = n0 + j, k = k0 + tx;
        if (k < K && n < N) out[(size_t)n * K + k] = tile[tx][j];
    }
}

// requant_scalar (int8_requant.rs:143-169): q = clamp(round_ties_even((float)(acc + bias[ch])
// * composite + y_zp), -128, 127), the add wrapping, multiply and add separate, ReLU after
// the saturation.
__global__ void __launch_bounds__(256)
requant_rows_kernel(const int32_t *__restrict__ acc, const int32_t *__restrict__ bias, float composite,
                    float y_zp, int relu, int8_t *__restrict__ out, size_t len, int c) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < len; i += (size_t)gridDim.x * blockDim.x) {
        uint32_t a = (uint32_t)acc[i];
        if (bias) a += (uint32_t)__ldg(bias + (int)(i % (size_t)c));
        const float v = __fadd_rn(__fmul_rn((float)(int32_t)a, composite), y_zp);
        int q = (int)fminf(fmaxf(rintf(v), -128.0f), 127.0f);
        if (v != v) q = 0;  // NaN -> 0, as Rust's saturating float-to-int cast does
        if (relu && q < 0) q = 0;
        out[i] = (int8_t)q;
    }
}

}  // namespace yscv

using namespace yscv;

struct yscv_cuda_registry {
    mutable std::shared_mutex mu;
    std::map<std::string, yscv_cuda_int4_weight *> int4;
    std::map<std::string, yscv_cuda_i8b *> i8b;
};

// container layout (little endian): 64-byte header, packed bytes (padded to 16), scales
namespace {
constexpr char kMagic[8] = {'Y', 'S', 'C', 'V', 'I', 'N', 'T', '4'};
constexpr uint32_t kVersion = 1;
constexpr size_t kHeader = 64;
struct ContainerHeader {
    char magic[8];
    uint32_t version, group_size;
    uint64_t m_w, k, packed_bytes, scale_count;
    uint8_t reserved[16];
};
static_assert(sizeof(ContainerHeader) == kHeader, "container header is 64 bytes");
size_t padded16(size_t v) { return (v + 15) / 16 * 16; }
}  // namespace

extern "C" {

/* ---- requant pass -------------------------------------------------------------------- */

int yscv_cuda_requant_i32_row_to_i8_dev(yscv_cuda_ctx *ctx, const int32_t *d_acc, const int32_t *d_bias,
                                        float composite, float y_zero_point, int relu, int8_t *d_out,
                                        size_t len, size_t c) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (c == 0 || len % c != 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "len=%zu must be a multiple of c=%zu > 0", len, c);
    if (len == 0) return YSCV_CUDA_OK;
    if (!d_acc || !d_out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    if (c >= (1u << 31)) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "dimension too large");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t want = (len + 255) / 256;
    const unsigned blocks = (unsigned)(want < (size_t)(16 * ctx->sm_count) ? want : (size_t)(16 * ctx->sm_count));
    requant_rows_kernel<<<blocks, 256, 0, ctx->stream>>>(d_acc, d_bias, composite, y_zero_point, relu, d_out, len, (int)c);
    YSCV_CUDA_TRY(cudaGetLastError());
    ctx->launches++;
    ctx->last_kernel = "requant_i32_row_to_i8";
    op_counters().requant_calls++;
    return YSCV_CUDA_OK;
}

int yscv_cuda_requant_i32_row_to_i8(yscv_cuda_ctx *ctx, const int32_t *acc, const int32_t *bias, float composite,
                                    float y_zero_point, int relu, int8_t *out, size_t len, size_t c) {
    if (!ctx) return fail(YSCV_CUDA_ERR_BAD_ARG, "ctx is null");
    if (c == 0 || len % c != 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "len=%zu must be a multiple of c=%zu > 0", len, c);
    if (len == 0) return YSCV_CUDA_OK;
    if (!acc || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    int rc;
    if ((rc = ctx->in0.reserve(len * 4)) || (rc = ctx->in1.reserve(c * 4)) || (rc = ctx->out0.reserve(len))) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in0.ptr, acc, len * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (bias) YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in1.ptr, bias, c * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = yscv_cuda_requant_i32_row_to_i8_dev(ctx, (const int32_t *)ctx->in0.ptr, bias ? (const int32_t *)ctx->in1.ptr : nullptr,
                                             composite, y_zero_point, relu, (int8_t *)ctx->out0.ptr, len, c);
    if (rc) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(out, ctx->out0.ptr, len, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

/* ---- MatMul / Gemm weight -> resident packed int4 ---------------------------------------- */

int yscv_cuda_int4_weight_from_f32(yscv_cuda_ctx *ctx, const float *weight, size_t dim0, size_t dim1,
                                   int layout, size_t group_size, yscv_cuda_int4_weight **out) {
    if (!ctx || !out) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    *out = nullptr;
    if (!weight) return fail(YSCV_CUDA_ERR_BAD_ARG, "null operand");
    // packed_int4.rs:54-58: an odd or zero group size is an error, not a skip
    if (group_size == 0 || (group_size & 1))
        return fail(YSCV_CUDA_ERR_BAD_ARG, "group_size must be even and > 0, got %zu", group_size);
    if (layout < 0 || layout > 2) return fail(YSCV_CUDA_ERR_BAD_ARG, "layout %d is not one of YSCV_CUDA_WEIGHT_*", layout);
    const bool transposed_source = layout != YSCV_CUDA_WEIGHT_GEMM_NK;   // [K,N] -> [N,K]
    const size_t m_w = transposed_source ? dim1 : dim0, k = transposed_source ? dim0 : dim1;
    // packed_int4.rs:102-104: silently skipped, the caller keeps the fp32 weight
    if (m_w == 0 || k == 0 || k % group_size != 0 || k * m_w < 32) return YSCV_CUDA_OK;
    if (m_w >= (1u << 30) || k >= (1u << 30)) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "dimension too large");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t wb = m_w * k * sizeof(float);
    int rc;
    if ((rc = ctx->in0.reserve(wb))) return rc;
    if (transposed_source && (rc = ctx->scratch.reserve(wb))) return rc;
    YSCV_CUDA_TRY(cudaMemcpyAsync(ctx->in0.ptr, weight, wb, cudaMemcpyHostToDevice, ctx->stream));
    const float *src = (const float *)ctx->in0.ptr;
    if (transposed_source) {
        dim3 grid((unsigned)((m_w + 31) / 32), (unsigned)((k + 31) / 32));
        if (grid.y > 65535) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "k=%zu too large for the transposing upload", k);
        transpose_f32_kernel<<<grid, 256, 0, ctx->stream>>>(src, (float *)ctx->scratch.ptr, (int)k, (int)m_w);
        YSCV_CUDA_TRY(cudaGetLastError());
        ctx->launches++;
        src = (const float *)ctx->scratch.ptr;
    }
    void *dp = nullptr, *ds = nullptr;
    YSCV_CUDA_TRY(cudaMalloc(&dp, m_w * k / 2));
    cudaError_t e = cudaMalloc(&ds, m_w * (k / group_size) * sizeof(float));
    if (e != cudaSuccess) {
        cudaFree(dp);
        return fail(YSCV_CUDA_ERR_CUDA, "cudaMalloc(scales): %s", cudaGetErrorString(e));
    }
    rc = pack_int4(ctx, src, m_w, k, group_size, (uint8_t *)dp, (float *)ds);
    if (!rc && cudaStreamSynchronize(ctx->stream) != cudaSuccess) rc = fail(YSCV_CUDA_ERR_CUDA, "packing failed");
    if (rc) {
        cudaFree(dp);
        cudaFree(ds);
        return rc;
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

size_t yscv_cuda_int4_weight_rows(const yscv_cuda_int4_weight *w) { return w ? w->m_w : 0; }
size_t yscv_cuda_int4_weight_k(const yscv_cuda_int4_weight *w) { return w ? w->k : 0; }
size_t yscv_cuda_int4_weight_group_size(const yscv_cuda_int4_weight *w) { return w ? w->group_size : 0; }

int yscv_cuda_int4_weight_download(yscv_cuda_ctx *ctx, const yscv_cuda_int4_weight *w, uint8_t *packed,
                                   float *scales) {
    if (!ctx || !w || !packed || !scales) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    YSCV_CUDA_TRY(cudaSetDevice(ctx->device));
    YSCV_CUDA_TRY(cudaMemcpyAsync(packed, w->d_packed, w->m_w * w->k / 2, cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaMemcpyAsync(scales, w->d_scales, w->m_w * (w->k / w->group_size) * sizeof(float),
                                  cudaMemcpyDeviceToHost, ctx->stream));
    YSCV_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YSCV_CUDA_OK;
}

/* ---- prepack gates ------------------------------------------------------------------------ */

int yscv_cuda_should_prepack_i8_b(size_t k, size_t n) {
    return ((k >= 4 && n % 16 == 0) || (k >= 512 && n >= 1024)) ? 1 : 0;
}

int yscv_cuda_should_use_prepacked_i8_b(size_t m, size_t k, size_t n) {
    return ((m >= 4 && k >= 4 && n >= 32 && n % 16 == 0) || (m <= 64 && k >= 512 && n >= 1024)) ? 1 : 0;
}

/* ---- name-keyed table of resident weights -------------------------------------------------- */

int yscv_cuda_registry_create(yscv_cuda_registry **out) {
    if (!out) return fail(YSCV_CUDA_ERR_BAD_ARG, "out is null");
    *out = new yscv_cuda_registry();
    return YSCV_CUDA_OK;
}

void yscv_cuda_registry_destroy(yscv_cuda_registry *reg) {
    if (!reg) return;
    for (auto &kv : reg->int4) yscv_cuda_int4_weight_free(kv.second);
    for (auto &kv : reg->i8b) yscv_cuda_i8b_free(kv.second);
    delete reg;
}

int yscv_cuda_registry_put_int4(yscv_cuda_registry *reg, const char *name, yscv_cuda_int4_weight *w) {
    if (!reg || !name || !w) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    std::unique_lock<std::shared_mutex> lock(reg->mu);
    auto it = reg->int4.find(name);
    if (it != reg->int4.end()) {
        if (it->second != w) yscv_cuda_int4_weight_free(it->second);  // HashMap::insert replaces
        it->second = w;
    } else {
        reg->int4.emplace(name, w);
    }
    return YSCV_CUDA_OK;
}

int yscv_cuda_registry_put_i8b(yscv_cuda_registry *reg, const char *name, yscv_cuda_i8b *b) {
    if (!reg || !name || !b) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    std::unique_lock<std::shared_mutex> lock(reg->mu);
    auto it = reg->i8b.find(name);
    if (it != reg->i8b.end()) {
        if (it->second != b) yscv_cuda_i8b_free(it->second);
        it->second = b;
    } else {
        reg->i8b.emplace(name, b);
    }
    return YSCV_CUDA_OK;
}

const yscv_cuda_int4_weight *yscv_cuda_registry_get_int4(const yscv_cuda_registry *reg, const char *name) {
    if (!reg || !name) return nullptr;
    std::shared_lock<std::shared_mutex> lock(reg->mu);
    auto it = reg->int4.find(name);
    return it == reg->int4.end() ? nullptr : it->second;
}

const yscv_cuda_i8b *yscv_cuda_registry_get_i8b(const yscv_cuda_registry *reg, const char *name) {
    if (!reg || !name) return nullptr;
    std::shared_lock<std::shared_mutex> lock(reg->mu);
    auto it = reg->i8b.find(name);
    return it == reg->i8b.end() ? nullptr : it->second;
}

size_t yscv_cuda_registry_len(const yscv_cuda_registry *reg) {
    if (!reg) return 0;
    std::shared_lock<std::shared_mutex> lock(reg->mu);
    return reg->int4.size() + reg->i8b.size();
}

int yscv_cuda_registry_register_matmul_weight(yscv_cuda_ctx *ctx, yscv_cuda_registry *reg, const char *name,
                                              const float *weight, size_t dim0, size_t dim1, int layout,
                                              size_t group_size, int *packed) {
    if (packed) *packed = 0;
    if (!reg || !name) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    yscv_cuda_int4_weight *w = nullptr;
    int rc = yscv_cuda_int4_weight_from_f32(ctx, weight, dim0, dim1, layout, group_size, &w);
    if (rc || !w) return rc;
    rc = yscv_cuda_registry_put_int4(reg, name, w);
    if (rc) {
        yscv_cuda_int4_weight_free(w);
        return rc;
    }
    if (packed) *packed = 1;
    return YSCV_CUDA_OK;
}

int yscv_cuda_registry_register_i8_weight(yscv_cuda_ctx *ctx, yscv_cuda_registry *reg, const char *name,
                                          const int8_t *b, size_t k, size_t n, int *prepacked) {
    if (prepacked) *prepacked = 0;
    if (!reg || !name) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (!yscv_cuda_should_prepack_i8_b(k, n)) return YSCV_CUDA_OK;  // plan/build.rs:1371-1377
    yscv_cuda_i8b *h = nullptr;
    int rc = yscv_cuda_pack_i8_b_for_matmul(ctx, b, k, n, &h);
    if (rc) return rc;
    rc = yscv_cuda_registry_put_i8b(reg, name, h);
    if (rc) {
        yscv_cuda_i8b_free(h);
        return rc;
    }
    if (prepacked) *prepacked = 1;
    return YSCV_CUDA_OK;
}

/* ---- container ------------------------------------------------------------------------------ */

size_t yscv_cuda_int4_container_size(size_t m_w, size_t k, size_t group_size) {
    if (group_size == 0 || k % group_size != 0) return 0;
    return kHeader + padded16(m_w * k / 2) + m_w * (k / group_size) * sizeof(float);
}

int yscv_cuda_int4_container_write(const uint8_t *packed, const float *scales, size_t m_w, size_t k,
                                   size_t group_size, uint8_t *dst, size_t capacity, size_t *written) {
    if (!packed || !scales || !dst) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (group_size == 0 || (group_size & 1) || k == 0 || k % group_size != 0 || m_w == 0)
        return fail(YSCV_CUDA_ERR_BAD_ARG, "not a packed int4 shape: m_w=%zu k=%zu group=%zu", m_w, k, group_size);
    const size_t need = yscv_cuda_int4_container_size(m_w, k, group_size);
    if (capacity < need) return fail(YSCV_CUDA_ERR_BAD_ARG, "container needs %zu bytes, buffer holds %zu", need, capacity);
    ContainerHeader h;
    memset(&h, 0, sizeof(h));
    memcpy(h.magic, kMagic, 8);
    h.version = kVersion;
    h.group_size = (uint32_t)group_size;
    h.m_w = m_w;
    h.k = k;
    h.packed_bytes = m_w * k / 2;
    h.scale_count = m_w * (k / group_size);
    memcpy(dst, &h, sizeof(h));
    memcpy(dst + kHeader, packed, h.packed_bytes);
    memset(dst + kHeader + h.packed_bytes, 0, padded16(h.packed_bytes) - h.packed_bytes);
    memcpy(dst + kHeader + padded16(h.packed_bytes), scales, h.scale_count * sizeof(float));
    if (written) *written = need;
    return YSCV_CUDA_OK;
}

int yscv_cuda_int4_container_read(const uint8_t *src, size_t len, size_t *m_w, size_t *k, size_t *group_size,
                                  const uint8_t **packed, const float **scales) {
    if (!src || !m_w || !k || !group_size || !packed || !scales) return fail(YSCV_CUDA_ERR_BAD_ARG, "null argument");
    if (len < kHeader) return fail(YSCV_CUDA_ERR_BAD_ARG, "container truncated: %zu bytes", len);
    ContainerHeader h;
    memcpy(&h, src, sizeof(h));
    if (memcmp(h.magic, kMagic, 8) != 0) return fail(YSCV_CUDA_ERR_BAD_ARG, "not a packed int4 container (bad magic)");
    if (h.version != kVersion) return fail(YSCV_CUDA_ERR_UNSUPPORTED, "container version %u", h.version);
    if (h.group_size == 0 || (h.group_size & 1) || h.k == 0 || h.k % h.group_size != 0 || h.m_w == 0 ||
        h.m_w >= (1u << 30) || h.k >= (1u << 30) || h.packed_bytes != h.m_w * h.k / 2 ||
        h.scale_count != h.m_w * (h.k / h.group_size))
        return fail(YSCV_CUDA_ERR_BAD_ARG, "container header is inconsistent");
    const size_t need = kHeader + padded16(h.packed_bytes) + h.scale_count * sizeof(float);
    if (len < need) return fail(YSCV_CUDA_ERR_BAD_ARG, "container truncated: %zu of %zu bytes", len, need);
    *m_w = h.m_w;
    *k = h.k;
    *group_size = h.group_size;
    *packed = src + kHeader;
    *scales = reinterpret_cast<const float *>(src + kHeader + padded16(h.packed_bytes));
    return YSCV_CUDA_OK;
}

int yscv_cuda_int4_weight_from_container(yscv_cuda_ctx *ctx, const uint8_t *src, size_t len,
                                         yscv_cuda_int4_weight **out) {
    if (!out) return fail(YSCV_CUDA_ERR_BAD_ARG, "out is null");
    *out = nullptr;
    size_t m_w, k, g;
    const uint8_t *packed;
    const float *scales;
    int rc = yscv_cuda_int4_container_read(src, len, &m_w, &k, &g, &packed, &scales);
    if (rc) return rc;
    // cudaMemcpy takes any host alignment: the scales need not be 4-byte aligned in `src`
    return yscv_cuda_int4_weight_upload(ctx, packed, scales, m_w, k, g, out);
}

int yscv_cuda_int4_to_matmulnbits(const uint8_t *src, uint8_t *dst, size_t bytes) {
    // q -> q + 8 on both nibbles is the same bit flip as the import
    return yscv_cuda_int4_from_matmulnbits(src, dst, bytes);
}

/* ---- counters and the dispatch report -------------------------------------------------------- */

void yscv_cuda_quant_stats_read(yscv_cuda_quant_stats *out) {
    if (!out) return;
    OpCounters &c = op_counters();
    out->int4_gemv_calls = c.int4_gemv_calls.load();
    out->int4_gemm_calls = c.int4_gemm_calls.load();
    out->int4_generic_calls = c.int4_generic_calls.load();
    out->int8_gemm_calls = c.int8_gemm_calls.load();
    out->qlinear_matmul_calls = c.qlinear_matmul_calls.load();
    out->matmul_integer_calls = c.matmul_integer_calls.load();
    out->requant_calls = c.requant_calls.load();
    out->decode_step_calls = c.decode_step_calls.load();
    out->cpu_fallbacks = 0;  // there is no CPU path in this library
}

void yscv_cuda_quant_stats_reset(void) {
    OpCounters &c = op_counters();
    c.int4_gemv_calls = 0;
    c.int4_gemm_calls = 0;
    c.int4_generic_calls = 0;
    c.int8_gemm_calls = 0;
    c.qlinear_matmul_calls = 0;
    c.matmul_integer_calls = 0;
    c.requant_calls = 0;
    c.decode_step_calls = 0;
}

const char *yscv_cuda_dispatch_report(const yscv_cuda_ctx *ctx) {
    static thread_local std::string s;
    if (!ctx) {
        s = "no context";
        return s.c_str();
    }
    char buf[768];
    snprintf(buf, sizeof(buf),
             "device %d: sm_100a, %d SMs; last kernel: %s; launches: %llu\n  int4: %s\n  int8: %s\n"
             "  cpu fallback: none (unsupported shapes return YSCV_CUDA_ERR_UNSUPPORTED)",
             ctx->device, ctx->sm_count, ctx->last_kernel, (unsigned long long)ctx->launches, ctx->report_int4,
             ctx->report_int8);
    s = buf;
    return s.c_str();
}

}  // extern "C"
