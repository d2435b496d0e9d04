// Internal definitions shared by the kernels and the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/yscv_cuda.h"

namespace yscv {

// Thread-local error text behind yscv_cuda_last_error().
std::string &last_error();
int fail(int status, const char *fmt, ...);

#define YSCV_CUDA_TRY(expr)                                                         \
    do {                                                                            \
        cudaError_t _e = (expr);                                                    \
        if (_e != cudaSuccess)                                                      \
            return ::yscv::fail(YSCV_CUDA_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, \
                                cudaGetErrorString(_e), __FILE__, __LINE__);        \
    } while (0)

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device); safe to call
// from several threads.
int ensure_dynamic_smem(const void *kernel, int device, int bytes);

// Process-wide operator counters, the counterpart of the reference's QuantRuntimeStats
// (crates/yscv-onnx/src/runner/quant_stats.rs:21-92): bumped by the entry points, read and
// reset through yscv_cuda_quant_stats / yscv_cuda_reset_quant_stats.
struct OpCounters {
    std::atomic<uint64_t> int4_gemv_calls{0}, int4_gemm_calls{0}, int4_generic_calls{0};
    std::atomic<uint64_t> int8_gemm_calls{0}, qlinear_matmul_calls{0}, matmul_integer_calls{0};
    std::atomic<uint64_t> requant_calls{0}, decode_step_calls{0};
};
OpCounters &op_counters();

// Grow-only device buffer owned by a context.
struct DeviceBuffer {
    void *ptr = nullptr;
    size_t bytes = 0;
    int reserve(size_t want);
    void release();
};

}  // namespace yscv

// ---- programmatic dependent launch ------------------------------------------------------
// A kernel launched through launch_pdl() may be scheduled while its predecessor in the
// stream is still draining. It must call pdl_wait() before it reads anything a predecessor
// wrote or writes anything a predecessor may still read; pdl_trigger() lets its own
// successor be scheduled early. Both are no-ops for a normally launched kernel.
// EVERY kernel launched through launch_pdl() MUST execute pdl_wait() on all paths, even one
// that touches nothing a predecessor wrote: a kernel that skips it can retire while its
// predecessor (which triggered early) is still running, and the next kernel's wait would then
// cover only the skipping kernel, not that predecessor.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

namespace yscv {
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
}  // namespace yscv
#endif

// Device status codes written by bounded waits inside kernels.
enum : int {
    YSCV_DEV_OK = 0,
    YSCV_DEV_MBARRIER_TIMEOUT = 1,
    YSCV_DEV_FLAG_TIMEOUT = 2,
    YSCV_DEV_POS_OVERFLOW = 3,  // the sequence position is outside [0, max_seq): nothing was appended
};

struct yscv_cuda_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int *d_status = nullptr;   // device status word
    uint64_t launches = 0;
    const char *last_kernel = "none";
    bool prefill_exact = false;  // int4 matmul with m > 16: fp32-exact kernel instead of bf16 MMA
    bool prefill_pairs = true;   // int4 prefill GEMM: CTA-pair kernel (cta_group::2) for large prefills
    int max_prefill_pairs = 0;   // CTA pairs of that kernel that can be resident at once (0: not asked yet)
    bool f32_tensor_cores = true;   // fp32 matmul with more than 8 rows: 3xTF32 tensor-core kernel (else the SIMT tiled kernel)
    bool attn_tensor_cores = true;  // decode attention over int8 caches: mma.sync kernel (else the fp32 loop)
    int int8_pairs = -1;         // int8 GEMM, CTA-pair kernel (cta_group::2): -1 where it measured faster, 0 never, 1 wherever the shape allows
    int max_pairs = 0;           // CTA pairs of that kernel that can be resident at once (0: not asked yet)
    // optional per-kernel event timing (yscv_cuda_ctx_profile_*)
    bool profiling = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_events;
    size_t prof_used = 0;
    void prof_begin();
    void prof_end();
    // staging for the host-pointer entry points
    yscv::DeviceBuffer in0, in1, in2, out0, out1;
    // scratch for kernels that need global memory beyond their operands
    yscv::DeviceBuffer scratch;
    yscv::DeviceBuffer scratch_attn;  // partial outputs of the split attention
    yscv::DeviceBuffer rowsum;        // row sums of A (int8 GEMM with a zero point on B)
    yscv::DeviceBuffer tmp_bt, tmp_colsum;  // B^T and column sums of the non-prepacked int8 entry point
    // int8 GEMM with a split tail: one slot of partial sums per CTA, four flags per CTA; every
    // launch that splits publishes a new epoch in the flags, so they are never reset
    yscv::DeviceBuffer gemm_ws, gemm_flags;
    int gemm_epoch = 0;
    bool int8_tail_split = true;
    // encoded TMA descriptors of the last few decode GEMV weight matrices (int4_gemv.cu)
    struct TmCacheEntry {
        const void *a = nullptr, *b = nullptr;
        int n = 0, k = 0, rows = 0, gs = 0;
        alignas(64) unsigned char w[128], s[128];
    };
    TmCacheEntry tm_cache[16];
    int tm_next = 0;
    // variant / tile report of the last int4 and int8 dispatch (yscv_cuda_dispatch_report)
    char report_int4[224] = "none";
    char report_int8[224] = "none";
};

struct yscv_cuda_int4_weight {
    const uint8_t *d_packed = nullptr;
    const float *d_scales = nullptr;
    size_t m_w = 0, k = 0, group_size = 0;
    bool owns = false;
    int device = 0;
};

// PackedI8B resident in HBM: B^T [n][kp] (kp = k rounded up to 16, zero padded)
// and the column sums of B over k.
struct yscv_cuda_i8b {
    int8_t *d_bt = nullptr;
    int32_t *d_colsum = nullptr;
    size_t k = 0, n = 0, kp = 0;
    int device = 0;
    int b_zp = 0;  // zero point of B (yscv_cuda_i8b_set_zero_point)
};

// One rank's view of a tensor-parallel group: its own exchange region and every peer's,
// mapped through CUDA IPC (tp_comm.cu).
struct yscv_cuda_tp_comm {
    int device = 0, rank = 0, world = 1;
    size_t cap_rows = 0, bytes = 0;
    void *local = nullptr;        // this rank's region (cudaMalloc)
    void *peer[8] = {};           // every rank's region as mapped in this process (peer[rank] == local)
    bool opened[8] = {};          // mapped with cudaIpcOpenMemHandle, to be closed
    void *standin = nullptr;      // test form: local stand-ins for the peers' regions that nobody writes
    unsigned int *d_seq = nullptr;  // steps run so far (tags of the exchanges)
    bool connected = false;
};
