// Internal definitions shared by the kernels and the C ABI.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
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
