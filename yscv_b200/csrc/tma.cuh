// TMA (cp.async.bulk[.tensor]) and mbarrier helpers for sm_100a, plus the host
// side that encodes tensor maps through the driver entry point (no link-time
// dependency on libcuda).
//
// Every wait is bounded: mbar_wait() gives up after a fixed number of probes,
// records YSCV_DEV_MBARRIER_TIMEOUT in the context's status word and returns
// false, so a kernel can never spin forever on a barrier nobody completes.
// No copy here uses cluster multicast.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace yscv {

// ---- host: tensor map encoding -------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Returns nullptr when the driver does not export cuTensorMapEncodeTiled.
EncodeTiledFn tensor_map_encoder();

// 2-D row-major tensor [rows][cols] of `elem_bytes` elements with row pitch
// `pitch_bytes`; box = [box_rows][box_cols]. Returns 0 on success.
int encode_2d(CUtensorMap *map, CUtensorMapDataType dtype, int elem_bytes, const void *base,
              uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows,
              uint32_t box_cols, CUtensorMapSwizzle swizzle);

// ---- device ---------------------------------------------------------------------

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait. `status` is the context's device status word (may be null).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *status) {
    // try_wait itself suspends the thread for a hardware-defined slice, so this
    // many probes is on the order of a second, far beyond any legitimate wait
    for (uint32_t i = 0; i < (1u << 22); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicExch(status, 1 /* YSCV_DEV_MBARRIER_TIMEOUT */);
    return false;
}

// 2-D tiled load: box at (x = innermost coordinate, y = row) -> smem, completes on `bar`.
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Linear bulk copy global -> shared; addresses 16-byte aligned, size % 16 == 0.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::
            "r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

// ---- clusters of two CTAs (tcgen05 cta_group::2 kernels) ---------------------------------
// Every cross-CTA signal is a remote arrival on a local mbarrier of the CTA that waits, through
// a mapa address; no multicast form is used anywhere.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
// Arrival on a barrier of either CTA of the cluster. Default semantics (release at CTA scope): what
// the arrival publishes here is shared memory of the arriving CTA already fenced for the async proxy
// (fence.proxy.async) or TMEM reads already fenced (tcgen05.fence::before_thread_sync); the
// cluster-scope release form costs a memory barrier per arrival, which stalled a kernel with one such
// arrival per warp and k block to 0.65 of its speed.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait on a barrier that a thread of the other CTA arrives on
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    if (status) atomicExch(status, 1 /* YSCV_DEV_MBARRIER_TIMEOUT */);
    return false;
}
// 2-D tiled load into this CTA's shared memory whose bytes complete on a barrier of either CTA
// of the pair (`bar`: a shared::cluster address). No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y,
                                                 uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%2, %3}], [%4];\n" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// Bounded wait by polling (test_wait never suspends the thread): for the waits of a cluster kernel
// that sit on its critical path once per k block.
__device__ __forceinline__ bool mbar_spin_cluster(uint32_t bar, uint32_t parity, int *status) {
    for (uint32_t i = 0; i < (1u << 26); ++i) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    if (status) atomicExch(status, 1 /* YSCV_DEV_MBARRIER_TIMEOUT */);
    return false;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace yscv
