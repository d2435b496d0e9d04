// Host side of tma.cuh: tensor-map encoding through the driver entry point.
#include "tma.cuh"

#include "common.cuh"

namespace yscv {

EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int encode_2d(CUtensorMap *map, CUtensorMapDataType dtype, int elem_bytes, const void *base,
              uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows,
              uint32_t box_cols, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return fail(YSCV_CUDA_ERR_CUDA, "driver does not export cuTensorMapEncodeTiled");
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15))
        return fail(YSCV_CUDA_ERR_BAD_ARG, "TMA operand must be 16-byte aligned (base %p, pitch %llu)",
                    base, (unsigned long long)pitch_bytes);
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    (void)elem_bytes;
    CUresult r = enc(map, dtype, 2, const_cast<void *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(YSCV_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed: %d", (int)r);
    return YSCV_CUDA_OK;
}

}  // namespace yscv
