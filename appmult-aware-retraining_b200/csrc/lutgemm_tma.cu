// Host side of the bulk-tensor operand loads: tensor-map encoding through the driver entry point, resolved at run
// time (the library does not link against the driver library).
#include "lutgemm_tma.cuh"

#include <cuda_runtime.h>

namespace lutgemm {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace

bool make_tensor_map_u8_2d(CUtensorMap *map, const void *base, unsigned long long width, unsigned long long height,
                           unsigned long long pitch, unsigned box_w, unsigned box_h) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || !base || width == 0 || height == 0) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch & 15) || (box_w & 15) || box_w > 256 || box_h > 256 || box_h == 0)
        return false;
    const cuuint64_t dims[2] = {width, height};
    const cuuint64_t strides[1] = {pitch};  // bytes, of the second dimension
    const cuuint32_t box[2] = {box_w, box_h};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace lutgemm
