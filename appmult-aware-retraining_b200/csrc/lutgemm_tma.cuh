// Tiled bulk-tensor (TMA) loads of operand-code tiles for the sm_100a LUT-GEMM kernels.
//
// The uint8 operand codes of a k chunk - 16 k x 256 rows of the transposed activation codes at[k][m], 16 k x 64
// columns of w[k][n] - are fetched by ONE elected thread with cp.async.bulk.tensor.2d straight into the shared-
// memory stage the kernel reads them from; completion is signalled on an mbarrier (complete_tx), which the
// consumers wait on with the library's bounded wait.  No registers and no shared-memory store instructions are
// spent on staging.  Every load is a plain single-CTA load from this GPU's own memory.
// Alignment rules the callers keep (the copy engine checks none of them at run time): the innermost coordinate is
// a multiple of 16 bytes, the global base address and row pitch are multiples of 16 bytes, the box's inner extent
// is a multiple of 16 bytes, box sides are at most 256.
#pragma once

#include <cuda.h>

#include "lutgemm_common.cuh"

namespace lutgemm {

// Encodes a 2-D uint8 tensor map: `width` bytes per row (innermost), `height` rows `pitch` bytes apart, tiles of
// box_w x box_h; elements outside [0,width) x [0,height) read as 0.  Returns false when the driver entry point is
// missing or the arguments break an alignment rule (the caller then keeps its vector-load path).
bool make_tensor_map_u8_2d(CUtensorMap *map, const void *base, unsigned long long width, unsigned long long height,
                           unsigned long long pitch, unsigned box_w, unsigned box_h);

__device__ __forceinline__ void tma_expect_bytes(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// orders this thread's (and, after a CTA barrier, the CTA's) earlier generic-proxy accesses to shared memory before
// the copy engine's writes that follow
__device__ __forceinline__ void tma_fence_before_load() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// box of the tensor map at (x, y) -> shared memory at dst; bytes are counted on `bar`
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

}  // namespace lutgemm
