// Tensor-map (TMA) helpers: host-side descriptor encoding through the driver entry point
// (no link-time dependency on libcuda) and the device-side tiled copy wrappers.
#pragma once

#include <cuda.h>

#include "izb_common.cuh"

namespace izb {

// Encodes a tiled tensor map of rank 2 or 3.  dims/box are in elements, innermost first;
// strides (rank-1 of them) are in bytes and must be multiples of 16.  Returns IZB_OK or a status.
int tma_encode(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

#ifdef __CUDACC__
// Tiled global->shared copies; the innermost coordinate times the element size must be a
// multiple of 16 bytes.  No cluster multicast anywhere: every CTA fetches its own tiles.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
            "r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
}
// Makes a tensor map that the host wrote into global memory visible to this thread's TMA unit.
__device__ __forceinline__ void tma_fence_descriptor(const CUtensorMap* map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(map) : "memory");
}
#endif

}  // namespace izb
