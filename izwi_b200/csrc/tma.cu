#include <cudaTypedefs.h>

#include <mutex>

#include "tma.cuh"

namespace izb {

namespace {
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_once;

void resolve() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
        g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    else
        (void)cudaGetLastError();
}
}  // namespace

int tma_encode(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    std::call_once(g_once, resolve);
    if (!g_encode) return IZB_ERR_NO_DEVICE;
    if (rank < 2 || rank > 3 || !izb_aligned(base, 16)) return IZB_ERR_BAD_ARG;
    cuuint64_t gdim[3], gstr[2];
    cuuint32_t bdim[3], estr[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        if (box[i] == 0 || box[i] > 256 || dims[i] == 0) return IZB_ERR_UNSUPPORTED;
    }
    for (int i = 0; i < rank - 1; ++i) {
        gstr[i] = strides_bytes[i];
        if (strides_bytes[i] % 16 != 0) return IZB_ERR_BAD_ARG;
    }
    const CUresult r = g_encode(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bdim,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? IZB_OK : IZB_ERR_UNSUPPORTED;
}

}  // namespace izb
