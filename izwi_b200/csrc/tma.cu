#include <cudaTypedefs.h>

#include <cstring>
#include <mutex>
#include <unordered_map>

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

namespace {
// Encoded maps are pure functions of (address, extents, strides, box, type, swizzle): a linear layer
// called again with the same buffers (every decode step, every layer of a captured pass) finds its
// two maps here instead of asking the driver again.  The table is dropped when it grows past a bound
// (a caller that streams through fresh buffers), never grown without limit.
struct MapKey {
    const void* base;
    uint64_t dims[3];
    uint64_t strides[2];
    uint32_t box[3];
    int32_t rank, dtype, swizzle;
    bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
        uint64_t h = 1469598103934665603ull;
        for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
        return static_cast<size_t>(h);
    }
};
static_assert(sizeof(MapKey) % 8 == 0, "MapKey is hashed in 8-byte words");
constexpr size_t kMapCacheLimit = 8192;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mutex;
}  // namespace

int tma_encode(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
               const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
    std::call_once(g_once, resolve);
    if (!g_encode) return IZB_ERR_NO_DEVICE;
    if (rank < 2 || rank > 3 || !izb_aligned(base, 16)) return IZB_ERR_BAD_ARG;
    MapKey key;
    std::memset(&key, 0, sizeof(key));  // padding too: the key is compared and hashed as bytes
    key.base = base;
    key.rank = rank;
    key.dtype = static_cast<int32_t>(dtype);
    key.swizzle = static_cast<int32_t>(swizzle);
    cuuint64_t gdim[3], gstr[2];
    cuuint32_t bdim[3], estr[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        key.dims[i] = dims[i];
        key.box[i] = box[i];
        if (box[i] == 0 || box[i] > 256 || dims[i] == 0) return IZB_ERR_UNSUPPORTED;
    }
    for (int i = 0; i < rank - 1; ++i) {
        gstr[i] = strides_bytes[i];
        key.strides[i] = strides_bytes[i];
        if (strides_bytes[i] % 16 != 0) return IZB_ERR_BAD_ARG;
    }
    {
        std::lock_guard<std::mutex> lock(g_maps_mutex);
        auto it = g_maps.find(key);
        if (it != g_maps.end()) {
            *out = it->second;
            return IZB_OK;
        }
    }
    const CUresult r = g_encode(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bdim,
                                estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return IZB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    if (g_maps.size() >= kMapCacheLimit) g_maps.clear();
    g_maps.emplace(key, *out);
    return IZB_OK;
}

}  // namespace izb
