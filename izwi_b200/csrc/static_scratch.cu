// A prefill-size linear layer over block-quantised weights that needs no caller workspace and
// performs no device allocation: the dequantised bf16 copy of the weights lives in a fixed
// array that is part of the library image.
#include <mutex>

#include "gemm_tc.cuh"
#include "izb_common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = IZB_STATIC_SCRATCH_BYTES;

// Resident on every GPU that loads the library, from load until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// In host code `g_static_scratch` is only a stand-in for the symbol, not a device address; the
// address a kernel can use has to be looked up once per device, with that device current.
int scratch_address(int device, void** out) {
    if (device < 0 || device >= kMaxDevices) return IZB_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[device]) {
        int current = -1;
        IZB_CUDA_TRY(cudaGetDevice(&current));
        if (current != device) IZB_CUDA_TRY(cudaSetDevice(device));
        void* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (current != device) (void)cudaSetDevice(current);
        if (err != cudaSuccess || !ptr) {
            (void)cudaGetLastError();
            return IZB_ERR_LAUNCH;
        }
        g_scratch_ptr[device] = ptr;
    }
    *out = g_scratch_ptr[device];
    return IZB_OK;
}

}  // namespace

extern "C" {

size_t izb_static_scratch_bytes(void) { return kStaticScratchBytes; }

int32_t izb_linear_quantized_static(izb_ctx* ctx, izb_stream stream, int32_t wfmt, const void* x, const void* w,
                                    const void* bias, void* y, int32_t y_dtype, int64_t M, int64_t N, int64_t K,
                                    int32_t epilogue) {
    if (!ctx) return IZB_ERR_BAD_ARG;
    if (wfmt != IZB_W_Q8_0 && wfmt != IZB_W_Q4_K) return IZB_ERR_BAD_ARG;
    if (M < 0 || N < 0 || K < 0) return IZB_ERR_BAD_ARG;
    if (M == 0 || N == 0) return IZB_OK;
    if (K == 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return IZB_ERR_UNSUPPORTED;
    if (K % (wfmt == IZB_W_Q8_0 ? 32 : 256) != 0) return IZB_ERR_BAD_ARG;  // a row is a whole number of blocks
    if (epilogue < IZB_EPI_NONE || epilogue > IZB_EPI_GLU) return IZB_ERR_BAD_ARG;
    if (y_dtype != IZB_BF16 && y_dtype != IZB_F32 && y_dtype != IZB_F16) return IZB_ERR_BAD_ARG;
    // the bf16 copy of the weights must fit the fixed array
    if (static_cast<unsigned long long>(N) * static_cast<unsigned long long>(K) * 2ull > kStaticScratchBytes)
        return IZB_ERR_SCRATCH_TOO_SMALL;
    if (!x || !w || !y) return IZB_ERR_BAD_ARG;
    void* scratch = nullptr;
    int rc = scratch_address(ctx->device, &scratch);
    if (rc != IZB_OK) return rc;
    // every element of the N*K region is rewritten here, so nothing left by an earlier call is read
    rc = izb_dequantize(ctx, stream, wfmt, w, N * K, IZB_BF16, scratch);
    if (rc != IZB_OK) return rc;
    const int n_out = (epilogue == IZB_EPI_SWIGLU || epilogue == IZB_EPI_GLU) ? static_cast<int>(N / 2) : static_cast<int>(N);
    return izb::gemm_tc_launch(ctx, static_cast<cudaStream_t>(stream), x, K, scratch, bias, y, n_out, y_dtype,
                               static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), epilogue, nullptr, 1);
}

}  // extern "C"
