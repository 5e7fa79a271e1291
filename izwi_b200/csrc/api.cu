// C ABI: context, block dequantisation, SwiGLU glue and the linear-layer entry points.
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include "izb_common.cuh"
#include "gemm_tc.cuh"
#include "skinny.cuh"

namespace izb {

// ---------------------------------------------------------------------------
// block dequantisation (bit-exact with GGML)
// ---------------------------------------------------------------------------
template <typename OutT>
__device__ __forceinline__ void store_val(OutT* out, long long i, float v);
template <>
__device__ __forceinline__ void store_val<float>(float* out, long long i, float v) {
    out[i] = v;
}
template <>
__device__ __forceinline__ void store_val<__nv_bfloat16>(__nv_bfloat16* out, long long i, float v) {
    out[i] = __float2bfloat16_rn(v);
}

// One thread per (block, 4 consecutive values): value = d * q.
template <typename OutT>
__global__ void dequant_q8_0_kernel(const uint8_t* __restrict__ raw, OutT* __restrict__ out, long long n_blocks) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_blocks * 8; i += stride) {
        const long long b = i >> 3;
        const int part = static_cast<int>(i & 7);
        const uint8_t* blk = raw + b * 34;
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(blk[0] | (blk[1] << 8))));
        const int8_t* q = reinterpret_cast<const int8_t*>(blk + 2 + part * 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) store_val(out, b * 32 + part * 4 + j, __fmul_rn(d, static_cast<float>(q[j])));
    }
}

// One thread per (super-block, sub-block, 4-value run): value = (d*sc)*q - (dmin*m), each
// product and the difference rounded on its own (no fused multiply-add), as GGML does.
template <typename OutT>
__global__ void dequant_q4_k_kernel(const uint8_t* __restrict__ raw, OutT* __restrict__ out, long long n_blocks) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_blocks * 64; i += stride) {
        const long long b = i >> 6;
        const int sub = static_cast<int>((i >> 3) & 7), part = static_cast<int>(i & 7);
        const uint8_t* blk = raw + b * 144;
        const uint16_t* hd = reinterpret_cast<const uint16_t*>(blk);
        const float d = __half2float(__ushort_as_half(hd[0])), dmin = __half2float(__ushort_as_half(hd[1]));
        const uint8_t* s = blk + 4;
        int sc, mn;
        if (sub < 4) {
            sc = s[sub] & 63;
            mn = s[sub + 4] & 63;
        } else {
            sc = (s[sub + 4] & 0x0F) | ((s[sub - 4] >> 6) << 4);
            mn = (s[sub + 4] >> 4) | ((s[sub] >> 6) << 4);
        }
        const float dsc = __fmul_rn(d, static_cast<float>(sc));
        const float dm = __fmul_rn(dmin, static_cast<float>(mn));
        const uint8_t* qs = blk + 16 + 32 * (sub >> 1) + part * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int q = (sub & 1) ? (qs[j] >> 4) : (qs[j] & 0x0F);
            store_val(out, b * 256 + sub * 32 + part * 4 + j, __fsub_rn(__fmul_rn(dsc, static_cast<float>(q)), dm));
        }
    }
}

// Q6_K: one thread per (super-block, 4-value run).  Value i of a block (half n = i / 128, group
// g = (i % 128) / 32, l = i % 32): low nibble from ql[64 n + 32 (g & 1) + l] (high nibble for
// g >= 2), bits 2g..2g+1 of qh[32 n + l], scale[8 n + l / 16 + 2 g]; value = (d * scale) * (code - 32).
template <typename OutT>
__global__ void dequant_q6_k_kernel(const uint8_t* __restrict__ raw, OutT* __restrict__ out, long long n_blocks) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_blocks * 64; i += stride) {
        const long long b = i >> 6;
        const int run = static_cast<int>(i & 63);  // values 4 run .. 4 run + 3 of the block
        const int n = run >> 5, g = (run >> 3) & 3, l0 = (run & 7) * 4;
        const uint8_t* blk = raw + b * 210;
        const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(blk[208] | (blk[209] << 8))));
        const float sc = static_cast<float>(reinterpret_cast<const int8_t*>(blk + 192)[8 * n + (l0 >> 4) + 2 * g]);
        const float dsc = __fmul_rn(d, sc);
        const uint8_t* ql = blk + 64 * n + 32 * (g & 1) + l0;
        const uint8_t* qh = blk + 128 + 32 * n + l0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int nib = g < 2 ? (ql[j] & 0x0F) : (ql[j] >> 4);
            const int q = (nib | (((qh[j] >> (2 * g)) & 3) << 4)) - 32;
            store_val(out, b * 256 + run * 4 + j, __fmul_rn(dsc, static_cast<float>(q)));
        }
    }
}

// Waits on a barrier that nothing ever completes, through the same bounded wait every pipeline
// kernel uses: it gives up after the limit, records it in the status word and returns normally.
__global__ void selftest_wait_kernel(int* status) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const bool done = mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag);
    if (!done && threadIdx.x == 0) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------
// out = silu(gate) * up
// ---------------------------------------------------------------------------
__device__ __forceinline__ float silu_mul_f(float g, float u) { return g / (1.0f + __expf(-g)) * u; }

__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                __nv_bfloat16* __restrict__ out, long long rows, long long cols, long long ldg,
                                long long ldu, long long ldo, int vec) {
    pdl_launch_dependents();
    pdl_wait();
    const long long cols_v = vec ? cols / 8 : cols;
    const long long total = rows * cols_v;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / cols_v, c = i % cols_v;
        if (vec) {
            const uint4 gv = *reinterpret_cast<const uint4*>(gate + r * ldg + c * 8);
            const uint4 uv = *reinterpret_cast<const uint4*>(up + r * ldu + c * 8);
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
            uint32_t ow[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                ow[j] = pack_bf16x2(silu_mul_f(bf16_lo_to_f32(gw[j]), bf16_lo_to_f32(uw[j])),
                                    silu_mul_f(bf16_hi_to_f32(gw[j]), bf16_hi_to_f32(uw[j])));
            *reinterpret_cast<uint4*>(out + r * ldo + c * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        } else {
            out[r * ldo + c] = __float2bfloat16_rn(
                silu_mul_f(__bfloat162float(gate[r * ldg + c]), __bfloat162float(up[r * ldu + c])));
        }
    }
}

// fp32 / fp16 activation rows -> dense bf16 rows (round to nearest even), the one rounding the
// bf16 x bf16 -> fp32 product applies to its left operand whatever type the caller holds it in.
template <typename T>
__global__ void cast_rows_bf16_kernel(const T* __restrict__ x, __nv_bfloat16* __restrict__ out, long long rows, long long cols,
                                      long long ldx) {
    pdl_launch_dependents();
    pdl_wait();
    const long long total = rows * cols, stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / cols, c = i % cols;
        float v;
        if constexpr (sizeof(T) == 4) v = x[r * ldx + c];
        else v = __half2float(x[r * ldx + c]);
        out[i] = __float2bfloat16_rn(v);
    }
}

static int grid_for(const izb_ctx* ctx, long long work_items, int threads) {
    const long long want = (work_items + threads - 1) / threads;
    const long long cap = static_cast<long long>(ctx->sm_count) * 16;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace izb

using namespace izb;

extern "C" {

int32_t izb_version(void) { return 100; }

int32_t izb_kernels_enabled(void) {
    static std::once_flag once;
    static int32_t enabled = 1;
    std::call_once(once, [] {
        const char* raw = std::getenv("IZWI_B200_KERNELS");
        if (!raw) return;  // unset: on
        std::string v(raw);
        const size_t a = v.find_first_not_of(" \t\r\n"), b = v.find_last_not_of(" \t\r\n");
        v = a == std::string::npos ? std::string() : v.substr(a, b - a + 1);
        for (char& c : v) c = static_cast<char>(std::tolower(static_cast<unsigned char>(c)));
        enabled = (v == "1" || v == "true" || v == "yes" || v == "on") ? 1 : 0;
    });
    return enabled;
}

const char* izb_status_string(int32_t status) {
    switch (status) {
        case IZB_OK: return "ok";
        case IZB_ERR_BAD_ARG: return "bad argument";
        case IZB_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case IZB_ERR_LAUNCH: return "CUDA launch or copy failed";
        case IZB_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case IZB_ERR_NO_DEVICE: return "no usable sm_100 device";
        case IZB_ERR_SCRATCH_TOO_SMALL: return "problem exceeds the library's fixed scratch array";
        default: return "unknown status";
    }
}

int32_t izb_ctx_create(int32_t device, izb_ctx** out) {
    if (!out || device < 0 || device >= IZB_MAX_DEVICES) return IZB_ERR_BAD_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device >= count) {
        (void)cudaGetLastError();
        return IZB_ERR_NO_DEVICE;
    }
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return IZB_ERR_NO_DEVICE;
    if (prop.major != 10) return IZB_ERR_NO_DEVICE;  // the kernels are sm_100a only
    int prev = 0;
    IZB_CUDA_TRY(cudaGetDevice(&prev));
    IZB_CUDA_TRY(cudaSetDevice(device));
    izb_ctx* ctx = new (std::nothrow) izb_ctx();
    if (!ctx) return IZB_ERR_LAUNCH;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->max_smem_optin = static_cast<int>(prop.sharedMemPerBlockOptin);
    ctx->launches.store(0);
    {
        const char* e = std::getenv("IZB_PDL");
        ctx->pdl = (e && e[0] == '0') ? 0 : 1;
    }
    ctx->d_status = nullptr;
    // one allocation: status words (padded to 64 bytes), then the arg-max keys and counters
    const size_t dev_bytes = 64 + static_cast<size_t>(IZB_ARGMAX_SPLIT_ROWS) * (sizeof(unsigned long long) + sizeof(unsigned int)) +
                             static_cast<size_t>(IZB_ROUTE_TILES) * sizeof(unsigned int);
    static_assert(IZB_STATUS_WORDS * sizeof(int) <= 64, "status words outgrew their slot");
    if (cudaMalloc(&ctx->d_status, dev_bytes) != cudaSuccess || cudaMemset(ctx->d_status, 0, dev_bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        delete ctx;
        (void)cudaSetDevice(prev);
        return IZB_ERR_LAUNCH;
    }
    ctx->d_argmax_keys = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(ctx->d_status) + 64);
    ctx->d_argmax_done = reinterpret_cast<unsigned int*>(ctx->d_argmax_keys + IZB_ARGMAX_SPLIT_ROWS);
    ctx->d_route_done = ctx->d_argmax_done + IZB_ARGMAX_SPLIT_ROWS;
    (void)cudaSetDevice(prev);
    *out = ctx;
    return IZB_OK;
}

int32_t izb_ctx_destroy(izb_ctx* ctx) {
    if (!ctx) return IZB_ERR_BAD_ARG;
    if (ctx->d_status) (void)cudaFree(ctx->d_status);
    delete ctx;
    return IZB_OK;
}

int32_t izb_ctx_check(izb_ctx* ctx, izb_stream stream) {
    if (!ctx) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int host[IZB_STATUS_WORDS] = {0};
    IZB_CUDA_TRY(cudaMemcpyAsync(host, ctx->d_status, sizeof(host), cudaMemcpyDeviceToHost, s));
    IZB_CUDA_TRY(cudaStreamSynchronize(s));
    bool any = false, waited = false;
    for (int i = 0; i < IZB_STATUS_WORDS; ++i) {
        any = any || host[i] != 0;
        waited = waited || (host[i] != 0 && i != 6);  // word 6: a token id outside the embedding table
    }
    if (any) {
        IZB_CUDA_TRY(cudaMemsetAsync(ctx->d_status, 0, sizeof(host), s));
        IZB_CUDA_TRY(cudaStreamSynchronize(s));
        return waited ? IZB_ERR_TIMEOUT : IZB_ERR_BAD_ARG;
    }
    return IZB_OK;
}

int64_t izb_ctx_launch_count(const izb_ctx* ctx) { return ctx ? ctx->launches.load() : 0; }

int32_t izb_ctx_selftest_wait_timeout(izb_ctx* ctx, izb_stream stream) {
    if (!ctx) return IZB_ERR_BAD_ARG;
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx->d_status + 7);
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_quantized_storage_bytes(int32_t wfmt, int64_t rows, int64_t cols, size_t* out_bytes) {
    if (!out_bytes || rows < 0 || cols < 0) return IZB_ERR_BAD_ARG;
    int64_t block, type;
    switch (wfmt) {
        case IZB_W_BF16: block = 1; type = 2; break;
        case IZB_W_Q8_0: block = 32; type = 34; break;
        case IZB_W_Q4_K: block = 256; type = 144; break;
        case IZB_W_Q6_K: block = 256; type = 210; break;
        default: return IZB_ERR_BAD_ARG;
    }
    if (cols != 0 && rows > INT64_MAX / cols) return IZB_ERR_BAD_ARG;  // element count overflows
    const int64_t elems = rows * cols;
    if (elems % block != 0) return IZB_ERR_BAD_ARG;
    if (elems / block > INT64_MAX / type) return IZB_ERR_BAD_ARG;
    *out_bytes = static_cast<size_t>(elems / block * type);
    return IZB_OK;
}

int32_t izb_dequantize(izb_ctx* ctx, izb_stream stream, int32_t wfmt, const void* raw, int64_t n_elems,
                       int32_t out_dtype, void* out) {
    if (!ctx || n_elems < 0) return IZB_ERR_BAD_ARG;
    if (out_dtype != IZB_F32 && out_dtype != IZB_BF16) return IZB_ERR_BAD_ARG;
    if (wfmt != IZB_W_Q8_0 && wfmt != IZB_W_Q4_K && wfmt != IZB_W_Q6_K) return IZB_ERR_UNSUPPORTED;
    const int64_t block = wfmt == IZB_W_Q8_0 ? 32 : 256;
    if (n_elems % block != 0) return IZB_ERR_BAD_ARG;
    if (n_elems == 0) return IZB_OK;
    if (!raw || !out || !izb_aligned(raw, 2) || !izb_aligned(out, out_dtype == IZB_F32 ? 4 : 2)) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long nb = n_elems / block;
    const uint8_t* r = static_cast<const uint8_t*>(raw);
    const int threads = 256;
    if (wfmt == IZB_W_Q8_0) {
        const int grid = grid_for(ctx, nb * 8, threads);
        if (out_dtype == IZB_F32)
            dequant_q8_0_kernel<float><<<grid, threads, 0, s>>>(r, static_cast<float*>(out), nb);
        else
            dequant_q8_0_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(r, static_cast<__nv_bfloat16*>(out), nb);
    } else if (wfmt == IZB_W_Q4_K) {
        const int grid = grid_for(ctx, nb * 64, threads);
        if (out_dtype == IZB_F32)
            dequant_q4_k_kernel<float><<<grid, threads, 0, s>>>(r, static_cast<float*>(out), nb);
        else
            dequant_q4_k_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(r, static_cast<__nv_bfloat16*>(out), nb);
    } else {
        const int grid = grid_for(ctx, nb * 64, threads);
        if (out_dtype == IZB_F32)
            dequant_q6_k_kernel<float><<<grid, threads, 0, s>>>(r, static_cast<float*>(out), nb);
        else
            dequant_q6_k_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(r, static_cast<__nv_bfloat16*>(out), nb);
    }
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_silu_mul(izb_ctx* ctx, izb_stream stream, const void* gate, const void* up, void* out, int64_t rows,
                     int64_t cols, int64_t ld_gate, int64_t ld_up, int64_t ld_out) {
    if (!ctx || rows < 0 || cols < 0) return IZB_ERR_BAD_ARG;
    if (rows == 0 || cols == 0) return IZB_OK;
    if (!gate || !up || !out) return IZB_ERR_BAD_ARG;
    if (ld_gate < cols || ld_up < cols || ld_out < cols) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(gate, 2) || !izb_aligned(up, 2) || !izb_aligned(out, 2)) return IZB_ERR_BAD_ARG;
    const bool vec = cols % 8 == 0 && ld_gate % 8 == 0 && ld_up % 8 == 0 && ld_out % 8 == 0 && izb_aligned(gate, 16) &&
                     izb_aligned(up, 16) && izb_aligned(out, 16);
    const long long items = rows * (vec ? cols / 8 : cols);
    const int threads = 256;
    IZB_CUDA_TRY(izb::launch_chained(ctx, silu_mul_kernel, dim3(grid_for(ctx, items, threads)), dim3(threads), 0,
                                     static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(gate),
                                     static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(out), rows, cols, ld_gate,
                                     ld_up, ld_out, vec ? 1 : 0));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

// Above this many token rows the tcgen05 GEMM takes over from the weight-streaming kernel.
static constexpr int64_t kStreamMaxM_bf16 = 32;
static constexpr int64_t kStreamMaxM_quant = 64;

// The weight-streaming kernels walk k in whole 256-value boxes of block-quantised rows (64 values of
// bf16 rows); other widths go to the tensor-core GEMM (block formats: through the bf16 copy).
static bool stream_width_ok(int32_t wfmt, int64_t K) { return K % (wfmt == IZB_W_BF16 ? 64 : 256) == 0; }

size_t izb_linear_workspace_bytes_ex(int32_t wfmt, int64_t M, int64_t N, int64_t K, int32_t epilogue) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const size_t dense = static_cast<size_t>(N) * static_cast<size_t>(K) * 2;
    if (wfmt == IZB_W_Q6_K) return dense;
    if (wfmt == IZB_W_Q8_0 || wfmt == IZB_W_Q4_K)
        return (M > kStreamMaxM_quant || epilogue != IZB_EPI_NONE || !stream_width_ok(wfmt, K)) ? dense : 0;
    return 0;
}

size_t izb_linear_workspace_bytes(int32_t wfmt, int64_t M, int64_t N, int64_t K) {
    return izb_linear_workspace_bytes_ex(wfmt, M, N, K, IZB_EPI_NONE);
}

int32_t izb_linear_fusion_max_tokens(int32_t wfmt) {
    if (wfmt != IZB_W_Q8_0 && wfmt != IZB_W_Q4_K) return 0;
    return skinny_gemv_max_tokens();
}

// Whether the one- and two-token integer-dot-product kernel takes this call with its prologue / residual inside.
static bool fuses_in_kernel(const izb_linear_args* a) {
    return (a->wfmt == IZB_W_Q8_0 || a->wfmt == IZB_W_Q4_K) && a->M <= izb_linear_fusion_max_tokens(a->wfmt) &&
           a->epilogue == IZB_EPI_NONE && stream_width_ok(a->wfmt, a->K);
}
static size_t align256(size_t v) { return (v + 255) / 256 * 256; }
// Bytes at the front of the workspace that the product itself uses: the bf16 copy of block-quantised
// weights on the routes that multiply one, or (3..16 tokens on the streaming route) the activations
// re-expressed for the integer tensor-core kernel.  The two never coincide.
static size_t product_workspace_bytes(const izb_linear_args* a) {
    const size_t dense = izb_linear_workspace_bytes_ex(a->wfmt, a->M, a->N, a->K, a->epilogue);
    if (dense) return dense;
    if (skinny_imma_format_ok(a->wfmt) && a->epilogue == IZB_EPI_NONE && a->M >= skinny_imma_min_tokens() && a->M <= skinny_imma_max_tokens())
        return skinny_imma_xq_bytes(16, a->K);
    return 0;
}

size_t izb_linear_workspace_bytes_args(const izb_linear_args* a) {
    if (!a || a->M <= 0 || a->N <= 0 || a->K <= 0) return 0;
    const size_t dense = product_workspace_bytes(a);
    const bool staged = a->x_dtype != IZB_BF16 || (a->prologue != IZB_PRO_NONE && !fuses_in_kernel(a));
    const size_t pro = staged ? align256(static_cast<size_t>(a->M) * static_cast<size_t>(a->K) * 2) : 0;
    return pro ? align256(dense) + pro : dense;
}

int32_t izb_linear(izb_ctx* ctx, izb_stream stream, const izb_linear_args* args) {
    if (!ctx || !args) return IZB_ERR_BAD_ARG;
    if (args->M < 0 || args->N < 0 || args->K < 0) return IZB_ERR_BAD_ARG;
    if (args->epilogue < IZB_EPI_NONE || args->epilogue > IZB_EPI_GLU) return IZB_ERR_BAD_ARG;
    if (args->prologue < IZB_PRO_NONE || args->prologue > IZB_PRO_SILU_MUL) return IZB_ERR_BAD_ARG;
    if (args->M == 0 || args->N == 0) return IZB_OK;
    if (args->K == 0) return IZB_ERR_UNSUPPORTED;
    if (args->M > INT32_MAX || args->N > INT32_MAX || args->K > INT32_MAX) return IZB_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (args->x_dtype != IZB_BF16) {
        // fp32 / fp16 activations: one cast launch writes the bf16 rows to the tail of the workspace
        if (args->x_dtype != IZB_F32 && args->x_dtype != IZB_F16) return IZB_ERR_BAD_ARG;
        if (args->prologue != IZB_PRO_NONE) return IZB_ERR_UNSUPPORTED;
        const size_t xb = args->x_dtype == IZB_F32 ? 4 : 2;
        const size_t dense = align256(product_workspace_bytes(args));
        const size_t rows = align256(static_cast<size_t>(args->M) * static_cast<size_t>(args->K) * 2);
        if (!args->workspace || !izb_aligned(args->workspace, 16) || args->workspace_bytes < dense + rows) return IZB_ERR_BAD_ARG;
        if (!args->x || !izb_aligned(args->x, xb) || args->ldx < args->K) return IZB_ERR_BAD_ARG;
        auto* xs = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(args->workspace) + dense);
        const int grid = grid_for(ctx, static_cast<long long>(args->M) * args->K, 256);
        if (args->x_dtype == IZB_F32)
            IZB_CUDA_TRY(launch_chained(ctx, cast_rows_bf16_kernel<float>, dim3(grid), dim3(256), 0, s, static_cast<const float*>(args->x),
                                        xs, static_cast<long long>(args->M), static_cast<long long>(args->K),
                                        static_cast<long long>(args->ldx)));
        else
            IZB_CUDA_TRY(launch_chained(ctx, cast_rows_bf16_kernel<__half>, dim3(grid), dim3(256), 0, s,
                                        static_cast<const __half*>(args->x), xs, static_cast<long long>(args->M),
                                        static_cast<long long>(args->K), static_cast<long long>(args->ldx)));
        ctx->launches.fetch_add(1, std::memory_order_relaxed);
        izb_linear_args plain = *args;
        plain.x = xs;
        plain.ldx = args->K;
        plain.x_dtype = IZB_BF16;
        plain.workspace_bytes = dense;
        if (dense == 0) plain.workspace = nullptr;
        return izb_linear(ctx, stream, &plain);
    }
    if (args->prologue != IZB_PRO_NONE && !fuses_in_kernel(args)) {
        // Routes whose kernel has no prologue stage (bf16 or Q6_K weights, more than two tokens, a fused
        // epilogue): the normalised rows (or the SiLU-multiply) are written once to the tail of the
        // workspace, bf16 as the reference's separate ops store them, and the product reads them there.
        // The residual still rides in the product's epilogue.
        const size_t dense = align256(product_workspace_bytes(args));
        const size_t pro = align256(static_cast<size_t>(args->M) * static_cast<size_t>(args->K) * 2);
        if (!args->workspace || !izb_aligned(args->workspace, 16) || args->workspace_bytes < dense + pro) return IZB_ERR_BAD_ARG;
        if (!args->x) return IZB_ERR_BAD_ARG;
        void* xs = static_cast<uint8_t*>(args->workspace) + dense;
        int rc;
        if (args->prologue == IZB_PRO_RMSNORM) {
            if (!args->norm_weight || args->ldx < args->K) return IZB_ERR_BAD_ARG;
            rc = izb_rms_norm(ctx, stream, args->x, args->norm_weight, nullptr, xs, nullptr, args->M, args->K, args->ldx, 0, args->K, 0,
                              args->norm_eps);
        } else {
            if (args->ldx < 2 * args->K) return IZB_ERR_BAD_ARG;
            rc = izb_silu_mul(ctx, stream, args->x, static_cast<const uint8_t*>(args->x) + static_cast<size_t>(args->K) * 2, xs, args->M,
                              args->K, args->ldx, args->ldx, args->K);
        }
        if (rc != IZB_OK) return rc;
        izb_linear_args plain = *args;
        plain.x = xs;
        plain.ldx = args->K;
        plain.prologue = IZB_PRO_NONE;
        plain.norm_weight = nullptr;
        plain.workspace_bytes = dense;  // what is left for the product itself
        if (dense == 0) plain.workspace = nullptr;
        return izb_linear(ctx, stream, &plain);
    }
    if (args->wfmt == IZB_W_Q6_K) {
        // no in-place kernel for 210-byte super-blocks: multiply the bf16 copy in the workspace
        const size_t need = static_cast<size_t>(args->N) * static_cast<size_t>(args->K) * 2;
        if (args->K % 256 != 0) return IZB_ERR_BAD_ARG;
        if (!args->workspace || args->workspace_bytes < need || !izb_aligned(args->workspace, 16)) return IZB_ERR_BAD_ARG;
        const int rc = izb_dequantize(ctx, stream, IZB_W_Q6_K, args->w, args->N * args->K, IZB_BF16, args->workspace);
        if (rc != IZB_OK) return rc;
        izb_linear_args dense = *args;
        dense.wfmt = IZB_W_BF16;
        dense.w = args->workspace;
        dense.workspace = nullptr;
        dense.workspace_bytes = 0;
        return izb_linear(ctx, stream, &dense);
    }
    const bool quant = args->wfmt == IZB_W_Q8_0 || args->wfmt == IZB_W_Q4_K;
    if (!quant && args->wfmt != IZB_W_BF16) return IZB_ERR_BAD_ARG;
    // a row must be a whole number of blocks, or the bytes of one row would run into the next
    if (quant && args->K % (args->wfmt == IZB_W_Q8_0 ? 32 : 256) != 0) return IZB_ERR_BAD_ARG;
    if (args->residual && (args->ld_residual < ((args->epilogue == IZB_EPI_SWIGLU || args->epilogue == IZB_EPI_GLU) ? args->N / 2 : args->N) || !izb_aligned(args->residual, 2)))
        return IZB_ERR_BAD_ARG;

    const void* w_dense = args->w;
    const bool streams = stream_width_ok(args->wfmt, args->K);
    bool use_gemm = !quant && (args->M > kStreamMaxM_bf16 || args->epilogue != IZB_EPI_NONE || !streams);
    if (quant && (args->M > kStreamMaxM_quant || args->epilogue != IZB_EPI_NONE || !streams)) {
        const size_t need = static_cast<size_t>(args->N) * static_cast<size_t>(args->K) * 2;
        if (args->workspace && args->workspace_bytes >= need && izb_aligned(args->workspace, 16)) {
            const int rc = izb_dequantize(ctx, stream, args->wfmt, args->w, args->N * args->K, IZB_BF16, args->workspace);
            if (rc != IZB_OK) return rc;
            w_dense = args->workspace;
            use_gemm = true;
        } else if (args->epilogue != IZB_EPI_NONE) {
            return IZB_ERR_BAD_ARG;  // a fused epilogue over block-quantised weights needs the workspace
        } else if (!streams) {
            return IZB_ERR_UNSUPPORTED;  // a row width the streaming kernels do not walk, and no workspace for the GEMM
        }
    }
    if (use_gemm) {
        if (!args->x || !args->y || !w_dense) return IZB_ERR_BAD_ARG;
        if (args->ldx < args->K) return IZB_ERR_BAD_ARG;
        return gemm_tc_launch(ctx, s, args->x, args->ldx, w_dense, args->bias, args->y, args->ldy, args->y_dtype,
                              static_cast<int>(args->M), static_cast<int>(args->N), static_cast<int>(args->K),
                              args->epilogue, nullptr, 1, args->residual, args->ld_residual);
    }
    // Token rows are processed 64 at a time by the weight-streaming kernel.
    const size_t ybytes = args->y_dtype == IZB_F32 ? 4 : 2;  // bf16 and fp16 are both two bytes
    for (int64_t m0 = 0; m0 < args->M; m0 += 64) {
        izb_linear_args a = *args;
        a.M = args->M - m0 < 64 ? args->M - m0 : 64;
        a.x = static_cast<const uint8_t*>(args->x) + static_cast<size_t>(m0) * args->ldx * 2;
        a.y = static_cast<uint8_t*>(args->y) + static_cast<size_t>(m0) * args->ldy * ybytes;
        if (args->residual) a.residual = static_cast<const uint8_t*>(args->residual) + static_cast<size_t>(m0) * args->ld_residual * 2;
        alignas(64) SkinnyProblem prob;
        SkinnyPlanHeader hdr;
        int rc = skinny_plan_build(ctx, &a, 1, &hdr, &prob);
        if (rc != IZB_OK) return rc;
        rc = skinny_launch(ctx, s, hdr, nullptr, &prob);
        if (rc != IZB_OK) return rc;
    }
    return IZB_OK;
}

static int32_t linear_typed(izb_ctx* ctx, izb_stream stream, int32_t wfmt, const void* x, const void* w,
                            const void* bias, void* y, int64_t M, int64_t N, int64_t K) {
    izb_linear_args a;
    std::memset(&a, 0, sizeof(a));
    a.wfmt = wfmt;
    a.y_dtype = IZB_BF16;
    a.x = x; a.w = w; a.bias = bias; a.y = y;
    a.M = M; a.N = N; a.K = K; a.ldx = K; a.ldy = N;
    return izb_linear(ctx, stream, &a);
}

int32_t izb_linear_bf16(izb_ctx* ctx, izb_stream stream, const void* x, const void* w, const void* bias, void* y,
                        int64_t M, int64_t N, int64_t K) {
    return linear_typed(ctx, stream, IZB_W_BF16, x, w, bias, y, M, N, K);
}
int32_t izb_linear_q8_0(izb_ctx* ctx, izb_stream stream, const void* x, const void* w, void* y, int64_t M, int64_t N,
                        int64_t K) {
    return linear_typed(ctx, stream, IZB_W_Q8_0, x, w, nullptr, y, M, N, K);
}
int32_t izb_linear_q4_k(izb_ctx* ctx, izb_stream stream, const void* x, const void* w, void* y, int64_t M, int64_t N,
                        int64_t K) {
    return linear_typed(ctx, stream, IZB_W_Q4_K, x, w, nullptr, y, M, N, K);
}

size_t izb_linear_group_plan_bytes(int32_t n_problems) {
    if (n_problems <= 0) return 0;
    return sizeof(SkinnyPlanHeader) + static_cast<size_t>(n_problems) * sizeof(SkinnyProblem);
}

int32_t izb_linear_group_plan(izb_ctx* ctx, const izb_linear_args* problems, int32_t n_problems, void* host_plan,
                              size_t host_plan_bytes) {
    if (!ctx || !problems || !host_plan || n_problems <= 0) return IZB_ERR_BAD_ARG;
    if (host_plan_bytes < izb_linear_group_plan_bytes(n_problems) || !izb_aligned(host_plan, 64)) return IZB_ERR_BAD_ARG;
    auto* hdr = static_cast<SkinnyPlanHeader*>(host_plan);
    auto* probs = reinterpret_cast<SkinnyProblem*>(static_cast<uint8_t*>(host_plan) + sizeof(SkinnyPlanHeader));
    return skinny_plan_build(ctx, problems, n_problems, hdr, probs);
}

int32_t izb_linear_group_launch(izb_ctx* ctx, izb_stream stream, const void* host_plan, const void* dev_plan) {
    if (!ctx || !host_plan || !dev_plan || !izb_aligned(dev_plan, 64)) return IZB_ERR_BAD_ARG;
    const auto* hdr = static_cast<const SkinnyPlanHeader*>(host_plan);
    const auto* dev = reinterpret_cast<const SkinnyProblem*>(static_cast<const uint8_t*>(dev_plan) + sizeof(SkinnyPlanHeader));
    return skinny_launch(ctx, static_cast<cudaStream_t>(stream), *hdr, dev, nullptr);
}

int32_t izb_linear_group_launch_host(izb_ctx* ctx, izb_stream stream, const void* host_plan, const void* dev_plan, const void* host_in,
                                     void* dev_in, size_t in_bytes, const void* dev_out, void* host_out, size_t out_bytes) {
    if (!ctx || (in_bytes && (!host_in || !dev_in)) || (out_bytes && (!dev_out || !host_out))) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_bytes) IZB_CUDA_TRY(cudaMemcpyAsync(dev_in, host_in, in_bytes, cudaMemcpyHostToDevice, s));
    const int32_t st = izb_linear_group_launch(ctx, stream, host_plan, dev_plan);
    if (st != IZB_OK) return st;
    if (out_bytes) IZB_CUDA_TRY(cudaMemcpyAsync(host_out, dev_out, out_bytes, cudaMemcpyDeviceToHost, s));
    IZB_CUDA_TRY(cudaStreamSynchronize(s));
    return IZB_OK;
}

}  // extern "C"
