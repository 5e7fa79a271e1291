// The convolution module of a Conformer encoder layer around its two pointwise (1x1) convolutions,
// which are linear layers and run on the GEMM: batch-norm folding at load time, and the depthwise
// convolution with the folded bias and the swish behind it in one pass over the activations.
// Activations stay [batch * frames, channels] (channels contiguous), the layout the surrounding
// linear layers produce and consume, so the reference's two transposes disappear.
#include "izb_common.cuh"

namespace {

__device__ __forceinline__ float swish_f(float v) { return v / (1.0f + __expf(-v)); }

// folded_w[c, j] = w[c, j] * scale[c], folded_b[c] = beta[c] - scale[c] * mean[c], scale = gamma / sqrt(var + eps)
// (gamma / beta null: 1 / 0).  fp32 in, bf16 out: runs once per layer at load time.
__global__ void fold_bn_kernel(const float* __restrict__ w, const float* __restrict__ gamma, const float* __restrict__ beta,
                               const float* __restrict__ mean, const float* __restrict__ var, float eps, int channels, int kernel,
                               __nv_bfloat16* __restrict__ folded_w, __nv_bfloat16* __restrict__ folded_b) {
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
        const float scale = (gamma ? gamma[c] : 1.0f) / sqrtf(var[c] + eps);
        for (int j = 0; j < kernel; ++j) folded_w[c * kernel + j] = __float2bfloat16_rn(w[c * kernel + j] * scale);
        folded_b[c] = __float2bfloat16_rn((beta ? beta[c] : 0.0f) - scale * mean[c]);
    }
}

// out[b, t, c] = act(bias[c] + sum_j w[c, j] * x[b, t + j - pad, c]), zero beyond the utterance's ends.
// A thread owns 8 channels (16 bytes of a row) and DW_T consecutive frames: it keeps the DW_T + kernel - 1
// input rows it needs in registers and walks the taps, so every input element is loaded once per
// DW_T outputs; neighbouring threads take neighbouring channel groups (whole rows are read contiguously).
constexpr int DW_T = 4;
constexpr int DW_MAX_KERNEL = 31;

__global__ void __launch_bounds__(128)
    depthwise_conv1d_kernel(const uint4* __restrict__ x, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ bias,
                            uint4* __restrict__ out, long long batch, int frames, int cgroups, int kernel, int pad, long long ldx_vec,
                            long long ldo_vec, int act) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const int t_tiles = (frames + DW_T - 1) / DW_T;
    const long long items = batch * t_tiles * cgroups;
    for (long long it = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; it < items;
         it += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int cg = static_cast<int>(it % cgroups);
        const long long bt = it / cgroups;
        const int tt = static_cast<int>(bt % t_tiles);
        const long long b = bt / t_tiles;
        const int t0 = tt * DW_T;
        float acc[DW_T][8];
#pragma unroll
        for (int i = 0; i < DW_T; ++i)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
        // walk the input rows t0 - pad .. t0 + DW_T - 1 + (kernel - 1 - pad); row r feeds output i with tap j = r - i + pad
        const int n_rows = DW_T + kernel - 1;
        for (int r = 0; r < n_rows; ++r) {
            const int t_in = t0 - pad + r;
            if (t_in < 0 || t_in >= frames) continue;
            const uint4 v = x[(b * frames + t_in) * ldx_vec + cg];
            const uint32_t q[4] = {v.x, v.y, v.z, v.w};
            float xv[8];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                xv[2 * e] = izb::bf16_lo_to_f32(q[e]);
                xv[2 * e + 1] = izb::bf16_hi_to_f32(q[e]);
            }
#pragma unroll
            for (int i = 0; i < DW_T; ++i) {
                const int j = r - i;  // tap index
                if (j < 0 || j >= kernel) continue;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][e] = fmaf(__bfloat162float(w[(cg * 8 + e) * kernel + j]), xv[e], acc[i][e]);
            }
        }
        float bv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) bv[e] = bias ? __bfloat162float(bias[cg * 8 + e]) : 0.f;
#pragma unroll
        for (int i = 0; i < DW_T; ++i) {
            if (t0 + i >= frames) break;
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float s = acc[i][e] + bv[e];
                o[e] = act ? swish_f(s) : s;
            }
            out[(b * frames + t0 + i) * ldo_vec + cg] = make_uint4(izb::pack_bf16x2(o[0], o[1]), izb::pack_bf16x2(o[2], o[3]),
                                                                   izb::pack_bf16x2(o[4], o[5]), izb::pack_bf16x2(o[6], o[7]));
        }
    }
}

}  // namespace

extern "C" {

int32_t izb_fold_depthwise_conv1d_batch_norm(izb_ctx* ctx, izb_stream stream, const float* conv_weight, const float* bn_weight,
                                             const float* bn_bias, const float* running_mean, const float* running_var, float eps,
                                             int64_t channels, int32_t kernel, void* folded_weight, void* folded_bias) {
    if (!ctx || channels <= 0 || kernel <= 0 || channels > INT32_MAX / kernel) return IZB_ERR_BAD_ARG;
    if (!conv_weight || !running_mean || !running_var || !folded_weight || !folded_bias || !(eps >= 0.f)) return IZB_ERR_BAD_ARG;
    if ((bn_weight == nullptr) != (bn_bias == nullptr)) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(conv_weight, 4) || !izb_aligned(running_mean, 4) || !izb_aligned(running_var, 4) || !izb_aligned(folded_weight, 2) ||
        !izb_aligned(folded_bias, 2))
        return IZB_ERR_BAD_ARG;
    const int grid = static_cast<int>((channels + 127) / 128);
    fold_bn_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(conv_weight, bn_weight, bn_bias, running_mean, running_var, eps,
                                                                        static_cast<int>(channels), kernel,
                                                                        static_cast<__nv_bfloat16*>(folded_weight),
                                                                        static_cast<__nv_bfloat16*>(folded_bias));
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_depthwise_conv1d_bias_swish(izb_ctx* ctx, izb_stream stream, const void* x, const void* weight, const void* bias, void* out,
                                        int64_t batch, int64_t frames, int64_t channels, int32_t kernel, int32_t padding,
                                        int64_t ld_x, int64_t ld_out, int32_t apply_swish) {
    if (!ctx || batch < 0 || frames < 0 || channels <= 0 || kernel <= 0 || padding < 0) return IZB_ERR_BAD_ARG;
    if (batch == 0 || frames == 0) return IZB_OK;
    if (!x || !weight || !out || ld_x < channels || ld_out < channels) return IZB_ERR_BAD_ARG;
    // "same" convolution, stride 1, dilation 1: what the Conformer block uses (padding = (kernel - 1) / 2)
    if (kernel > DW_MAX_KERNEL || kernel % 2 == 0 || padding != (kernel - 1) / 2) return IZB_ERR_UNSUPPORTED;
    if (channels % 8 != 0 || ld_x % 8 != 0 || ld_out % 8 != 0 || frames > INT32_MAX) return IZB_ERR_UNSUPPORTED;
    if (!izb_aligned(x, 16) || !izb_aligned(out, 16) || !izb_aligned(weight, 2) || (bias && !izb_aligned(bias, 2))) return IZB_ERR_BAD_ARG;
    const long long items = batch * ((frames + DW_T - 1) / DW_T) * (channels / 8);
    const long long cap = static_cast<long long>(ctx->sm_count) * 16, blocks = (items + 127) / 128;
    const int grid = static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
    IZB_CUDA_TRY(izb::launch_chained(ctx, depthwise_conv1d_kernel, dim3(grid), dim3(128), 0, static_cast<cudaStream_t>(stream),
                                     static_cast<const uint4*>(x), static_cast<const __nv_bfloat16*>(weight),
                                     static_cast<const __nv_bfloat16*>(bias), static_cast<uint4*>(out), static_cast<long long>(batch),
                                     static_cast<int>(frames), static_cast<int>(channels / 8), kernel, padding,
                                     static_cast<long long>(ld_x / 8), static_cast<long long>(ld_out / 8), apply_swish ? 1 : 0));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // extern "C"
