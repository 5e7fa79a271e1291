// MLX affine-packed weights -> dense rows: the load-time expansion the reference does on the host for
// MLX-exported checkpoints (crates/izwi-core/src/models/shared/weights/mlx.rs:140-256), here on the device so that
// a packed checkpoint can be uploaded as it is stored.  HBM-bound: one thread per packed word, coalesced reads of
// the words and writes of the pack values behind them.
#include "izb_common.cuh"

namespace {

template <typename W>
__global__ void mlx_affine_kernel(const W* __restrict__ packed, const float* __restrict__ scales, const float* __restrict__ biases,
                                  long long out_dim, long long in_dim, long long packed_in, int pack, int bits, long long groups,
                                  int transposed, int out_dtype, void* __restrict__ out) {
    const long long group_size = in_dim / groups;
    const unsigned int mask = (1u << bits) - 1u;  // bits <= 8
    const long long total = out_dim * packed_in;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / packed_in, pcol = i - row * packed_in;
        const unsigned int word = static_cast<unsigned int>(packed[i]);
        for (int pi = 0; pi < pack; ++pi) {
            const long long col = pcol * pack + pi;
            const long long g = col / group_size;
            const long long pidx = transposed ? g * out_dim + row : row * groups + g;
            const float q = static_cast<float>((word >> (pi * bits)) & mask);
            // product and sum rounded separately, as the host code computes them
            const float v = __fadd_rn(__fmul_rn(q, scales[pidx]), biases ? biases[pidx] : 0.0f);
            izb::store_typed(out, out_dtype, row * in_dim + col, v);
        }
    }
}

}  // namespace

extern "C" int32_t izb_dequantize_mlx_affine(izb_ctx* ctx, izb_stream stream, const void* packed, int32_t word_bits, int64_t packed_in,
                                             const float* scales, const float* biases, int64_t groups, int32_t params_transposed,
                                             int64_t out_dim, int64_t in_dim, int32_t out_dtype, void* out) {
    if (!ctx || out_dim < 0 || in_dim < 0) return IZB_ERR_BAD_ARG;
    if (word_bits != 32 && word_bits != 8) return IZB_ERR_BAD_ARG;
    if (out_dtype != IZB_F32 && out_dtype != IZB_BF16 && out_dtype != IZB_F16) return IZB_ERR_BAD_ARG;
    // the reference's shape rules (mlx.rs:104-136, 78-95)
    if (packed_in <= 0 || in_dim <= 0 || in_dim % packed_in != 0) return IZB_ERR_BAD_ARG;
    const int64_t pack = in_dim / packed_in;
    if (pack > word_bits || word_bits % pack != 0) return IZB_ERR_BAD_ARG;
    const int64_t bits = word_bits / pack;
    if (bits == 0 || bits > 8) return IZB_ERR_BAD_ARG;
    if (groups <= 0 || in_dim % groups != 0) return IZB_ERR_BAD_ARG;
    if (out_dim == 0) return IZB_OK;
    if (!packed || !scales || !out) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(packed, word_bits / 8) || !izb_aligned(scales, 4) || (biases && !izb_aligned(biases, 4)) ||
        !izb_aligned(out, out_dtype == IZB_F32 ? 4 : 2))
        return IZB_ERR_BAD_ARG;
    if (out_dim > INT64_MAX / in_dim) return IZB_ERR_BAD_ARG;
    const long long total = out_dim * packed_in;
    const long long cap = static_cast<long long>(ctx->sm_count) * 16, want = (total + 255) / 256;
    const int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (word_bits == 32)
        mlx_affine_kernel<uint32_t><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(packed), scales, biases, out_dim, in_dim, packed_in,
                                                          static_cast<int>(pack), static_cast<int>(bits), groups, params_transposed ? 1 : 0,
                                                          out_dtype, out);
    else
        mlx_affine_kernel<uint8_t><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(packed), scales, biases, out_dim, in_dim, packed_in,
                                                         static_cast<int>(pack), static_cast<int>(bits), groups, params_transposed ? 1 : 0,
                                                         out_dtype, out);
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}
