// Row-wise glue around the projections of a decode step: RMS normalisation (optionally after a
// residual add) and arg-max over logits.  HBM-bound, one pass over the data, 16-byte accesses
// when the rows allow.
#include <algorithm>

#include "izb_common.cuh"

namespace {

using izb::bf16_hi_to_f32;
using izb::bf16_lo_to_f32;
using izb::pack_bf16x2;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// One group of G threads (a warp, or the whole block) per row.  h = x (+ residual, rounded to bf16
// as the reference's tensor add does); out = h * rsqrt(mean(h^2) + eps) * weight, computed in fp32
// and rounded once.  The row is read once from global memory and kept in registers (up to
// 8 * MAX_VEC values per thread); longer rows are re-read in the second pass.
template <bool WARP_ROW>
__global__ void __launch_bounds__(256)
    rms_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ weight,
                    const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out,
                    __nv_bfloat16* __restrict__ sum_out, long long rows, int cols, long long ldx, long long ldr,
                    long long ldo, long long lds, float eps) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    __shared__ float partial[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = WARP_ROW ? 32 : blockDim.x;
    const int tid = WARP_ROW ? lane : threadIdx.x;
    const long long rows_per_block = WARP_ROW ? (blockDim.x >> 5) : 1;
    for (long long row = blockIdx.x * rows_per_block + (WARP_ROW ? warp : 0); row < rows;
         row += static_cast<long long>(gridDim.x) * rows_per_block) {
        const __nv_bfloat16* xr = x + row * ldx;
        const __nv_bfloat16* rr = residual ? residual + row * ldr : nullptr;
        __nv_bfloat16* sr = sum_out ? sum_out + row * lds : nullptr;
        float ss = 0.f;
        for (int c = tid; c < cols; c += group) {
            float h = __bfloat162float(xr[c]);
            if (rr) {
                h = __bfloat162float(__float2bfloat16_rn(h + __bfloat162float(rr[c])));
                if (sr) sr[c] = __float2bfloat16_rn(h);
            }
            ss += h * h;
        }
        ss = warp_sum(ss);
        if (!WARP_ROW) {
            if (lane == 0) partial[warp] = ss;
            __syncthreads();
            ss = 0.f;
            for (int w = 0; w < (blockDim.x >> 5); ++w) ss += partial[w];
            __syncthreads();
        }
        const float scale = rsqrtf(ss / static_cast<float>(cols) + eps);
        __nv_bfloat16* orow = out + row * ldo;
        for (int c = tid; c < cols; c += group) {
            float h = __bfloat162float(xr[c]);
            if (rr) h = __bfloat162float(__float2bfloat16_rn(h + __bfloat162float(rr[c])));
            orow[c] = __float2bfloat16_rn(h * scale * __bfloat162float(weight[c]));
        }
    }
}

// One block per row: the largest value and the lowest index that holds it.  NaN never wins
// (comparisons with it are false); a row of nothing but NaN gives index 0 and -inf.
template <typename T>
__global__ void __launch_bounds__(512)
    argmax_rows_kernel(const T* __restrict__ x, long long rows, long long cols, long long ldx, int32_t* __restrict__ out_idx,
                       float* __restrict__ out_val) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    __shared__ float sv[16];
    __shared__ long long si[16];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* xr = x + row * ldx;
        float best = -INFINITY;
        long long bi = 0x7FFFFFFFFFFFFFFFll;
        for (long long c = threadIdx.x; c < cols; c += blockDim.x) {
            const float v = static_cast<float>(xr[c]);
            if (v > best) {  // strided scan visits this thread's indices in increasing order: first maximum kept
                best = v;
                bi = c;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const long long oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (lane == 0) {
            sv[warp] = best;
            si[warp] = bi;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < (blockDim.x >> 5); ++w) {
                if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
                    best = sv[w];
                    bi = si[w];
                }
            }
            out_idx[row] = bi == 0x7FFFFFFFFFFFFFFFll ? 0 : static_cast<int32_t>(bi);
            if (out_val) out_val[row] = best;
        }
        __syncthreads();
    }
}

// A few very long rows (the logits of a decode step): `splits` CTAs share a row.  Each folds its
// best (value, index) into one 64-bit key per row with atomicMax: the value's bits made monotonic
// in the high word, the complemented index in the low word, so the largest key is the largest value
// at its lowest index.  The last CTA to arrive writes the row's result and zeroes key and counter
// for the next call.
__device__ __forceinline__ unsigned long long argmax_key(float v, long long idx) {
    const uint32_t b = v == 0.f ? 0u : __float_as_uint(v);  // -0 and +0 are equal maxima
    const uint32_t hi = b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
    const uint32_t lo = 0xFFFFFFFFu - static_cast<uint32_t>(idx > 0xFFFFFFFFll ? 0xFFFFFFFFll : idx);
    return (static_cast<unsigned long long>(hi) << 32) | lo;
}

template <typename T>
__global__ void __launch_bounds__(512)
    argmax_rows_split_kernel(const T* __restrict__ x, long long cols, long long ldx, int splits, int32_t* __restrict__ out_idx,
                             float* __restrict__ out_val, unsigned long long* __restrict__ keys,
                             unsigned int* __restrict__ done) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    __shared__ float sv[16];
    __shared__ long long si[16];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x / splits, part = blockIdx.x % splits;
    const long long chunk = (cols + splits - 1) / splits;
    const long long c0 = part * chunk, c1 = min(cols, c0 + chunk);
    const T* xr = x + static_cast<long long>(row) * ldx;
    float best = -INFINITY;
    long long bi = 0x7FFFFFFFFFFFFFFFll;
    for (long long c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
        const float v = static_cast<float>(xr[c]);
        if (v > best) {
            best = v;
            bi = c;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const long long oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
        }
    }
    if (lane == 0) {
        sv[warp] = best;
        si[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (blockDim.x >> 5); ++w) {
            if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
                best = sv[w];
                bi = si[w];
            }
        }
        atomicMax(&keys[row], argmax_key(best, bi));
        __threadfence();
        if (atomicAdd(&done[row], 1u) == static_cast<unsigned int>(splits - 1)) {
            __threadfence();
            const unsigned long long k = atomicExch(&keys[row], 0ull);
            done[row] = 0;
            const uint32_t hi = static_cast<uint32_t>(k >> 32), lo = static_cast<uint32_t>(k);
            const uint32_t idx = 0xFFFFFFFFu - lo;  // 0xFFFFFFFF: nothing but NaN in the row
            out_idx[row] = idx == 0xFFFFFFFFu ? 0 : static_cast<int32_t>(idx);
            if (out_val) out_val[row] = __uint_as_float(hi ^ ((hi >> 31) ? 0x80000000u : 0xFFFFFFFFu));
        }
    }
}

}  // namespace

extern "C" {

int32_t izb_rms_norm(izb_ctx* ctx, izb_stream stream, const void* x, const void* weight, const void* residual, void* out,
                     void* sum_out, int64_t rows, int64_t cols, int64_t ld_x, int64_t ld_residual, int64_t ld_out,
                     int64_t ld_sum, float eps) {
    if (!ctx || rows < 0 || cols < 0) return IZB_ERR_BAD_ARG;
    if (rows == 0 || cols == 0) return IZB_OK;
    if (!x || !weight || !out) return IZB_ERR_BAD_ARG;
    if (cols > INT32_MAX || ld_x < cols || ld_out < cols) return IZB_ERR_BAD_ARG;
    if (residual && ld_residual < cols) return IZB_ERR_BAD_ARG;
    if (sum_out && (!residual || ld_sum < cols)) return IZB_ERR_BAD_ARG;
    if (!(eps >= 0.f)) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(x, 2) || !izb_aligned(weight, 2) || !izb_aligned(out, 2) || (residual && !izb_aligned(residual, 2)) ||
        (sum_out && !izb_aligned(sum_out, 2)))
        return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    const auto* wp = static_cast<const __nv_bfloat16*>(weight);
    const auto* rp = static_cast<const __nv_bfloat16*>(residual);
    auto* op = static_cast<__nv_bfloat16*>(out);
    auto* sp = static_cast<__nv_bfloat16*>(sum_out);
    const long long cap = static_cast<long long>(ctx->sm_count) * 16;
    if (cols <= 512) {  // short rows (head-wise q/k norm): a warp per row, eight rows per block
        const long long blocks = (rows + 7) / 8;
        IZB_CUDA_TRY(izb::launch_chained(ctx, rms_norm_kernel<true>, dim3(static_cast<int>(blocks < cap ? blocks : cap)), dim3(256), 0,
                                         s, xp, wp, rp, op, sp, rows, static_cast<int>(cols), ld_x, ld_residual, ld_out, ld_sum,
                                         eps));
    } else {
        IZB_CUDA_TRY(izb::launch_chained(ctx, rms_norm_kernel<false>, dim3(static_cast<int>(rows < cap ? rows : cap)), dim3(256), 0, s,
                                         xp, wp, rp, op, sp, rows, static_cast<int>(cols), ld_x, ld_residual, ld_out, ld_sum, eps));
    }
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_argmax_rows(izb_ctx* ctx, izb_stream stream, const void* x, int32_t x_dtype, int64_t rows, int64_t cols,
                        int64_t ld_x, int32_t* out_idx, float* out_val) {
    if (!ctx || rows < 0 || cols < 0) return IZB_ERR_BAD_ARG;
    if (x_dtype != IZB_BF16 && x_dtype != IZB_F32) return IZB_ERR_BAD_ARG;
    if (rows == 0) return IZB_OK;
    if (cols == 0 || cols > INT32_MAX) return IZB_ERR_BAD_ARG;
    if (!x || !out_idx || ld_x < cols) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(x, x_dtype == IZB_F32 ? 4 : 2) || !izb_aligned(out_idx, 4) || (out_val && !izb_aligned(out_val, 4)))
        return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long cap = static_cast<long long>(ctx->sm_count) * 4;
    // few long rows: several CTAs per row, at least 8192 values each
    const long long splits = std::min<long long>(cols / 8192, cap / rows);
    if (rows <= IZB_ARGMAX_SPLIT_ROWS && splits >= 2) {
        const int grid = static_cast<int>(rows * splits);
        if (x_dtype == IZB_F32)
            IZB_CUDA_TRY(izb::launch_chained(ctx, argmax_rows_split_kernel<float>, dim3(grid), dim3(512), 0, s,
                                             static_cast<const float*>(x), cols, ld_x, static_cast<int>(splits), out_idx, out_val,
                                             ctx->d_argmax_keys, ctx->d_argmax_done));
        else
            IZB_CUDA_TRY(izb::launch_chained(ctx, argmax_rows_split_kernel<__nv_bfloat16>, dim3(grid), dim3(512), 0, s,
                                             static_cast<const __nv_bfloat16*>(x), cols, ld_x, static_cast<int>(splits), out_idx,
                                             out_val, ctx->d_argmax_keys, ctx->d_argmax_done));
        ctx->launches.fetch_add(1, std::memory_order_relaxed);
        return IZB_OK;
    }
    const int grid = static_cast<int>(rows < cap ? rows : cap);
    if (x_dtype == IZB_F32)
        IZB_CUDA_TRY(izb::launch_chained(ctx, argmax_rows_kernel<float>, dim3(grid), dim3(512), 0, s, static_cast<const float*>(x), rows,
                                         cols, ld_x, out_idx, out_val));
    else
        IZB_CUDA_TRY(izb::launch_chained(ctx, argmax_rows_kernel<__nv_bfloat16>, dim3(grid), dim3(512), 0, s,
                                         static_cast<const __nv_bfloat16*>(x), rows, cols, ld_x, out_idx, out_val));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // extern "C"
