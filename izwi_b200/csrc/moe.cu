// Mixture-of-experts glue around the grouped GEMM: top-k routing, the stable (expert, token)
// permutation, row gather and the weighted combine.  The rules (this project's specification,
// the reference has no MoE code): experts are chosen by logit, ties go to the lowest expert id;
// weights are the softmax over the chosen logits; permuted rows are ordered by expert and, inside
// one expert, by ascending (token, slot); the combine adds slots in ascending slot order in fp32.
#include <cstring>

#include "gemm_tc.cuh"
#include <cstdlib>

#include "izb_common.cuh"

namespace izb {

constexpr int MOE_MAX_EXPERTS = 512;
constexpr int MOE_MAX_TOPK = 32;

// Top-k of one token's logits by one warp.  Each lane keeps experts lane, lane+32, ...; k rounds of
// warp arg-max (largest logit, lowest expert id among equals); weights = softmax over the chosen logits.
__device__ __forceinline__ void topk_row(const volatile float* row, int lane, int E, int k, int* idx_row, float* wts_row) {
    float v[MOE_MAX_EXPERTS / 32];
#pragma unroll
    for (int i = 0; i < MOE_MAX_EXPERTS / 32; ++i) {
        const int e = lane + 32 * i;
        v[i] = e < E ? row[e] : -INFINITY;
    }
    float first = 0.f, sum = 0.f, mine = 0.f;
    for (int j = 0; j < k; ++j) {
        float best = -INFINITY;
        int best_e = 0x7FFFFFFF;
#pragma unroll
        for (int i = 0; i < MOE_MAX_EXPERTS / 32; ++i) {
            const int e = lane + 32 * i;
            if (e < E && (v[i] > best || (v[i] == best && e < best_e))) {
                best = v[i];
                best_e = e;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, off);
            const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, off);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        if (best_e == 0x7FFFFFFF) best_e = j < E ? j : 0;  // every remaining logit is -inf or NaN
        if ((best_e & 31) == lane) {
#pragma unroll
            for (int i = 0; i < MOE_MAX_EXPERTS / 32; ++i)
                if (i == (best_e >> 5)) v[i] = -INFINITY;
        }
        if (j == 0) first = best;
        const float ex = expf(best - first);
        sum += ex;
        if (lane == j) mine = ex;
        if (lane == 0) idx_row[j] = best_e;
    }
    if (lane < k) wts_row[lane] = mine / sum;
}

// One warp per token.
__global__ void moe_topk_kernel(const float* __restrict__ logits, int T, int E, int k, int* __restrict__ idx,
                                float* __restrict__ wts) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < T; t += gridDim.x * warps_per_block)
        topk_row(logits + static_cast<long long>(t) * E, lane, E, k, idx + static_cast<long long>(t) * k,
                 wts + static_cast<long long>(t) * k);
}

// Router and top-k in one launch: logits[T, E] = x[T, H] . w[E, H]^T + bias (fp32), then the top-k of
// every token.  A CTA computes 16 tokens x (8 NG) experts with mma.sync m16n8k16: warp (ng, ks) owns
// the 8 experts of group ng and every KS-th 32-value block of H; both operands are read straight
// from global memory (the router weight is a few hundred KB and stays in L2) with 16-byte loads under
// a permutation of k that is the same for both, so each lane's 16 bytes are its fragments of two
// k-steps.  The k-slices meet through shared memory, the logits go to global memory, and the last
// CTA of a token tile to finish (a counter per tile, left at zero again) picks the experts of its 16
// tokens, one warp per token.  NG x KS = 8 warps: (4, 2) in general, (1, 8) for a single token tile,
// where E / 8 CTAs each stream eight rows of the weight instead of E / 32 CTAs thirty-two.
// (A single token tile as one cluster of eight CTAs, the logits meeting in CTA 0's shared memory instead of the
// counter and the last CTA's trip to L2, was measured: 0.0336 ms per one-token layer against 0.0307, since eight
// CTAs halve the loads in flight per expert row.)
constexpr int ROUTE_TOKENS = 16;
constexpr int ROUTE_WARPS = 8;
constexpr int ROUTE_MAX_TILES = 1024;

template <int NG, int KS>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
    moe_route_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ bias, int T, int H, int E, int k, float* __restrict__ logits,
                     int* __restrict__ idx, float* __restrict__ wts, unsigned int* __restrict__ tile_done) {
    static_assert(NG * KS == ROUTE_WARPS, "eight warps");
    __shared__ float part[KS][NG][32][4];
    __shared__ int is_last;
    izb::pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int ng = warp % NG, ks = warp / NG;
    const int tok0 = blockIdx.x * ROUTE_TOKENS;
    const int n0 = (blockIdx.y * NG + ng) * 8;  // first expert of this warp's group
    const bool live = n0 < E;
    // rows past the end repeat the last token (their results are not stored)
    const int r_lo = min(tok0 + g, T - 1), r_hi = min(tok0 + g + 8, T - 1);
    izb::pdl_wait();  // x is the output of the kernel before this one
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        const uint4* xa = reinterpret_cast<const uint4*>(x + r_lo * ldx) + t4;
        const uint4* xb = reinterpret_cast<const uint4*>(x + r_hi * ldx) + t4;
        const uint4* wr = reinterpret_cast<const uint4*>(w + static_cast<long long>(min(n0 + g, E - 1)) * H) + t4;
        const int n_blk = H / 32;
#pragma unroll(KS == 8 ? 8 : 4)  // a single token tile: the eight steps of H = 2048 in one batch of loads
        for (int b = ks; b < n_blk; b += KS) {
            const uint4 a_lo = xa[b * 4], a_hi = xb[b * 4], bw = wr[b * 4];
            mma_bf16_16816(acc, a_lo.x, a_hi.x, a_lo.y, a_hi.y, bw.x, bw.y);
            mma_bf16_16816(acc, a_lo.z, a_hi.z, a_lo.w, a_hi.w, bw.z, bw.w);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) part[ks][ng][lane][i] = acc[i];
    __syncthreads();
    if (ks == 0 && live) {
#pragma unroll
        for (int s2 = 1; s2 < KS; ++s2)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[i] += part[s2][ng][lane][i];
        // c0, c1: token g, experts n0 + 2 t4, + 1; c2, c3: token g + 8
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int tok = tok0 + g + (i >> 1) * 8, e = n0 + 2 * t4 + (i & 1);
            if (tok < T && e < E) logits[static_cast<long long>(tok) * E + e] = acc[i] + (bias ? __bfloat162float(bias[e]) : 0.f);
        }
    }
    // the last CTA of this token tile to get here sees every group's logits and picks the experts
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(&tile_done[blockIdx.x], 1u);
        is_last = prev == gridDim.y - 1;
        if (is_last) tile_done[blockIdx.x] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int tt = warp; tt < ROUTE_TOKENS; tt += ROUTE_WARPS) {
        const int tok = tok0 + tt;
        if (tok < T)
            topk_row(logits + static_cast<long long>(tok) * E, lane, E, k,
                     idx + static_cast<long long>(tok) * k, wts + static_cast<long long>(tok) * k);
    }
}

// ---------------------------------------------------------------------------
// A handful of tokens (decode): no permutation, no gather, no grouped GEMM.  Every (token, expert) pair
// streams its expert's rows once with 16-byte loads (a warp per output, fp32 accumulation, one shuffle
// reduction): two launches behind the router, HBM-bound on the 8 experts' 9.4 MB each instead of
// launch-bound on six kernels.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float dot8(uint4 a, uint4 b, float acc) {
    const uint32_t x[4] = {a.x, a.y, a.z, a.w}, y[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc = fmaf(izb::bf16_lo_to_f32(x[i]), izb::bf16_lo_to_f32(y[i]), acc);
        acc = fmaf(izb::bf16_hi_to_f32(x[i]), izb::bf16_hi_to_f32(y[i]), acc);
    }
    return acc;
}

// hidden[p][i] = silu(gate_i . x_t) * (up_i . x_t) for pair p = (t, j), expert idx[p]; grid (outputs / 8, pairs).
// A warp owns output i: its gate row and its up row, sixteen 16-byte loads per lane and pass of 2048 values of H,
// all issued before the first product.  The loads of the first pass go out before the token's row is staged in
// shared memory, so that the two trips to memory overlap.
constexpr int MOE_SMALL_HB = 8;  // 16-byte units per lane, row and pass
struct MoeSmallRows {
    uint4 g[MOE_SMALL_HB], u[MOE_SMALL_HB];
};
__device__ __forceinline__ void moe_small_load(MoeSmallRows& r, const uint4* g, const uint4* u, int c0, int h_units, int lane) {
#pragma unroll
    for (int m = 0; m < MOE_SMALL_HB; ++m) {
        const int c = c0 + 32 * m + lane;
        r.g[m] = c < h_units ? g[c] : make_uint4(0u, 0u, 0u, 0u);
        r.u[m] = c < h_units ? u[c] : make_uint4(0u, 0u, 0u, 0u);
    }
}
__device__ __forceinline__ void moe_small_dot(const MoeSmallRows& r, const uint4* xs, int c0, int h_units, int lane, float& ag, float& au) {
#pragma unroll
    for (int m = 0; m < MOE_SMALL_HB; ++m) {
        const int c = c0 + 32 * m + lane;
        if (c < h_units) {
            const uint4 xv = xs[c];
            ag = dot8(r.g[m], xv, ag);
            au = dot8(r.u[m], xv, au);
        }
    }
}
__global__ void __launch_bounds__(256)
    moe_small_gate_up_kernel(const uint4* __restrict__ x, long long ldx_units, const int* __restrict__ idx,
                             const uint4* __restrict__ w_gate_up, int h_units, int I, int top_k, __nv_bfloat16* __restrict__ hidden) {
    extern __shared__ uint4 xs[];  // the token's row
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const int p = blockIdx.y, t = p / top_k, e = idx[p];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint4* base = w_gate_up + static_cast<long long>(e) * 2 * I * h_units;
    int i = blockIdx.x * 8 + warp;
    MoeSmallRows r;
    bool loaded = false;  // the first pass of the first row is in flight while the token's row is staged
    if (i < I) {
        moe_small_load(r, base + static_cast<long long>(i) * h_units, base + static_cast<long long>(I + i) * h_units, 0, h_units, lane);
        loaded = true;
    }
    for (int c = threadIdx.x; c < h_units; c += blockDim.x) xs[c] = x[static_cast<long long>(t) * ldx_units + c];
    __syncthreads();
    for (; i < I; i += gridDim.x * 8) {
        const uint4* g = base + static_cast<long long>(i) * h_units;
        const uint4* u = base + static_cast<long long>(I + i) * h_units;
        float ag = 0.f, au = 0.f;
        for (int c0 = 0; c0 < h_units; c0 += 32 * MOE_SMALL_HB) {
            if (!loaded) moe_small_load(r, g, u, c0, h_units, lane);
            loaded = false;
            moe_small_dot(r, xs, c0, h_units, lane, ag, au);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ag += __shfl_xor_sync(0xFFFFFFFFu, ag, o);
            au += __shfl_xor_sync(0xFFFFFFFFu, au, o);
        }
        if (lane == 0) hidden[static_cast<long long>(p) * I + i] = __float2bfloat16_rn(ag / (1.0f + __expf(-ag)) * au);
    }
}

// y[t][n] = sum_j wts[t][j] * (down_{e_j}[n] . hidden[t][j]); grid (outputs / 8, tokens).
// A warp owns one output row n.  Its weights are top_k short rows (I values each) in top_k different matrices: the
// loads of four experts' rows (up to sixteen 16-byte loads per lane) are issued together, before the first product,
// so that a row costs two trips to memory instead of one per expert; the expert ids and routing weights are asked
// for before the token's hidden rows are staged, so that those trips overlap too.
constexpr int MOE_SMALL_JB = 4;  // experts per batch of loads
constexpr int MOE_SMALL_CB = 4;  // 16-byte units per lane and expert in a batch (128 units = 1024 values of I per pass)
__global__ void __launch_bounds__(256)
    moe_small_down_kernel(const uint4* __restrict__ hidden, const int* __restrict__ idx, const float* __restrict__ wts,
                          const uint4* __restrict__ w_down, int H, int i_units, int top_k, __nv_bfloat16* __restrict__ y) {
    extern __shared__ uint4 hs[];  // [top_k][i_units]
    __shared__ int s_e[32];
    __shared__ float s_w[32];
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const int t = blockIdx.y;
    if (threadIdx.x < top_k && threadIdx.x < 32) {
        s_e[threadIdx.x] = idx[t * top_k + threadIdx.x];
        s_w[threadIdx.x] = wts[t * top_k + threadIdx.x];
    }
    for (int c = threadIdx.x; c < top_k * i_units; c += blockDim.x) hs[c] = hidden[static_cast<long long>(t) * top_k * i_units + c];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int n = blockIdx.x * 8 + warp; n < H; n += gridDim.x * 8) {
        float out = 0.f;
        for (int j0 = 0; j0 < top_k; j0 += MOE_SMALL_JB) {
            float acc[MOE_SMALL_JB];
#pragma unroll
            for (int jj = 0; jj < MOE_SMALL_JB; ++jj) acc[jj] = 0.f;
            for (int c0 = 0; c0 < i_units; c0 += 32 * MOE_SMALL_CB) {
                uint4 wv[MOE_SMALL_JB][MOE_SMALL_CB];
#pragma unroll
                for (int jj = 0; jj < MOE_SMALL_JB; ++jj) {
                    const int j = min(j0 + jj, top_k - 1);  // past the last expert: its row again, weight 0 below
                    const uint4* row = w_down + (static_cast<long long>(s_e[j]) * H + n) * i_units;
#pragma unroll
                    for (int m = 0; m < MOE_SMALL_CB; ++m) {
                        const int c = c0 + 32 * m + lane;
                        wv[jj][m] = c < i_units ? row[c] : make_uint4(0u, 0u, 0u, 0u);
                    }
                }
#pragma unroll
                for (int jj = 0; jj < MOE_SMALL_JB; ++jj) {
                    const int j = min(j0 + jj, top_k - 1);
#pragma unroll
                    for (int m = 0; m < MOE_SMALL_CB; ++m) {
                        const int c = c0 + 32 * m + lane;
                        if (c < i_units) acc[jj] = dot8(wv[jj][m], hs[j * i_units + c], acc[jj]);
                    }
                }
            }
#pragma unroll
            for (int jj = 0; jj < MOE_SMALL_JB; ++jj)
                if (j0 + jj < top_k) out = fmaf(s_w[j0 + jj], acc[jj], out);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) out += __shfl_xor_sync(0xFFFFFFFFu, out, o);
        if (lane == 0) y[static_cast<long long>(t) * H + n] = __float2bfloat16_rn(out);
    }
}

// One block per expert e, every warp owning one contiguous range of the pairs.  Pass 1: each warp
// counts, in its range, the pairs routed to e and (summed over the block) to experts below e: the
// segment start and, by a scan over the warps, where each warp's hits begin.  Pass 2: each warp walks
// its range again in order and hands out positions, so equal experts keep ascending pair order.  No
// block depends on another, and inside a block the warps meet once.
__global__ void moe_permute_kernel(const int* __restrict__ idx, int pairs, int E, int* __restrict__ offsets,
                                   int* __restrict__ perm, int* __restrict__ inv) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    __shared__ int warp_equal[32], warp_below[32];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // ranges are whole multiples of 32 pairs so that a warp's lanes read consecutive pairs
    const int per_warp = ((pairs + nwarps - 1) / nwarps + 31) / 32 * 32;
    const int lo = min(warp * per_warp, pairs), hi = min(lo + per_warp, pairs);

    int below = 0, equal = 0;
    for (int p = lo + lane; p < hi; p += 32) {
        const int x = idx[p];
        below += x < e;
        equal += x == e;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        below += __shfl_xor_sync(0xFFFFFFFFu, below, off);
        equal += __shfl_xor_sync(0xFFFFFFFFu, equal, off);
    }
    if (lane == 0) {
        warp_below[warp] = below;
        warp_equal[warp] = equal;
    }
    __syncthreads();
    int base = 0, before = 0, total = 0;
    for (int w = 0; w < nwarps; ++w) {
        base += warp_below[w];
        if (w < warp) before += warp_equal[w];
        total += warp_equal[w];
    }
    if (threadIdx.x == 0) {
        offsets[e] = base;
        if (e == E - 1) offsets[E] = base + total;
    }
    int at = base + before;
    for (int p0 = lo; p0 < hi; p0 += 32) {
        const int p = p0 + lane;
        const bool hit = p < hi && idx[p] == e;
        const unsigned ballot = __ballot_sync(0xFFFFFFFFu, hit);
        if (hit) {
            const int pos = at + __popc(ballot & ((1u << lane) - 1u));
            perm[pos] = p;
            inv[p] = pos;
        }
        at += __popc(ballot);
    }
}

// x_perm[r] = x[perm[r] / k], 16 bytes per thread.
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ perm, int k, int rows,
                                  int vec_per_row, long long ldx_vec, uint4* __restrict__ out) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const long long total = static_cast<long long>(rows) * vec_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int r = static_cast<int>(i / vec_per_row), c = static_cast<int>(i % vec_per_row);
        out[i] = x[static_cast<long long>(perm[r] / k) * ldx_vec + c];
    }
}

// y[t] = sum over slots (ascending) of w[t, slot] * yp[inv[t*k + slot]], fp32 accumulate, 8 columns per thread.
__global__ void moe_combine_kernel(const uint4* __restrict__ yp, const int* __restrict__ inv, const float* __restrict__ wts,
                                   int T, int k, int vec_per_row, uint4* __restrict__ y) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const long long total = static_cast<long long>(T) * vec_per_row;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int t = static_cast<int>(i / vec_per_row), c = static_cast<int>(i % vec_per_row);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < k; ++s) {
            const float w = wts[static_cast<long long>(t) * k + s];
            const uint4 v = yp[static_cast<long long>(inv[static_cast<long long>(t) * k + s]) * vec_per_row + c];
            const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                acc[2 * j] = fmaf(w, bf16_lo_to_f32(q[j]), acc[2 * j]);
                acc[2 * j + 1] = fmaf(w, bf16_hi_to_f32(q[j]), acc[2 * j + 1]);
            }
        }
        y[i] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                          pack_bf16x2(acc[6], acc[7]));
    }
}

static int blocks_for(const izb_ctx* ctx, long long items, int threads) {
    const long long want = (items + threads - 1) / threads, cap = static_cast<long long>(ctx->sm_count) * 16;
    return static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace izb

using namespace izb;

extern "C" {

int32_t izb_moe_topk(izb_ctx* ctx, izb_stream stream, const void* logits, int64_t T, int64_t E, int32_t top_k,
                     void* idx_out, void* weights_out) {
    if (!ctx || T < 0 || E <= 0 || top_k <= 0) return IZB_ERR_BAD_ARG;
    if (E > MOE_MAX_EXPERTS || top_k > MOE_MAX_TOPK || top_k > E) return IZB_ERR_UNSUPPORTED;
    if (T == 0) return IZB_OK;
    if (!logits || !idx_out || !weights_out) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(logits, 4) || !izb_aligned(idx_out, 4) || !izb_aligned(weights_out, 4)) return IZB_ERR_BAD_ARG;
    const int threads = 128;
    IZB_CUDA_TRY(izb::launch_chained(ctx, moe_topk_kernel, dim3(blocks_for(ctx, T * 32, threads)), dim3(threads), 0,
                                     static_cast<cudaStream_t>(stream), static_cast<const float*>(logits), static_cast<int>(T),
                                     static_cast<int>(E), top_k, static_cast<int*>(idx_out), static_cast<float*>(weights_out)));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_moe_route(izb_ctx* ctx, izb_stream stream, const void* x, int64_t ld_x, const void* w_router,
                      const void* router_bias, int64_t T, int64_t H, int64_t E, int32_t top_k, void* logits_out,
                      void* idx_out, void* weights_out) {
    if (!ctx || T < 0 || H <= 0 || E <= 0 || top_k <= 0 || ld_x < H) return IZB_ERR_BAD_ARG;
    if (E > MOE_MAX_EXPERTS || top_k > MOE_MAX_TOPK || top_k > E) return IZB_ERR_UNSUPPORTED;
    if (T == 0) return IZB_OK;
    if (!x || !w_router || !logits_out || !idx_out || !weights_out) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(logits_out, 4) || !izb_aligned(idx_out, 4) || !izb_aligned(weights_out, 4)) return IZB_ERR_BAD_ARG;
    if (router_bias && !izb_aligned(router_bias, 2)) return IZB_ERR_BAD_ARG;
    const int64_t tiles = (T + ROUTE_TOKENS - 1) / ROUTE_TOKENS;
    const bool fused = H % 32 == 0 && ld_x % 8 == 0 && izb_aligned(x, 16) && izb_aligned(w_router, 16) &&
                       tiles <= ROUTE_MAX_TILES && T <= INT32_MAX / E;
    if (!fused) {
        // shapes the fused kernel does not take: the linear layer, then the top-k kernel
        izb_linear_args r;
        memset(&r, 0, sizeof(r));
        r.wfmt = IZB_W_BF16;
        r.y_dtype = IZB_F32;
        r.x = x; r.w = w_router; r.bias = router_bias; r.y = logits_out;
        r.M = T; r.N = E; r.K = H; r.ldx = ld_x; r.ldy = E;
        const int rc = izb_linear(ctx, stream, &r);
        if (rc != IZB_OK) return rc;
        return izb_moe_topk(ctx, stream, logits_out, T, E, top_k, idx_out, weights_out);
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto* xp = static_cast<const __nv_bfloat16*>(x);
    const auto* wp = static_cast<const __nv_bfloat16*>(w_router);
    const auto* bp = static_cast<const __nv_bfloat16*>(router_bias);
    auto* lp = static_cast<float*>(logits_out);
    auto* ip = static_cast<int*>(idx_out);
    auto* op = static_cast<float*>(weights_out);
    const int Ti = static_cast<int>(T), Hi = static_cast<int>(H), Ei = static_cast<int>(E);
    if (tiles == 1) {
        const dim3 grid(1, static_cast<unsigned>((E + 7) / 8));
        IZB_CUDA_TRY(izb::launch_chained(ctx, moe_route_kernel<1, 8>, grid, dim3(ROUTE_WARPS * 32), 0, s, xp, ld_x, wp, bp, Ti, Hi, Ei,
                                         top_k, lp, ip, op, ctx->d_route_done));
    } else {
        const dim3 grid(static_cast<unsigned>(tiles), static_cast<unsigned>((E + 31) / 32));
        IZB_CUDA_TRY(izb::launch_chained(ctx, moe_route_kernel<4, 2>, grid, dim3(ROUTE_WARPS * 32), 0, s, xp, ld_x, wp, bp, Ti, Hi, Ei,
                                         top_k, lp, ip, op, ctx->d_route_done));
    }
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_moe_permute(izb_ctx* ctx, izb_stream stream, const void* idx, int64_t pairs, int64_t E, void* offsets_out,
                        void* perm_out, void* inv_out) {
    if (!ctx || pairs < 0 || E <= 0) return IZB_ERR_BAD_ARG;
    if (E > 65535 || pairs > INT32_MAX) return IZB_ERR_UNSUPPORTED;
    if (!offsets_out || (pairs > 0 && (!idx || !perm_out || !inv_out))) return IZB_ERR_BAD_ARG;
    // 1024 threads: the in-order pass costs three block barriers per 1024 pairs
    IZB_CUDA_TRY(izb::launch_chained(ctx, moe_permute_kernel, dim3(static_cast<int>(E)), dim3(pairs >= 4096 ? 1024 : 256), 0,
                                     static_cast<cudaStream_t>(stream), static_cast<const int*>(idx), static_cast<int>(pairs),
                                     static_cast<int>(E), static_cast<int*>(offsets_out), static_cast<int*>(perm_out),
                                     static_cast<int*>(inv_out)));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_moe_gather(izb_ctx* ctx, izb_stream stream, const void* x, int64_t ldx, const void* perm, int32_t top_k,
                       int64_t rows, int64_t H, void* x_perm) {
    if (!ctx || rows < 0 || H <= 0 || top_k <= 0 || ldx < H) return IZB_ERR_BAD_ARG;
    if (rows == 0) return IZB_OK;
    if (!x || !perm || !x_perm) return IZB_ERR_BAD_ARG;
    if (H % 8 != 0 || ldx % 8 != 0 || !izb_aligned(x, 16) || !izb_aligned(x_perm, 16)) return IZB_ERR_UNSUPPORTED;
    const int threads = 256;
    IZB_CUDA_TRY(izb::launch_chained(ctx, moe_gather_kernel, dim3(blocks_for(ctx, rows * (H / 8), threads)), dim3(threads), 0,
                                     static_cast<cudaStream_t>(stream), static_cast<const uint4*>(x), static_cast<const int*>(perm),
                                     top_k, static_cast<int>(rows), static_cast<int>(H / 8), static_cast<long long>(ldx / 8),
                                     static_cast<uint4*>(x_perm)));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_moe_grouped_gemm(izb_ctx* ctx, izb_stream stream, const void* x_perm, const void* w, const void* offsets,
                             void* y, int32_t y_dtype, int64_t rows, int64_t N, int64_t K, int64_t E, int32_t epilogue) {
    if (!ctx || rows < 0 || N <= 0 || K <= 0 || E <= 0) return IZB_ERR_BAD_ARG;
    if (rows == 0) return IZB_OK;
    if (rows > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return IZB_ERR_UNSUPPORTED;
    if (!offsets) return IZB_ERR_BAD_ARG;
    const int64_t n_out = (epilogue == IZB_EPI_SWIGLU || epilogue == IZB_EPI_GLU) ? N / 2 : N;
    return gemm_tc_launch(ctx, static_cast<cudaStream_t>(stream), x_perm, K, w, nullptr, y, n_out, y_dtype,
                          static_cast<int>(rows), static_cast<int>(N), static_cast<int>(K), epilogue,
                          static_cast<const int*>(offsets), static_cast<int>(E));
}

int32_t izb_moe_combine(izb_ctx* ctx, izb_stream stream, const void* y_perm, const void* inv, const void* weights,
                        int64_t T, int32_t top_k, int64_t H, void* y) {
    if (!ctx || T < 0 || H <= 0 || top_k <= 0) return IZB_ERR_BAD_ARG;
    if (T == 0) return IZB_OK;
    if (!y_perm || !inv || !weights || !y) return IZB_ERR_BAD_ARG;
    if (H % 8 != 0 || !izb_aligned(y_perm, 16) || !izb_aligned(y, 16)) return IZB_ERR_UNSUPPORTED;
    const int threads = 256;
    IZB_CUDA_TRY(izb::launch_chained(ctx, moe_combine_kernel, dim3(blocks_for(ctx, T * (H / 8), threads)), dim3(threads), 0,
                                     static_cast<cudaStream_t>(stream), static_cast<const uint4*>(y_perm),
                                     static_cast<const int*>(inv), static_cast<const float*>(weights), static_cast<int>(T), top_k,
                                     static_cast<int>(H / 8), static_cast<uint4*>(y)));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// whole MoE feed-forward layer out of the pieces above
// ---------------------------------------------------------------------------
namespace {
struct MoeWorkspace {
    size_t logits, idx, wts, offsets, perm, inv, x_perm, hidden, y_perm, total;
};
size_t align_up(size_t v) { return (v + 255) / 256 * 256; }
MoeWorkspace moe_layout(int64_t T, int64_t H, int64_t I, int64_t E, int64_t k) {
    MoeWorkspace w;
    size_t at = 0;
    const size_t pairs = static_cast<size_t>(T) * static_cast<size_t>(k);
    w.logits = at; at = align_up(at + static_cast<size_t>(T) * E * 4);
    w.idx = at; at = align_up(at + pairs * 4);
    w.wts = at; at = align_up(at + pairs * 4);
    w.offsets = at; at = align_up(at + (static_cast<size_t>(E) + 1) * 4);
    w.perm = at; at = align_up(at + pairs * 4);
    w.inv = at; at = align_up(at + pairs * 4);
    w.x_perm = at; at = align_up(at + pairs * H * 2);
    w.hidden = at; at = align_up(at + pairs * I * 2);
    w.y_perm = at; at = align_up(at + pairs * H * 2);
    w.total = at;
    return w;
}
// The pair-streaming path reads an expert's weights once per pair routed to it: right for a few decode tokens
// (IZB_MOE_SMALL_MAX_PAIRS, default 32 = four tokens at top-8), wrong as soon as experts repeat.
bool moe_small_path(const izb_ctx* ctx, const izb_moe_args* a, int64_t pairs) {
    static const int max_pairs = [] {
        const char* e = std::getenv("IZB_MOE_SMALL_MAX_PAIRS");
        return e ? std::atoi(e) : 32;
    }();
    if (pairs > max_pairs) return false;
    if (a->H % 8 != 0 || a->I % 8 != 0 || a->top_k > 32) return false;
    if (!izb_aligned(a->x, 16) || !izb_aligned(a->w_gate_up, 16) || !izb_aligned(a->w_down, 16) || !izb_aligned(a->y, 2)) return false;
    return a->H * 2 <= 48 * 1024 && static_cast<int64_t>(a->top_k) * a->I * 2 <= 48 * 1024 && ctx != nullptr;
}
}  // namespace

extern "C" {

size_t izb_moe_workspace_bytes(int64_t T, int64_t H, int64_t I, int64_t E, int32_t top_k) {
    if (T <= 0 || H <= 0 || I <= 0 || E <= 0 || top_k <= 0) return 0;
    return moe_layout(T, H, I, E, top_k).total;
}

int32_t izb_moe_forward(izb_ctx* ctx, izb_stream stream, const izb_moe_args* a) {
    if (!ctx || !a) return IZB_ERR_BAD_ARG;
    if (a->T < 0 || a->H <= 0 || a->I <= 0 || a->E <= 0 || a->top_k <= 0) return IZB_ERR_BAD_ARG;
    if (a->T == 0) return IZB_OK;
    if (!a->x || !a->w_router || !a->w_gate_up || !a->w_down || !a->y || !a->workspace) return IZB_ERR_BAD_ARG;
    const MoeWorkspace L = moe_layout(a->T, a->H, a->I, a->E, a->top_k);
    if (a->workspace_bytes < L.total || !izb_aligned(a->workspace, 256)) return IZB_ERR_BAD_ARG;
    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    const int64_t pairs = a->T * a->top_k;

    int rc = izb_moe_route(ctx, stream, a->x, a->H, a->w_router, a->router_bias, a->T, a->H, a->E, a->top_k, ws + L.logits,
                           ws + L.idx, ws + L.wts);
    if (rc != IZB_OK) return rc;
    if (moe_small_path(ctx, a, pairs)) {
        // a handful of tokens: every pair streams its expert's rows (two launches behind the router)
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const int h_units = static_cast<int>(a->H / 8), i_units = static_cast<int>(a->I / 8);
        const int gx = static_cast<int>((a->I + 7) / 8), dx = static_cast<int>((a->H + 7) / 8);
        IZB_CUDA_TRY(izb::launch_chained(ctx, moe_small_gate_up_kernel, dim3(gx, static_cast<unsigned>(pairs)), dim3(256),
                                         static_cast<size_t>(a->H) * 2, s, static_cast<const uint4*>(a->x), static_cast<long long>(h_units),
                                         reinterpret_cast<const int*>(ws + L.idx), static_cast<const uint4*>(a->w_gate_up), h_units,
                                         static_cast<int>(a->I), a->top_k, reinterpret_cast<__nv_bfloat16*>(ws + L.hidden)));
        IZB_CUDA_TRY(izb::launch_chained(ctx, moe_small_down_kernel, dim3(dx, static_cast<unsigned>(a->T)), dim3(256),
                                         static_cast<size_t>(a->top_k) * a->I * 2, s, reinterpret_cast<const uint4*>(ws + L.hidden),
                                         reinterpret_cast<const int*>(ws + L.idx), reinterpret_cast<const float*>(ws + L.wts),
                                         static_cast<const uint4*>(a->w_down), static_cast<int>(a->H), i_units, a->top_k,
                                         static_cast<__nv_bfloat16*>(a->y)));
        ctx->launches.fetch_add(2, std::memory_order_relaxed);
        return IZB_OK;
    }
    rc = izb_moe_permute(ctx, stream, ws + L.idx, pairs, a->E, ws + L.offsets, ws + L.perm, ws + L.inv);
    if (rc != IZB_OK) return rc;
    rc = izb_moe_gather(ctx, stream, a->x, a->H, ws + L.perm, a->top_k, pairs, a->H, ws + L.x_perm);
    if (rc != IZB_OK) return rc;
    rc = izb_moe_grouped_gemm(ctx, stream, ws + L.x_perm, a->w_gate_up, ws + L.offsets, ws + L.hidden, IZB_BF16, pairs,
                              2 * a->I, a->H, a->E, IZB_EPI_SWIGLU);
    if (rc != IZB_OK) return rc;
    rc = izb_moe_grouped_gemm(ctx, stream, ws + L.hidden, a->w_down, ws + L.offsets, ws + L.y_perm, IZB_BF16, pairs,
                              a->H, a->I, a->E, IZB_EPI_NONE);
    if (rc != IZB_OK) return rc;
    return izb_moe_combine(ctx, stream, ws + L.y_perm, ws + L.inv, ws + L.wts, a->T, a->top_k, a->H, a->y);
}

}  // extern "C"
