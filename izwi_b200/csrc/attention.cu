// The step between the QKV and O projections of a decode token: rotary embedding of q and k, and
// single-query grouped-query attention over a head-major KV cache (flash-decoding: the cache is
// split over CTAs, each keeps a running max / sum / weighted value sum, a second kernel merges).
// HBM-bound on the K and V bytes, which every CTA reads exactly once, coalesced.
#include "izb_common.cuh"

namespace {

constexpr int ATT_THREADS = 128;  // 4 warps; also the number of cache positions per tile
constexpr int ATT_MAX_G = 8;      // query heads per KV head

// out_first = x1 cos - x2 sin, out_second = x1 sin + x2 cos over the two halves of every head
// (the non-interleaved form), fp32 arithmetic, one rounding.  In place.
__global__ void rope_pair_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                 const __nv_bfloat16* __restrict__ cos_half, const __nv_bfloat16* __restrict__ sin_half,
                                 long long tokens, int q_heads, int k_heads, int head_dim, long long ld_q, long long ld_k) {
    const int half = head_dim >> 1;
    const long long per_tok = static_cast<long long>(q_heads + k_heads) * half;
    const long long total = tokens * per_tok;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = i / per_tok;
        const int r = static_cast<int>(i - t * per_tok);
        const int head = r / half, j = r - head * half;
        __nv_bfloat16* base = head < q_heads ? q + t * ld_q + static_cast<long long>(head) * head_dim
                                             : k + t * ld_k + static_cast<long long>(head - q_heads) * head_dim;
        const float c = __bfloat162float(cos_half[t * half + j]), s = __bfloat162float(sin_half[t * half + j]);
        const float x1 = __bfloat162float(base[j]), x2 = __bfloat162float(base[j + half]);
        base[j] = __float2bfloat16_rn(x1 * c - x2 * s);
        base[j + half] = __float2bfloat16_rn(x1 * s + x2 * c);
    }
}

// k, v [batch, kv_heads, head_dim] of the new token -> position `pos` of the head-major caches.
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                 __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, long long batch, int kv_heads,
                                 int head_dim, long long pos, long long cap, long long ld_k, long long ld_v) {
    const long long per = static_cast<long long>(kv_heads) * head_dim, total = batch * per;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long b = i / per;
        const int r = static_cast<int>(i - b * per);
        const int kh = r / head_dim, d = r - kh * head_dim;
        const long long dst = ((b * kv_heads + kh) * cap + pos) * head_dim + d;
        kc[dst] = k[b * ld_k + r];
        vc[dst] = v[b * ld_v + r];
    }
}

// One warp per head row of the fused QKV output of one decode token per sequence:
//   q rows: RMS-normalise with q_w (optional), rotate, write to q_out;
//   k rows: the same with k_w, written into position `pos` of the head-major K cache;
//   v rows: copied into the V cache.
// fp32 arithmetic, one rounding (the unfused sequence rounds after the norm and again after the rotation).
template <int D>
__global__ void __launch_bounds__(256)
    qk_norm_rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_qkv, const __nv_bfloat16* __restrict__ q_w,
                               const __nv_bfloat16* __restrict__ k_w, float eps, const __nv_bfloat16* __restrict__ cos_half,
                               const __nv_bfloat16* __restrict__ sin_half, __nv_bfloat16* __restrict__ q_out, long long ld_q_out,
                               __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, long long batch, int heads,
                               int kv_heads, long long pos, long long cap) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    constexpr int E = D / 32;  // elements per lane; the rotation partner of element j is j +- D/2: lane ^ 16
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rows_per_tok = heads + 2 * kv_heads;
    const long long rows = batch * rows_per_tok;
    for (long long row = static_cast<long long>(blockIdx.x) * 8 + warp; row < rows; row += static_cast<long long>(gridDim.x) * 8) {
        const long long b = row / rows_per_tok;
        const int r = static_cast<int>(row - b * rows_per_tok);
        const __nv_bfloat16* src = qkv + b * ld_qkv + static_cast<long long>(r) * D + lane * E;
        float x[E];
#pragma unroll
        for (int j = 0; j < E; ++j) x[j] = __bfloat162float(src[j]);
        __nv_bfloat16* dst;
        if (r >= heads + kv_heads) {  // v: straight into the cache
            dst = vc + ((b * kv_heads + (r - heads - kv_heads)) * cap + pos) * D + lane * E;
        } else {
            const bool is_q = r < heads;
            const __nv_bfloat16* w = is_q ? q_w : k_w;
            if (w) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < E; ++j) ss += x[j] * x[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                const float scale = rsqrtf(ss / static_cast<float>(D) + eps);
#pragma unroll
                for (int j = 0; j < E; ++j) x[j] = x[j] * scale * __bfloat162float(w[lane * E + j]);
            }
            // lanes 0..15 hold the first half (x1), lanes 16..31 the second (x2) of the same pair index
            const int jh = (lane & 15) * E;
#pragma unroll
            for (int j = 0; j < E; ++j) {
                const float other = __shfl_xor_sync(0xFFFFFFFFu, x[j], 16);
                const float c = __bfloat162float(cos_half[b * (D / 2) + jh + j]), s = __bfloat162float(sin_half[b * (D / 2) + jh + j]);
                x[j] = lane < 16 ? x[j] * c - other * s : other * s + x[j] * c;
            }
            dst = is_q ? q_out + b * ld_q_out + static_cast<long long>(r) * D + lane * E
                       : kc + ((b * kv_heads + (r - heads)) * cap + pos) * D + lane * E;
        }
#pragma unroll
        for (int j = 0; j < E; ++j) dst[j] = __float2bfloat16_rn(x[j]);
    }
}

struct AttShared {
    float m[ATT_MAX_G], l[ATT_MAX_G], alpha[ATT_MAX_G];
};

// grid (splits, kv_heads, batch).  G query heads share the K / V rows of their KV head.
template <int D, int G>
__global__ void __launch_bounds__(ATT_THREADS)
    decode_gqa_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                      const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out, float* __restrict__ part,
                      int heads, int kv_heads, int g_real, long long ld_q_tok, long long ld_out_tok, long long kv_cap,
                      int kv_len, float scale) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    constexpr int DV = D / 32;  // output values per lane
    extern __shared__ float dyn[];
    float* S = dyn;                        // [G][ATT_THREADS]: scores, then probabilities of the tile
    float* red = S + G * ATT_THREADS;      // [4][G][D] cross-warp sums
    __shared__ AttShared sh;

    const int split = blockIdx.x, n_splits = gridDim.x, kh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = ((kv_len + n_splits - 1) / n_splits + ATT_THREADS - 1) / ATT_THREADS * ATT_THREADS;
    const int t_begin = split * per, t_end = min(kv_len, t_begin + per);

    // Scores on mma.sync (16 cache positions x 8 head columns x 16 d per instruction, K rows as the A
    // operand, q as B).  Any permutation of d is free as long as both operands use it: lane (gq, tq)
    // takes d = 32 tq .. 32 tq + 31 (16 tq .. for d = 64) of its rows, i.e. 16-byte loads, and step s
    // consumes words 2s, 2s + 1 of them.  The q fragments stay in registers for the whole CTA.
    constexpr int STEPS = D / 16;  // MMA steps per row; words of one lane's share of a row = 2 STEPS
    const int gq = lane >> 2, tq = lane & 3;
    uint32_t qf[STEPS][2];
    {
        uint4 tmp[STEPS / 2];
#pragma unroll
        for (int j = 0; j < STEPS / 2; ++j) tmp[j] = make_uint4(0u, 0u, 0u, 0u);
        if (gq < g_real) {
            const uint4* qr = reinterpret_cast<const uint4*>(q + b * ld_q_tok + static_cast<long long>(kh * g_real + gq) * D +
                                                             tq * (D / 4));
#pragma unroll
            for (int j = 0; j < STEPS / 2; ++j) tmp[j] = qr[j];
        }
#pragma unroll
        for (int j = 0; j < STEPS / 2; ++j) {
            qf[2 * j][0] = tmp[j].x; qf[2 * j][1] = tmp[j].y;
            qf[2 * j + 1][0] = tmp[j].z; qf[2 * j + 1][1] = tmp[j].w;
        }
    }
    if (tid < G) {
        sh.m[tid] = -INFINITY;
        sh.l[tid] = 0.f;
    }
    float acc[G][DV];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < DV; ++j) acc[g][j] = 0.f;
    __syncthreads();

    const __nv_bfloat16* kbase = kc + (static_cast<long long>(b) * kv_heads + kh) * kv_cap * D;
    const __nv_bfloat16* vbase = vc + (static_cast<long long>(b) * kv_heads + kh) * kv_cap * D;

    for (int t0 = t_begin; t0 < t_end; t0 += ATT_THREADS) {
        const int n = min(ATT_THREADS, t_end - t0);
        // ---- scores: warp w takes positions 32 w .. 32 w + 31 of the tile, sixteen per MMA group ----
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
            const int r0 = warp * 32 + grp * 16 + gq, r1 = r0 + 8;  // this lane's two rows inside the tile
            uint4 ka[STEPS / 2], kb[STEPS / 2];
#pragma unroll
            for (int j = 0; j < STEPS / 2; ++j) ka[j] = kb[j] = make_uint4(0u, 0u, 0u, 0u);
            if (r0 < n) {
                const uint4* kr = reinterpret_cast<const uint4*>(kbase + static_cast<long long>(t0 + r0) * D + tq * (D / 4));
#pragma unroll
                for (int j = 0; j < STEPS / 2; ++j) ka[j] = kr[j];
            }
            if (r1 < n) {
                const uint4* kr = reinterpret_cast<const uint4*>(kbase + static_cast<long long>(t0 + r1) * D + tq * (D / 4));
#pragma unroll
                for (int j = 0; j < STEPS / 2; ++j) kb[j] = kr[j];
            }
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < STEPS / 2; ++j) {
                izb::mma_bf16_16816(c, ka[j].x, kb[j].x, ka[j].y, kb[j].y, qf[2 * j][0], qf[2 * j][1]);
                izb::mma_bf16_16816(c, ka[j].z, kb[j].z, ka[j].w, kb[j].w, qf[2 * j + 1][0], qf[2 * j + 1][1]);
            }
            // c0, c1: position r0 x heads 2 tq, 2 tq + 1;  c2, c3: position r1
            if (2 * tq < G) {
                S[(2 * tq) * ATT_THREADS + r0] = r0 < n ? c[0] * scale : -INFINITY;
                S[(2 * tq) * ATT_THREADS + r1] = r1 < n ? c[2] * scale : -INFINITY;
            }
            if (2 * tq + 1 < G) {
                S[(2 * tq + 1) * ATT_THREADS + r0] = r0 < n ? c[1] * scale : -INFINITY;
                S[(2 * tq + 1) * ATT_THREADS + r1] = r1 < n ? c[3] * scale : -INFINITY;
            }
        }
        __syncthreads();
        // ---- running max and sum per query head: warp w takes heads w, w + 4 ----
        for (int g = warp; g < G; g += 4) {
            float v[4], mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] = S[g * ATT_THREADS + lane + 32 * j];
                mx = fmaxf(mx, v[j]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
            const float m_old = sh.m[g], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p = __expf(v[j] - m_new);  // -inf (past the end) -> 0
                S[g * ATT_THREADS + lane + 32 * j] = p;
                sum += p;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
            if (lane == 0) {
                const float a = __expf(m_old - m_new);  // first tile: exp(-inf) = 0
                sh.alpha[g] = a;
                sh.m[g] = m_new;
                sh.l[g] = sh.l[g] * a + sum;
            }
        }
        __syncthreads();
        // ---- weighted values: warp w takes positions w, w + 4, ...; lane owns DV output values ----
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float a = sh.alpha[g];
#pragma unroll
            for (int j = 0; j < DV; ++j) acc[g][j] *= a;
        }
        for (int i = warp; i < n; i += 4) {
            const __nv_bfloat16* vr = vbase + static_cast<long long>(t0 + i) * D + lane * DV;
            float vv[DV];
            if constexpr (DV == 4) {
                const uint2 w = *reinterpret_cast<const uint2*>(vr);
                vv[0] = izb::bf16_lo_to_f32(w.x); vv[1] = izb::bf16_hi_to_f32(w.x);
                vv[2] = izb::bf16_lo_to_f32(w.y); vv[3] = izb::bf16_hi_to_f32(w.y);
            } else {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(vr);
                vv[0] = izb::bf16_lo_to_f32(w); vv[1] = izb::bf16_hi_to_f32(w);
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float p = S[g * ATT_THREADS + i];
#pragma unroll
                for (int j = 0; j < DV; ++j) acc[g][j] = fmaf(p, vv[j], acc[g][j]);
            }
        }
        __syncthreads();  // S is rewritten by the next tile
    }

    // ---- sum the four warps' partial outputs ----
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < DV; ++j) red[(warp * G + g) * D + lane * DV + j] = acc[g][j];
    __syncthreads();
    for (int i = tid; i < g_real * D; i += ATT_THREADS) {
        const int g = i / D, d = i - g * D;
        const float v = red[(0 * G + g) * D + d] + red[(1 * G + g) * D + d] + red[(2 * G + g) * D + d] + red[(3 * G + g) * D + d];
        const int head = kh * g_real + g;
        if (n_splits == 1) {
            out[b * ld_out_tok + static_cast<long long>(head) * D + d] = __float2bfloat16_rn(v / sh.l[g]);
        } else {
            // partials: [batch][head][split][D + 2] = unnormalised sum, then max and sum of weights
            float* p = part + ((static_cast<long long>(b) * heads + head) * n_splits + split) * (D + 2);
            p[d] = v;
            if (d == 0) {
                p[D] = sh.m[g];
                p[D + 1] = sh.l[g];
            }
        }
    }
}

// grid (heads, batch): merges the splits' (max, sum, weighted values).
template <int D>
__global__ void __launch_bounds__(D)
    decode_gqa_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int heads, int n_splits,
                            long long ld_out_tok) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const float* p = part + (static_cast<long long>(b) * heads + head) * n_splits * (D + 2);
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, p[s * (D + 2) + D]);
    float num = 0.f, den = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float w = __expf(p[s * (D + 2) + D] - m);  // a split past the end carries max = -inf, weight 0
        num = fmaf(w, p[s * (D + 2) + d], num);
        den = fmaf(w, p[s * (D + 2) + D + 1], den);
    }
    out[b * ld_out_tok + static_cast<long long>(head) * D + d] = __float2bfloat16_rn(num / den);
}

int att_splits(const izb_ctx* ctx, int64_t batch, int64_t kv_heads, int64_t kv_len) {
    const int64_t tiles = (kv_len + ATT_THREADS - 1) / ATT_THREADS;
    // about six CTAs of four warps per SM: the loads of a cache position are a dependent chain
    int64_t want = (6 * static_cast<int64_t>(ctx ? ctx->sm_count : 148) + batch * kv_heads - 1) / (batch * kv_heads);
    if (want < 1) want = 1;
    if (want > tiles) want = tiles;
    if (want > 64) want = 64;
    return static_cast<int>(want);
}

template <int D, int G>
int launch_att(izb_ctx* ctx, cudaStream_t s, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
               __nv_bfloat16* out, float* part, int batch, int heads, int kv_heads, int g_real, long long ld_q,
               long long ld_out, long long kv_cap, int kv_len, float scale, int splits) {
    const size_t smem = static_cast<size_t>(G * ATT_THREADS + 4 * G * D) * sizeof(float);
    auto kern = decode_gqa_kernel<D, G>;
    static std::atomic<int> smem_set[IZB_MAX_DEVICES];
    const int slot = ctx->device;
    if (smem > 48 * 1024 && smem_set[slot].load(std::memory_order_relaxed) < static_cast<int>(smem)) {
        IZB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        smem_set[slot].store(static_cast<int>(smem), std::memory_order_relaxed);
    }
    IZB_CUDA_TRY(izb::launch_chained(ctx, kern, dim3(splits, kv_heads, batch), dim3(ATT_THREADS), smem, s, q, k, v, out, part, heads,
                                     kv_heads, g_real, ld_q, ld_out, kv_cap, kv_len, scale));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    if (splits > 1) {
        IZB_CUDA_TRY(izb::launch_chained(ctx, decode_gqa_merge_kernel<D>, dim3(heads, batch), dim3(D), 0, s,
                                         static_cast<const float*>(part), out, heads, splits, ld_out));
        ctx->launches.fetch_add(1, std::memory_order_relaxed);
    }
    return IZB_OK;
}

template <int D>
int launch_att_g(izb_ctx* ctx, cudaStream_t s, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                 __nv_bfloat16* out, float* part, int batch, int heads, int kv_heads, int g, long long ld_q, long long ld_out,
                 long long kv_cap, int kv_len, float scale, int splits) {
    if (g == 1) return launch_att<D, 1>(ctx, s, q, k, v, out, part, batch, heads, kv_heads, g, ld_q, ld_out, kv_cap, kv_len, scale, splits);
    if (g == 2) return launch_att<D, 2>(ctx, s, q, k, v, out, part, batch, heads, kv_heads, g, ld_q, ld_out, kv_cap, kv_len, scale, splits);
    if (g <= 4) return launch_att<D, 4>(ctx, s, q, k, v, out, part, batch, heads, kv_heads, g, ld_q, ld_out, kv_cap, kv_len, scale, splits);
    return launch_att<D, 8>(ctx, s, q, k, v, out, part, batch, heads, kv_heads, g, ld_q, ld_out, kv_cap, kv_len, scale, splits);
}

}  // namespace

extern "C" {

int32_t izb_rope_pair(izb_ctx* ctx, izb_stream stream, void* q, void* k, const void* cos_half, const void* sin_half,
                      int64_t tokens, int32_t q_heads, int32_t k_heads, int32_t head_dim, int64_t ld_q, int64_t ld_k) {
    if (!ctx || tokens < 0 || q_heads < 0 || k_heads < 0 || head_dim <= 0 || (head_dim & 1)) return IZB_ERR_BAD_ARG;
    if (tokens == 0 || q_heads + k_heads == 0) return IZB_OK;
    if (!cos_half || !sin_half || (q_heads && !q) || (k_heads && !k)) return IZB_ERR_BAD_ARG;
    if (ld_q < static_cast<int64_t>(q_heads) * head_dim || ld_k < static_cast<int64_t>(k_heads) * head_dim) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(q, 2) || !izb_aligned(k, 2) || !izb_aligned(cos_half, 2) || !izb_aligned(sin_half, 2)) return IZB_ERR_BAD_ARG;
    const long long total = tokens * static_cast<long long>(q_heads + k_heads) * (head_dim / 2);
    const long long cap = static_cast<long long>(ctx->sm_count) * 16;
    const long long blocks = (total + 255) / 256;
    rope_pair_kernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(cos_half),
        static_cast<const __nv_bfloat16*>(sin_half), tokens, q_heads, k_heads, head_dim, ld_q, ld_k);
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_kv_append(izb_ctx* ctx, izb_stream stream, const void* k, const void* v, void* k_cache, void* v_cache,
                      int64_t batch, int32_t kv_heads, int32_t head_dim, int64_t pos, int64_t kv_capacity, int64_t ld_k,
                      int64_t ld_v) {
    if (!ctx || batch < 0 || kv_heads <= 0 || head_dim <= 0) return IZB_ERR_BAD_ARG;
    if (batch == 0) return IZB_OK;
    if (!k || !v || !k_cache || !v_cache || pos < 0 || pos >= kv_capacity) return IZB_ERR_BAD_ARG;
    const int64_t per = static_cast<int64_t>(kv_heads) * head_dim;
    if (ld_k < per || ld_v < per) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(k, 2) || !izb_aligned(v, 2) || !izb_aligned(k_cache, 2) || !izb_aligned(v_cache, 2)) return IZB_ERR_BAD_ARG;
    const long long total = batch * per, cap = static_cast<long long>(ctx->sm_count) * 8, blocks = (total + 255) / 256;
    kv_append_kernel<<<static_cast<int>(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), static_cast<__nv_bfloat16*>(k_cache),
        static_cast<__nv_bfloat16*>(v_cache), batch, kv_heads, head_dim, pos, kv_capacity, ld_k, ld_v);
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_qk_norm_rope_append(izb_ctx* ctx, izb_stream stream, const void* qkv, int64_t ld_qkv, const void* q_norm_weight,
                                const void* k_norm_weight, float eps, const void* cos_half, const void* sin_half, void* q_out,
                                int64_t ld_q_out, void* k_cache, void* v_cache, int64_t batch, int32_t heads, int32_t kv_heads,
                                int32_t head_dim, int64_t pos, int64_t kv_capacity) {
    if (!ctx || batch < 0 || heads <= 0 || kv_heads <= 0) return IZB_ERR_BAD_ARG;
    if (batch == 0) return IZB_OK;
    if (head_dim != 64 && head_dim != 128) return IZB_ERR_UNSUPPORTED;
    if (!qkv || !cos_half || !sin_half || !q_out || !k_cache || !v_cache) return IZB_ERR_BAD_ARG;
    if ((q_norm_weight == nullptr) != (k_norm_weight == nullptr) || !(eps >= 0.f)) return IZB_ERR_BAD_ARG;
    if (pos < 0 || pos >= kv_capacity) return IZB_ERR_BAD_ARG;
    if (ld_qkv < static_cast<int64_t>(heads + 2 * kv_heads) * head_dim || ld_q_out < static_cast<int64_t>(heads) * head_dim)
        return IZB_ERR_BAD_ARG;
    if (!izb_aligned(qkv, 2) || !izb_aligned(q_out, 2) || !izb_aligned(k_cache, 2) || !izb_aligned(v_cache, 2)) return IZB_ERR_BAD_ARG;
    const long long rows = batch * (heads + 2 * kv_heads), blocks = (rows + 7) / 8, cap = static_cast<long long>(ctx->sm_count) * 8;
    const int grid = static_cast<int>(blocks < cap ? blocks : cap);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto* in = static_cast<const __nv_bfloat16*>(qkv);
    const auto* qw = static_cast<const __nv_bfloat16*>(q_norm_weight);
    const auto* kw = static_cast<const __nv_bfloat16*>(k_norm_weight);
    const auto* cs = static_cast<const __nv_bfloat16*>(cos_half);
    const auto* sn = static_cast<const __nv_bfloat16*>(sin_half);
    auto* qo = static_cast<__nv_bfloat16*>(q_out);
    auto* kc = static_cast<__nv_bfloat16*>(k_cache);
    auto* vc = static_cast<__nv_bfloat16*>(v_cache);
    if (head_dim == 128)
        IZB_CUDA_TRY(izb::launch_chained(ctx, qk_norm_rope_append_kernel<128>, dim3(grid), dim3(256), 0, s, in, ld_qkv, qw, kw, eps, cs,
                                         sn, qo, ld_q_out, kc, vc, batch, heads, kv_heads, pos, kv_capacity));
    else
        IZB_CUDA_TRY(izb::launch_chained(ctx, qk_norm_rope_append_kernel<64>, dim3(grid), dim3(256), 0, s, in, ld_qkv, qw, kw, eps, cs,
                                         sn, qo, ld_q_out, kc, vc, batch, heads, kv_heads, pos, kv_capacity));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

size_t izb_decode_gqa_attention_workspace_bytes(const izb_ctx* ctx, int64_t batch, int32_t heads, int32_t kv_heads,
                                                int32_t head_dim, int64_t kv_len) {
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || kv_len <= 0) return 0;
    const int splits = att_splits(ctx, batch, kv_heads, kv_len);
    if (splits <= 1) return 0;
    return static_cast<size_t>(batch) * heads * splits * (head_dim + 2) * sizeof(float);
}

int32_t izb_decode_gqa_attention(izb_ctx* ctx, izb_stream stream, const void* q, const void* k_cache, const void* v_cache,
                                 void* out, int64_t batch, int32_t heads, int32_t kv_heads, int32_t head_dim, int64_t kv_len,
                                 int64_t kv_capacity, int64_t ld_q, int64_t ld_out, float scale, void* workspace,
                                 size_t workspace_bytes) {
    if (!ctx || batch < 0 || heads <= 0 || kv_heads <= 0) return IZB_ERR_BAD_ARG;
    if (batch == 0) return IZB_OK;
    if (!q || !k_cache || !v_cache || !out) return IZB_ERR_BAD_ARG;
    if (head_dim != 64 && head_dim != 128) return IZB_ERR_UNSUPPORTED;
    if (heads % kv_heads != 0 || heads / kv_heads > ATT_MAX_G) return IZB_ERR_UNSUPPORTED;
    if (kv_len <= 0 || kv_len > kv_capacity || kv_len > INT32_MAX || batch > 65535 || kv_heads > 65535) return IZB_ERR_BAD_ARG;
    if (ld_q < static_cast<int64_t>(heads) * head_dim || ld_out < static_cast<int64_t>(heads) * head_dim) return IZB_ERR_BAD_ARG;
    // q and the caches are read with 16-byte loads: the base and every token row must sit on that boundary
    if (!izb_aligned(q, 16) || ld_q % 8 != 0 || !izb_aligned(out, 2) || !izb_aligned(k_cache, 16) || !izb_aligned(v_cache, 16))
        return IZB_ERR_BAD_ARG;
    const int splits = att_splits(ctx, batch, kv_heads, kv_len);
    const size_t need = splits > 1 ? static_cast<size_t>(batch) * heads * splits * (head_dim + 2) * sizeof(float) : 0;
    if (need && (!workspace || workspace_bytes < need || !izb_aligned(workspace, 4))) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto* qp = static_cast<const __nv_bfloat16*>(q);
    const auto* kp = static_cast<const __nv_bfloat16*>(k_cache);
    const auto* vp = static_cast<const __nv_bfloat16*>(v_cache);
    auto* op = static_cast<__nv_bfloat16*>(out);
    float* part = static_cast<float*>(workspace);
    const int g = heads / kv_heads;
    if (head_dim == 128)
        return launch_att_g<128>(ctx, s, qp, kp, vp, op, part, static_cast<int>(batch), heads, kv_heads, g, ld_q, ld_out,
                                 kv_capacity, static_cast<int>(kv_len), scale, splits);
    return launch_att_g<64>(ctx, s, qp, kp, vp, op, part, static_cast<int>(batch), heads, kv_heads, g, ld_q, ld_out, kv_capacity,
                            static_cast<int>(kv_len), scale, splits);
}

}  // extern "C"
