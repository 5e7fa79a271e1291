// What a prompt needs beyond the projections before the first decode step can run: embedding rows,
// the q/k head norms + rotation + cache append for a run of tokens, and causal attention of those
// tokens over the cache they have just extended.  The decode step itself (one token per sequence)
// lives in attention.cu; the projections run on the GEMM whatever the token count.
#include <cstring>

#include "izb_common.cuh"

namespace {

// out[t, :] = table[ids[t], :], 16 bytes per thread; an id outside [0, vocab) gives a zero row and
// raises the status word (the host reports it as a bad argument after the fact).
__global__ void embed_rows_kernel(const uint4* __restrict__ table, const int* __restrict__ ids, long long tokens, int vec_per_row,
                                  long long vocab, uint4* __restrict__ out, long long ld_out_vec, int* status) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const long long total = tokens * vec_per_row;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = i / vec_per_row;
        const int c = static_cast<int>(i - t * vec_per_row);
        const long long id = ids[t];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (id >= 0 && id < vocab) v = table[id * vec_per_row + c];
        else if (c == 0) atomicExch(status, 8);
        out[t * ld_out_vec + c] = v;
    }
}

// One warp per head row of the fused QKV output of `q_len` consecutive tokens per sequence (token
// i of sequence b is row b * q_len + i of qkv and sits at cache position pos0 + i):
//   q rows: RMS-normalise with q_w (optional), rotate by the token's table row, write to q_out;
//   k rows: the same with k_w, written into the K cache; v rows: copied into the V cache.
// fp32 arithmetic, one rounding.
template <int D>
__global__ void __launch_bounds__(256)
    qk_norm_rope_append_seq_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_qkv, const __nv_bfloat16* __restrict__ q_w,
                                   const __nv_bfloat16* __restrict__ k_w, float eps, const __nv_bfloat16* __restrict__ cos_half,
                                   const __nv_bfloat16* __restrict__ sin_half, __nv_bfloat16* __restrict__ q_out,
                                   long long ld_q_out, __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                   long long batch, long long q_len, int heads, int kv_heads, long long pos0, long long cap) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    constexpr int E = D / 32;  // elements per lane; the rotation partner of element j is j +- D/2: lane ^ 16
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rows_per_tok = heads + 2 * kv_heads;
    const long long rows = batch * q_len * rows_per_tok;
    for (long long row = static_cast<long long>(blockIdx.x) * 8 + warp; row < rows; row += static_cast<long long>(gridDim.x) * 8) {
        const long long tok = row / rows_per_tok;  // b * q_len + i
        const int r = static_cast<int>(row - tok * rows_per_tok);
        const long long b = tok / q_len, i = tok - b * q_len, pos = pos0 + i;
        const __nv_bfloat16* src = qkv + tok * ld_qkv + static_cast<long long>(r) * D + lane * E;
        float x[E];
#pragma unroll
        for (int j = 0; j < E; ++j) x[j] = __bfloat162float(src[j]);
        __nv_bfloat16* dst;
        if (r >= heads + kv_heads) {
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
            const int jh = (lane & 15) * E;
#pragma unroll
            for (int j = 0; j < E; ++j) {
                const float other = __shfl_xor_sync(0xFFFFFFFFu, x[j], 16);
                const float c = __bfloat162float(cos_half[i * (D / 2) + jh + j]), s = __bfloat162float(sin_half[i * (D / 2) + jh + j]);
                x[j] = lane < 16 ? x[j] * c - other * s : other * s + x[j] * c;
            }
            dst = is_q ? q_out + tok * ld_q_out + static_cast<long long>(r) * D + lane * E
                       : kc + ((b * kv_heads + (r - heads)) * cap + pos) * D + lane * E;
        }
#pragma unroll
        for (int j = 0; j < E; ++j) dst[j] = __float2bfloat16_rn(x[j]);
    }
}

// Causal attention of a run of new tokens over a head-major cache: one warp per (sequence, token,
// query head).  Keys are taken 32 at a time, one per lane: the lane reads its key row (16-byte loads)
// against the query held in registers, the warp keeps a running maximum and sum, then every lane
// takes D / 32 consecutive output columns and adds p_j * V[j] for the 32 keys in turn (V rows read
// coalesced).  The cache is read once per query head; a prompt is attended once per request, so
// this is sized for correctness at any length rather than for the tensor cores.
template <int D>
__global__ void __launch_bounds__(128)
    prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
                             const __nv_bfloat16* __restrict__ vc, __nv_bfloat16* __restrict__ out, long long batch, long long q_len,
                             int heads, int kv_heads, long long pos0, long long cap, long long ld_q, long long ld_out, float scale) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    constexpr int E = D / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long items = batch * q_len * heads;
    const int group = heads / kv_heads;
    for (long long it = static_cast<long long>(blockIdx.x) * 4 + warp; it < items; it += static_cast<long long>(gridDim.x) * 4) {
        const long long tok = it / heads;
        const int h = static_cast<int>(it - tok * heads);
        const long long b = tok / q_len, i = tok - b * q_len;
        const long long n_keys = pos0 + i + 1;  // the token sees the cache up to and including itself
        const __nv_bfloat16* kbase = kc + (b * kv_heads + h / group) * cap * D;
        const __nv_bfloat16* vbase = vc + (b * kv_heads + h / group) * cap * D;
        // the whole query row in every lane, as packed bf16 pairs
        uint32_t qreg[D / 2];
        const uint4* qrow = reinterpret_cast<const uint4*>(q + tok * ld_q + static_cast<long long>(h) * D);
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            const uint4 v = qrow[j];
            qreg[4 * j] = v.x; qreg[4 * j + 1] = v.y; qreg[4 * j + 2] = v.z; qreg[4 * j + 3] = v.w;
        }
        float m = -INFINITY, l = 0.f, acc[E];
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = 0.f;
        for (long long k0 = 0; k0 < n_keys; k0 += 32) {
            const long long key = k0 + lane;
            float s = -INFINITY;
            if (key < n_keys) {
                const uint4* krow = reinterpret_cast<const uint4*>(kbase + key * D);
                float dot = 0.f;
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    const uint4 kv = krow[j];
                    const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        dot = fmaf(izb::bf16_lo_to_f32(qreg[4 * j + w]), izb::bf16_lo_to_f32(kw[w]), dot);
                        dot = fmaf(izb::bf16_hi_to_f32(qreg[4 * j + w]), izb::bf16_hi_to_f32(kw[w]), dot);
                    }
                }
                s = dot * scale;
            }
            float tile_max = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xFFFFFFFFu, tile_max, o));
            const float m_new = fmaxf(m, tile_max);  // finite: the tile holds at least one key
            const float corr = __expf(m - m_new);
            const float p = key < n_keys ? __expf(s - m_new) : 0.f;
            float psum = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xFFFFFFFFu, psum, o);
            l = l * corr + psum;
            m = m_new;
#pragma unroll
            for (int e = 0; e < E; ++e) acc[e] *= corr;
            const int in_tile = static_cast<int>(n_keys - k0 < 32 ? n_keys - k0 : 32);
            for (int j = 0; j < in_tile; ++j) {
                const float pj = __shfl_sync(0xFFFFFFFFu, p, j);
                const __nv_bfloat16* vrow = vbase + (k0 + j) * D + lane * E;
                if (E == 4) {
                    const uint2 vv = *reinterpret_cast<const uint2*>(vrow);
                    acc[0] = fmaf(pj, izb::bf16_lo_to_f32(vv.x), acc[0]);
                    acc[1] = fmaf(pj, izb::bf16_hi_to_f32(vv.x), acc[1]);
                    acc[2] = fmaf(pj, izb::bf16_lo_to_f32(vv.y), acc[2]);
                    acc[3] = fmaf(pj, izb::bf16_hi_to_f32(vv.y), acc[3]);
                } else {
                    const uint32_t vv = *reinterpret_cast<const uint32_t*>(vrow);
                    acc[0] = fmaf(pj, izb::bf16_lo_to_f32(vv), acc[0]);
                    acc[1] = fmaf(pj, izb::bf16_hi_to_f32(vv), acc[1]);
                }
            }
        }
        __nv_bfloat16* dst = out + tok * ld_out + static_cast<long long>(h) * D + lane * E;
#pragma unroll
        for (int e = 0; e < E; ++e) dst[e] = __float2bfloat16_rn(acc[e] / l);
    }
}

int grid_cap(const izb_ctx* ctx, long long blocks, int per_sm) {
    const long long cap = static_cast<long long>(ctx->sm_count) * per_sm;
    return static_cast<int>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace

extern "C" {

int32_t izb_embed_rows(izb_ctx* ctx, izb_stream stream, const void* table, int64_t vocab, int64_t hidden, const int32_t* ids,
                       int64_t tokens, void* out, int64_t ld_out) {
    if (!ctx || vocab <= 0 || hidden <= 0 || tokens < 0 || ld_out < hidden) return IZB_ERR_BAD_ARG;
    if (tokens == 0) return IZB_OK;
    if (!table || !ids || !out) return IZB_ERR_BAD_ARG;
    if (hidden % 8 != 0 || ld_out % 8 != 0 || !izb_aligned(table, 16) || !izb_aligned(out, 16) || !izb_aligned(ids, 4))
        return IZB_ERR_BAD_ARG;
    const long long items = tokens * (hidden / 8);
    IZB_CUDA_TRY(izb::launch_chained(ctx, embed_rows_kernel, dim3(grid_cap(ctx, (items + 255) / 256, 16)), dim3(256), 0,
                                     static_cast<cudaStream_t>(stream), static_cast<const uint4*>(table), ids,
                                     static_cast<long long>(tokens), static_cast<int>(hidden / 8), static_cast<long long>(vocab),
                                     static_cast<uint4*>(out), static_cast<long long>(ld_out / 8), ctx->d_status + 6));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_qk_norm_rope_append_seq(izb_ctx* ctx, izb_stream stream, const void* qkv, int64_t ld_qkv, const void* q_norm_weight,
                                    const void* k_norm_weight, float eps, const void* cos_half, const void* sin_half, void* q_out,
                                    int64_t ld_q_out, void* k_cache, void* v_cache, int64_t batch, int64_t q_len, int32_t heads,
                                    int32_t kv_heads, int32_t head_dim, int64_t pos0, int64_t kv_capacity) {
    if (!ctx || batch < 0 || q_len < 0 || heads <= 0 || kv_heads <= 0) return IZB_ERR_BAD_ARG;
    if (batch == 0 || q_len == 0) return IZB_OK;
    if (!qkv || !cos_half || !sin_half || !q_out || !k_cache || !v_cache) return IZB_ERR_BAD_ARG;
    if (head_dim != 64 && head_dim != 128) return IZB_ERR_UNSUPPORTED;
    if ((q_norm_weight == nullptr) != (k_norm_weight == nullptr) || !(eps >= 0.f)) return IZB_ERR_BAD_ARG;
    if (pos0 < 0 || pos0 + q_len > kv_capacity) return IZB_ERR_BAD_ARG;
    if (ld_qkv < static_cast<int64_t>(heads + 2 * kv_heads) * head_dim || ld_q_out < static_cast<int64_t>(heads) * head_dim)
        return IZB_ERR_BAD_ARG;
    if (!izb_aligned(qkv, 2) || !izb_aligned(q_out, 2) || !izb_aligned(k_cache, 2) || !izb_aligned(v_cache, 2)) return IZB_ERR_BAD_ARG;
    const long long rows = batch * q_len * (heads + 2 * kv_heads);
    const int grid = grid_cap(ctx, (rows + 7) / 8, 8);
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
        IZB_CUDA_TRY(izb::launch_chained(ctx, qk_norm_rope_append_seq_kernel<128>, dim3(grid), dim3(256), 0, s, in, ld_qkv, qw, kw, eps,
                                         cs, sn, qo, ld_q_out, kc, vc, batch, q_len, heads, kv_heads, pos0, kv_capacity));
    else
        IZB_CUDA_TRY(izb::launch_chained(ctx, qk_norm_rope_append_seq_kernel<64>, dim3(grid), dim3(256), 0, s, in, ld_qkv, qw, kw, eps,
                                         cs, sn, qo, ld_q_out, kc, vc, batch, q_len, heads, kv_heads, pos0, kv_capacity));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_prefill_gqa_attention(izb_ctx* ctx, izb_stream stream, const void* q, const void* k_cache, const void* v_cache,
                                  void* out, int64_t batch, int64_t q_len, int32_t heads, int32_t kv_heads, int32_t head_dim,
                                  int64_t pos0, int64_t kv_capacity, int64_t ld_q, int64_t ld_out, float scale) {
    if (!ctx || batch < 0 || q_len < 0 || heads <= 0 || kv_heads <= 0) return IZB_ERR_BAD_ARG;
    if (batch == 0 || q_len == 0) return IZB_OK;
    if (!q || !k_cache || !v_cache || !out) return IZB_ERR_BAD_ARG;
    if (head_dim != 64 && head_dim != 128) return IZB_ERR_UNSUPPORTED;
    if (heads % kv_heads != 0) return IZB_ERR_UNSUPPORTED;
    if (pos0 < 0 || pos0 + q_len > kv_capacity) return IZB_ERR_BAD_ARG;
    if (ld_q < static_cast<int64_t>(heads) * head_dim || ld_out < static_cast<int64_t>(heads) * head_dim) return IZB_ERR_BAD_ARG;
    // q and the K rows are read with 16-byte loads, V with 8- or 4-byte loads
    if (!izb_aligned(q, 16) || ld_q % 8 != 0 || !izb_aligned(k_cache, 16) || !izb_aligned(v_cache, 16) || !izb_aligned(out, 2))
        return IZB_ERR_BAD_ARG;
    const long long items = batch * q_len * heads;
    const int grid = grid_cap(ctx, (items + 3) / 4, 16);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const auto* qp = static_cast<const __nv_bfloat16*>(q);
    const auto* kp = static_cast<const __nv_bfloat16*>(k_cache);
    const auto* vp = static_cast<const __nv_bfloat16*>(v_cache);
    auto* op = static_cast<__nv_bfloat16*>(out);
    if (head_dim == 128)
        IZB_CUDA_TRY(izb::launch_chained(ctx, prefill_attention_kernel<128>, dim3(grid), dim3(128), 0, s, qp, kp, vp, op, batch, q_len,
                                         heads, kv_heads, pos0, kv_capacity, ld_q, ld_out, scale));
    else
        IZB_CUDA_TRY(izb::launch_chained(ctx, prefill_attention_kernel<64>, dim3(grid), dim3(128), 0, s, qp, kp, vp, op, batch, q_len,
                                         heads, kv_heads, pos0, kv_capacity, ld_q, ld_out, scale));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // extern "C"
