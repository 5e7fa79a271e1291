// Paged KV cache for decode attention: fixed-size pages of [page_size tokens, kv_heads, head_dim] per
// sequence, dense (bf16) or quantised the way the reference's KvPage is
// (crates/izwi-core/src/models/shared/attention/paged.rs):
//   Int8  (:158-199)  u8 = round(clamp(x / scale, -127, 127)) + 128 with ONE scale per page,
//                     scale = max(max|x| / 127, 1e-8) (1 for an all-zero page); the reference does this
//                     arithmetic in the cache's dtype, so every product here is rounded to bf16 as well;
//   Q4_0  (:200-343)  blocks of 32 consecutive values, scale = max|x| / 7 (1 if all zero),
//                     q = clamp(round(x / scale), -7, 7) + 8, two codes per byte, low nibble first.
// Appending to a partly filled page re-quantises the whole page from its dequantised (bf16) contents
// plus the new rows, exactly as `append_to_pages` (:345-388) rebuilds its last page.
// Attention (`paged_decode_attention`, :486-628) walks the pages of a sequence with a running maximum
// and sum; here pages are dequantised in registers on the way, never materialised.
// Sequence lengths live on the device, so a decode step that grows the cache can be replayed from a
// CUDA graph.
#include "izb_common.cuh"

namespace {

constexpr int PA_THREADS = 128;
constexpr int PA_MAX_G = 8;

__device__ __forceinline__ float bf16_rn(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct Pages {
    void* k_values;
    void* v_values;
    float* k_scales;
    float* v_scales;
    const int* page_table;  // [batch, max_pages]
    int quant, page_size, kv_heads, head_dim;
    long long max_pages;
};

__device__ __forceinline__ long long page_elems(const Pages& p) { return static_cast<long long>(p.page_size) * p.kv_heads * p.head_dim; }

// value `e` (flat index inside the page) of a stored page, as the bf16 value the reference's
// `to_dense` yields
__device__ __forceinline__ float load_dense(const Pages& p, const void* values, const float* scales, long long page, long long e) {
    const long long pe = page_elems(p);
    if (p.quant == 0) return __bfloat162float(static_cast<const __nv_bfloat16*>(values)[page * pe + e]);
    if (p.quant == 1) {
        const float c = static_cast<float>(static_cast<const unsigned char*>(values)[page * pe + e]) - 128.0f;
        const float s = scales[page];
        return fabsf(s - 1.0f) < 1.1920929e-7f ? c : bf16_rn(c * bf16_rn(s));
    }
    const unsigned char byte = static_cast<const unsigned char*>(values)[(page * pe + e) >> 1];
    const int code = (e & 1) ? (byte >> 4) : (byte & 0x0F);
    return bf16_rn(static_cast<float>(code - 8) * scales[page * (pe / 32) + (e >> 5)]);
}

// One CTA per (sequence, K or V, touched page).  `old_len` tokens are in the cache, `n_new` arrive (rows
// of `src`, [kv_heads * head_dim] values each, ld apart).  The CTA rebuilds its page: the tokens it
// already holds are taken dequantised, the new ones from src, and the whole page is quantised anew.
__global__ void __launch_bounds__(256)
    pages_append_kernel(Pages p, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, long long ld_k,
                        long long ld_v, const int* __restrict__ seq_lens, int n_new, int pages_per_call, int* status) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    __shared__ float red[8];
    __shared__ float page_scale;
    const int b = blockIdx.z, which = blockIdx.y;
    const int old_len = seq_lens[b];
    const int first_page = old_len / p.page_size;
    const int pg = first_page + blockIdx.x;  // logical page of the sequence this CTA rebuilds
    const int new_len = old_len + n_new;
    if (static_cast<long long>(pg) * p.page_size >= new_len || blockIdx.x >= pages_per_call) return;
    if (pg >= p.max_pages) {
        if (threadIdx.x == 0) atomicExch(status, 9);  // the page table is too short for this sequence
        return;
    }
    const long long page = p.page_table[static_cast<long long>(b) * p.max_pages + pg];
    void* values = which == 0 ? p.k_values : p.v_values;
    float* scales = which == 0 ? p.k_scales : p.v_scales;
    const __nv_bfloat16* src = which == 0 ? k : v;
    const long long ld = which == 0 ? ld_k : ld_v;
    const int row = p.kv_heads * p.head_dim;
    const int tok0 = pg * p.page_size;                        // first token of this page
    const int held = min(max(old_len - tok0, 0), p.page_size);  // tokens of it already stored
    const int upto = min(new_len - tok0, p.page_size);          // tokens it holds after this call
    const long long pe = page_elems(p);
    // value e of the page after the append, before quantisation
    auto merged = [&](long long e) -> float {
        const int t = static_cast<int>(e / row);
        if (t < held) return load_dense(p, values, scales, page, e);
        return __bfloat162float(src[(static_cast<long long>(b) * n_new + (tok0 + t - old_len)) * ld + (e - static_cast<long long>(t) * row)]);
    };
    const long long n = static_cast<long long>(upto) * row;
    if (p.quant == 0) {
        auto* out = static_cast<__nv_bfloat16*>(values) + page * pe;
        for (long long e = static_cast<long long>(held) * row + threadIdx.x; e < n; e += blockDim.x) out[e] = __float2bfloat16_rn(merged(e));
        return;
    }
    if (p.quant == 1) {
        // one scale for the page: largest magnitude first
        float mx = 0.f;
        for (long long e = threadIdx.x; e < n; e += blockDim.x) mx = fmaxf(mx, fabsf(merged(e)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
        __syncthreads();
        if (threadIdx.x == 0) {
            float m = 0.f;
            for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
            page_scale = m > 0.f ? fmaxf(__fdiv_rn(m, 127.0f), 1e-8f) : 1.0f;
        }
        __syncthreads();
        const float scale = page_scale;
        const float inv_bf = bf16_rn(__fdiv_rn(1.0f, scale));
        // every value is read (with the old scale) and rewritten by one thread, in that order, and by no other
        auto* out = static_cast<unsigned char*>(values) + page * pe;
        for (long long e0 = threadIdx.x; e0 < n; e0 += static_cast<long long>(blockDim.x) * 4) {
            float x[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const long long e = e0 + static_cast<long long>(j) * blockDim.x;
                x[j] = e < n ? merged(e) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const long long e = e0 + static_cast<long long>(j) * blockDim.x;
                if (e < n) {
                    const float q = roundf(fminf(fmaxf(bf16_rn(x[j] * inv_bf), -127.0f), 127.0f));
                    out[e] = static_cast<unsigned char>(static_cast<int>(q) + 128);
                }
            }
        }
        __syncthreads();  // the new scale is stored only after every value has been re-read with the old one
        if (threadIdx.x == 0) scales[page] = scale;
        return;
    }
    // Q4_0: a warp takes blocks of 32 values, a lane one value
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    auto* out = static_cast<unsigned char*>(values) + ((page * pe) >> 1);
    float* sc = scales + page * (pe / 32);
    for (long long blk = warp; blk < n / 32; blk += nwarps) {
        const float x = merged(blk * 32 + lane);
        float mx = fabsf(x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        const float scale = mx > 0.f ? __fdiv_rn(mx, 7.0f) : 1.0f;
        const float inv = __fdiv_rn(1.0f, scale);
        const int code = static_cast<int>(fminf(fmaxf(roundf(x * inv), -7.0f), 7.0f)) + 8;
        const int hi = __shfl_down_sync(0xFFFFFFFFu, code, 1);
        __syncwarp();
        if ((lane & 1) == 0) out[blk * 16 + (lane >> 1)] = static_cast<unsigned char>((code & 0x0F) | ((hi & 0x0F) << 4));
        if (lane == 0) sc[blk] = scale;
    }
}

// Dense copy of a sequence's pages: out[b, t, :] for t < seq_lens[b] (materialize_pages, :390-405).
__global__ void pages_materialize_kernel(Pages p, int which, const int* __restrict__ seq_lens, __nv_bfloat16* __restrict__ out,
                                         long long ld_tok, long long ld_batch) {
    const int b = blockIdx.y;
    const int row = p.kv_heads * p.head_dim;
    const long long n = static_cast<long long>(seq_lens[b]) * row;
    const void* values = which == 0 ? p.k_values : p.v_values;
    const float* scales = which == 0 ? p.k_scales : p.v_scales;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long t = i / row, c = i - t * row;
        const long long page = p.page_table[static_cast<long long>(b) * p.max_pages + t / p.page_size];
        const long long e = (t % p.page_size) * row + c;
        out[b * ld_batch + t * ld_tok + c] = __float2bfloat16_rn(load_dense(p, values, scales, page, e));
    }
}

// grid (splits, kv_heads, batch), 128 threads.  A warp takes tokens w, w + 4, ... of the CTA's share of
// the sequence; a lane holds D / 32 consecutive channels of the key / value row and of the G query
// heads that share this KV head.  Scores: per-lane partial dot products, one butterfly per head.
// Every warp keeps its own running maximum, sum and output; the four warps and then the splits are
// merged with the usual rescaling.
template <int D>
__global__ void __launch_bounds__(PA_THREADS)
    paged_attention_kernel(Pages p, const __nv_bfloat16* __restrict__ q, const int* __restrict__ seq_lens, float* __restrict__ part,
                           __nv_bfloat16* __restrict__ out, int heads, long long ld_q, long long ld_out, float scale, int splits) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    constexpr int E = D / 32;
    __shared__ float sm_m[4][PA_MAX_G], sm_l[4][PA_MAX_G], sm_acc[4][PA_MAX_G][D];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
    const int G = heads / p.kv_heads;
    const int len = seq_lens[b];
    const int per = (len + splits - 1) / splits;
    const int t_lo = split * per, t_hi = min(len, t_lo + per);
    const int row = p.kv_heads * D;
    const long long pe = page_elems(p);

    float qv[PA_MAX_G][E];
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g)
#pragma unroll
        for (int e = 0; e < E; ++e)
            qv[g][e] = g < G ? __bfloat162float(q[b * ld_q + static_cast<long long>(kh * G + g) * D + lane * E + e]) * scale : 0.f;
    float m[PA_MAX_G], l[PA_MAX_G], acc[PA_MAX_G][E];
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
    }
    for (int t = t_lo + warp; t < t_hi; t += 4) {
        const long long page = p.page_table[static_cast<long long>(b) * p.max_pages + t / p.page_size];
        const long long e0 = static_cast<long long>(t % p.page_size) * row + kh * D + lane * E;
        float kx[E], vx[E];
        if (p.quant == 0) {
            const __nv_bfloat16* kr = static_cast<const __nv_bfloat16*>(p.k_values) + page * pe + e0;
            const __nv_bfloat16* vr = static_cast<const __nv_bfloat16*>(p.v_values) + page * pe + e0;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                kx[e] = __bfloat162float(kr[e]);
                vx[e] = __bfloat162float(vr[e]);
            }
        } else {
#pragma unroll
            for (int e = 0; e < E; ++e) {
                kx[e] = load_dense(p, p.k_values, p.k_scales, page, e0 + e);
                vx[e] = load_dense(p, p.v_values, p.v_scales, page, e0 + e);
            }
        }
#pragma unroll
        for (int g = 0; g < PA_MAX_G; ++g) {
            if (g >= G) break;
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < E; ++e) s = fmaf(qv[g][e], kx[e], s);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
            const float m_new = fmaxf(m[g], s);
            const float corr = __expf(m[g] - m_new), pr = __expf(s - m_new);
            l[g] = l[g] * corr + pr;
            m[g] = m_new;
#pragma unroll
            for (int e = 0; e < E; ++e) acc[g][e] = fmaf(pr, vx[e], acc[g][e] * corr);
        }
    }
    // ---- merge the four warps ----
#pragma unroll
    for (int g = 0; g < PA_MAX_G; ++g) {
        if (g >= G) break;
        if (lane == 0) {
            sm_m[warp][g] = m[g];
            sm_l[warp][g] = l[g];
        }
#pragma unroll
        for (int e = 0; e < E; ++e) sm_acc[warp][g][lane * E + e] = acc[g][e];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * D; i += PA_THREADS) {
        const int g = i / D, d = i - g * D;
        float mm = -INFINITY;
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm_m[w][g]);
        float ll = 0.f, a = 0.f;
        for (int w = 0; w < 4; ++w) {
            const float c = sm_m[w][g] == -INFINITY ? 0.f : __expf(sm_m[w][g] - mm);
            ll += sm_l[w][g] * c;
            a += sm_acc[w][g][d] * c;
        }
        const int head = kh * G + g;
        if (splits == 1) {
            out[b * ld_out + static_cast<long long>(head) * D + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
        } else {
            float* dst = part + ((static_cast<long long>(b) * heads + head) * splits + split) * (D + 2);
            dst[2 + d] = a;
            if (d == 0) {
                dst[0] = mm;
                dst[1] = ll;
            }
        }
    }
}

template <int D>
__global__ void paged_merge_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int heads, int splits, long long ld_out) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    const float* src = part + (static_cast<long long>(b) * heads + head) * splits * (D + 2);
    float mm = -INFINITY;
    for (int s = 0; s < splits; ++s) mm = fmaxf(mm, src[s * (D + 2)]);
    float ll = 0.f, a = 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = src[s * (D + 2)];
        const float c = ms == -INFINITY ? 0.f : __expf(ms - mm);
        ll += src[s * (D + 2) + 1] * c;
        a += src[s * (D + 2) + 2 + d] * c;
    }
    out[b * ld_out + static_cast<long long>(head) * D + d] = __float2bfloat16_rn(ll > 0.f ? a / ll : 0.f);
}

int pages_from(const izb_kv_pages* a, Pages* p) {
    if (!a || !a->k_values || !a->v_values || !a->page_table) return IZB_ERR_BAD_ARG;
    if (a->quantization < IZB_KV_NONE || a->quantization > IZB_KV_Q4_0) return IZB_ERR_BAD_ARG;
    if (a->page_size <= 0 || a->kv_heads <= 0 || a->max_pages_per_seq <= 0) return IZB_ERR_BAD_ARG;
    if (a->head_dim != 64 && a->head_dim != 128) return IZB_ERR_UNSUPPORTED;
    if (a->quantization != IZB_KV_NONE && (!a->k_scales || !a->v_scales)) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(a->k_values, 16) || !izb_aligned(a->v_values, 16) || !izb_aligned(a->page_table, 4)) return IZB_ERR_BAD_ARG;
    p->k_values = a->k_values; p->v_values = a->v_values;
    p->k_scales = a->k_scales; p->v_scales = a->v_scales;
    p->page_table = a->page_table;
    p->quant = a->quantization; p->page_size = a->page_size; p->kv_heads = a->kv_heads; p->head_dim = a->head_dim;
    p->max_pages = a->max_pages_per_seq;
    return IZB_OK;
}

int paged_splits(const izb_ctx* ctx, int64_t batch, int kv_heads, int64_t max_len) {
    int64_t want = (4 * static_cast<int64_t>(ctx ? ctx->sm_count : 148) + batch * kv_heads - 1) / (batch * kv_heads);
    const int64_t tiles = (max_len + 63) / 64;
    if (want > tiles) want = tiles;
    if (want > 64) want = 64;
    return static_cast<int>(want < 1 ? 1 : want);
}

}  // namespace

extern "C" {

size_t izb_kv_page_bytes(int32_t quantization, int32_t page_size, int32_t kv_heads, int32_t head_dim) {
    if (page_size <= 0 || kv_heads <= 0 || head_dim <= 0) return 0;
    const size_t elems = static_cast<size_t>(page_size) * kv_heads * head_dim;
    return quantization == IZB_KV_NONE ? elems * 2 : quantization == IZB_KV_INT8 ? elems : quantization == IZB_KV_Q4_0 ? elems / 2 : 0;
}

size_t izb_kv_page_scales(int32_t quantization, int32_t page_size, int32_t kv_heads, int32_t head_dim) {
    if (page_size <= 0 || kv_heads <= 0 || head_dim <= 0) return 0;
    const size_t elems = static_cast<size_t>(page_size) * kv_heads * head_dim;
    return quantization == IZB_KV_INT8 ? 1 : quantization == IZB_KV_Q4_0 ? elems / 32 : 0;
}

int32_t izb_kv_pages_append(izb_ctx* ctx, izb_stream stream, const izb_kv_pages* pages, const void* k, const void* v, int64_t batch,
                            int64_t n_new, int64_t ld_k, int64_t ld_v, const int32_t* seq_lens) {
    Pages p;
    if (!ctx || batch < 0 || n_new < 0) return IZB_ERR_BAD_ARG;
    const int rc = pages_from(pages, &p);
    if (rc != IZB_OK) return rc;
    if (batch == 0 || n_new == 0) return IZB_OK;
    const int64_t row = static_cast<int64_t>(p.kv_heads) * p.head_dim;
    if (!k || !v || !seq_lens || ld_k < row || ld_v < row || !izb_aligned(k, 2) || !izb_aligned(v, 2)) return IZB_ERR_BAD_ARG;
    if (batch > 65535 || n_new > (1 << 24)) return IZB_ERR_UNSUPPORTED;
    // pages a call can touch per sequence: the partly filled last one, then whole new ones
    const int pages_per_call = static_cast<int>((n_new + p.page_size - 1) / p.page_size) + 1;
    IZB_CUDA_TRY(izb::launch_chained(ctx, pages_append_kernel, dim3(pages_per_call, 2, static_cast<unsigned>(batch)), dim3(256), 0,
                                     static_cast<cudaStream_t>(stream), p, static_cast<const __nv_bfloat16*>(k),
                                     static_cast<const __nv_bfloat16*>(v), static_cast<long long>(ld_k), static_cast<long long>(ld_v),
                                     seq_lens, static_cast<int>(n_new), pages_per_call, ctx->d_status + 6));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_kv_pages_materialize(izb_ctx* ctx, izb_stream stream, const izb_kv_pages* pages, int32_t which, int64_t batch,
                                 const int32_t* seq_lens, void* out, int64_t ld_token, int64_t ld_batch) {
    Pages p;
    if (!ctx || batch < 0 || (which != 0 && which != 1)) return IZB_ERR_BAD_ARG;
    const int rc = pages_from(pages, &p);
    if (rc != IZB_OK) return rc;
    if (batch == 0) return IZB_OK;
    if (!out || !seq_lens || ld_token < static_cast<int64_t>(p.kv_heads) * p.head_dim || !izb_aligned(out, 2) || batch > 65535)
        return IZB_ERR_BAD_ARG;
    pages_materialize_kernel<<<dim3(ctx->sm_count * 2, static_cast<unsigned>(batch)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        p, which, seq_lens, static_cast<__nv_bfloat16*>(out), ld_token, ld_batch);
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

size_t izb_paged_decode_gqa_attention_workspace_bytes(const izb_ctx* ctx, int64_t batch, int32_t heads, int32_t kv_heads,
                                                      int32_t head_dim, int64_t max_seq_len) {
    if (batch <= 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) return 0;
    const int splits = paged_splits(ctx, batch, kv_heads, max_seq_len);
    return splits <= 1 ? 0 : static_cast<size_t>(batch) * heads * splits * (head_dim + 2) * sizeof(float);
}

int32_t izb_paged_decode_gqa_attention(izb_ctx* ctx, izb_stream stream, const void* q, const izb_kv_pages* pages,
                                       const int32_t* seq_lens, void* out, int64_t batch, int32_t heads, int64_t max_seq_len,
                                       int64_t ld_q, int64_t ld_out, float scale, void* workspace, size_t workspace_bytes) {
    Pages p;
    if (!ctx || batch < 0 || heads <= 0 || max_seq_len <= 0) return IZB_ERR_BAD_ARG;
    const int rc = pages_from(pages, &p);
    if (rc != IZB_OK) return rc;
    if (batch == 0) return IZB_OK;
    if (!q || !out || !seq_lens) return IZB_ERR_BAD_ARG;
    if (heads % p.kv_heads != 0 || heads / p.kv_heads > PA_MAX_G) return IZB_ERR_UNSUPPORTED;
    if (batch > 65535 || p.kv_heads > 65535) return IZB_ERR_BAD_ARG;
    if (ld_q < static_cast<int64_t>(heads) * p.head_dim || ld_out < static_cast<int64_t>(heads) * p.head_dim) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(q, 2) || !izb_aligned(out, 2)) return IZB_ERR_BAD_ARG;
    const int splits = paged_splits(ctx, batch, p.kv_heads, max_seq_len);
    const size_t need = splits > 1 ? static_cast<size_t>(batch) * heads * splits * (p.head_dim + 2) * sizeof(float) : 0;
    if (need && (!workspace || workspace_bytes < need || !izb_aligned(workspace, 4))) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid(splits, p.kv_heads, static_cast<unsigned>(batch));
    const auto* qp = static_cast<const __nv_bfloat16*>(q);
    auto* op = static_cast<__nv_bfloat16*>(out);
    float* part = static_cast<float*>(workspace);
    if (p.head_dim == 128)
        IZB_CUDA_TRY(izb::launch_chained(ctx, paged_attention_kernel<128>, grid, dim3(PA_THREADS), 0, s, p, qp, seq_lens, part, op, heads,
                                         static_cast<long long>(ld_q), static_cast<long long>(ld_out), scale, splits));
    else
        IZB_CUDA_TRY(izb::launch_chained(ctx, paged_attention_kernel<64>, grid, dim3(PA_THREADS), 0, s, p, qp, seq_lens, part, op, heads,
                                         static_cast<long long>(ld_q), static_cast<long long>(ld_out), scale, splits));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    if (splits > 1) {
        if (p.head_dim == 128)
            IZB_CUDA_TRY(izb::launch_chained(ctx, paged_merge_kernel<128>, dim3(heads, static_cast<unsigned>(batch)), dim3(128), 0, s,
                                             static_cast<const float*>(part), op, heads, splits, static_cast<long long>(ld_out)));
        else
            IZB_CUDA_TRY(izb::launch_chained(ctx, paged_merge_kernel<64>, dim3(heads, static_cast<unsigned>(batch)), dim3(64), 0, s,
                                             static_cast<const float*>(part), op, heads, splits, static_cast<long long>(ld_out)));
        ctx->launches.fetch_add(1, std::memory_order_relaxed);
    }
    return IZB_OK;
}

}  // extern "C"
