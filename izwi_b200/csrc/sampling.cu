// Token choice beyond arg-max, on the device: temperature, top-k, top-p (nucleus) and the draw itself,
// one CTA per logits row, so that a decode step never copies a vocabulary-long row to the host.
// The rules are those of the reference's host-side samplers (`sample_from_logits`,
// models/architectures/lfm25_audio/sampling.rs:65-160; `sample_semantic`,
// models/architectures/qwen3/tts/mod.rs:2293-2440):
//   temperature <= 1e-5: the arg-max;  otherwise v = logit / temperature over the finite logits;
//   top_k > 0: keep the k largest (equal values: lowest index first);
//   p = softmax(v) over what is kept;  top_p < 1: keep the smallest prefix, in descending order of p,
//   whose mass reaches max(top_p, 1e-6), renormalise;
//   walk the kept candidates (descending order if top-k or top-p cut anything, index order
//   otherwise) and return the first whose cumulative mass reaches the uniform draw u.
// The draw u in [0, 1) comes from the caller (one float per row on the device), so the host keeps its
// own generator and the result is a pure function of (logits, parameters, u).
//
// No sort: positions in descending order are found by a radix descent over an order-preserving
// 32-bit key of the value (four passes of 256-bin histograms of count and mass), with masses
// exp(v - max) kept as 32.32 fixed point in 64-bit integers, so sums do not depend on the order in
// which threads add them and every run gives the same token.
#include <cmath>

#include "izb_common.cuh"

namespace {

constexpr int SMP_THREADS = 1024;

struct SampleShared {
    unsigned int cnt[256];
    unsigned long long mass[256];
    unsigned int warp_cnt[SMP_THREADS / 32];
    unsigned long long warp_mass[SMP_THREADS / 32];
    float red_f[SMP_THREADS / 32];
    int red_i[SMP_THREADS / 32];
    // results of a step, written by thread 0
    unsigned int sel_prefix, sel_cnt_before;
    unsigned long long sel_mass_before;
    unsigned long long total_mass;
    unsigned int total_cnt;
    float vmax;
    int answer;
};

__device__ __forceinline__ float load_logit(const void* row, int dtype, int i) {
    return dtype == IZB_F32 ? static_cast<const float*>(row)[i] : __bfloat162float(static_cast<const __nv_bfloat16*>(row)[i]);
}
// larger value <-> larger key
__device__ __forceinline__ unsigned int order_key(float v) {
    const unsigned int u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long mass_of(float v, float vmax) {
    return static_cast<unsigned long long>(__expf(v - vmax) * 4294967296.0f);  // 32.32 fixed point, at most 2^32
}

// One radix descent in descending key order.  by_mass: stop at the first position whose cumulative
// mass reaches `target_mass`; else at position `target_cnt` (1-based).  Leaves in shared memory the
// full key of the group of equal values in which the target falls, and the count and mass of all
// elements with a larger key.
__device__ void descend(SampleShared& sh, const void* row, int dtype, int cols, float inv_t, float vmax, bool by_mass,
                        unsigned long long target_mass, unsigned int target_cnt) {
    unsigned int prefix = 0, cnt_before = 0;
    unsigned long long mass_before = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = threadIdx.x; i < 256; i += SMP_THREADS) {
            sh.cnt[i] = 0;
            sh.mass[i] = 0;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < cols; i += SMP_THREADS) {
            const float raw = load_logit(row, dtype, i);
            if (!isfinite(raw)) continue;
            const float v = raw * inv_t;
            const unsigned int key = order_key(v);
            if (pass > 0 && (key >> (shift + 8)) != (prefix >> (shift + 8))) continue;
            const unsigned int bin = (key >> shift) & 255u;
            atomicAdd(&sh.cnt[bin], 1u);
            atomicAdd(&sh.mass[bin], mass_of(v, vmax));
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int bin = 255;
            for (; bin > 0; --bin) {
                const bool reached = by_mass ? (mass_before + sh.mass[bin] >= target_mass) : (cnt_before + sh.cnt[bin] >= target_cnt);
                if (reached) break;
                cnt_before += sh.cnt[bin];
                mass_before += sh.mass[bin];
            }
            sh.sel_prefix = prefix | (static_cast<unsigned int>(bin) << shift);
            sh.sel_cnt_before = cnt_before;
            sh.sel_mass_before = mass_before;
        }
        __syncthreads();
        prefix = sh.sel_prefix;
        cnt_before = sh.sel_cnt_before;
        mass_before = sh.sel_mass_before;
        __syncthreads();
    }
}

// Index of the r-th (1-based) element, in index order, whose key equals `key`; the last such element if the
// group has fewer than r members (a target at the very end of the mass).
__device__ int nth_with_key(SampleShared& sh, const void* row, int dtype, int cols, float inv_t, unsigned int key, unsigned int r) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned int seen = 0;
    if (threadIdx.x == 0) {
        sh.answer = -1;
        sh.red_i[0] = -1;
    }
    __syncthreads();
    for (int base = 0; base < cols; base += SMP_THREADS) {
        const int i = base + threadIdx.x;
        bool hit = false;
        if (i < cols) {
            const float raw = load_logit(row, dtype, i);
            hit = isfinite(raw) && order_key(raw * inv_t) == key;
        }
        const unsigned int ballot = __ballot_sync(0xFFFFFFFFu, hit);
        if (lane == 0) sh.warp_cnt[warp] = __popc(ballot);
        __syncthreads();
        unsigned int before = seen, chunk = 0;
        for (int w = 0; w < SMP_THREADS / 32; ++w) {
            if (w < warp) before += sh.warp_cnt[w];
            chunk += sh.warp_cnt[w];
        }
        if (hit) {
            if (before + __popc(ballot & ((1u << lane) - 1u)) + 1 == r) sh.answer = i;  // this hit's 1-based rank
            atomicMax(&sh.red_i[0], i);
        }
        __syncthreads();
        seen += chunk;
        if (sh.answer >= 0) break;
        __syncthreads();
    }
    __syncthreads();
    return sh.answer >= 0 ? sh.answer : sh.red_i[0];
}

__global__ void __launch_bounds__(SMP_THREADS)
    sample_rows_kernel(const void* __restrict__ logits, int dtype, int cols, long long ld, float temperature, int top_k, float top_p,
                       const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ SampleShared sh;
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const void* row = static_cast<const uint8_t*>(logits) + static_cast<size_t>(blockIdx.x) * ld * (dtype == IZB_F32 ? 4 : 2);

    // ---- the largest finite logit and its lowest index; how many are finite ----
    float best = -INFINITY;
    int best_i = 0x7FFFFFFF;
    unsigned int finite = 0;
    for (int i = threadIdx.x; i < cols; i += SMP_THREADS) {
        const float v = load_logit(row, dtype, i);
        if (isfinite(v)) {
            ++finite;
            if (v > best) {
                best = v;
                best_i = i;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_i, o);
        finite += __shfl_xor_sync(0xFFFFFFFFu, finite, o);
        if (ob > best || (ob == best && oi < best_i)) {
            best = ob;
            best_i = oi;
        }
    }
    if (lane == 0) {
        sh.red_f[warp] = best;
        sh.red_i[warp] = best_i;
        sh.warp_cnt[warp] = finite;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float b = -INFINITY;
        int bi = 0x7FFFFFFF;
        unsigned int n = 0;
        for (int w = 0; w < SMP_THREADS / 32; ++w) {
            n += sh.warp_cnt[w];
            if (sh.red_f[w] > b || (sh.red_f[w] == b && sh.red_i[w] < bi)) {
                b = sh.red_f[w];
                bi = sh.red_i[w];
            }
        }
        sh.vmax = b;
        sh.answer = bi == 0x7FFFFFFF ? 0 : bi;
        sh.total_cnt = n;
    }
    __syncthreads();
    const unsigned int n_finite = sh.total_cnt;
    const int argmax = sh.answer;
    if (temperature <= 1e-5f || n_finite == 0) {  // greedy, or nothing to draw from
        if (threadIdx.x == 0) out[blockIdx.x] = argmax;
        return;
    }
    const float inv_t = 1.0f / fmaxf(temperature, 1e-5f);
    const float vmax = sh.vmax * inv_t;
    __syncthreads();

    // ---- total mass of the finite logits ----
    unsigned long long part = 0;
    for (int i = threadIdx.x; i < cols; i += SMP_THREADS) {
        const float raw = load_logit(row, dtype, i);
        if (isfinite(raw)) part += mass_of(raw * inv_t, vmax);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
    if (lane == 0) sh.warp_mass[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long z = 0;
        for (int w = 0; w < SMP_THREADS / 32; ++w) z += sh.warp_mass[w];
        sh.total_mass = z;
    }
    __syncthreads();
    unsigned long long z_kept = sh.total_mass;
    const float u = fminf(fmaxf(uniform[blockIdx.x], 0.0f), 0.99999994f);
    const bool cut_k = top_k > 0 && static_cast<unsigned int>(top_k) < n_finite;
    const bool cut_p = top_p < 1.0f;

    if (!cut_k && !cut_p) {
        // ---- index order: first index whose running mass reaches u * Z ----
        unsigned long long target = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(z_kept));
        if (target < 1) target = 1;
        unsigned long long run = 0;
        if (threadIdx.x == 0) sh.answer = -1;
        __syncthreads();
        for (int base = 0; base < cols; base += SMP_THREADS) {
            const int i = base + threadIdx.x;
            unsigned long long m = 0;
            if (i < cols) {
                const float raw = load_logit(row, dtype, i);
                if (isfinite(raw)) m = mass_of(raw * inv_t, vmax);
            }
            unsigned long long incl = m;  // inclusive scan inside the warp
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += up;
            }
            if (lane == 31) sh.warp_mass[warp] = incl;
            __syncthreads();
            unsigned long long before = run, chunk = 0;
            for (int w = 0; w < SMP_THREADS / 32; ++w) {
                if (w < warp) before += sh.warp_mass[w];
                chunk += sh.warp_mass[w];
            }
            const unsigned long long cum = before + incl;
            // the one element at which the running mass crosses the target
            if (m > 0 && cum >= target && cum - m < target) sh.answer = i;
            __syncthreads();
            run += chunk;
            if (sh.answer >= 0) break;
            __syncthreads();
        }
        __syncthreads();
        if (threadIdx.x == 0) out[blockIdx.x] = sh.answer >= 0 ? sh.answer : argmax;
        return;
    }

    // ---- descending order ----
    if (cut_k) {
        descend(sh, row, dtype, cols, inv_t, vmax, false, 0, static_cast<unsigned int>(top_k));
        // the group of equal values in which position k falls: (k - larger) of its members are kept
        const unsigned long long m_tie = mass_of(__uint_as_float((sh.sel_prefix & 0x80000000u) ? (sh.sel_prefix & 0x7FFFFFFFu) : ~sh.sel_prefix), vmax);
        z_kept = sh.sel_mass_before + static_cast<unsigned long long>(static_cast<unsigned int>(top_k) - sh.sel_cnt_before) * m_tie;
        __syncthreads();
    }
    if (cut_p) {
        const double cutoff = fmax(static_cast<double>(top_p), 1e-6) * static_cast<double>(z_kept);
        unsigned long long target = static_cast<unsigned long long>(cutoff);
        if (target < 1) target = 1;
        if (target > z_kept) target = z_kept;
        descend(sh, row, dtype, cols, inv_t, vmax, true, target, 0);
        const unsigned long long m_tie = mass_of(__uint_as_float((sh.sel_prefix & 0x80000000u) ? (sh.sel_prefix & 0x7FFFFFFFu) : ~sh.sel_prefix), vmax);
        unsigned long long r = m_tie ? (target - sh.sel_mass_before + m_tie - 1) / m_tie : 1;  // members of the group inside the nucleus
        if (r < 1) r = 1;
        const unsigned long long z_p = sh.sel_mass_before + r * m_tie;
        z_kept = z_p < z_kept ? z_p : z_kept;
        __syncthreads();
    }
    {
        unsigned long long target = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(z_kept));
        if (target < 1) target = 1;
        if (target > z_kept) target = z_kept;
        descend(sh, row, dtype, cols, inv_t, vmax, true, target, 0);
        const unsigned int key = sh.sel_prefix;
        const unsigned long long m_tie = mass_of(__uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key), vmax);
        unsigned long long r = m_tie ? (target - sh.sel_mass_before + m_tie - 1) / m_tie : 1;
        if (r < 1) r = 1;
        __syncthreads();
        const int idx = nth_with_key(sh, row, dtype, cols, inv_t, key, static_cast<unsigned int>(r > 0xFFFFFFFFull ? 0xFFFFFFFFull : r));
        if (threadIdx.x == 0) out[blockIdx.x] = idx >= 0 ? idx : argmax;
    }
}

}  // namespace

extern "C" {

int32_t izb_sample_rows(izb_ctx* ctx, izb_stream stream, const void* logits, int32_t dtype, int64_t rows, int64_t cols, int64_t ld,
                        float temperature, int32_t top_k, float top_p, const float* uniform, int32_t* out_idx) {
    if (!ctx || rows < 0 || cols <= 0 || ld < cols || top_k < 0) return IZB_ERR_BAD_ARG;
    if (dtype != IZB_F32 && dtype != IZB_BF16) return IZB_ERR_BAD_ARG;
    if (!(top_p >= 0.0f) || !(temperature == temperature)) return IZB_ERR_BAD_ARG;
    if (rows == 0) return IZB_OK;
    if (!logits || !out_idx || !izb_aligned(logits, dtype == IZB_F32 ? 4 : 2) || !izb_aligned(out_idx, 4)) return IZB_ERR_BAD_ARG;
    if (temperature > 1e-5f && (!uniform || !izb_aligned(uniform, 4))) return IZB_ERR_BAD_ARG;
    if (cols > INT32_MAX || rows > 65535 * 64) return IZB_ERR_UNSUPPORTED;
    IZB_CUDA_TRY(izb::launch_chained(ctx, sample_rows_kernel, dim3(static_cast<unsigned>(rows)), dim3(SMP_THREADS), 0,
                                     static_cast<cudaStream_t>(stream), logits, dtype, static_cast<int>(cols),
                                     static_cast<long long>(ld), temperature, top_k, top_p, uniform, out_idx));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // extern "C"
