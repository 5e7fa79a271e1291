// Block-quantised linear layers for 17..64 tokens: dequantise into shared memory, multiply on tcgen05.
//
// Same plan, descriptors and TMA producer as the weight-streaming kernel (skinny.cu), but the
// consumers do not multiply: eight warps turn each 64-k slice of a 128-row weight tile into bf16
// values (block scale applied) laid out as a K-major, 128-byte-swizzled UMMA operand, and one
// thread issues tcgen05.mma (128 weight rows x up to 64 tokens x 16) against the activation slice
// the producer already placed in the ring in exactly that operand layout.  The accumulator lives in
// TMEM; the dequantisation cost per weight no longer grows with the token count.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "skinny.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace izb {

constexpr int STC_DQ_WARPS = 8;                       // dequantise (all) + epilogue (first four)
constexpr int STC_THREADS = 32 * (STC_DQ_WARPS + 2);  // + producer warp + MMA warp
constexpr int STC_TILE_ROWS = 128;
constexpr int STC_ABUF_BYTES = STC_TILE_ROWS * 128;   // one 64-k operand slice: 128 rows x 128 bytes
constexpr int STC_NA = 4;  // operand slices in flight between the dequantising warps and the MMA thread

struct StcShared {
    unsigned long long full[SK_MAX_STAGES];
    unsigned long long empty[SK_MAX_STAGES];
    unsigned long long a_ready[STC_NA];
    unsigned long long a_free[STC_NA];
    unsigned long long acc_full, acc_empty, drain;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts128v(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Four int8 codes of a word times the block scale -> two bf16x2 registers (natural k order).
__device__ __forceinline__ void s8x4_scaled_bf16(uint32_t w, float d, uint32_t& p01, uint32_t& p23) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = __uint_as_float(prmt(u, 0x4B000000u, 0x7440)) - 8388736.0f;
    const float f1 = __uint_as_float(prmt(u, 0x4B000000u, 0x7441)) - 8388736.0f;
    const float f2 = __uint_as_float(prmt(u, 0x4B000000u, 0x7442)) - 8388736.0f;
    const float f3 = __uint_as_float(prmt(u, 0x4B000000u, 0x7443)) - 8388736.0f;
    p01 = pack_bf16x2(f0 * d, f1 * d);
    p23 = pack_bf16x2(f2 * d, f3 * d);
}

// Q8_0: one 64-k slice = one pair of blocks (68 bytes, see skinny.cu).  Warp w owns rows
// 16w..16w+15; lane (g, t) lifts codes 4t..4t+3 of each 16-code quarter and writes 8 bytes.
__device__ __forceinline__ void dequant_slice_q8_0(uint32_t wpair, uint32_t abuf, int warp, int g, int t) {
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        const int row = warp * 16 + rr * 8 + g;
        const uint32_t wr = wpair + static_cast<uint32_t>(row * 272);
        const uint32_t w0 = lds32(wr), w8 = lds32(wr + 32);
        const uint32_t l0 = lds32(wr + 4 * t), l1 = lds32(wr + 4 * t + 4);
        const uint32_t h0 = lds32(wr + 16 + 4 * t), h1 = lds32(wr + 20 + 4 * t);
        const uint32_t q2 = lds32(wr + 36 + 4 * t), q3 = lds32(wr + 52 + 4 * t);
        const uint32_t cw[4] = {prmt(l0, l1, 0x5432), prmt(h0, h1, 0x5432), q2, q3};
        const float d0 = half_bits_to_f32(w0), d1 = half_bits_to_f32(w8 >> 16);
        const uint32_t dst = abuf + static_cast<uint32_t>(row * 128 + (t & 1) * 8);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t p01, p23;
            s8x4_scaled_bf16(cw[q], q < 2 ? d0 : d1, p01, p23);
            // codes of quarter q, lane t: k = 16 q + 4 t .. +3 -> 16-byte chunk 2 q + t/2, half t%2
            sts64(dst + static_cast<uint32_t>(((2 * q + (t >> 1)) ^ (row & 7)) << 4), p01, p23);
        }
    }
}

// Q4_K: one 64-k slice = code group j of a super-block (32 bytes: low nibbles sub-block 2j, high
// nibbles 2j+1).  Thread (row, HI) owns one sub-block of one row: 32 code bytes -> 32 weights;
// warps 0..3 take the low nibbles, warps 4..7 the high ones, so the nibble choice never diverges.
template <bool HI>
__device__ __forceinline__ void dequant_slice_q4_k(uint32_t wsb, int wrow, int j, uint32_t abuf, int row) {
    const uint32_t base = wsb + static_cast<uint32_t>(row * wrow);
    const uint4 hd = lds128(base);
    const int s = 2 * j + (HI ? 1 : 0);  // sub-block index 0..7
    uint32_t sc, mn;
    if (s < 4) {
        sc = (hd.y >> (8 * s)) & 0x3Fu;
        mn = (hd.z >> (8 * s)) & 0x3Fu;
    } else {
        sc = ((hd.w >> (8 * (s - 4))) & 0x0Fu) | (((hd.y >> (8 * (s - 4) + 6)) & 0x3u) << 4);
        mn = ((hd.w >> (8 * (s - 4) + 4)) & 0x0Fu) | (((hd.z >> (8 * (s - 4) + 6)) & 0x3u) << 4);
    }
    const float dsc = half_bits_to_f32(hd.x) * static_cast<float>(sc);
    const float dm = half_bits_to_f32(hd.x >> 16) * static_cast<float>(mn);
    const uint32_t s2 = bcast_bf16x2(dsc);
    const uint32_t c2 = bcast_bf16x2(-fmaf(16.0f, bf16_hi_to_f32(s2), dm));  // weight = (16+n)*s - (16*s + dm)
    const uint4 c0 = lds128(base + static_cast<uint32_t>(16 + j * 32));
    const uint4 c1 = lds128(base + static_cast<uint32_t>(16 + j * 32 + 16));
    const uint32_t words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const uint32_t dst = abuf + static_cast<uint32_t>(row * 128);
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // four 16-byte chunks of 8 weights = two code words each
        uint32_t out[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = words[2 * c + h];
            // bytes (0,1) and (2,3) spread into the two halves of a word: natural k order
            const uint32_t v01 = prmt(w, 0u, 0x4140), v23 = prmt(w, 0u, 0x4342);
            // nibble n -> bf16 16+n (0x4180 | n<<3), then one fma with the sub-block's scale pair
            const uint32_t n01 = lop3<0xEA>(HI ? (v01 >> 1) : (v01 << 3), 0x00780078u, 0x41804180u);
            const uint32_t n23 = lop3<0xEA>(HI ? (v23 >> 1) : (v23 << 3), 0x00780078u, 0x41804180u);
            out[2 * h] = hfma2_bf16(n01, s2, c2);
            out[2 * h + 1] = hfma2_bf16(n23, s2, c2);
        }
        sts128v(dst + static_cast<uint32_t>((((HI ? 4 : 0) + c) ^ (row & 7)) << 4), out[0], out[1], out[2], out[3]);
    }
}

template <int FMT>
__global__ void __launch_bounds__(STC_THREADS)
    skinny_tc_kernel(const SkinnyProblem* __restrict__ probs, const __grid_constant__ SkinnyProblem single, int n_probs,
                     int total_tiles, int n_stages, int stage_bytes, int lite_bytes, int mp, int y_dtype, int* status) {
    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    __shared__ StcShared sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const SkinnyProblem* plist = probs ? probs : &single;

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.empty[s]), 1);
        }
        for (int b = 0; b < STC_NA; ++b) {
            mbar_init(smem_u32(&sh.a_ready[b]), STC_DQ_WARPS);
            mbar_init(smem_u32(&sh.a_free[b]), 1);
        }
        mbar_init(smem_u32(&sh.acc_full), 1);
        mbar_init(smem_u32(&sh.acc_empty), 4);
        mbar_init(smem_u32(&sh.drain), 1);
        sh.abort_flag = 0;
        mbar_fence_init();
    }
    ProbLite* lite = reinterpret_cast<ProbLite*>(dyn_smem);
    const int n_cached = min(n_probs, lite_bytes / static_cast<int>(sizeof(ProbLite)));
    for (int i = threadIdx.x; i < n_cached; i += blockDim.x) lite[i] = lite_from(plist[i]);
    if (warp == STC_DQ_WARPS + 1) tc_alloc(smem_u32(&sh.tmem_base), 64);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    volatile int* abort_flag = &sh.abort_flag;
    const uint32_t tmem_base = sh.tmem_base;
    const uint32_t abuf0 = smem_u32(dyn_smem) + static_cast<uint32_t>(lite_bytes);
    const uint32_t stage0 = abuf0 + STC_NA * STC_ABUF_BYTES;
    bool ok = true;

    if (warp == STC_DQ_WARPS) {
        // ---------------- TMA producer (one lane) ----------------
        if (lane == 0) {
            int stage = 0, p = -1;
            uint32_t phase = 0;
            long long issued = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int np = find_problem(lite, n_cached, plist, n_probs, tile);
                const bool moved = np != p;
                p = np;
                const SkinnyProblem* P = plist + p;
                if (moved && probs) {
                    tma_fence_descriptor(&P->tmap_w);
                    tma_fence_descriptor(&P->tmap_x);
                }
                const ProbLite L = p < n_cached ? lite[p] : lite_from(*P);
                const int row0 = (tile - L.tile_start) * STC_TILE_ROWS;
                const int xchunks = L.nb * (L.kbox >> 6);
                for (int c = 0; c < L.n_chunks; ++c) {
                    if (!mbar_wait_bounded(smem_u32(&sh.empty[stage]), phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fbar = smem_u32(&sh.full[stage]);
                    const uint32_t sbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                    mbar_expect_tx(fbar, static_cast<uint32_t>(L.stage_tx));
                    tma_load_3d(sbase, &P->tmap_w, 0, row0, c * L.nb, fbar);
                    tma_load_3d(sbase + static_cast<uint32_t>(L.x_off), &P->tmap_x, 0, 0, c * xchunks, fbar);
                    ++issued;
                    if (++stage == n_stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                const long long first = issued > n_stages ? issued - n_stages : 0;
                for (long long f = first; f < issued; ++f) {
                    const uint32_t bar = smem_u32(&sh.full[f % n_stages]);
                    const uint32_t par = static_cast<uint32_t>((f / n_stages) & 1);
                    const long long t0 = clock64();
                    while (!mbar_try_wait(bar, par)) {
                        if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) break;
                    }
                }
            }
        }
    } else if (warp == STC_DQ_WARPS + 1) {
        // ---------------- MMA issuer (one lane) ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(mp);
            int stage = 0, it = 0;
            uint32_t phase = 0;
            unsigned int kbi = 0;  // 64-k slices issued so far by this CTA
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int p = find_problem(lite, n_cached, plist, n_probs, tile);
                const ProbLite L = p < n_cached ? lite[p] : lite_from(plist[p]);
                const int slices = L.nb * (L.kbox >> 6);
                if (!mbar_wait_bounded(smem_u32(&sh.acc_empty), static_cast<uint32_t>(it & 1) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                for (int c = 0; c < L.n_chunks && ok; ++c) {
                    if (!mbar_wait_bounded(smem_u32(&sh.full[stage]), phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t xbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes) +
                                           static_cast<uint32_t>(L.x_off);
                    for (int kb = 0; kb < slices; ++kb, ++kbi) {
                        const int buf = kbi % STC_NA;
                        if (!mbar_wait_bounded(smem_u32(&sh.a_ready[buf]), (kbi / STC_NA) & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint64_t adesc = umma_desc_k_major_sw128(abuf0 + static_cast<uint32_t>(buf * STC_ABUF_BYTES));
                        const uint64_t bdesc = umma_desc_k_major_sw128(xbase + static_cast<uint32_t>(kb * mp * 128));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tc_mma_f16(tmem_base, adesc + static_cast<uint64_t>(2 * k), bdesc + static_cast<uint64_t>(2 * k),
                                       idesc, (c | kb | k) != 0 ? 1u : 0u);
                        tc_commit(smem_u32(&sh.a_free[buf]));
                    }
                    if (!ok) break;
                    tc_commit(smem_u32(&sh.empty[stage]));  // raw weights and activations of this stage are consumed
                    if (++stage == n_stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&sh.acc_full));
            }
            tc_commit(smem_u32(&sh.drain));
            const long long t0 = clock64();
            while (!mbar_try_wait(smem_u32(&sh.drain), 0)) {
                if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                    ok = false;
                    break;
                }
            }
        }
    } else {
        // ---------------- dequantise (8 warps) + epilogue (warps 0..3) ----------------
        const int g = lane >> 2, t = lane & 3;
        int stage = 0, it = 0;
        uint32_t phase = 0;
        unsigned int kbi = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int p = find_problem(lite, n_cached, plist, n_probs, tile);
            const ProbLite L = p < n_cached ? lite[p] : lite_from(plist[p]);
            const int row0 = (tile - L.tile_start) * STC_TILE_ROWS;
            const int per_box = L.kbox >> 6;  // 64-k slices per weight box
            for (int c = 0; c < L.n_chunks && ok; ++c) {
                if (!mbar_wait_bounded(smem_u32(&sh.full[stage]), phase, abort_flag)) {
                    ok = false;
                    break;
                }
                const uint32_t wbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                for (int kb = 0; kb < L.nb * per_box; ++kb, ++kbi) {
                    const int buf = kbi % STC_NA;
                    if (!mbar_wait_bounded(smem_u32(&sh.a_free[buf]), ((kbi / STC_NA) & 1u) ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t abuf = abuf0 + static_cast<uint32_t>(buf * STC_ABUF_BYTES);
                    const uint32_t wbox = wbase + static_cast<uint32_t>((kb / per_box) * L.w_box_bytes);
                    const int in_box = kb % per_box;
                    if constexpr (FMT == IZB_W_Q8_0) {
                        dequant_slice_q8_0(wbox + static_cast<uint32_t>(in_box * 68), abuf, warp, g, t);
                    } else {
                        const uint32_t wsb = wbox + static_cast<uint32_t>((in_box >> 2) * 144);
                        if (warp < 4) dequant_slice_q4_k<false>(wsb, L.w_row_bytes, in_box & 3, abuf, threadIdx.x);
                        else dequant_slice_q4_k<true>(wsb, L.w_row_bytes, in_box & 3, abuf, threadIdx.x - 128);
                    }
                    fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sh.a_ready[buf]));
                }
                if (++stage == n_stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (!ok) break;
            if (warp < 4) {
                // accumulator: lane = weight row (32 per warp), column = token
                if (!mbar_wait_bounded(smem_u32(&sh.acc_full), static_cast<uint32_t>(it & 1), abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const int row = row0 + warp * 32 + lane;
                const float b = (L.bias && row < L.N) ? __bfloat162float(L.bias[row]) : 0.f;
                for (int cc = 0; cc < mp; cc += 32) {
                    float v[32];
                    tc_ld_32x32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(cc), v);
                    if (row < L.N) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int tok = cc + i;
                            if (tok < L.M) {
                                const long long idx = static_cast<long long>(tok) * L.ldy + row;
                                if (y_dtype == IZB_F32) static_cast<float*>(L.y)[idx] = v[i] + b;
                                else static_cast<__nv_bfloat16*>(L.y)[idx] = __float2bfloat16_rn(v[i] + b);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sh.acc_empty));
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == STC_DQ_WARPS + 1) {
        __syncwarp();
        tc_fence_after();
        tc_dealloc(tmem_base, 64);
    }
    if ((!ok || sh.abort_flag) && lane == 0) atomicExch(status, 4);
}

int skinny_tc_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev_probs,
                     const SkinnyProblem* single) {
    if (h.magic != SK_PLAN_MAGIC || !h.tc) return IZB_ERR_BAD_ARG;
    if (!dev_probs && !single) return IZB_ERR_BAD_ARG;
    static const SkinnyProblem dummy = {};
    const SkinnyProblem& s = single ? *single : dummy;
    const int mp = h.nt * 8;
    static std::atomic<int> smem_set[2][16];
    const int slot = ctx->device & 15, which = h.fmt == IZB_W_Q8_0 ? 0 : 1;
    if (smem_set[which][slot].load(std::memory_order_relaxed) < h.smem_bytes) {
        if (which == 0)
            IZB_CUDA_TRY(cudaFuncSetAttribute(skinny_tc_kernel<IZB_W_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem_bytes));
        else
            IZB_CUDA_TRY(cudaFuncSetAttribute(skinny_tc_kernel<IZB_W_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem_bytes));
        smem_set[which][slot].store(h.smem_bytes, std::memory_order_relaxed);
    }
    if (which == 0)
        skinny_tc_kernel<IZB_W_Q8_0><<<h.grid, STC_THREADS, h.smem_bytes, stream>>>(
            dev_probs, s, h.n_probs, h.total_tiles, h.n_stages, h.stage_bytes, h.lite_bytes, mp, h.y_dtype, ctx->d_status + 3);
    else
        skinny_tc_kernel<IZB_W_Q4_K><<<h.grid, STC_THREADS, h.smem_bytes, stream>>>(
            dev_probs, s, h.n_probs, h.total_tiles, h.n_stages, h.stage_bytes, h.lite_bytes, mp, h.y_dtype, ctx->d_status + 3);
    IZB_CUDA_TRY(cudaGetLastError());
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // namespace izb
