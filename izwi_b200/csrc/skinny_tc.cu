// Block-quantised linear layers for 17..64 tokens: dequantise into shared memory, multiply on tcgen05.
//
// Same plan, descriptors and TMA producer as the weight-streaming kernel (skinny.cu), but the
// consumers do not multiply: sixteen warps turn each 256-k box of a 128-row weight tile into bf16
// values (block scale applied) laid out as four K-major, 128-byte-swizzled UMMA operand slices (one
// thread per row and slice), and one thread issues tcgen05.mma (128 weight rows x up to 64 tokens
// x 16) against the activation slices the producer already placed in the ring in exactly that
// operand layout.  Two accumulators alternate in TMEM, so a tile's read-out overlaps the next
// tile; the dequantisation cost per weight no longer grows with the token count.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include <type_traits>

#include "skinny.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace izb {

constexpr int STC_DQ_WARPS = 16;                      // dequantise + epilogue
constexpr int STC_EPI_WARPS = STC_DQ_WARPS;  // every converting warp reads out 16 token columns of its lane quarter
constexpr int STC_WPROD_WARP = STC_DQ_WARPS, STC_XPROD_WARP = STC_DQ_WARPS + 1, STC_MMA_WARP = STC_DQ_WARPS + 2;
constexpr int STC_THREADS = 32 * (STC_DQ_WARPS + 3);  // + two producer warps + MMA warp
constexpr int STC_MAX_X_STAGES = 4;
constexpr int STC_TILE_ROWS = 128;
constexpr int STC_ABUF_BYTES = STC_TILE_ROWS * 128;   // one 64-k operand slice: 128 rows x 128 bytes
constexpr int STC_NA = 4;        // operand slices of one 256-k weight box; warps 4q..4q+3 own slice q
constexpr int STC_ACC_COLS = 64; // fp32 columns of one accumulator (tokens); two accumulators alternate

struct StcShared {
    unsigned long long full_w[SK_MAX_STAGES];   // raw weight boxes: filled by TMA ...
    unsigned long long empty_w[SK_MAX_STAGES];  // ... released by the converting warps once loaded into registers
    unsigned long long full_x[STC_MAX_X_STAGES];   // activation slices: filled by TMA ...
    unsigned long long empty_x[STC_MAX_X_STAGES];  // ... released when the MMAs that read them complete
    unsigned long long a_ready[2];  // per 32-k half of all four slices: written by all converting warps
    unsigned long long a_free[2];   // the MMAs that read that half have completed
    unsigned long long acc_full[2], acc_empty[2], drain;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void sts128v(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Four int8 codes of a word times the block scale -> two bf16x2 registers (natural k order).
// Code byte u = s + 128 dropped into mantissa bits 8..15 of 2^15 gives the float 32768 + u exactly;
// one fma with the scale d and c = -32896 d (exact in fp32: 257 * 2^7 times an 11-bit scale)
// yields d * s with a single rounding.
__device__ __forceinline__ void s8x4_scaled_bf16(uint32_t w, float d, float c, uint32_t& p01, uint32_t& p23) {
    const uint32_t u = w ^ 0x80808080u;
    const float f0 = fmaf(__uint_as_float(prmt(u, 0x47000000u, 0x7404)), d, c);
    const float f1 = fmaf(__uint_as_float(prmt(u, 0x47000000u, 0x7414)), d, c);
    const float f2 = fmaf(__uint_as_float(prmt(u, 0x47000000u, 0x7424)), d, c);
    const float f3 = fmaf(__uint_as_float(prmt(u, 0x47000000u, 0x7434)), d, c);
    p01 = pack_bf16x2(f0, f1);
    p23 = pack_bf16x2(f2, f3);
}

// Q8_0, one 32-code block -> four 16-byte chunks of one operand row.  q[0..7]: the block's code words.
__device__ __forceinline__ void q8_block_to_row(const uint32_t (&q)[8], uint32_t dbits, uint32_t dst_row, int chunk0,
                                                int row) {
    const float d = half_bits_to_f32(dbits);
    const float c = -32896.0f * d;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint32_t o0, o1, o2, o3;
        s8x4_scaled_bf16(q[2 * ch], d, c, o0, o1);
        s8x4_scaled_bf16(q[2 * ch + 1], d, c, o2, o3);
        sts128v(dst_row + static_cast<uint32_t>(((chunk0 + ch) ^ (row & 7)) << 4), o0, o1, o2, o3);
    }
}

// Q4_K, one sub-block of 32 codes (low or high nibbles of eight code words) -> four chunks of a row.
// nibble n -> bf16 16+n (0x4180 | n<<3), then one fma with the sub-block's scale pair.
template <bool HI>
__device__ __forceinline__ void q4_sub_to_row(const uint32_t (&words)[8], uint32_t s2, uint32_t c2, uint32_t dst_row,
                                              int row) {
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
        uint32_t out[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t w = words[2 * ch + h];
            const uint32_t ws = HI ? (w >> 1) : (w << 3);  // nibble of every byte now at bits 3..6 of that byte
            // bytes (0,1) and (2,3) spread into the two halves of a word: natural k order
            const uint32_t v01 = prmt(ws, 0u, 0x4140), v23 = prmt(ws, 0u, 0x4342);
            out[2 * h] = hfma2_bf16(lop3<0xEA>(v01, 0x00780078u, 0x41804180u), s2, c2);
            out[2 * h + 1] = hfma2_bf16(lop3<0xEA>(v23, 0x00780078u, 0x41804180u), s2, c2);
        }
        sts128v(dst_row + static_cast<uint32_t>((((HI ? 4 : 0) + ch) ^ (row & 7)) << 4), out[0], out[1], out[2], out[3]);
    }
}

// 6-bit scale and minimum of sub-block S from the twelve packed bytes (hd.y, hd.z, hd.w) of a super-block.
template <int S>
__device__ __forceinline__ void q4_scale_min(const uint4& hd, uint32_t& sc, uint32_t& mn) {
    if constexpr (S < 4) {
        sc = (hd.y >> (8 * S)) & 0x3Fu;
        mn = (hd.z >> (8 * S)) & 0x3Fu;
    } else {
        sc = ((hd.w >> (8 * (S - 4))) & 0x0Fu) | (((hd.y >> (8 * (S - 4) + 6)) & 0x3u) << 4);
        mn = ((hd.w >> (8 * (S - 4) + 4)) & 0x0Fu) | (((hd.z >> (8 * (S - 4) + 6)) & 0x3u) << 4);
    }
}

// One thread's share of one 256-k weight box: row `row`, 64-k slice Q, written as the two 32-k halves
// of operand buffer Q.  Each half is handed to the MMA thread on its own barrier, so the half being
// multiplied and the half being written overlap.  n = boxes this thread has converted so far.
template <int FMT, int Q>
__device__ __forceinline__ bool convert_box(StcShared& sh, uint32_t wrow, uint32_t ebar, uint32_t abuf0, int row, int lane,
                                            unsigned int n, volatile int* abort_flag) {
    const uint32_t dst_row = abuf0 + static_cast<uint32_t>(Q * STC_ABUF_BYTES + row * 128);
    const uint32_t par = (n & 1u) ^ 1u;
    if constexpr (FMT == IZB_W_Q8_0) {
        // row = eight 34-byte blocks; slice Q = bytes [68 Q, 68 Q + 68) = words Q .. Q+16 of the five
        // 16-byte units that start at byte 64 Q (rows are 272 bytes apart: conflict-free 16-byte loads)
        uint32_t W[20];
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            const uint4 v = lds128(wrow + static_cast<uint32_t>(64 * Q + 16 * i));
            W[4 * i] = v.x; W[4 * i + 1] = v.y; W[4 * i + 2] = v.z; W[4 * i + 3] = v.w;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(ebar);  // the raw box is in registers: its stage may be refilled
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = prmt(W[Q + i], W[Q + i + 1], 0x5432);  // codes start 2 bytes into word Q
        if (!mbar_wait_bounded(smem_u32(&sh.a_free[0]), par, abort_flag)) return false;
        q8_block_to_row(q, W[Q] & 0xFFFFu, dst_row, 0, row);
        fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.a_ready[0]));
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = W[Q + 9 + i];  // second block: scale in the top half of word Q+8
        if (!mbar_wait_bounded(smem_u32(&sh.a_free[1]), par, abort_flag)) return false;
        q8_block_to_row(q, W[Q + 8] >> 16, dst_row, 4, row);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.a_ready[1]));
    } else {
        // row = one 144-byte super-block; slice Q = code group Q: low nibbles sub-block 2Q, high 2Q+1
        const uint4 hd = lds128(wrow);
        const uint4 c0 = lds128(wrow + static_cast<uint32_t>(16 + Q * 32));
        const uint4 c1 = lds128(wrow + static_cast<uint32_t>(32 + Q * 32));
        const uint32_t words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        __syncwarp();
        if (lane == 0) mbar_arrive(ebar);  // the raw box is in registers: its stage may be refilled
        const float d = half_bits_to_f32(hd.x), dmin = half_bits_to_f32(hd.x >> 16);
        uint32_t sc, mn;
        q4_scale_min<2 * Q>(hd, sc, mn);
        uint32_t s2 = bcast_bf16x2(d * static_cast<float>(sc));
        // weight = (16+n)*s - (16*s + dmin*m), s already rounded to bf16
        uint32_t c2 = bcast_bf16x2(-fmaf(16.0f, bf16_hi_to_f32(s2), dmin * static_cast<float>(mn)));
        if (!mbar_wait_bounded(smem_u32(&sh.a_free[0]), par, abort_flag)) return false;
        q4_sub_to_row<false>(words, s2, c2, dst_row, row);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.a_ready[0]));
        q4_scale_min<2 * Q + 1>(hd, sc, mn);
        s2 = bcast_bf16x2(d * static_cast<float>(sc));
        c2 = bcast_bf16x2(-fmaf(16.0f, bf16_hi_to_f32(s2), dmin * static_cast<float>(mn)));
        if (!mbar_wait_bounded(smem_u32(&sh.a_free[1]), par, abort_flag)) return false;
        q4_sub_to_row<true>(words, s2, c2, dst_row, row);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sh.a_ready[1]));
    }
    return true;
}

// Accumulator -> y for one finished tile: warp w reads TMEM lanes 32 (w%4) .. +31 (weight rows) and
// token columns 16 (w/4) .. +15; every store instruction writes 32 consecutive rows of one token.
template <typename T>
__device__ __forceinline__ void stc_store_cols(T* y, long long ldy, const float (&v)[16], float b, int n_tok) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        if (i < n_tok) {
            if constexpr (sizeof(T) == 4) *y = v[i] + b;
            else if constexpr (std::is_same<T, __half>::value) *y = __float2half_rn(v[i] + b);
            else *y = __float2bfloat16_rn(v[i] + b);
        }
        y += ldy;
    }
}
__device__ __forceinline__ void stc_epilogue(const ProbLite& L, const SkinnyProblem& full, int row0, uint32_t tmem_acc, int warp,
                                             int lane, int mp, int y_dtype) {
    const int cc = (warp >> 2) * 16;
    if (cc >= mp) return;
    const int row = row0 + (warp & 3) * 32 + lane;
    float v[16];
    tc_ld_32x16(tmem_acc + (static_cast<uint32_t>((warp & 3) * 32) << 16) + static_cast<uint32_t>(cc), v);
    if (row >= L.N || cc >= L.M) return;
    if (L.extras && full.residual) {
        // residual [token, row] added in fp32 with the bias, before the one rounding
#pragma unroll
        for (int j = 0; j < 16; ++j)
            if (cc + j < L.M) v[j] += __bfloat162float(full.residual[static_cast<long long>(cc + j) * full.ld_res + row]);
    }
    const float b = L.bias ? __bfloat162float(L.bias[row]) : 0.f;
    const long long first = static_cast<long long>(cc) * L.ldy + row;
    if (y_dtype == IZB_F32) stc_store_cols(static_cast<float*>(L.y) + first, L.ldy, v, b, L.M - cc);
    else if (y_dtype == IZB_F16) stc_store_cols(static_cast<__half*>(L.y) + first, L.ldy, v, b, L.M - cc);
    else stc_store_cols(static_cast<__nv_bfloat16*>(L.y) + first, L.ldy, v, b, L.M - cc);
}

// Waits (bounded) for every copy a producer still has in flight on ring `full`, so that no TMA
// write lands in shared memory after the CTA has gone.
__device__ __forceinline__ void stc_drain_ring(unsigned long long* full, int n_stages, long long issued) {
    const long long first = issued > n_stages ? issued - n_stages : 0;
    for (long long f = first; f < issued; ++f) {
        const uint32_t bar = smem_u32(&full[f % n_stages]);
        const uint32_t par = static_cast<uint32_t>((f / n_stages) & 1);
        const long long t0 = clock64();
        while (!mbar_try_wait(bar, par)) {
            if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) break;
        }
    }
}

template <int FMT>
__global__ void __launch_bounds__(STC_THREADS, 1)
    skinny_tc_kernel(const SkinnyProblem* __restrict__ probs, const __grid_constant__ SkinnyProblem single, int n_probs,
                     int total_tiles, int w_stages, int w_stage_bytes, int x_stages, int lite_bytes, int mp, int y_dtype,
                     int* status) {
    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    __shared__ StcShared sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const SkinnyProblem* plist = probs ? probs : &single;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < w_stages; ++s) {
            mbar_init(smem_u32(&sh.full_w[s]), 1);
            mbar_init(smem_u32(&sh.empty_w[s]), STC_DQ_WARPS);
        }
        for (int s = 0; s < x_stages; ++s) {
            mbar_init(smem_u32(&sh.full_x[s]), 1);
            mbar_init(smem_u32(&sh.empty_x[s]), 1);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(smem_u32(&sh.a_ready[h]), STC_DQ_WARPS);
            mbar_init(smem_u32(&sh.a_free[h]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&sh.acc_full[a]), 1);
            mbar_init(smem_u32(&sh.acc_empty[a]), STC_EPI_WARPS);
        }
        mbar_init(smem_u32(&sh.drain), 1);
        sh.abort_flag = 0;
        mbar_fence_init();
    }
    ProbLite* lite = reinterpret_cast<ProbLite*>(dyn_smem);
    const int n_cached = min(n_probs, lite_bytes / static_cast<int>(sizeof(ProbLite)));
    for (int i = threadIdx.x; i < n_cached; i += blockDim.x) lite[i] = lite_from(plist[i]);
    if (warp == STC_MMA_WARP) tc_alloc(smem_u32(&sh.tmem_base), 2 * STC_ACC_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();  // activations and the output buffer belong to the kernels before this one

    volatile int* abort_flag = &sh.abort_flag;
    const uint32_t tmem_base = sh.tmem_base;
    // dynamic shared memory: [descriptor cache][4 operand slices][activation ring][raw weight ring]
    const uint32_t x_stage_bytes = static_cast<uint32_t>(STC_NA * mp * 128);
    const uint32_t abuf0 = smem_u32(dyn_smem) + static_cast<uint32_t>(lite_bytes);
    const uint32_t xring0 = abuf0 + STC_NA * STC_ABUF_BYTES;
    const uint32_t wring0 = xring0 + static_cast<uint32_t>(x_stages) * x_stage_bytes;
    bool ok = true;

    if (warp == STC_WPROD_WARP || warp == STC_XPROD_WARP) {
        // ---------------- TMA producers (one lane each): raw weight boxes / activation slices ----------------
        if (lane == 0) {
            const bool is_w = warp == STC_WPROD_WARP;
            unsigned long long* full = is_w ? sh.full_w : sh.full_x;
            unsigned long long* empty = is_w ? sh.empty_w : sh.empty_x;
            const int n_stages = is_w ? w_stages : x_stages;
            int stage = 0, p = -1;
            uint32_t phase = 0;
            long long issued = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int np = find_problem(lite, n_cached, plist, n_probs, tile);
                const bool moved = np != p;
                p = np;
                const SkinnyProblem* P = plist + p;
                if (moved && probs) tma_fence_descriptor(is_w ? &P->tmap_w : &P->tmap_x);
                const ProbLite L = p < n_cached ? lite[p] : lite_from(*P);
                const int row0 = (tile - L.tile_start) * STC_TILE_ROWS;
                for (int c = 0; c < L.n_chunks; ++c) {
                    if (!mbar_wait_bounded_relaxed(smem_u32(&empty[stage]), phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fbar = smem_u32(&full[stage]);
                    if (is_w) {
                        mbar_expect_tx(fbar, static_cast<uint32_t>(L.w_box_bytes));
                        tma_load_3d(wring0 + static_cast<uint32_t>(stage * w_stage_bytes), &P->tmap_w, 0, row0, c, fbar);
                    } else {
                        mbar_expect_tx(fbar, x_stage_bytes);
                        tma_load_3d(xring0 + static_cast<uint32_t>(stage) * x_stage_bytes, &P->tmap_x, 0, 0, c * STC_NA, fbar);
                    }
                    ++issued;
                    if (++stage == n_stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) stc_drain_ring(full, n_stages, issued);
        }
    } else if (warp == STC_MMA_WARP) {
        // ---------------- MMA issuer (one lane) ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(mp);
            int stage = 0, it = 0;
            uint32_t phase = 0;
            unsigned int n = 0;  // weight boxes multiplied so far by this CTA
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int p = find_problem(lite, n_cached, plist, n_probs, tile);
                const int n_chunks = p < n_cached ? lite[p].n_chunks : plist[p].n_chunks;
                const int acc = it & 1;
                const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(acc * STC_ACC_COLS);
                if (!mbar_wait_bounded(smem_u32(&sh.acc_empty[acc]), static_cast<uint32_t>((it >> 1) & 1) ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                for (int c = 0; c < n_chunks && ok; ++c, ++n) {
                    if (!mbar_wait_bounded(smem_u32(&sh.full_x[stage]), phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t xbase = xring0 + static_cast<uint32_t>(stage) * x_stage_bytes;
                    // first halves of all four slices, then second halves: the tensor core works on
                    // the first halves while the converting warps still write the second ones
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (!mbar_wait_bounded(smem_u32(&sh.a_ready[h]), n & 1u, abort_flag)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
#pragma unroll
                        for (int q = 0; q < STC_NA; ++q) {
                            const uint64_t adesc = umma_desc_k_major_sw128(abuf0 + static_cast<uint32_t>(q * STC_ABUF_BYTES));
                            const uint64_t bdesc = umma_desc_k_major_sw128(xbase + static_cast<uint32_t>(q * mp * 128));
#pragma unroll
                            for (int k = 2 * h; k < 2 * h + 2; ++k)
                                tc_mma_f16(tmem_acc, adesc + static_cast<uint64_t>(2 * k), bdesc + static_cast<uint64_t>(2 * k),
                                           idesc, (c | q | k) != 0 ? 1u : 0u);
                        }
                        tc_commit(smem_u32(&sh.a_free[h]));
                    }
                    if (!ok) break;
                    tc_commit(smem_u32(&sh.empty_x[stage]));  // the activation slices of this stage are consumed
                    if (++stage == x_stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&sh.acc_full[acc]));
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
        // ---------------- dequantise (16 warps) + epilogue (warps 0..7) ----------------
        // warps that share a scheduler (same warp % 4) convert the same slice: one code path each
        const int q = warp & 3;                   // the 64-k slice of every box this warp converts
        const int row = (warp >> 2) * 32 + lane;  // its row of the 128-row tile
        int stage = 0, it = 0;
        uint32_t phase = 0;
        unsigned int n = 0;
        int prev_p = 0, prev_row0 = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int p = find_problem(lite, n_cached, plist, n_probs, tile);
            const int n_chunks = p < n_cached ? lite[p].n_chunks : plist[p].n_chunks;
            const int w_row_bytes = p < n_cached ? lite[p].w_row_bytes : plist[p].w_row_bytes;
            const int row0 = (tile - (p < n_cached ? lite[p].tile_start : plist[p].tile_start)) * STC_TILE_ROWS;
            for (int c = 0; c < n_chunks && ok; ++c, ++n) {
                if (!mbar_wait_bounded(smem_u32(&sh.full_w[stage]), phase, abort_flag)) {
                    ok = false;
                    break;
                }
                const uint32_t wrow = wring0 + static_cast<uint32_t>(stage * w_stage_bytes + row * w_row_bytes);
                const uint32_t ebar = smem_u32(&sh.empty_w[stage]);
                switch (q) {
                    case 0: ok = convert_box<FMT, 0>(sh, wrow, ebar, abuf0, row, lane, n, abort_flag); break;
                    case 1: ok = convert_box<FMT, 1>(sh, wrow, ebar, abuf0, row, lane, n, abort_flag); break;
                    case 2: ok = convert_box<FMT, 2>(sh, wrow, ebar, abuf0, row, lane, n, abort_flag); break;
                    default: ok = convert_box<FMT, 3>(sh, wrow, ebar, abuf0, row, lane, n, abort_flag); break;
                }
                if (++stage == w_stages) {
                    stage = 0;
                    phase ^= 1u;
                }
                // the previous tile's accumulator is read out one box into this tile: its last MMAs
                // have had time to finish, and the tensor core already works on this tile meanwhile
                if (c == 0 && it > 0 && warp < STC_EPI_WARPS && ok) {
                    const int acc = (it - 1) & 1;
                    if (!mbar_wait_bounded(smem_u32(&sh.acc_full[acc]), static_cast<uint32_t>(((it - 1) >> 1) & 1), abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    stc_epilogue(prev_p < n_cached ? lite[prev_p] : lite_from(plist[prev_p]), plist[prev_p], prev_row0,
                                 tmem_base + static_cast<uint32_t>(acc * STC_ACC_COLS), warp, lane, mp, y_dtype);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&sh.acc_empty[acc]));
                }
            }
            prev_p = p;
            prev_row0 = row0;
        }
        if (ok && it > 0 && warp < STC_EPI_WARPS) {
            const int acc = (it - 1) & 1;
            if (mbar_wait_bounded(smem_u32(&sh.acc_full[acc]), static_cast<uint32_t>(((it - 1) >> 1) & 1), abort_flag)) {
                tc_fence_after();
                stc_epilogue(prev_p < n_cached ? lite[prev_p] : lite_from(plist[prev_p]), plist[prev_p], prev_row0,
                             tmem_base + static_cast<uint32_t>(acc * STC_ACC_COLS), warp, lane, mp, y_dtype);
                tc_fence_before();
            } else {
                ok = false;
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == STC_MMA_WARP) {
        __syncwarp();
        tc_fence_after();
        tc_dealloc(tmem_base, 2 * STC_ACC_COLS);
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
    static std::atomic<int> smem_set[2][IZB_MAX_DEVICES];
    const int slot = ctx->device, which = h.fmt == IZB_W_Q8_0 ? 0 : 1;
    if (smem_set[which][slot].load(std::memory_order_relaxed) < h.smem_bytes) {
        if (which == 0)
            IZB_CUDA_TRY(cudaFuncSetAttribute(skinny_tc_kernel<IZB_W_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem_bytes));
        else
            IZB_CUDA_TRY(cudaFuncSetAttribute(skinny_tc_kernel<IZB_W_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem_bytes));
        smem_set[which][slot].store(h.smem_bytes, std::memory_order_relaxed);
    }
    if (which == 0)
        IZB_CUDA_TRY(launch_chained(ctx, skinny_tc_kernel<IZB_W_Q8_0>, dim3(h.grid), dim3(STC_THREADS), h.smem_bytes, stream, dev_probs,
                                    s, h.n_probs, h.total_tiles, h.n_stages, h.stage_bytes, h.x_stages, h.lite_bytes, mp, h.y_dtype,
                                    ctx->d_status + 3));
    else
        IZB_CUDA_TRY(launch_chained(ctx, skinny_tc_kernel<IZB_W_Q4_K>, dim3(h.grid), dim3(STC_THREADS), h.smem_bytes, stream, dev_probs,
                                    s, h.n_probs, h.total_tiles, h.n_stages, h.stage_bytes, h.x_stages, h.lite_bytes, mp, h.y_dtype,
                                    ctx->d_status + 3));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // namespace izb
