// Small-M linear layers: the persistent weight-streaming kernel and its host planner.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "skinny.cuh"
#include "tma.cuh"

namespace izb {

// Row permutations that make the shared-memory loads bank-conflict free under the 128-byte
// swizzle (16-byte chunk index ^= row & 7).  Fragment row/column g of an mma maps to
// shared-memory row perm(g) inside its group of eight.
//   kPermQuad: for 16-byte loads by lane quads   [0,4,1,5,2,6,3,7]
//   kPermPair: for  8-byte loads by lane quads   [0,2,4,6,1,3,5,7]
__device__ __forceinline__ int perm_quad(int g) { return (g >> 1) | ((g & 1) << 2); }
__device__ __forceinline__ int perm_pair(int g) { return ((g & 3) << 1) | (g >> 2); }

// The few descriptor fields the inner loops need, copied to registers once per tile (the
// descriptor itself lives in global or parameter memory).
struct StageGeom {
    int nb, kbox, w_row_bytes, w_box_bytes;
};

// ---------------------------------------------------------------------------
// consumer inner loops: one pipeline stage
//   wbase/xbase: shared-memory byte addresses of the stage's weight / activation regions
//   the activation region is [k/64 chunks][8*NT token rows][128 bytes], swizzled
//   rowbase: first row (inside the tile) of this warp; g = lane/4, t = lane%4
// ---------------------------------------------------------------------------

// bf16: one weight box = 64 k = [TILE_ROWS][128 bytes], swizzled like the activations.
template <int NT, int RT, int KS>
__device__ __forceinline__ void stage_bf16(float (&acc)[RT][NT][4], uint32_t wbase, uint32_t xbase,
                                           const StageGeom P, int rowbase, int ks, int g, int t) {
    const int pg = perm_quad(g);
    for (int b = ks; b < P.nb; b += KS) {
        const uint32_t wbox = wbase + static_cast<uint32_t>(b * P.w_box_bytes);
        const uint32_t xbox = xbase + static_cast<uint32_t>(b * (NT * 1024));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t col = static_cast<uint32_t>(((4 * h + t) ^ pg) << 4);
            uint4 wa[RT], wb[RT];
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                const uint32_t ra = wbox + static_cast<uint32_t>((rowbase + rt * 16 + pg) * 128) + col;
                wa[rt] = lds128(ra);
                wb[rt] = lds128(ra + 8 * 128);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint4 xb = lds128(xbox + static_cast<uint32_t>((nt * 8 + pg) * 128) + col);
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    mma_bf16_16816(acc[rt][nt], wa[rt].x, wb[rt].x, wa[rt].y, wb[rt].y, xb.x, xb.y);
                    mma_bf16_16816(acc[rt][nt], wa[rt].z, wb[rt].z, wa[rt].w, wb[rt].w, xb.z, xb.w);
                }
            }
        }
    }
}

// Q8_0: one weight box = 256 k = [TILE_ROWS][272 bytes] = 4 pairs of 34-byte blocks.
// A pair is 68 bytes = 17 aligned words:
//   word 0 = [d0 | q0[0..1]], words 1..7 = q0[2..29], word 8 = [q0[30..31] | d1], words 9..16 = q1[0..31].
// Block 0's codes sit half a word off, so each logical word is funnelled out of two neighbours.
// The integer codes go through the tensor core exactly as fp16 (an int8 -> fp16 lift costs a
// third of the int8 -> bf16 one), against activations converted bf16 -> fp16 on the fly; the
// block scale is applied in fp32.
template <int NT, int RT, int KS>
__device__ __forceinline__ void stage_q8_0(float (&acc)[RT][NT][4], uint32_t wbase, uint32_t xbase,
                                           const StageGeom P, int rowbase, int ks, int g, int t) {
    const int pg = perm_pair(g);
    const int units = P.nb * 4;
    for (int u = ks; u < units; u += KS) {
        const uint32_t wbox = wbase + static_cast<uint32_t>((u >> 2) * P.w_box_bytes + (u & 3) * 68);
        const uint32_t xchunk = xbase + static_cast<uint32_t>(u * (NT * 1024));
        // activations of this pair for every token group, converted once and reused by all row tiles;
        // step s covers k = 16 s + 4 t .. +3 of the pair: byte 32 s + 8 t of the 128-byte token row
        uint2 xv[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint32_t xr = xchunk + static_cast<uint32_t>((nt * 8 + pg) * 128 + (t & 1) * 8);
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint2 v = lds64(xr + static_cast<uint32_t>(((2 * s + (t >> 1)) ^ pg) << 4));
                xv[nt][s].x = bf16x2_to_f16x2(v.x);
                xv[nt][s].y = bf16x2_to_f16x2(v.y);
            }
        }
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
            uint32_t a[4][4];  // [step][a0..a3]
            float d[2][2];     // [block][row a / row b]
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint32_t wr = wbox + static_cast<uint32_t>((rowbase + rt * 16 + g + half * 8) * 272);
                const uint32_t w0 = lds32(wr), w8 = lds32(wr + 32);
                const uint32_t l0 = lds32(wr + 4 * t), l1 = lds32(wr + 4 * t + 4);
                const uint32_t h0 = lds32(wr + 16 + 4 * t), h1 = lds32(wr + 20 + 4 * t);
                const uint32_t q2 = lds32(wr + 36 + 4 * t), q3 = lds32(wr + 52 + 4 * t);
                const uint32_t q0 = prmt(l0, l1, 0x5432), q1 = prmt(h0, h1, 0x5432);
                d[0][half] = half_bits_to_f32(w0);
                d[1][half] = half_bits_to_f32(w8 >> 16);
                s8x4_to_f16x4(q0, a[0][half], a[0][half + 2]);
                s8x4_to_f16x4(q1, a[1][half], a[1][half + 2]);
                s8x4_to_f16x4(q2, a[2][half], a[2][half + 2]);
                s8x4_to_f16x4(q3, a[3][half], a[3][half + 2]);
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    float tmp[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_f16_16816(tmp, a[2 * b][0], a[2 * b][1], a[2 * b][2], a[2 * b][3], xv[nt][2 * b].x,
                                  xv[nt][2 * b].y);
                    mma_f16_16816(tmp, a[2 * b + 1][0], a[2 * b + 1][1], a[2 * b + 1][2], a[2 * b + 1][3],
                                  xv[nt][2 * b + 1].x, xv[nt][2 * b + 1].y);
                    acc[rt][nt][0] = fmaf(d[b][0], tmp[0], acc[rt][nt][0]);
                    acc[rt][nt][1] = fmaf(d[b][0], tmp[1], acc[rt][nt][1]);
                    acc[rt][nt][2] = fmaf(d[b][1], tmp[2], acc[rt][nt][2]);
                    acc[rt][nt][3] = fmaf(d[b][1], tmp[3], acc[rt][nt][3]);
                }
            }
        }
    }
}

// Q4_K: one weight box = kbox/256 super-blocks of 144 bytes per row.
// Super-block = [d, dmin (fp16) | 12 scale bytes | 4 groups of 32 code bytes]; group j holds
// sub-block 2j in the low nibbles and 2j+1 in the high nibbles.  A nibble n is lifted to the bf16
// value 16+n with one shift and one logic op (0x4180 | n<<3), then one bf16x2 fma with the
// sub-block's (d*sc) and -(16*d*sc + dmin*m) turns it into the dequantised weight.  Lane t of a
// quad decodes the scales of sub-blocks 2t and 2t+1 and hands them round by shuffle.
template <int NT, int RT, int KS>
__device__ __forceinline__ void stage_q4_k(float (&acc)[RT][NT][4], uint32_t wbase, uint32_t xbase,
                                           const StageGeom P, int rowbase, int ks, int g, int t, int lane) {
    const int pg = perm_quad(g);
    const int sbb = P.kbox >> 8;  // super-blocks per box
    const int nsb = P.nb * sbb;
    const int wrow = P.w_row_bytes;
    for (int sb = ks; sb < nsb; sb += KS) {
        const uint32_t wsb = wbase + static_cast<uint32_t>((sb / sbb) * P.w_box_bytes + (sb % sbb) * 144);
        uint32_t my_s[RT][2][2], my_c[RT][2][2];  // [tile][row a/b][own sub-block 0/1]
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint4 hd = lds128(wsb + static_cast<uint32_t>((rowbase + rt * 16 + g + half * 8) * wrow));
                const float dd = half_bits_to_f32(hd.x), dmin = half_bits_to_f32(hd.x >> 16);
                const uint32_t sc_lo = hd.y & 0x3F3F3F3Fu, mn_lo = hd.z & 0x3F3F3F3Fu;
                const uint32_t sc_hi = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
                const uint32_t mn_hi = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
                const uint32_t scw = (t < 2 ? sc_lo : sc_hi) >> ((t & 1) * 16);
                const uint32_t mnw = (t < 2 ? mn_lo : mn_hi) >> ((t & 1) * 16);
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const float dsc = dd * static_cast<float>((scw >> (8 * s)) & 0xFFu);
                    const float dm = dmin * static_cast<float>((mnw >> (8 * s)) & 0xFFu);
                    const float dsc_r = __bfloat162float(__float2bfloat16_rn(dsc));
                    my_s[rt][half][s] = bcast_bf16x2(dsc);
                    my_c[rt][half][s] = bcast_bf16x2(-(16.0f * dsc_r + dm));
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int src = (lane & ~3) | j;
            uint32_t a[RT][4][4];  // [tile][step = sub*2 + word][a0..a3]
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint32_t s0 = __shfl_sync(0xFFFFFFFFu, my_s[rt][half][0], src);
                    const uint32_t s1 = __shfl_sync(0xFFFFFFFFu, my_s[rt][half][1], src);
                    const uint32_t c0 = __shfl_sync(0xFFFFFFFFu, my_c[rt][half][0], src);
                    const uint32_t c1 = __shfl_sync(0xFFFFFFFFu, my_c[rt][half][1], src);
                    const uint2 wv = lds64(wsb + static_cast<uint32_t>((rowbase + rt * 16 + g + half * 8) * wrow) +
                                           static_cast<uint32_t>(16 + j * 32 + t * 8));
#pragma unroll
                    for (int wd = 0; wd < 2; ++wd) {
                        const uint32_t w = wd ? wv.y : wv.x;
                        // low nibbles (sub-block 2j): bytes 0,2 then bytes 1,3
                        a[rt][wd][half] = hfma2_bf16(lop3<0xEA>(w << 3, 0x00780078u, 0x41804180u), s0, c0);
                        a[rt][wd][half + 2] = hfma2_bf16(lop3<0xEA>(w >> 5, 0x00780078u, 0x41804180u), s0, c0);
                        // high nibbles (sub-block 2j+1)
                        a[rt][2 + wd][half] = hfma2_bf16(lop3<0xEA>(w >> 1, 0x00780078u, 0x41804180u), s1, c1);
                        a[rt][2 + wd][half + 2] = hfma2_bf16(lop3<0xEA>(w >> 9, 0x00780078u, 0x41804180u), s1, c1);
                    }
                }
            }
            // group j of super-block sb is activation chunk sb*4 + j: bytes [0,64) = sub-block 2j, [64,128) = 2j+1
            const uint32_t xchunk = xbase + static_cast<uint32_t>((sb * 4 + j) * (NT * 1024));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t xr = xchunk + static_cast<uint32_t>((nt * 8 + pg) * 128);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    const uint4 xq = lds128(xr + static_cast<uint32_t>(((4 * sub + t) ^ pg) << 4));
                    // word 0 covers x[0..3] -> operand pairs (x0,x2),(x1,x3); word 1 covers x[4..7]
                    const uint32_t b00 = prmt(xq.x, xq.y, 0x5410), b01 = prmt(xq.x, xq.y, 0x7632);
                    const uint32_t b10 = prmt(xq.z, xq.w, 0x5410), b11 = prmt(xq.z, xq.w, 0x7632);
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt) {
                        mma_bf16_16816(acc[rt][nt], a[rt][sub * 2][0], a[rt][sub * 2][1], a[rt][sub * 2][2],
                                       a[rt][sub * 2][3], b00, b01);
                        mma_bf16_16816(acc[rt][nt], a[rt][sub * 2 + 1][0], a[rt][sub * 2 + 1][1], a[rt][sub * 2 + 1][2],
                                       a[rt][sub * 2 + 1][3], b10, b11);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
struct SkinnyShared {
    unsigned long long full[SK_MAX_STAGES];
    unsigned long long empty[SK_MAX_STAGES];
    int abort_flag;
};

template <int FMT, int NT, int RT, int KS>
__global__ void __launch_bounds__(SK_THREADS)
    skinny_kernel(const SkinnyProblem* __restrict__ probs, const __grid_constant__ SkinnyProblem single, int n_probs,
                  int total_tiles, int n_stages, int stage_bytes, int red_bytes, int lite_bytes, int y_dtype,
                  int* status) {
    constexpr int RG = SK_CONSUMER_WARPS / KS;
    constexpr int TILE_ROWS = RG * RT * 16;
    constexpr int ACC = RT * NT * 4;

    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    __shared__ SkinnyShared sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const SkinnyProblem* plist = probs ? probs : &single;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.empty[s]), SK_CONSUMER_WARPS);
        }
        sh.abort_flag = 0;
        mbar_fence_init();
    }
    // dynamic shared memory: [descriptor cache][k-split reduction buffer][stage ring]
    ProbLite* lite = reinterpret_cast<ProbLite*>(dyn_smem);
    const int n_cached = min(n_probs, lite_bytes / static_cast<int>(sizeof(ProbLite)));
    for (int i = threadIdx.x; i < n_cached; i += blockDim.x) lite[i] = lite_from(plist[i]);  // the plan: written by the host
    __syncthreads();
    pdl_wait();  // activations and the output buffer belong to the kernels before this one

    volatile int* abort_flag = &sh.abort_flag;
    const uint32_t stage0 = smem_u32(dyn_smem) + static_cast<uint32_t>(lite_bytes + red_bytes);

    if (warp == SK_CONSUMER_WARPS) {
        // ---------------- producer: one lane issues two tiled copies per stage ----------------
        if (lane != 0) return;
        int stage = 0;
        uint32_t phase = 0;
        long long issued = 0;
        bool ok = true;
        int p = -1;
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
            const int row0 = (tile - L.tile_start) * TILE_ROWS;
            const int n_chunks = L.n_chunks, nb = L.nb, x_off = L.x_off;
            const uint32_t tx = static_cast<uint32_t>(L.stage_tx);
            const int xchunks = nb * (L.kbox >> 6);
            for (int c = 0; c < n_chunks; ++c) {
                if (!mbar_wait_bounded(smem_u32(&sh.empty[stage]), phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                const uint32_t fbar = smem_u32(&sh.full[stage]);
                const uint32_t sbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                mbar_expect_tx(fbar, tx);
                tma_load_3d(sbase, &P->tmap_w, 0, row0, c * nb, fbar);
                tma_load_3d(sbase + static_cast<uint32_t>(x_off), &P->tmap_x, 0, 0, c * xchunks, fbar);
                ++issued;
                if (++stage == n_stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        if (ok) {
            // Drain: every stage handed out has been read back by all consumers.
            for (int s = 0; s < n_stages && ok; ++s) {
                if (!mbar_wait_bounded(smem_u32(&sh.empty[stage]), phase ^ 1u, abort_flag)) ok = false;
                if (++stage == n_stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        if (!ok) {
            // A wait gave up: let the copies still in flight land before the CTA's shared memory goes away.
            const long long first = issued > n_stages ? issued - n_stages : 0;
            for (long long f = first; f < issued; ++f) {
                const uint32_t bar = smem_u32(&sh.full[f % n_stages]);
                const uint32_t par = static_cast<uint32_t>((f / n_stages) & 1);
                const long long t0 = clock64();
                while (!mbar_try_wait(bar, par)) {
                    if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) break;
                }
            }
            atomicExch(status, 1);
        }
        return;
    }

    // ---------------- consumers ----------------
    const int g = lane >> 2, t = lane & 3;
    const int rg = warp / KS, ks = warp % KS;
    const int rowbase = rg * RT * 16;
    float* red = reinterpret_cast<float*>(dyn_smem + lite_bytes);

    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int p = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        p = find_problem(lite, n_cached, plist, n_probs, tile);
        const ProbLite PD = p < n_cached ? lite[p] : lite_from(plist[p]);
        const int row0 = (tile - PD.tile_start) * TILE_ROWS;
        const int n_chunks = PD.n_chunks;
        const uint32_t x_off = static_cast<uint32_t>(PD.x_off);
        const StageGeom P = {PD.nb, PD.kbox, PD.w_row_bytes, PD.w_box_bytes};

        float acc[RT][NT][4];
#pragma unroll
        for (int rt = 0; rt < RT; ++rt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[rt][nt][i] = 0.f;

        for (int c = 0; c < n_chunks; ++c) {
            if (ok && !mbar_wait_bounded(smem_u32(&sh.full[stage]), phase, abort_flag)) ok = false;
            if (ok) {
                const uint32_t wbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                const uint32_t xbase = wbase + x_off;
                if constexpr (FMT == IZB_W_BF16)
                    stage_bf16<NT, RT, KS>(acc, wbase, xbase, P, rowbase, ks, g, t);
                else if constexpr (FMT == IZB_W_Q8_0)
                    stage_q8_0<NT, RT, KS>(acc, wbase, xbase, P, rowbase, ks, g, t);
                else
                    stage_q4_k<NT, RT, KS>(acc, wbase, xbase, P, rowbase, ks, g, t, lane);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.empty[stage]));
            if (++stage == n_stages) {
                stage = 0;
                phase ^= 1u;
            }
        }

        if constexpr (KS > 1) {
            // k-slices 1..KS-1 park their partial sums in shared memory; slice 0 adds them up.
            if (ks > 0) {
                float* dst = red + ((ks - 1) * RG + rg) * ACC * 32 + lane;
#pragma unroll
                for (int rt = 0; rt < RT; ++rt)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) dst[((rt * NT + nt) * 4 + i) * 32] = acc[rt][nt][i];
            }
            named_bar_sync(1, SK_CONSUMER_WARPS * 32);
            if (ks == 0) {
#pragma unroll
                for (int s = 1; s < KS; ++s) {
                    const float* src = red + ((s - 1) * RG + rg) * ACC * 32 + lane;
#pragma unroll
                    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[rt][nt][i] += src[((rt * NT + nt) * 4 + i) * 32];
                }
            }
            named_bar_sync(2, SK_CONSUMER_WARPS * 32);  // the buffer is free for the next tile
        }

        if (ks == 0 && ok) {
            // Fragment row g sits in tile row perm(g) for bf16 (swizzled tile), g otherwise;
            // fragment column n sits in token perm(n) of its group of eight.
            const int rsel = FMT == IZB_W_BF16 ? perm_quad(g) : g;
            const int N = PD.N, M = PD.M, ldy = PD.ldy;
            const __nv_bfloat16* bias = PD.bias;
            void* y = PD.y;
            // a residual (rare: the descriptor says so) is added in fp32 with the bias, before the one rounding
            const __nv_bfloat16* res = PD.extras ? plist[p].residual : nullptr;
            const int ld_res = res ? plist[p].ld_res : 0;
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int row = row0 + rowbase + rt * 16 + rsel + half * 8;
                    if (row < N) {
                        const float b = bias ? __bfloat162float(bias[row]) : 0.f;
#pragma unroll
                        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                            for (int i = 0; i < 2; ++i) {
                                const int n = 2 * t + i;
                                const int tok = nt * 8 + (FMT == IZB_W_Q8_0 ? perm_pair(n) : perm_quad(n));
                                if (tok < M)
                                    store_typed(y, y_dtype, static_cast<long long>(tok) * ldy + row,
                                              acc[rt][nt][half * 2 + i] + b +
                                                  (res ? __bfloat162float(res[static_cast<long long>(tok) * ld_res + row]) : 0.f));
                            }
                        }
                    }
                }
            }
        }
    }
    if (!ok && lane == 0) atomicExch(status, 1);
}

// ---------------------------------------------------------------------------
// host: planning and launch
// ---------------------------------------------------------------------------
namespace {

int env_int(const char* name, int dflt) {
    const char* v = std::getenv(name);
    if (!v || !*v) return dflt;
    return std::atoi(v);
}

template <int FMT, int NT, int RT, int KS>
int launch_one(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
               const SkinnyProblem& single) {
    auto kern = skinny_kernel<FMT, NT, RT, KS>;
    // The opt-in shared-memory ceiling is per function and per device; raise it only when it grows.
    static std::atomic<int> smem_set[IZB_MAX_DEVICES];
    const int dev_slot = ctx->device;
    if (smem_set[dev_slot].load(std::memory_order_relaxed) < h.smem_bytes) {
        IZB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem_bytes));
        smem_set[dev_slot].store(h.smem_bytes, std::memory_order_relaxed);
    }
    IZB_CUDA_TRY(launch_chained(ctx, kern, dim3(h.grid), dim3(SK_THREADS), h.smem_bytes, stream, dev, single, h.n_probs,
                                h.total_tiles, h.n_stages, h.stage_bytes, h.red_bytes, h.lite_bytes, h.y_dtype, ctx->d_status));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

template <int FMT, int NT, int RT>
int launch_ks(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
              const SkinnyProblem& single) {
    switch (h.ks) {
        case 1:
            if constexpr (RT <= 2) return launch_one<FMT, NT, RT, 1>(ctx, stream, h, dev, single);
            return IZB_ERR_UNSUPPORTED;
        case 2: return launch_one<FMT, NT, RT, 2>(ctx, stream, h, dev, single);
        case 4: return launch_one<FMT, NT, RT, 4>(ctx, stream, h, dev, single);
        default: return IZB_ERR_UNSUPPORTED;
    }
}

template <int FMT, int NT>
int launch_cfg(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
               const SkinnyProblem& single) {
    switch (h.rt) {
        case 1: return launch_ks<FMT, NT, 1>(ctx, stream, h, dev, single);
        case 2:
            if constexpr (NT <= 4) return launch_ks<FMT, NT, 2>(ctx, stream, h, dev, single);
            return IZB_ERR_UNSUPPORTED;
        case 4:
            if constexpr (NT <= 2) return launch_ks<FMT, NT, 4>(ctx, stream, h, dev, single);
            return IZB_ERR_UNSUPPORTED;
        default: return IZB_ERR_UNSUPPORTED;
    }
}

template <int FMT>
int launch_fmt(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
               const SkinnyProblem& single) {
    switch (h.nt) {
        case 1: return launch_cfg<FMT, 1>(ctx, stream, h, dev, single);
        case 2: return launch_cfg<FMT, 2>(ctx, stream, h, dev, single);
        case 4: return launch_cfg<FMT, 4>(ctx, stream, h, dev, single);
        case 8: return launch_cfg<FMT, 8>(ctx, stream, h, dev, single);
        default: return IZB_ERR_UNSUPPORTED;
    }
}

struct BoxGeom {
    int kbox;         // k values per weight box
    int w_row_bytes;  // bytes per row of a box
};

BoxGeom box_geom(int fmt, int K, bool tc = false) {
    switch (fmt) {
        case IZB_W_BF16: return {64, 128};
        case IZB_W_Q8_0: return {256, 272};
        default:
            // two super-blocks per box keep the 8-byte code loads conflict free (288 = 32 mod 128);
            // an odd super-block count per row falls back to one (144-byte rows, 2-way conflicts)
            // (the tcgen05 variant reads a row per thread and keeps stages small: always one)
            return (K % 512 == 0 && !tc) ? BoxGeom{512, 288} : BoxGeom{256, 144};
    }
}

}  // namespace

int skinny_gemv_max_tokens() { return std::max(0, std::min(env_int("IZB_SKINNY_GEMV_MAX_M", 2), 4)); }

int skinny_plan_build(const izb_ctx* ctx, const izb_linear_args* probs, int n, SkinnyPlanHeader* hdr,
                      SkinnyProblem* out) {
    if (!ctx || !probs || !hdr || !out || n <= 0) return IZB_ERR_BAD_ARG;
    const int fmt = probs[0].wfmt, y_dtype = probs[0].y_dtype;
    if (fmt != IZB_W_BF16 && fmt != IZB_W_Q8_0 && fmt != IZB_W_Q4_K) return IZB_ERR_BAD_ARG;
    if (y_dtype != IZB_BF16 && y_dtype != IZB_F32 && y_dtype != IZB_F16) return IZB_ERR_BAD_ARG;
    const int kalign = fmt == IZB_W_BF16 ? 64 : 256;

    int64_t max_m = 0;
    bool any_extras = false;
    for (int i = 0; i < n; ++i) {
        const izb_linear_args& a = probs[i];
        if (a.wfmt != fmt || a.y_dtype != y_dtype) return IZB_ERR_BAD_ARG;
        if (a.x_dtype != IZB_BF16) return IZB_ERR_UNSUPPORTED;  // the plan holds no staging rows: izb_linear casts
        if (!a.x || !a.w || !a.y) return IZB_ERR_BAD_ARG;
        if (a.M <= 0 || a.N <= 0 || a.K <= 0) return IZB_ERR_BAD_ARG;
        if (a.M > 64) return IZB_ERR_UNSUPPORTED;
        if (a.N > (1 << 24) || a.K > (1 << 20)) return IZB_ERR_UNSUPPORTED;
        if (a.K % kalign != 0) return IZB_ERR_UNSUPPORTED;
        if (a.ldx < a.K || a.ldy < a.N || a.ldx % 8 != 0) return IZB_ERR_BAD_ARG;
        if (!izb_aligned(a.x, 16) || !izb_aligned(a.w, 16)) return IZB_ERR_BAD_ARG;
        if (!izb_aligned(a.y, y_dtype == IZB_F32 ? 4 : 2)) return IZB_ERR_BAD_ARG;
        if (a.bias && !izb_aligned(a.bias, 2)) return IZB_ERR_BAD_ARG;
        max_m = std::max<int64_t>(max_m, a.M);
        if (a.prologue < IZB_PRO_NONE || a.prologue > IZB_PRO_SILU_MUL) return IZB_ERR_BAD_ARG;
        if (a.prologue == IZB_PRO_RMSNORM && (!a.norm_weight || !izb_aligned(a.norm_weight, 16))) return IZB_ERR_BAD_ARG;
        if (a.prologue == IZB_PRO_SILU_MUL && a.ldx < 2 * a.K) return IZB_ERR_BAD_ARG;
        if (a.residual && (a.ld_residual < a.N || a.ld_residual > INT32_MAX || !izb_aligned(a.residual, 2))) return IZB_ERR_BAD_ARG;
        any_extras = any_extras || a.prologue != IZB_PRO_NONE || a.residual != nullptr;
    }
    if (skinny_imma_takes(probs, n)) return skinny_imma_plan_build(ctx, probs, n, hdr, out);
    const int nt = max_m <= 8 ? 1 : max_m <= 16 ? 2 : max_m <= 32 ? 4 : 8;
    const int mp = nt * 8;
    // wide token groups over block-quantised weights: dequantise once into shared memory, multiply
    // on tcgen05.  Measured crossover against the mma.sync consumers: Q4_K from 17 tokens, Q8_0 from 33.
    const bool tc = fmt != IZB_W_BF16 && nt >= env_int("IZB_SKINNY_TC_MIN_NT", fmt == IZB_W_Q8_0 ? 8 : 4);
    // one to four tokens over block-quantised weights: integer dot products against activations in
    // 16-bit block fixed point (skinny_gemv.cu); gemv = tokens the kernel is instantiated for
    const int gemv = (fmt != IZB_W_BF16 && max_m <= skinny_gemv_max_tokens()) ? (max_m <= 1 ? 1 : max_m <= 2 ? 2 : 4) : 0;
    bool any_prologue = false;
    for (int i = 0; i < n; ++i) any_prologue = any_prologue || probs[i].prologue != IZB_PRO_NONE;
    if (any_prologue && !gemv) return IZB_ERR_UNSUPPORTED;  // only that kernel takes a prologue; every kernel adds a residual
    const bool one_sb = tc || gemv != 0;  // one Q4_K super-block per box row

    // measured best residency: three CTAs per SM for Q8_0 (most ALU work per byte), two otherwise
    // measured best residency: three CTAs per SM for Q8_0 at up to 16 tokens (most ALU work per
    // byte), two otherwise; wide token groups need the whole SM's shared memory for one CTA
    int ctas_per_sm = std::max(1, env_int("IZB_SKINNY_CTAS_PER_SM", gemv ? 4 : (fmt == IZB_W_Q8_0 && nt <= 2) ? 3 : 2));
    if ((nt == 8 || tc) && !env_int("IZB_SKINNY_CTAS_PER_SM", 0)) ctas_per_sm = 1;
    if (gemv && !env_int("IZB_SKINNY_CTAS_PER_SM", 0)) {
        // a lone projection of a decode step has fewer 64-row tiles than four per SM: fewer CTAs per
        // SM then, each with a deeper ring, since with so few CTAs it is the bytes in flight per CTA
        // that set the rate
        int64_t tiles = 0;
        for (int i = 0; i < n; ++i) tiles += (probs[i].N + 63) / 64;
        ctas_per_sm = static_cast<int>(std::min<int64_t>(4, std::max<int64_t>(1, (tiles + ctx->sm_count - 1) / ctx->sm_count)));
    }
    const int stage_target = std::max(4, env_int("IZB_SKINNY_STAGE_KB", 24)) * 1024;
    const int max_grid = ctx->sm_count * ctas_per_sm;
    // barriers (+ gemv: k-half sums, and with one CTA per SM room for the partial sums of a cluster's other CTAs)
    const int static_smem = gemv ? 384 + 512 * gemv + (ctas_per_sm == 1 ? 2048 * gemv : 0) : static_cast<int>(sizeof(SkinnyShared));
    const int budget = ctx->max_smem_optin / ctas_per_sm - 2048 - static_smem;

    // Bytes of the smallest possible stage (one weight box + its activation chunks) of a row tile.
    auto min_stage = [&](int rows) {
        int worst = 0;
        for (int i = 0; i < n; ++i) {
            const BoxGeom bg = box_geom(fmt, static_cast<int>(probs[i].K), one_sb);
            worst = std::max(worst, rows * bg.w_row_bytes + (bg.kbox / 64) * mp * 128);
        }
        return worst;
    };

    // Row tile = 16 * RT * (4 / KS) rows: RT row tiles per warp share every converted activation
    // fragment, KS warps split k.  Candidates in order of preference per format; the first that
    // leaves every CTA a few tiles to balance with and room for two stages wins, else the
    // smallest tile (most CTAs busy on a single small problem).
    struct Cand { int rt, ks; };
    static const Cand pref_q8[] = {{2, 2}, {2, 1}, {1, 1}, {1, 2}, {1, 4}};   // up to 16 tokens
    static const Cand pref_q8w[] = {{2, 1}, {1, 1}, {2, 2}, {1, 2}, {1, 4}};  // 17..64 tokens
    static const Cand pref_q4[] = {{2, 1}, {2, 2}, {1, 1}, {1, 2}, {1, 4}};
    static const Cand pref_bf[] = {{2, 1}, {1, 1}, {1, 2}, {1, 4}};
    const Cand* pref = fmt == IZB_W_Q8_0 ? (nt <= 2 ? pref_q8 : pref_q8w) : fmt == IZB_W_Q4_K ? pref_q4 : pref_bf;
    const int n_pref = fmt == IZB_W_BF16 ? 4 : 5;
    int rt = 1, ks = 4;
    const int forced_rt = env_int("IZB_SKINNY_RT", 0), forced_ks = env_int("IZB_SKINNY_KS", 0);
    const int forced_rows = env_int("IZB_SKINNY_TILE_ROWS", 0);
    if (tc) {
        rt = 2;  // 128-row tiles = the 128 TMEM lanes of one accumulator
        ks = 1;
    } else if (gemv) {
        rt = 2;  // 64-row tiles: two warps per k-half, one row per thread
        ks = 2;
    } else if (forced_rt && forced_ks) {
        rt = forced_rt;
        ks = forced_ks;
        if (rt * nt > 8 || (rt == 4 && ks == 1)) return IZB_ERR_UNSUPPORTED;
    } else {
        for (int c = 0; c < n_pref; ++c) {
            const int rows = 16 * pref[c].rt * (SK_CONSUMER_WARPS / pref[c].ks);
            if (pref[c].rt * nt > 8) continue;
            if (forced_rows) {
                if (rows == forced_rows) { rt = pref[c].rt; ks = pref[c].ks; break; }
                continue;
            }
            int64_t tiles = 0;
            for (int i = 0; i < n; ++i) tiles += (probs[i].N + rows - 1) / rows;
            if (tiles >= 2LL * max_grid && 2 * min_stage(rows) <= budget) { rt = pref[c].rt; ks = pref[c].ks; break; }
        }
    }
    const int tile_rows = 16 * rt * (SK_CONSUMER_WARPS / ks);
    const int rg = SK_CONSUMER_WARPS / ks;

    int stage_bytes = 0, tile_cursor = 0, xq_stage = 0;
    for (int i = 0; i < n; ++i) {
        const izb_linear_args& a = probs[i];
        SkinnyProblem& q = out[i];
        std::memset(&q, 0, sizeof(q));
        const int K = static_cast<int>(a.K), N = static_cast<int>(a.N), M = static_cast<int>(a.M);
        const BoxGeom bg = box_geom(fmt, K, one_sb);
        const int boxes_total = K / bg.kbox;
        const int box_stage = tile_rows * bg.w_row_bytes + (bg.kbox / 64) * (gemv ? gemv : mp) * 128;
        // k-boxes per stage: fill the stage target, keep every k-slice busy, divide the row evenly
        int nb = tc ? 1 : std::max(1, std::min(boxes_total, stage_target / box_stage));  // tc: one box per stage
        const int units_per_box = fmt == IZB_W_BF16 ? 1 : fmt == IZB_W_Q8_0 ? 4 : bg.kbox / 256;
        while (nb * units_per_box < ks && nb < boxes_total && (nb + 1) * box_stage <= 2 * stage_target) ++nb;
        while (nb > 1 && boxes_total % nb != 0) --nb;
        nb = std::min(nb, 256);

        q.y = a.y;
        q.bias = static_cast<const __nv_bfloat16*>(a.bias);
        q.N = N; q.K = K; q.M = M;
        q.ldy = static_cast<int>(a.ldy);
        q.tile_start = tile_cursor;
        q.nb = nb;
        q.kbox = bg.kbox;
        q.n_chunks = (boxes_total + nb - 1) / nb;
        q.w_row_bytes = bg.w_row_bytes;
        q.w_box_bytes = tile_rows * bg.w_row_bytes;
        q.x_off = (nb * q.w_box_bytes + 1023) / 1024 * 1024;
        // gemv: only the tokens the kernel is instantiated for are copied, unswizzled (no tensor-core read)
        const int x_rows = gemv ? gemv : mp;
        const bool silu_mul = a.prologue == IZB_PRO_SILU_MUL;  // gate and up chunks travel side by side
        const int x_half = nb * (bg.kbox / 64) * x_rows * 128;
        const int x_bytes = silu_mul ? 2 * x_half : x_half;
        q.norm_w = static_cast<const __nv_bfloat16*>(a.prologue == IZB_PRO_RMSNORM ? a.norm_weight : nullptr);
        q.residual = static_cast<const __nv_bfloat16*>(a.residual);
        q.ld_res = static_cast<int>(a.ld_residual);
        q.prologue = a.prologue;
        q.eps = a.norm_eps;
        q.up_chunk0 = K / 64;
        q.x_half = x_half;
        q.stage_tx = nb * q.w_box_bytes + x_bytes;
        // tc: weights and activations travel in separate rings; stage_bytes describes the weight ring
        // gemv: converted activations (576 bytes per token and box) live beside the ring, one slot per stage
        xq_stage = std::max(xq_stage, gemv ? nb * gemv * 576 : 0);
        stage_bytes = std::max(stage_bytes, tc ? q.x_off : (q.x_off + x_bytes + 1023) / 1024 * 1024);
        tile_cursor += (N + tile_rows - 1) / tile_rows;

        // weights: [k-box][row][elements of one box row]
        int rc;
        if (fmt == IZB_W_BF16) {
            const uint64_t dims[3] = {64, static_cast<uint64_t>(N), static_cast<uint64_t>(boxes_total)};
            const uint64_t strides[2] = {static_cast<uint64_t>(K) * 2, 128};
            const uint32_t box[3] = {64, static_cast<uint32_t>(tile_rows), static_cast<uint32_t>(nb)};
            rc = tma_encode(&q.tmap_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.w, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_128B);
        } else {
            const uint64_t row_bytes = fmt == IZB_W_Q8_0 ? static_cast<uint64_t>(K) / 32 * 34
                                                         : static_cast<uint64_t>(K) / 256 * 144;
            const uint32_t words = static_cast<uint32_t>(bg.w_row_bytes / 4);
            const uint64_t dims[3] = {words, static_cast<uint64_t>(N), static_cast<uint64_t>(boxes_total)};
            const uint64_t strides[2] = {row_bytes, static_cast<uint64_t>(bg.w_row_bytes)};
            const uint32_t box[3] = {words, static_cast<uint32_t>(tile_rows), static_cast<uint32_t>(nb)};
            rc = tma_encode(&q.tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, a.w, dims, strides, box,
                            CU_TENSOR_MAP_SWIZZLE_NONE);
        }
        if (rc != IZB_OK) return rc;
        // activations: [k/64][token][64 bf16]; rows past M read as zero
        {
            const uint64_t dims[3] = {64, static_cast<uint64_t>(M), static_cast<uint64_t>((silu_mul ? 2 * K : K) / 64)};
            const uint64_t strides[2] = {static_cast<uint64_t>(a.ldx) * 2, 128};
            const uint32_t box[3] = {64, static_cast<uint32_t>(x_rows), static_cast<uint32_t>(nb * (bg.kbox / 64))};
            rc = tma_encode(&q.tmap_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.x, dims, strides, box,
                            gemv ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc != IZB_OK) return rc;
        }
    }

    // A lone small projection: split the k chunks of every row tile over a cluster of CTAs, as many as
    // keep the grid within one CTA per SM (skinny_gemv.cu); each CTA then needs a ring no deeper than its share.
    int ksplit = 1, ring_cap = GV_MAX_STAGES;
    const int ksplit_max = std::min(env_int("IZB_SKINNY_GEMV_KSPLIT", 8), 8);
    if (gemv && gemv <= 2 && ctas_per_sm == 1 && ksplit_max > 1) {
        int min_chunks = INT32_MAX, max_chunks = 0;
        for (int i = 0; i < n; ++i) {
            min_chunks = std::min(min_chunks, out[i].n_chunks);
            max_chunks = std::max(max_chunks, out[i].n_chunks);
        }
        while (ksplit * 2 <= ksplit_max && ksplit * 2 <= min_chunks && tile_cursor * ksplit * 2 <= ctx->sm_count) ksplit *= 2;
        if (ksplit > 1) ring_cap = std::max(2, (max_chunks + ksplit - 1) / ksplit);
    }

    const int lite_bytes = (std::min(n, SK_LITE_MAX) * static_cast<int>(sizeof(ProbLite)) + 1023) / 1024 * 1024;
    // this region holds: tc, the four 16 KB operand slices; gemv, the converted activations of every stage;
    // otherwise the k-split partial sums
    int red_raw = tc ? 4 * 128 * 128 : ks > 1 ? (ks - 1) * rg * (rt * nt * 4) * 32 * 4 : 0;
    if (gemv) {
        int s = std::min(GV_MAX_STAGES, ring_cap);
        while (s > 2 && lite_bytes + (s * xq_stage + 1023) / 1024 * 1024 + s * stage_bytes > budget) --s;
        red_raw = s * xq_stage;
    }
    const int red_bytes = (red_raw + 1023) / 1024 * 1024;
    int n_stages = (budget - red_bytes - lite_bytes) / stage_bytes;
    int x_stages = 0;
    const int forced_stages = env_int("IZB_SKINNY_STAGES", 0);
    if (tc) {
        // two rings: raw weight boxes (released as soon as they are in registers) and activation
        // slices (released when the MMAs complete); grow them in turn while they fit
        const int x_stage = 4 * mp * 128;
        int room = budget - red_bytes - lite_bytes - 2 * stage_bytes - 2 * x_stage;
        if (room < 0) return IZB_ERR_UNSUPPORTED;
        n_stages = 2;
        x_stages = 2;
        for (bool grew = true; grew;) {
            grew = false;
            if (n_stages < std::min(4, SK_MAX_STAGES) && room >= stage_bytes) { ++n_stages; room -= stage_bytes; grew = true; }
            if (x_stages < 3 && room >= x_stage) { ++x_stages; room -= x_stage; grew = true; }
        }
        if (forced_stages) n_stages = std::min(forced_stages, n_stages);
    } else {
        if (forced_stages) n_stages = forced_stages;
        n_stages = std::min(n_stages, gemv ? std::min(GV_MAX_STAGES, ring_cap) : SK_MAX_STAGES);
        if (n_stages < 2) {
            // A single stage pair must still fit one CTA per SM.
            n_stages = 2;
            if (lite_bytes + red_bytes + 2 * stage_bytes > ctx->max_smem_optin - 2048) return IZB_ERR_UNSUPPORTED;
        }
    }

    std::memset(hdr, 0, sizeof(*hdr));
    hdr->magic = SK_PLAN_MAGIC;
    hdr->fmt = fmt;
    hdr->nt = nt;
    hdr->rt = rt;
    hdr->ks = ks;
    hdr->n_probs = n;
    hdr->total_tiles = tile_cursor;
    hdr->n_stages = n_stages;
    hdr->stage_bytes = stage_bytes;
    hdr->red_bytes = red_bytes;
    hdr->lite_bytes = lite_bytes;
    hdr->tc = tc ? 1 : 0;
    hdr->x_stages = x_stages;
    hdr->gemv = gemv;
    hdr->xq_stage_bytes = xq_stage;
    hdr->extras = any_extras ? 1 : 0;
    hdr->smem_bytes = lite_bytes + red_bytes + n_stages * stage_bytes + x_stages * 4 * mp * 128 + 1024;  // slack to align the ring to 1024 bytes
    hdr->grid = std::min(tile_cursor, max_grid);
    hdr->y_dtype = y_dtype;
    hdr->ksplit = 1;
    if (ksplit > 1) {
        hdr->ksplit = ksplit;
        hdr->grid = tile_cursor * ksplit;
        if (!skinny_gemv_clusters_fit(ctx, *hdr)) {  // the device cannot hold all clusters at once: no split
            hdr->ksplit = 1;
            hdr->grid = std::min(tile_cursor, max_grid);
        }
    }
    return IZB_OK;
}

int skinny_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev_probs,
                  const SkinnyProblem* single) {
    if (h.magic != SK_PLAN_MAGIC) return IZB_ERR_BAD_ARG;
    if (!dev_probs && !single) return IZB_ERR_BAD_ARG;
    if (h.imma) return skinny_imma_launch(ctx, stream, h, dev_probs, single);
    if (h.tc) return skinny_tc_launch(ctx, stream, h, dev_probs, single);
    if (h.gemv) return skinny_gemv_launch(ctx, stream, h, dev_probs, single);
    static const SkinnyProblem dummy = {};
    const SkinnyProblem& s = single ? *single : dummy;
    switch (h.fmt) {
        case IZB_W_BF16: return launch_fmt<IZB_W_BF16>(ctx, stream, h, dev_probs, s);
        case IZB_W_Q8_0: return launch_fmt<IZB_W_Q8_0>(ctx, stream, h, dev_probs, s);
        case IZB_W_Q4_K: return launch_fmt<IZB_W_Q4_K>(ctx, stream, h, dev_probs, s);
        default: return IZB_ERR_BAD_ARG;
    }
}

}  // namespace izb
