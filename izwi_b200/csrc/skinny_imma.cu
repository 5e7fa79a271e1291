// Block-quantised linear layers for 3..16 tokens: integer tensor-core products.
//
// The weights stay the integers they are stored as (Q8_0: int8 codes; Q4_K: 4-bit codes) and feed
// mma.sync.m16n8k32 (int8 x int8 -> int32) as the 16-row operand; the activations are re-expressed
// once per launch, by a small kernel in front of this one, as 16-bit block fixed point
// (X = round(x * 2^(14-e)), e the exponent of the 32-value block's maximum), split into a signed
// high-byte plane and an unsigned low-byte plane.  Per 32-k block and 16 x 8 (row, token) tile:
//   c  = codes . X_high             (mma, s8 x s8)
//   c  = (c << 8) + codes . X_low   (mma, s8 x u8, accumulating)
//   acc += float(c) * d_row * 2^(e-14)
// which costs about two instructions per weight for 8 tokens and three for 16, against three to four
// for lifting every code to a floating-point operand; the sums are exact in int32.
//
// Layout of the converted activations (global memory, then one bulk copy per pipeline stage):
// per 32-k block [high plane: MP tokens x 32 bytes][low plane: MP x 32][2^(e-14): MP floats]
// [2^(e-14) * sum of X: MP floats], MP = 8 or 16.  Inside a token's 32 bytes the values sit in the order
// the weight fragments come out of shared memory without shuffles (see imma_convert_kernel).
//
// Tile = 64 weight rows; the 4 consumer warps split the k of every 256-k box between them (each byte of a
// stage is read from shared memory once) and add their sums up when the tile ends.  One more warp issues
// the copies: the tiled weight copies of its first stages go out before the wait on the kernel in front,
// since weights depend on nobody.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "skinny.cuh"
#include "tma.cuh"

namespace izb {

constexpr int IM_CONSUMER_WARPS = 4;
constexpr int IM_THREADS = 32 * (IM_CONSUMER_WARPS + 1);
constexpr int IM_TILE_ROWS = 64;
constexpr int IM_MAX_STAGES = 8;
constexpr int IM_BLOCK_BYTES_PER_TOKEN = 72;  // 32 high bytes, 32 low bytes, scale, scaled sum

struct ImShared {
    unsigned long long full[IM_MAX_STAGES];
    unsigned long long empty[IM_MAX_STAGES];
    int abort_flag;
};

// ---------------------------------------------------------------------------
// Activations -> block fixed point.  One warp per (token, 256-k box); lane = 8 consecutive values,
// the four lanes of a 32-value block agree on its exponent by shuffle.
//
// Order inside a token's 32 bytes ("position words" P0..P7, four values each):
//   odd blocks of a Q8_0 row:  Pj = values 4j .. 4j+3.
//   Q4_K: a thread's fragment registers hold code bytes 4t..4t+3 and 16+4t..16+4t+3 of a sub-block (ldmatrix),
//   so P(2t) = values 4t .. 4t+3 and P(2t+1) = values 16+4t .. 16+4t+3.
//   even blocks of a Q8_0 row: the block's 32 codes start two bytes into a word (behind the fp16 scale),
//   so its aligned words hold codes (0,1) | 2..5 | 6..9 | ... | 26..29 | (30,31); the consumer glues the
//   two halves into one word and takes the rest as they are: P0 = values (0,1,30,31), Pj = 4j-2 .. 4j+1.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    imma_convert_kernel(const SkinnyProblem* __restrict__ probs, const __grid_constant__ SkinnyProblem single, int fmt, int mp) {
    pdl_launch_dependents();
    pdl_wait();
    const SkinnyProblem& P = probs ? probs[blockIdx.y] : single;
    const int lane = threadIdx.x & 31;
    const int boxes = P.K / 256;
    const int items = mp * boxes;
    const int warps_per_grid = static_cast<int>(gridDim.x) * 8;
    for (int it = static_cast<int>(blockIdx.x) * 8 + (threadIdx.x >> 5); it < items; it += warps_per_grid) {
        const int m = it % mp, box = it / mp;
        const int blk = box * 8 + (lane >> 2), u = lane & 3;  // 32-value block of the row, 8-value unit inside it
        uint8_t* dst = P.xq + static_cast<size_t>(blk) * (IM_BLOCK_BYTES_PER_TOKEN * mp);
        uint32_t hi[2] = {0, 0}, lo[2] = {0, 0};
        float xs = 0.f, sx = 0.f;
        if (m < P.M) {
            const uint4 v = *reinterpret_cast<const uint4*>(P.x_rows + static_cast<size_t>(m) * P.ldx + box * 256 + lane * 8);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t amax = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) amax = max(amax, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
            amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
            amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
            const uint32_t eb = amax >> 7;  // biased exponent of the block maximum
            // X = x * 2^(14-e) rounds into [-32640, 32640]; blocks below 2^-111 count as zero, Inf / NaN poison the scale
            const float sf = (eb >= 16u && eb < 255u) ? __uint_as_float((268u - eb) << 23) : 0.f;
            xs = eb == 255u ? __uint_as_float(0x7FC00000u) : eb >= 16u ? __uint_as_float((eb - 14u) << 23) : 0.f;
            int X[8], isum = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                X[2 * i] = __float2int_rn(__uint_as_float(w[i] << 16) * sf);
                X[2 * i + 1] = __float2int_rn(__uint_as_float(w[i] & 0xFFFF0000u) * sf);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) isum += X[i];
            isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 1);
            isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 2);
            sx = xs * static_cast<float>(isum);
            // bytes 0 (low) and 1 (high) of four values each into one word per plane
            const uint32_t u0 = prmt(X[0], X[1], 0x5140), v0 = prmt(X[2], X[3], 0x5140);
            const uint32_t u1 = prmt(X[4], X[5], 0x5140), v1 = prmt(X[6], X[7], 0x5140);
            hi[0] = prmt(u0, v0, 0x7632); hi[1] = prmt(u1, v1, 0x7632);
            lo[0] = prmt(u0, v0, 0x5410); lo[1] = prmt(u1, v1, 0x5410);
        }
        // the second word of the unit before this one; unit 0 takes unit 3's (values 28..31)
        const int from = (lane & ~3) | ((u + 3) & 3);
        const uint32_t ph = __shfl_sync(0xFFFFFFFFu, hi[1], from), pl = __shfl_sync(0xFFFFFFFFu, lo[1], from);
        if (fmt == IZB_W_Q8_0 && ((lane >> 2) & 1) == 0) {
            // even block: natural words N(2u), N(2u+1) -> position words P(2u), P(2u+1)
            const uint32_t h1 = prmt(hi[0], hi[1], 0x5432), l1 = prmt(lo[0], lo[1], 0x5432);
            hi[0] = u == 0 ? prmt(hi[0], ph, 0x7610) : prmt(ph, hi[0], 0x5432);
            lo[0] = u == 0 ? prmt(lo[0], pl, 0x7610) : prmt(pl, lo[0], 0x5432);
            hi[1] = h1;
            lo[1] = l1;
        }
        if (fmt == IZB_W_Q8_0) {
            *reinterpret_cast<uint2*>(dst + m * 32 + u * 8) = make_uint2(hi[0], hi[1]);
            *reinterpret_cast<uint2*>(dst + mp * 32 + m * 32 + u * 8) = make_uint2(lo[0], lo[1]);
        } else {
            // natural word j -> position word 2j (j < 4) or 2(j - 4) + 1: this lane holds words 2u and 2u + 1
            const int p0 = u < 2 ? 4 * u : 4 * u - 7, p1 = u < 2 ? 4 * u + 2 : 4 * u - 5;
            uint32_t* hp = reinterpret_cast<uint32_t*>(dst + m * 32);
            uint32_t* lp = reinterpret_cast<uint32_t*>(dst + mp * 32 + m * 32);
            hp[p0] = hi[0]; hp[p1] = hi[1];
            lp[p0] = lo[0]; lp[p1] = lo[1];
        }
        if (u == 0) {
            *reinterpret_cast<float*>(dst + mp * 64 + m * 4) = xs;
            *reinterpret_cast<float*>(dst + mp * 68 + m * 4) = sx;
        }
    }
}

// ---------------------------------------------------------------------------
// The consumers split k: warp w takes 32-k blocks 2w and 2w + 1 of every 256-k box for all 64 rows of
// the tile (four 16-row operand tiles), so every byte of the stage is read from shared memory once.
// g = lane / 4 (rows g and g + 8 of an operand tile; token g of a group), t = lane % 4.
// ---------------------------------------------------------------------------
constexpr uint32_t IM_MAGIC = 0x4B400000u;  // 1.5 * 2^23: as an accumulator's start value it makes the int32 sum v
constexpr float IM_MAGIC_F = 12582912.0f;   // read back, as a float, 1.5 * 2^23 + v exactly for |v| < 2^22

// D(16x8, s32) = A(16x32) * B(32x8) + IM_MAGIC
template <bool A_SIGNED, bool B_SIGNED>
__device__ __forceinline__ void mma_i8_magic(uint32_t (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (A_SIGNED && B_SIGNED)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(IM_MAGIC));
    else if constexpr (A_SIGNED && !B_SIGNED)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(IM_MAGIC));
    else if constexpr (!A_SIGNED && B_SIGNED)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(IM_MAGIC));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(IM_MAGIC));
}

// codes . (256 * X_high + X_low) of one 32-k block as a float (both partial sums are below 2^22 in magnitude)
template <bool A_SIGNED>
__device__ __forceinline__ void im_block_dot(float (&f)[4], const uint32_t (&a)[4], uint2 bh, uint2 bl) {
    uint32_t ch[4], cl[4];
    mma_i8_magic<A_SIGNED, true>(ch, a, bh.x, bh.y);
    mma_i8_magic<A_SIGNED, false>(cl, a, bl.x, bl.y);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = fmaf(__uint_as_float(ch[i]) - IM_MAGIC_F, 256.0f, __uint_as_float(cl[i]) - IM_MAGIC_F);
}

// The activations of one 32-k block for this thread: both planes of token g and the scales of tokens 2t, 2t + 1, per group.
template <int NG>
struct ImB {
    uint2 bh[NG], bl[NG], xs[NG], sx[NG];
};
template <int NG, bool WITH_SUMS>
__device__ __forceinline__ void im_load_b(ImB<NG>& B, uint32_t xb, int mp, int g, int t) {
#pragma unroll
    for (int n = 0; n < NG; ++n) {
        const uint32_t tok = static_cast<uint32_t>((8 * n + g) * 32 + 8 * t);
        B.bh[n] = lds64(xb + tok);
        B.bl[n] = lds64(xb + static_cast<uint32_t>(32 * mp) + tok);
        B.xs[n] = lds64(xb + static_cast<uint32_t>(64 * mp + (8 * n + 2 * t) * 4));
        if (WITH_SUMS) B.sx[n] = lds64(xb + static_cast<uint32_t>(68 * mp + (8 * n + 2 * t) * 4));
    }
}

// Q8_0: blocks 2w, 2w + 1 (the 68 bytes from byte 68 w of a 272-byte box row) of the 64 rows.
template <int NG>
__device__ __forceinline__ void im_box_q8_0(float (&acc)[4][NG][4], uint32_t box, uint32_t xq_box, int blk_bytes, int mp, int w,
                                            int g, int t) {
    ImB<NG> B[2];
    im_load_b<NG, false>(B[0], xq_box + static_cast<uint32_t>((2 * w) * blk_bytes), mp, g, t);
    im_load_b<NG, false>(B[1], xq_box + static_cast<uint32_t>((2 * w + 1) * blk_bytes), mp, g, t);
    // every load of this warp's share of the box first (they issue in program order), then the products
    uint32_t a[4][2][4];  // [operand tile][block][fragment register: (row g, word 0), (g + 8, word 0), (g, word 1), (g + 8, word 1)]
    float d[4][2][2];     // [operand tile][block][row]
#pragma unroll
    for (int rt = 0; rt < 4; ++rt) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t row = box + static_cast<uint32_t>((16 * rt + g + 8 * r) * 272 + 68 * w);
            const uint32_t e0 = lds32(row), e8 = lds32(row + 32);
            const uint32_t w0 = lds32(row + static_cast<uint32_t>(8 * t)), w1 = lds32(row + static_cast<uint32_t>(8 * t + 4));
            a[rt][0][r] = t == 0 ? prmt(e0, e8, 0x5432) : w0;  // codes (0, 1, 30, 31) glued from the two half words
            a[rt][0][2 + r] = w1;
            a[rt][1][r] = lds32(row + static_cast<uint32_t>(36 + 8 * t));
            a[rt][1][2 + r] = lds32(row + static_cast<uint32_t>(40 + 8 * t));
            d[rt][0][r] = half_bits_to_f32(e0);
            d[rt][1][r] = half_bits_to_f32(e8 >> 16);
        }
    }
#pragma unroll
    for (int rt = 0; rt < 4; ++rt) {
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
            for (int n = 0; n < NG; ++n) {
                float f[4];
                im_block_dot<true>(f, a[rt][b], B[b].bh[n], B[b].bl[n]);
                const float x0 = __uint_as_float(B[b].xs[n].x), x1 = __uint_as_float(B[b].xs[n].y);
                acc[rt][n][0] = fmaf(f[0], d[rt][b][0] * x0, acc[rt][n][0]);
                acc[rt][n][1] = fmaf(f[1], d[rt][b][0] * x1, acc[rt][n][1]);
                acc[rt][n][2] = fmaf(f[2], d[rt][b][1] * x0, acc[rt][n][2]);
                acc[rt][n][3] = fmaf(f[3], d[rt][b][1] * x1, acc[rt][n][3]);
            }
        }
    }
}

// 6-bit scale and minimum of sub-block s from the 12 packed bytes (words y, z, w of the super-block header)
__device__ __forceinline__ void q4k_scale_min(uint32_t y, uint32_t z, uint32_t w, int s, int& sc, int& mn) {
    if (s < 4) {
        sc = static_cast<int>((y >> (8 * s)) & 63u);
        mn = static_cast<int>((z >> (8 * s)) & 63u);
    } else {
        const int sh = 8 * (s - 4);
        sc = static_cast<int>(((w >> sh) & 0xFu) | (((y >> (sh + 6)) & 3u) << 4));
        mn = static_cast<int>(((w >> (sh + 4)) & 0xFu) | (((z >> (sh + 6)) & 3u) << 4));
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Q4_K: code group w (32 bytes: low nibbles = sub-block 2w, high nibbles = 2w + 1) of the 64 rows' 144-byte super-blocks.
template <int NG>
__device__ __forceinline__ void im_box_q4_k(float (&acc)[4][NG][4], uint32_t box, uint32_t xq_box, int blk_bytes, int mp, int w,
                                            int g, int t, int lane) {
    ImB<NG> B[2];
    im_load_b<NG, true>(B[0], xq_box + static_cast<uint32_t>((2 * w) * blk_bytes), mp, g, t);
    im_load_b<NG, true>(B[1], xq_box + static_cast<uint32_t>((2 * w + 1) * blk_bytes), mp, g, t);
    // ldmatrix: lane i names row i % 8 of 8x16-byte matrix i / 8: rows 0-7 / 8-15 of the operand tile, first / second 16 code bytes
    const uint32_t lm_off = static_cast<uint32_t>((((lane >> 3) & 1) * 8 + (lane & 7)) * 144 + 16 + 32 * w + (lane >> 4) * 16);
    uint32_t q[4][4];
    uint4 hd[4][2];
#pragma unroll
    for (int rt = 0; rt < 4; ++rt) {
        ldmatrix_x4(q[rt], box + static_cast<uint32_t>(16 * rt * 144) + lm_off);
#pragma unroll
        for (int r = 0; r < 2; ++r) hd[rt][r] = lds128(box + static_cast<uint32_t>((16 * rt + g + 8 * r) * 144));
    }
#pragma unroll
    for (int rt = 0; rt < 4; ++rt) {
        float dsc[2][2], dmn[2][2];  // [sub-block of the pair][row]
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float d = half_bits_to_f32(hd[rt][r].x), dmin = half_bits_to_f32(hd[rt][r].x >> 16);
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                int sc, mn;
                q4k_scale_min(hd[rt][r].y, hd[rt][r].z, hd[rt][r].w, 2 * w + b, sc, mn);
                dsc[b][r] = d * (__uint_as_float(IM_MAGIC + static_cast<uint32_t>(sc)) - IM_MAGIC_F);  // the 6-bit integers, lifted exactly
                dmn[b][r] = dmin * (__uint_as_float(IM_MAGIC + static_cast<uint32_t>(mn)) - IM_MAGIC_F);
            }
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            uint32_t a[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = (b ? q[rt][i] >> 4 : q[rt][i]) & 0x0F0F0F0Fu;
#pragma unroll
            for (int n = 0; n < NG; ++n) {
                float f[4];
                im_block_dot<false>(f, a, B[b].bh[n], B[b].bl[n]);
                const float x0 = __uint_as_float(B[b].xs[n].x), x1 = __uint_as_float(B[b].xs[n].y);
                const float s0 = __uint_as_float(B[b].sx[n].x), s1 = __uint_as_float(B[b].sx[n].y);
                acc[rt][n][0] = fmaf(f[0], dsc[b][0] * x0, fmaf(-dmn[b][0], s0, acc[rt][n][0]));
                acc[rt][n][1] = fmaf(f[1], dsc[b][0] * x1, fmaf(-dmn[b][0], s1, acc[rt][n][1]));
                acc[rt][n][2] = fmaf(f[2], dsc[b][1] * x0, fmaf(-dmn[b][1], s0, acc[rt][n][2]));
                acc[rt][n][3] = fmaf(f[3], dsc[b][1] * x1, fmaf(-dmn[b][1], s1, acc[rt][n][3]));
            }
        }
    }
}

// Walks the (tile, chunk) items of one CTA in launch order.
struct ImItems {
    const ProbLite* lite;
    const SkinnyProblem* plist;
    int n_cached, n_probs, total_tiles, tile_step;
    int tile, c, p;
    ProbLite L;
    __device__ __forceinline__ void load() {
        if (tile < total_tiles) {
            p = find_problem(lite, n_cached, plist, n_probs, tile);
            L = p < n_cached ? lite[p] : lite_from(plist[p]);
        }
    }
    __device__ __forceinline__ void start(int first) {
        tile = first;
        c = 0;
        load();
    }
    __device__ __forceinline__ bool valid() const { return tile < total_tiles; }
    __device__ __forceinline__ void next() {
        if (++c == L.n_chunks) {
            c = 0;
            tile += tile_step;
            load();
        }
    }
};

template <int FMT, int NG>
__global__ void __launch_bounds__(IM_THREADS)
    skinny_imma_kernel(const SkinnyProblem* __restrict__ probs, const __grid_constant__ SkinnyProblem single, int n_probs,
                       int total_tiles, int n_stages, int stage_bytes, int lite_bytes, int y_dtype, int* status) {
    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    __shared__ ImShared sh;
    constexpr int MP = 8 * NG;
    constexpr int BLK = IM_BLOCK_BYTES_PER_TOKEN * MP;  // converted activations of one 32-k block
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const SkinnyProblem* plist = probs ? probs : &single;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.empty[s]), IM_CONSUMER_WARPS);
        }
        sh.abort_flag = 0;
        mbar_fence_init();
    }
    ProbLite* lite = reinterpret_cast<ProbLite*>(dyn_smem);
    const int n_cached = min(n_probs, lite_bytes / static_cast<int>(sizeof(ProbLite)));
    for (int i = threadIdx.x; i < n_cached; i += blockDim.x) lite[i] = lite_from(plist[i]);  // the plan: written by the host
    __syncthreads();

    volatile int* abort_flag = &sh.abort_flag;
    const uint32_t stage0 = smem_u32(dyn_smem) + static_cast<uint32_t>(lite_bytes);

    if (warp == IM_CONSUMER_WARPS) {
        // ---------------- producer ----------------
        if (lane != 0) return;
        ImItems it{lite, plist, n_cached, n_probs, total_tiles, static_cast<int>(gridDim.x), 0, 0, 0, {}};
        // weights of the first ring-full of stages: nobody writes them, so they need not wait for the kernel in front
        int pre = 0, last_p = -1;
        for (it.start(static_cast<int>(blockIdx.x)); it.valid() && pre < n_stages; it.next(), ++pre) {
            const SkinnyProblem* P = plist + it.p;
            if (it.p != last_p && probs) tma_fence_descriptor(&P->tmap_w);
            last_p = it.p;
            const uint32_t fbar = smem_u32(&sh.full[pre]);
            mbar_expect_tx(fbar, static_cast<uint32_t>(it.L.stage_tx));
            tma_load_3d(stage0 + static_cast<uint32_t>(pre) * static_cast<uint32_t>(stage_bytes), &P->tmap_w, 0,
                        (it.tile - it.L.tile_start) * IM_TILE_ROWS, it.c * it.L.nb, fbar);
        }
        pdl_wait();  // the converted activations come from the kernel in front
        int stage = 0;
        uint32_t phase = 0;
        long long issued = 0;
        bool ok = true;
        last_p = -1;
        for (it.start(static_cast<int>(blockIdx.x)); it.valid(); it.next()) {
            const SkinnyProblem* P = plist + it.p;
            const uint32_t fbar = smem_u32(&sh.full[stage]);
            const uint32_t sbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
            if (issued >= pre) {
                if (!mbar_wait_bounded(smem_u32(&sh.empty[stage]), phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                if (it.p != last_p && probs) tma_fence_descriptor(&P->tmap_w);
                mbar_expect_tx(fbar, static_cast<uint32_t>(it.L.stage_tx));
                tma_load_3d(sbase, &P->tmap_w, 0, (it.tile - it.L.tile_start) * IM_TILE_ROWS, it.c * it.L.nb, fbar);
            }
            last_p = it.p;
            const uint32_t xq_bytes = static_cast<uint32_t>(it.L.nb * 8 * BLK);
            bulk_g2s(sbase + static_cast<uint32_t>(it.L.x_off), P->xq + static_cast<size_t>(it.c) * xq_bytes, xq_bytes, fbar);
            ++issued;
            if (++stage == n_stages) {
                stage = 0;
                phase ^= 1u;
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
            atomicExch(status, 5);
        }
        return;
    }

    // ---------------- consumers: warp w takes blocks 2w, 2w + 1 of every box, all 64 rows ----------------
    pdl_wait();
    const int g = lane >> 2, t = lane & 3;
    float* red = reinterpret_cast<float*>(dyn_smem + lite_bytes + n_stages * stage_bytes);  // [warp][operand tile][NG * 4][lane]
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = static_cast<int>(blockIdx.x); tile < total_tiles; tile += static_cast<int>(gridDim.x)) {
        const int p = find_problem(lite, n_cached, plist, n_probs, tile);
        const ProbLite L = p < n_cached ? lite[p] : lite_from(plist[p]);
        float acc[4][NG][4];
#pragma unroll
        for (int rt = 0; rt < 4; ++rt)
#pragma unroll
            for (int n = 0; n < NG; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[rt][n][i] = 0.f;
        for (int c = 0; c < L.n_chunks; ++c) {
            if (ok && !mbar_wait_bounded(smem_u32(&sh.full[stage]), phase, abort_flag)) ok = false;
            if (ok) {
                const uint32_t sbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                for (int b = 0; b < L.nb; ++b) {
                    const uint32_t box = sbase + static_cast<uint32_t>(b * L.w_box_bytes);
                    const uint32_t xq_box = sbase + static_cast<uint32_t>(L.x_off + b * 8 * BLK);
                    if constexpr (FMT == IZB_W_Q8_0) im_box_q8_0<NG>(acc, box, xq_box, BLK, MP, warp, g, t);
                    else im_box_q4_k<NG>(acc, box, xq_box, BLK, MP, warp, g, t, lane);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.empty[stage]));
            if (++stage == n_stages) {
                stage = 0;
                phase ^= 1u;
            }
        }
        // every warp parks its share of k; warp w then sums and stores operand tile w
        named_bar_sync(1, IM_CONSUMER_WARPS * 32);  // the sums of the tile before this one have been read
#pragma unroll
        for (int rt = 0; rt < 4; ++rt)
#pragma unroll
            for (int n = 0; n < NG; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) red[((warp * 4 + rt) * NG * 4 + n * 4 + i) * 32 + lane] = acc[rt][n][i];
        named_bar_sync(1, IM_CONSUMER_WARPS * 32);
        if (ok) {
            // sum[n][0..3] = (row g, token 8n + 2t), (g, 2t + 1), (g + 8, 2t), (g + 8, 2t + 1) of operand tile `warp`
            const int row0 = (tile - L.tile_start) * IM_TILE_ROWS + warp * 16;
            const __nv_bfloat16* residual = L.extras ? plist[p].residual : nullptr;
            const int ld_res = residual ? plist[p].ld_res : 0;
#pragma unroll
            for (int n = 0; n < NG; ++n) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float v = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < IM_CONSUMER_WARPS; ++w2) v += red[((w2 * 4 + warp) * NG * 4 + n * 4 + i) * 32 + lane];
                    const int grow = row0 + g + 8 * (i >> 1), tok = 8 * n + 2 * t + (i & 1);
                    if (grow >= L.N || tok >= L.M) continue;
                    v += L.bias ? __bfloat162float(L.bias[grow]) : 0.f;
                    if (residual) v += __bfloat162float(residual[static_cast<long long>(tok) * ld_res + grow]);
                    store_typed(L.y, y_dtype, static_cast<long long>(tok) * L.ldy + grow, v);
                }
            }
        }
    }
    if (!ok && lane == 0) atomicExch(status, 5);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace {
int im_env_int(const char* name, int fallback) {
    const char* e = std::getenv(name);
    return (e && *e) ? std::atoi(e) : fallback;
}
}  // namespace

// Where the kernel is the default, from measurement on the Qwen3-0.6B projection stack: Q8_0 weights and
// 3..8 tokens (0.85 of the HBM copy rate against 0.78 for the floating-point mma.sync consumers).  With 9..16
// tokens, and over Q4_K weights at any count, the older kernels are faster (the per-block float epilogue
// grows with the token count; a Q4_K byte carries twice the weights): those variants stay reachable
// through the two variables below and are covered by the tests.
int skinny_imma_min_tokens() { return std::max(2, im_env_int("IZB_SKINNY_IMMA_MIN_M", 3)); }
int skinny_imma_max_tokens() { return std::min(16, im_env_int("IZB_SKINNY_IMMA_MAX_M", 8)); }
bool skinny_imma_format_ok(int fmt) { return fmt == IZB_W_Q8_0 || (fmt == IZB_W_Q4_K && im_env_int("IZB_SKINNY_IMMA_Q4_K", 0) != 0); }

size_t skinny_imma_xq_bytes(int64_t M, int64_t K) {
    if (M <= 0 || M > 16 || K <= 0 || K % 256 != 0) return 0;
    const size_t mp = M <= 8 ? 8 : 16;
    return static_cast<size_t>(K / 32) * IM_BLOCK_BYTES_PER_TOKEN * mp;
}

bool skinny_imma_takes(const izb_linear_args* probs, int n) {
    if (n <= 0) return false;
    const int fmt = probs[0].wfmt;
    if (!skinny_imma_format_ok(fmt)) return false;
    int64_t max_m = 0;
    for (int i = 0; i < n; ++i) {
        const izb_linear_args& a = probs[i];
        if (a.prologue != IZB_PRO_NONE || a.K % 256 != 0 || a.M <= 0 || a.M > 16) return false;
        if (!a.workspace || !izb_aligned(a.workspace, 16) || a.workspace_bytes < skinny_imma_xq_bytes(16, a.K)) return false;
        max_m = std::max<int64_t>(max_m, a.M);
    }
    return max_m >= skinny_imma_min_tokens() && max_m <= skinny_imma_max_tokens();
}

static int ring_lite_bytes(int n) { return (std::min(n, SK_LITE_MAX) * static_cast<int>(sizeof(ProbLite)) + 1023) / 1024 * 1024; }
static int ring_red_bytes(int ng) { return IM_CONSUMER_WARPS * 4 * ng * 4 * 32 * 4; }  // every consumer warp's sums of a tile
// Shared memory left for the stage ring of one CTA when `ctas_per_sm` share an SM.
static int budget_for_ring(const izb_ctx* ctx, int ctas_per_sm, int n, int ng) {
    return ctx->max_smem_optin / ctas_per_sm - 2048 - static_cast<int>(sizeof(ImShared)) - ring_lite_bytes(n) - ring_red_bytes(ng) - 1024;
}

// Fills the plan for the integer tensor-core kernel; the arguments were validated by the caller.
int skinny_imma_plan_build(const izb_ctx* ctx, const izb_linear_args* probs, int n, SkinnyPlanHeader* hdr, SkinnyProblem* out) {
    const int fmt = probs[0].wfmt;
    int64_t max_m = 0;
    for (int i = 0; i < n; ++i) max_m = std::max<int64_t>(max_m, probs[i].M);
    const int ng = max_m <= 8 ? 1 : 2, mp = 8 * ng;
    const int w_row_bytes = fmt == IZB_W_Q8_0 ? 272 : 144;
    const int w_box_bytes = IM_TILE_ROWS * w_row_bytes;
    const int xq_box = 8 * IM_BLOCK_BYTES_PER_TOKEN * mp;
    // two CTAs per SM measured best (a third leaves each a ring too shallow); fewer when two stages of one box do not fit
    int ctas_per_sm = std::max(1, std::min(4, im_env_int("IZB_IMMA_CTAS_PER_SM", 2)));
    while (ctas_per_sm > 1 && budget_for_ring(ctx, ctas_per_sm, n, ng) < 2 * (w_box_bytes + xq_box + 1024)) --ctas_per_sm;
    const int lite_bytes = ring_lite_bytes(n), red_bytes = ring_red_bytes(ng);
    const int budget = budget_for_ring(ctx, ctas_per_sm, n, ng);
    int stage_target = std::max(8, im_env_int("IZB_IMMA_STAGE_KB", 28)) * 1024;
    // a stage target that leaves no room for two stages shrinks to the largest that does (never below one box)
    stage_target = std::max(w_box_bytes + xq_box, std::min(stage_target, budget_for_ring(ctx, ctas_per_sm, n, ng) / 2 - 1024));

    int stage_bytes = 0, tile_cursor = 0;
    for (int i = 0; i < n; ++i) {
        const izb_linear_args& a = probs[i];
        SkinnyProblem& q = out[i];
        std::memset(&q, 0, sizeof(q));
        const int K = static_cast<int>(a.K), N = static_cast<int>(a.N);
        const int boxes_total = K / 256;
        int nb = std::max(1, std::min(boxes_total, stage_target / (w_box_bytes + xq_box)));
        while (nb > 1 && boxes_total % nb != 0) --nb;
        q.y = a.y;
        q.bias = static_cast<const __nv_bfloat16*>(a.bias);
        q.N = N; q.K = K; q.M = static_cast<int>(a.M);
        q.ldy = static_cast<int>(a.ldy);
        q.tile_start = tile_cursor;
        q.nb = nb;
        q.kbox = 256;
        q.n_chunks = boxes_total / nb;
        q.w_row_bytes = w_row_bytes;
        q.w_box_bytes = w_box_bytes;
        q.x_off = (nb * w_box_bytes + 127) / 128 * 128;
        q.stage_tx = nb * w_box_bytes + nb * xq_box;
        q.residual = static_cast<const __nv_bfloat16*>(a.residual);
        q.ld_res = static_cast<int>(a.ld_residual);
        q.xq = static_cast<uint8_t*>(a.workspace);
        q.x_rows = static_cast<const __nv_bfloat16*>(a.x);
        q.ldx = static_cast<int>(a.ldx);
        stage_bytes = std::max(stage_bytes, (q.x_off + nb * xq_box + 1023) / 1024 * 1024);
        tile_cursor += (N + IM_TILE_ROWS - 1) / IM_TILE_ROWS;

        const uint64_t row_bytes = fmt == IZB_W_Q8_0 ? static_cast<uint64_t>(K) / 32 * 34 : static_cast<uint64_t>(K) / 256 * 144;
        const uint32_t words = static_cast<uint32_t>(w_row_bytes / 4);
        const uint64_t dims[3] = {words, static_cast<uint64_t>(N), static_cast<uint64_t>(boxes_total)};
        const uint64_t strides[2] = {row_bytes, static_cast<uint64_t>(w_row_bytes)};
        const uint32_t box[3] = {words, static_cast<uint32_t>(IM_TILE_ROWS), static_cast<uint32_t>(nb)};
        const int rc = tma_encode(&q.tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, a.w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != IZB_OK) return rc;
    }
    int n_stages = std::min(IM_MAX_STAGES, budget / stage_bytes);
    const int forced = im_env_int("IZB_IMMA_STAGES", 0);
    if (forced) n_stages = std::min(forced, n_stages);
    if (n_stages < 2) return IZB_ERR_UNSUPPORTED;

    std::memset(hdr, 0, sizeof(*hdr));
    hdr->magic = SK_PLAN_MAGIC;
    hdr->fmt = fmt;
    hdr->nt = ng;
    hdr->rt = 1;
    hdr->ks = 1;
    hdr->n_probs = n;
    hdr->total_tiles = tile_cursor;
    hdr->n_stages = n_stages;
    hdr->stage_bytes = stage_bytes;
    hdr->lite_bytes = lite_bytes;
    hdr->imma = ng;
    hdr->ksplit = 1;
    hdr->smem_bytes = lite_bytes + n_stages * stage_bytes + red_bytes + 1024;
    hdr->grid = std::min(tile_cursor, ctx->sm_count * ctas_per_sm);
    hdr->y_dtype = probs[0].y_dtype;
    int max_items = 0;
    for (int i = 0; i < n; ++i) max_items = std::max(max_items, mp * out[i].K / 256);
    hdr->conv_grid = std::max(1, std::min((max_items + 7) / 8, 64));
    return IZB_OK;
}

template <int FMT, int NG>
static int imma_launch_one(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
                           const SkinnyProblem& single) {
    auto kern = skinny_imma_kernel<FMT, NG>;
    static std::atomic<int> smem_set[IZB_MAX_DEVICES];
    if (smem_set[ctx->device].load(std::memory_order_relaxed) < h.smem_bytes) {
        IZB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem_bytes));
        smem_set[ctx->device].store(h.smem_bytes, std::memory_order_relaxed);
    }
    IZB_CUDA_TRY(launch_chained(ctx, imma_convert_kernel, dim3(h.conv_grid, h.n_probs), dim3(256), 0, stream, dev, single, h.fmt, 8 * NG));
    IZB_CUDA_TRY(launch_chained(ctx, kern, dim3(h.grid), dim3(IM_THREADS), h.smem_bytes, stream, dev, single, h.n_probs, h.total_tiles,
                                h.n_stages, h.stage_bytes, h.lite_bytes, h.y_dtype, ctx->d_status + 4));
    ctx->launches.fetch_add(2, std::memory_order_relaxed);
    return IZB_OK;
}

int skinny_imma_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev_probs,
                       const SkinnyProblem* single) {
    if (h.magic != SK_PLAN_MAGIC || h.imma < 1 || h.imma > 2) return IZB_ERR_BAD_ARG;
    if (!dev_probs && !single) return IZB_ERR_BAD_ARG;
    static const SkinnyProblem dummy = {};
    const SkinnyProblem& s = single ? *single : dummy;
    if (h.fmt == IZB_W_Q8_0)
        return h.imma == 1 ? imma_launch_one<IZB_W_Q8_0, 1>(ctx, stream, h, dev_probs, s) : imma_launch_one<IZB_W_Q8_0, 2>(ctx, stream, h, dev_probs, s);
    if (h.fmt == IZB_W_Q4_K)
        return h.imma == 1 ? imma_launch_one<IZB_W_Q4_K, 1>(ctx, stream, h, dev_probs, s) : imma_launch_one<IZB_W_Q4_K, 2>(ctx, stream, h, dev_probs, s);
    return IZB_ERR_BAD_ARG;
}

}  // namespace izb
