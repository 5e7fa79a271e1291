// Integer dot products of block-quantised weight rows against activations in 16-bit block fixed
// point: the device functions shared by the kernels that keep the weight codes integers
// (skinny_gemv.cu: one launch per projection group; decode_token.cu: one launch per token).
//
// Each 32-value block of the activations is X = round(x * 2^(14-e)), e the exponent of the block
// maximum, split into a signed high byte and an unsigned low byte; a 256-k box of one token is
// [256 high bytes][256 low bytes][8 block scales 2^(e-14)][8 scaled block sums] = GV_XQ_BYTES.
#pragma once

#include "skinny.cuh"

namespace izb {

// converted activations of one token and one 256-k box: high bytes, low bytes, 8 block scales, 8 block sums
constexpr int GV_XQ_BYTES = 256 + 256 + 32 + 32;
constexpr int GV_XQ_XL = 256, GV_XQ_XS = 512, GV_XQ_SX = 544;

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(static_cast<uint32_t>(c)));
    return static_cast<int>(d);
}
__device__ __forceinline__ void sts64v(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.b32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts32f(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float lds32f(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// 1 / x to within one ulp on the special-function unit (an IEEE division costs some twenty instructions,
// and the single converting warp does eight per lane and stage); 1 / inf = 0.
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// Exact int32 -> fp32 for |v| < 2^22 on the integer and fp32 pipes (the conversion unit runs at a
// quarter of their rate): 1.5 * 2^23 + v is representable, so its bit pattern is the magic's plus v.
__device__ __forceinline__ float small_int_to_f32(int v) {
    return __int_as_float(0x4B400000 + v) - 12582912.0f;
}

// Eight fixed-point values of one lane -> the two byte planes, plus (one lane in four) the block's
// scale and scaled sum.
__device__ __forceinline__ void gv_store_unit(const int (&X)[8], float xs, uint32_t dst, int lane) {
    int isum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) isum += X[i];
    isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 1);
    isum += __shfl_xor_sync(0xFFFFFFFFu, isum, 2);
    // bytes 0 (low) and 1 (high) of four values each into one word per plane
    const uint32_t u0 = prmt(X[0], X[1], 0x5140), v0 = prmt(X[2], X[3], 0x5140);
    const uint32_t u1 = prmt(X[4], X[5], 0x5140), v1 = prmt(X[6], X[7], 0x5140);
    sts64v(dst + static_cast<uint32_t>(8 * lane), prmt(u0, v0, 0x7632), prmt(u1, v1, 0x7632));
    sts64v(dst + static_cast<uint32_t>(GV_XQ_XL + 8 * lane), prmt(u0, v0, 0x5410), prmt(u1, v1, 0x5410));
    if ((lane & 3) == 0) {
        sts32f(dst + static_cast<uint32_t>(GV_XQ_XS + lane), xs);  // block lane/4: 4 bytes each
        sts32f(dst + static_cast<uint32_t>(GV_XQ_SX + lane), xs * static_cast<float>(isum));
    }
}

// One lane's share of the conversion: 8 consecutive activations (one 16-byte unit) of one token;
// the four lanes of a 32-value block agree on the block exponent by shuffle.
__device__ __forceinline__ void gv_convert_unit(const uint4 v, uint32_t dst, int lane) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t amax = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) amax = max(amax, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const uint32_t eb = amax >> 7;  // biased exponent of the block maximum
    // X = x * 2^(14-e) rounds into [-32640, 32640]; blocks below 2^-111 count as zero, Inf/NaN poison the scale
    const float sf = (eb >= 16u && eb < 255u) ? __uint_as_float((268u - eb) << 23) : 0.f;
    const float xs = eb == 255u ? __uint_as_float(0x7FC00000u) : eb >= 16u ? __uint_as_float((eb - 14u) << 23) : 0.f;
    int X[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        X[2 * i] = __float2int_rn(__uint_as_float(w[i] << 16) * sf);
        X[2 * i + 1] = __float2int_rn(__uint_as_float(w[i] & 0xFFFF0000u) * sf);
    }
    gv_store_unit(X, xs, dst, lane);
}

// The same for eight fp32 values (activations that went through a fused prologue): fp32 mantissas
// can round up to 2^15, which the signed high byte cannot hold, so the top is clamped to 32767.
__device__ __forceinline__ void gv_convert_unit_f32(const float (&v)[8], uint32_t dst, int lane) {
    uint32_t amax = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = max(amax, __float_as_uint(v[i]) & 0x7FFFFFFFu);
    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    const uint32_t eb = amax >> 23;
    const float sf = (eb >= 16u && eb < 255u) ? __uint_as_float((268u - eb) << 23) : 0.f;
    const float xs = eb == 255u ? __uint_as_float(0x7FC00000u) : eb >= 16u ? __uint_as_float((eb - 14u) << 23) : 0.f;
    int X[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) X[i] = min(__float2int_rn(v[i] * sf), 32767);
    gv_store_unit(X, xs, dst, lane);
}

// Q8_0: blocks 2P and 2P+1 (P = 0..3: pair of the 256-k box) of one row against MT tokens.
// The pair is the 68 bytes from byte 68 P of the row = words P .. P+16 of the five 16-byte units
// that start at byte 64 P (see skinny_tc.cu for the same extraction).
template <int P, int MT>
__device__ __forceinline__ void gv_pair_q8_0(float (&acc)[MT], uint32_t wrow, uint32_t xq, int xq_tok_stride) {
    uint32_t W[20];
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        const uint4 v = lds128(wrow + static_cast<uint32_t>(64 * P + 16 * i));
        W[4 * i] = v.x; W[4 * i + 1] = v.y; W[4 * i + 2] = v.z; W[4 * i + 3] = v.w;
    }
    uint32_t q[2][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        q[0][i] = prmt(W[P + i], W[P + i + 1], 0x5432);  // codes start 2 bytes into word P
        q[1][i] = W[P + 9 + i];
    }
    const float d0 = half_bits_to_f32(W[P]), d1 = half_bits_to_f32(W[P + 8] >> 16);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        const uint32_t xm = xq + static_cast<uint32_t>(m * xq_tok_stride);
        const float xs0 = lds32f(xm + static_cast<uint32_t>(GV_XQ_XS + 8 * P));
        const float xs1 = lds32f(xm + static_cast<uint32_t>(GV_XQ_XS + 8 * P + 4));
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            int th[2] = {0, 0}, tl[2] = {0, 0};  // two chains each: the dot products of a block are independent
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint4 xh = lds128(xm + static_cast<uint32_t>(64 * P + 32 * b + 16 * i));
                const uint4 xl = lds128(xm + static_cast<uint32_t>(GV_XQ_XL + 64 * P + 32 * b + 16 * i));
                th[0] = dp4a_ss(q[b][4 * i], xh.x, th[0]); tl[0] = dp4a_su(q[b][4 * i], xl.x, tl[0]);
                th[1] = dp4a_ss(q[b][4 * i + 1], xh.y, th[1]); tl[1] = dp4a_su(q[b][4 * i + 1], xl.y, tl[1]);
                th[0] = dp4a_ss(q[b][4 * i + 2], xh.z, th[0]); tl[0] = dp4a_su(q[b][4 * i + 2], xl.z, tl[0]);
                th[1] = dp4a_ss(q[b][4 * i + 3], xh.w, th[1]); tl[1] = dp4a_su(q[b][4 * i + 3], xl.w, tl[1]);
            }
            // |sum of 32 code * byte products| < 2^20: exact through the magic-number conversion
            const float t = fmaf(small_int_to_f32(th[0] + th[1]), 256.0f, small_int_to_f32(tl[0] + tl[1]));
            acc[m] = fmaf((b ? d1 : d0) * (b ? xs1 : xs0), t, acc[m]);
        }
    }
}

// Q4_K: sub-blocks 4 KH .. 4 KH + 3 (code groups 2 KH, 2 KH + 1) of one 144-byte super-block row.
template <int KH, int MT>
__device__ __forceinline__ void gv_half_q4_k(float (&acc)[MT], uint32_t wrow, uint32_t xq, int xq_tok_stride) {
    const uint4 hd = lds128(wrow);
    const float d = half_bits_to_f32(hd.x), dmin = half_bits_to_f32(hd.x >> 16);
    uint32_t sc4, mn4;  // the four 6-bit scales / minimums of this half, one per byte
    if (KH == 0) {
        sc4 = hd.y & 0x3F3F3F3Fu;
        mn4 = hd.z & 0x3F3F3F3Fu;
    } else {
        sc4 = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
        mn4 = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
    }
    // the four scale * d and minimum * dmin products of this half (6-bit integers lifted exactly)
    float dsc[4], dm[4];
#pragma unroll
    for (int sl = 0; sl < 4; ++sl) {
        dsc[sl] = d * small_int_to_f32(static_cast<int>((sc4 >> (8 * sl)) & 0xFFu)) * ((sl & 1) ? 0.0625f : 1.0f);
        dm[sl] = dmin * small_int_to_f32(static_cast<int>((mn4 >> (8 * sl)) & 0xFFu));
    }
    uint4 xsv[MT], sxv[MT];  // block scales and block sums of the activations for sub-blocks 4 KH .. 4 KH + 3
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        xsv[m] = lds128(xq + static_cast<uint32_t>(m * xq_tok_stride + GV_XQ_XS + 16 * KH));
        sxv[m] = lds128(xq + static_cast<uint32_t>(m * xq_tok_stride + GV_XQ_SX + 16 * KH));
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {  // code group 2 KH + j: low nibbles sub-block s, high nibbles s + 1
        const uint4 c0 = lds128(wrow + static_cast<uint32_t>(16 + (2 * KH + j) * 32));
        const uint4 c1 = lds128(wrow + static_cast<uint32_t>(32 + (2 * KH + j) * 32));
        const uint32_t cw[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            const int sl = 2 * j + hi;  // sub-block inside this half
            uint32_t n[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) n[i] = hi ? (cw[i] & 0xF0F0F0F0u) : (cw[i] & 0x0F0F0F0Fu);  // hi: 16 n (scale / 16)
            const int s = 4 * KH + sl;  // sub-block of the super-block = 32-value block of the box
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint32_t xm = xq + static_cast<uint32_t>(m * xq_tok_stride);
                int th[2] = {0, 0}, tl[2] = {0, 0};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const uint4 xh = lds128(xm + static_cast<uint32_t>(32 * s + 16 * i));
                    const uint4 xl = lds128(xm + static_cast<uint32_t>(GV_XQ_XL + 32 * s + 16 * i));
                    th[0] = dp4a_us(n[4 * i], xh.x, th[0]); tl[0] = dp4a_uu(n[4 * i], xl.x, tl[0]);
                    th[1] = dp4a_us(n[4 * i + 1], xh.y, th[1]); tl[1] = dp4a_uu(n[4 * i + 1], xl.y, tl[1]);
                    th[0] = dp4a_us(n[4 * i + 2], xh.z, th[0]); tl[0] = dp4a_uu(n[4 * i + 2], xl.z, tl[0]);
                    th[1] = dp4a_us(n[4 * i + 3], xh.w, th[1]); tl[1] = dp4a_uu(n[4 * i + 3], xl.w, tl[1]);
                }
                // |sum| <= 32 * 240 * 255 < 2^21: exact through the magic-number conversion
                const float t = fmaf(small_int_to_f32(th[0] + th[1]), 256.0f, small_int_to_f32(tl[0] + tl[1]));
                const float xs = __uint_as_float(sl == 0 ? xsv[m].x : sl == 1 ? xsv[m].y : sl == 2 ? xsv[m].z : xsv[m].w);
                const float sx = __uint_as_float(sl == 0 ? sxv[m].x : sl == 1 ? sxv[m].y : sl == 2 ? sxv[m].z : sxv[m].w);
                acc[m] = fmaf(dsc[sl] * xs, t, acc[m]);
                acc[m] = fmaf(-dm[sl], sx, acc[m]);
            }
        }
    }
}

}  // namespace izb
