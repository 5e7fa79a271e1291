// Dense bf16 GEMM on tcgen05 tensor cores with TMEM accumulators (see gemm_tc.cuh).
#include <algorithm>
#include <cstring>
#include <cstdlib>

#include "gemm_tc.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace izb {

constexpr int GT_BM = 128;       // rows of X per tile = TMEM lanes
constexpr int GT_BK = 64;        // k per pipeline stage = one 128-byte swizzle row of bf16
constexpr int GT_UMMA_K = 16;    // k per tcgen05.mma (bf16)
constexpr int GT_EPI_WARPS = 8;   // two warps per TMEM lane quarter, each takes half of the tile's columns
constexpr int GT_THREADS = 32 * (2 + GT_EPI_WARPS);  // producer warp, MMA warp, epilogue warps
constexpr int GT_MAX_STAGES = 8;
constexpr int GT_MAX_EXPERTS = 256;
constexpr int GT_GROUP_M = 16;  // row blocks per rasterisation band
constexpr int GT_STAGING_PER_WARP = 32 * 128;  // 32 rows x 128 bytes of output staging per epilogue warp

struct GemmShared {
    unsigned long long full[GT_MAX_STAGES];
    unsigned long long empty[GT_MAX_STAGES];
    unsigned long long tmem_full[2];
    unsigned long long tmem_empty[2];
    unsigned long long drain;
    uint32_t tmem_base;
    int abort_flag;
    int tile_prefix[GT_MAX_EXPERTS + 1];  // grouped: first m-tile of each expert
};

struct TileCoord {
    int m0;        // first row of X
    int rows_end;  // rows at or past this are not stored
    int n_blk;     // column block (in units of the tile's output columns)
    int expert;
};

__device__ __forceinline__ TileCoord tile_coord(int tile, int m_tiles, int n_tiles, const GemmParams& p, const int* prefix) {
    TileCoord c;
    // Band rasterisation: tiles are walked in bands of GT_GROUP_M row blocks, column-major inside a
    // band, so the CTAs running at one time cover a near-square patch of the output; each X and W
    // tile is then shared by a dozen CTAs through L2 instead of one W tile by all of them.
    const int band_tiles = GT_GROUP_M * n_tiles;
    const int band = tile / band_tiles, within = tile - band * band_tiles;
    const int gm = min(GT_GROUP_M, m_tiles - band * GT_GROUP_M);
    const int mt = band * GT_GROUP_M + within % gm;
    c.n_blk = within / gm;
    if (p.seg_offsets == nullptr) {
        c.expert = 0;
        c.m0 = mt * GT_BM;
        c.rows_end = p.M;
    } else {
        int lo = 0, hi = p.n_experts;  // last expert whose first tile is <= mt
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= mt) lo = mid; else hi = mid;
        }
        c.expert = lo;
        c.m0 = p.seg_offsets[lo] + (mt - prefix[lo]) * GT_BM;
        c.rows_end = p.seg_offsets[lo + 1];
    }
    return c;
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }
// x * sigmoid(x) = 0.5 x (1 + tanh(x / 2)): one special-function instruction per element
// (tanh.approx, relative error ~2^-11, below the bf16 rounding of the result).
// tanh-form GELU, 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), on the same instruction.
__device__ __forceinline__ float gelu_tanh(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * fmaf(0.044715f * x * x, x, x)));
    return fmaf(0.5f * x, t, 0.5f * x);
}
// sigmoid(x) = 0.5 (1 + tanh(x / 2)) on the same instruction
__device__ __forceinline__ float sigmoid_fast(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
}
__device__ __forceinline__ float silu(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f * x, t, 0.5f * x);
}

// d (16 bytes of one output row: kind 0 = eight bf16, 1 = eight fp16, 2 = four fp32) plus the bf16 residual values
// behind rs, of which `valid` exist.  A call, not inline code: it sits in the eight-fold unrolled flush loop of the
// epilogue, which should stay small.
__device__ __noinline__ uint4 gt_add_residual(uint4 d, const __nv_bfloat16* rs, int valid, int kind) {
    uint32_t w[4] = {d.x, d.y, d.z, d.w};
    if (kind == 2) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (e < valid) w[e] = __float_as_uint(__uint_as_float(w[e]) + __bfloat162float(rs[e]));
    } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float r_lo = 2 * e < valid ? __bfloat162float(rs[2 * e]) : 0.f;
            const float r_hi = 2 * e + 1 < valid ? __bfloat162float(rs[2 * e + 1]) : 0.f;
            if (kind == 1) {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[e]);
                w[e] = pack_f16x2(__low2float(h) + r_lo, __high2float(h) + r_hi);
            } else {
                w[e] = pack_bf16x2(bf16_lo_to_f32(w[e]) + r_lo, bf16_hi_to_f32(w[e]) + r_hi);
            }
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// EPI, OUT: the epilogue and the output type, compile-time choices: the epilogue loop of an instantiation holds its own activation only
// (the erf / tanh / sigmoid bodies are 32-fold unrolled; all of them behind run-time branches in one loop made
// the epilogue warps wait for instruction fetch).
template <int EPI, int OUT>
__global__ void __launch_bounds__(GT_THREADS, 1)
    gemm_tc_kernel(const __grid_constant__ GemmParams p, int n_stages, int* status) {
    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    __shared__ GemmShared sh;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bn = p.bn;
    // gated epilogues: the tile's accumulator holds the matching columns of both row halves of W side by side
    constexpr bool swiglu = EPI == GEMM_EPI_SWIGLU || EPI == GEMM_EPI_GLU;
    constexpr bool glu = EPI == GEMM_EPI_GLU;
    const int out_cols = swiglu ? bn / 2 : bn;  // output columns one tile produces
    const uint32_t a_bytes = GT_BM * GT_BK * 2, b_bytes = static_cast<uint32_t>(bn) * GT_BK * 2;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    const uint32_t smem0 = smem_u32(dyn_smem);
    const int n_kb = (p.K + GT_BK - 1) / GT_BK;
    volatile int* abort_flag = &sh.abort_flag;
    constexpr bool f32_out = OUT == IZB_F32, f16_out = OUT == IZB_F16;  // the output type, compile-time like the epilogue
    const uint32_t stage_out = smem0 + static_cast<uint32_t>(n_stages) * stage_bytes;  // output staging after the ring
    // 16-byte global stores need an aligned base and row stride
    const bool vec_ok = (reinterpret_cast<uintptr_t>(p.y) & 15) == 0 && (p.ldy * (f32_out ? 4 : 2)) % 16 == 0;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&sh.tmem_full[a]), 1);
            mbar_init(smem_u32(&sh.tmem_empty[a]), GT_EPI_WARPS);
        }
        mbar_init(smem_u32(&sh.drain), 1);
        sh.abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tc_alloc(smem_u32(&sh.tmem_base), 512);
    pdl_wait();  // the expert offsets, the activations and the output buffer belong to the kernels before this one
    if (threadIdx.x == 0 && p.seg_offsets != nullptr) {
        // grouped: m-tile prefix over the expert segments
        int acc = 0;
        for (int e = 0; e < p.n_experts; ++e) {
            sh.tile_prefix[e] = acc;
            acc += (p.seg_offsets[e + 1] - p.seg_offsets[e] + GT_BM - 1) / GT_BM;
        }
        sh.tile_prefix[p.n_experts] = acc;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    const uint32_t tmem_base = sh.tmem_base;
    const int m_tiles = p.seg_offsets ? sh.tile_prefix[p.n_experts] : (p.M + GT_BM - 1) / GT_BM;
    const int n_tiles = (p.n_out + out_cols - 1) / out_cols;
    const int total_tiles = m_tiles * n_tiles;
    bool ok = true;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            long long issued = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const TileCoord c = tile_coord(tile, m_tiles, n_tiles, p, sh.tile_prefix);
                const int n0 = c.n_blk * out_cols;
                for (int kb = 0; kb < n_kb; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(&sh.empty[stage]), phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    const uint32_t fbar = smem_u32(&sh.full[stage]);
                    const uint32_t sa = smem0 + static_cast<uint32_t>(stage) * stage_bytes, sb = sa + a_bytes;
                    mbar_expect_tx(fbar, stage_bytes);
                    tma_load_2d(sa, &p.tmap_a, kb * GT_BK, c.m0, fbar);
                    if (swiglu) {
                        tma_load_3d(sb, &p.tmap_b, kb * GT_BK, n0, c.expert, fbar);
                        tma_load_3d(sb + b_bytes / 2, &p.tmap_b, kb * GT_BK, p.n_out + n0, c.expert, fbar);
                    } else {
                        tma_load_3d(sb, &p.tmap_b, kb * GT_BK, n0, c.expert, fbar);
                    }
                    ++issued;
                    if (++stage == n_stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                // let copies still in flight land before shared memory is released
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
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16(bn);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
                if (!mbar_wait_bounded(smem_u32(&sh.tmem_empty[acc]), acc_phase ^ 1u, abort_flag)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
                for (int kb = 0; kb < n_kb; ++kb) {
                    if (!mbar_wait_bounded(smem_u32(&sh.full[stage]), phase, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem0 + static_cast<uint32_t>(stage) * stage_bytes, sb = sa + a_bytes;
                    const uint64_t adesc = umma_desc_k_major_sw128(sa), bdesc = umma_desc_k_major_sw128(sb);
#pragma unroll
                    for (int k = 0; k < GT_BK / GT_UMMA_K; ++k) {
                        // 16 bf16 = 32 bytes further along the swizzle row: +2 in 16-byte units
                        tc_mma_f16(d_tmem, adesc + static_cast<uint64_t>(2 * k), bdesc + static_cast<uint64_t>(2 * k), idesc,
                                   (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&sh.empty[stage]));  // slot free once these MMAs have read it
                    if (++stage == n_stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                tc_commit(smem_u32(&sh.tmem_full[acc]));  // accumulator complete
            }
            // every MMA issued by this thread has retired before TMEM is released
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
        // ---------------- epilogue: warps 2..9, TMEM lane group = warp % 4, column half = (warp-2)/4 ----
        const int lg = warp & 3;
        const int ew = warp - 2;
        // narrow tiles (fewer than 64 output columns) are handled by the first warp of each lane group
        const int cc_begin = out_cols >= 64 ? (ew >> 2) * (out_cols / 2) : 0;
        const int cc_end = out_cols >= 64 ? cc_begin + out_cols / 2 : ((ew >> 2) == 0 ? out_cols : 0);
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = static_cast<uint32_t>((it >> 1) & 1);
            const TileCoord c = tile_coord(tile, m_tiles, n_tiles, p, sh.tile_prefix);
            if (ok && !mbar_wait_bounded(smem_u32(&sh.tmem_full[acc]), acc_phase, abort_flag)) ok = false;
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + static_cast<uint32_t>(acc * 256);
            const __nv_bfloat16* bias = p.bias ? p.bias + static_cast<long long>(c.expert) * p.N : nullptr;
            const int col_base = c.n_blk * out_cols;
            // Staging: each thread owns one output row, but a row-per-thread store scatters 16-byte
            // pieces over 32 rows.  The warp parks 128 bytes per row in shared memory (16-byte chunks
            // XOR-swizzled by row) and writes them back 8 lanes per row, i.e. whole 128-byte lines.
            const int cols_per_flush = f32_out ? 32 : 64;
            const uint32_t stg = stage_out + static_cast<uint32_t>(ew) * GT_STAGING_PER_WARP;
            for (int cc = cc_begin; cc < cc_end; cc += 32) {
                float v[32];
                tc_ld_32x32(t_row + static_cast<uint32_t>(cc), v);
                const int col0 = col_base + cc;
                // The mode tests sit outside the element loops on purpose: inside, the compiler turns
                // them into selects and evaluates erf and exp for every element of every mode.
                if constexpr (swiglu) {
                    float u[32];
                    tc_ld_32x32(t_row + static_cast<uint32_t>(bn / 2 + cc), u);
                    if (bias) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            if (col0 + i < p.n_out) {
                                v[i] += __bfloat162float(bias[col0 + i]);
                                u[i] += __bfloat162float(bias[p.n_out + col0 + i]);
                            }
                        }
                    }
                    if constexpr (glu) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = v[i] * sigmoid_fast(u[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = silu(v[i]) * u[i];
                    }
                } else {
                    if (bias) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < p.n_out) v[i] += __bfloat162float(bias[col0 + i]);
                    }
                    if constexpr (EPI == GEMM_EPI_GELU) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = gelu_erf(v[i]);
                    } else if constexpr (EPI == GEMM_EPI_SILU) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = silu(v[i]);
                    } else if constexpr (EPI == GEMM_EPI_GELU_TANH) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
                    }
                }
                // park this thread's 32 values in its staging row
                const uint32_t my_row = stg + static_cast<uint32_t>(lane) * 128;
                if constexpr (f32_out) {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        sts128(my_row + static_cast<uint32_t>((q ^ (lane & 7)) << 4), __float_as_uint(v[4 * q]),
                               __float_as_uint(v[4 * q + 1]), __float_as_uint(v[4 * q + 2]), __float_as_uint(v[4 * q + 3]));
                } else {
                    const int half = ((cc - cc_begin) >> 5) & 1;  // first or second 64 bytes of the 128-byte row
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t dst = my_row + static_cast<uint32_t>(((half * 4 + q) ^ (lane & 7)) << 4);
                        if constexpr (f16_out)
                            sts128(dst, pack_f16x2(v[8 * q], v[8 * q + 1]), pack_f16x2(v[8 * q + 2], v[8 * q + 3]),
                                   pack_f16x2(v[8 * q + 4], v[8 * q + 5]), pack_f16x2(v[8 * q + 6], v[8 * q + 7]));
                        else
                            sts128(dst, pack_bf16x2(v[8 * q], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                                   pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
                    }
                }
                const int rel = cc - cc_begin;
                const bool row_full = f32_out || ((rel >> 5) & 1) || cc + 32 >= cc_end;
                if (!row_full) continue;
                __syncwarp();
                const int flush_rel = f32_out ? rel : (rel & ~63);
                const int flush_col0 = col_base + cc_begin + flush_rel;
                const int valid_cols = min(cols_per_flush, rel + 32 - flush_rel);
                const int vec = f32_out ? 4 : 8;  // elements per 16 bytes
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = 4 * j + (lane >> 3), ch = lane & 7;
                    const long long grow = static_cast<long long>(c.m0) + lg * 32 + r;
                    const int col = flush_col0 + ch * vec;
                    if (grow < c.rows_end && ch * vec < valid_cols && col < p.n_out) {
                        uint4 d = lds128(stg + static_cast<uint32_t>(r * 128 + ((ch ^ (r & 7)) << 4)));
                        if (p.residual)  // the residual rides in here, where a lane holds 16 contiguous bytes of one output row
                            d = gt_add_residual(d, p.residual + grow * p.ld_res + col, p.n_out - col, f32_out ? 2 : (f16_out ? 1 : 0));
                        if constexpr (f32_out) {
                            float* dst = static_cast<float*>(p.y) + grow * p.ldy + col;
                            if (vec_ok && col + 4 <= p.n_out) {
                                *reinterpret_cast<uint4*>(dst) = d;
                            } else {
                                const uint32_t w[4] = {d.x, d.y, d.z, d.w};
                                for (int e = 0; e < 4 && col + e < p.n_out; ++e) dst[e] = __uint_as_float(w[e]);
                            }
                        } else {
                            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.y) + grow * p.ldy + col;
                            if (vec_ok && col + 8 <= p.n_out) {
                                *reinterpret_cast<uint4*>(dst) = d;
                            } else {
                                const uint32_t w[4] = {d.x, d.y, d.z, d.w};
                                for (int e = 0; e < 8 && col + e < p.n_out; ++e)
                                    reinterpret_cast<unsigned short*>(dst)[e] =
                                        static_cast<unsigned short>((w[e >> 1] >> ((e & 1) * 16)) & 0xFFFFu);
                            }
                        }
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.tmem_empty[acc]));
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tc_dealloc(tmem_base, 512);
    }
    if ((!ok || sh.abort_flag) && lane == 0) atomicExch(status, 2);
}

int gemm_tc_launch(izb_ctx* ctx, cudaStream_t stream, const void* x, long long ldx, const void* w, const void* bias,
                   void* y, long long ldy, int y_dtype, int M, int N, int K, int epilogue, const int* seg_offsets,
                   int n_experts, const void* residual, long long ld_res) {
    if (!ctx || !x || !w || !y) return IZB_ERR_BAD_ARG;
    if (M <= 0 || N <= 0 || K <= 0 || n_experts <= 0) return IZB_ERR_BAD_ARG;
    if (K % 8 != 0 || ldx % 8 != 0 || ldx < K) return IZB_ERR_UNSUPPORTED;
    if (!izb_aligned(x, 16) || !izb_aligned(w, 16)) return IZB_ERR_BAD_ARG;
    if (y_dtype != IZB_BF16 && y_dtype != IZB_F32 && y_dtype != IZB_F16) return IZB_ERR_BAD_ARG;
    if (epilogue < GEMM_EPI_NONE || epilogue > GEMM_EPI_GLU) return IZB_ERR_BAD_ARG;
    if (seg_offsets && n_experts > GT_MAX_EXPERTS) return IZB_ERR_UNSUPPORTED;
    if (!seg_offsets && n_experts != 1) return IZB_ERR_BAD_ARG;
    const bool swiglu = epilogue == GEMM_EPI_SWIGLU || epilogue == GEMM_EPI_GLU;  // gated: two row halves of W per output column
    if (swiglu && N % 2 != 0) return IZB_ERR_BAD_ARG;
    const int n_out = swiglu ? N / 2 : N;
    if (ldy < n_out) return IZB_ERR_BAD_ARG;
    if (residual && (ld_res < n_out || !izb_aligned(residual, 2))) return IZB_ERR_BAD_ARG;

    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    // Accumulator width.  Tiles are dealt round-robin to one CTA per SM, so a pass costs
    // ceil(tiles / SMs) rounds of one tile each; a tile's time grows with its width plus a fixed part
    // (the 128-row operand is fetched whatever the width).  The width with the cheapest pass wins,
    // wider on ties: 375 x 4096 takes 128 (96 tiles, one round) rather than 64 (192 tiles, two rounds).
    // Grouped: the row tiles are only known on the device; half a tile per non-empty expert is the
    // expected padding of ragged segments.
    const long long m_tiles = seg_offsets ? (static_cast<long long>(M) + GT_BM - 1) / GT_BM + (std::min(n_experts, M) + 1) / 2
                                          : (static_cast<long long>(M) + GT_BM - 1) / GT_BM;
    int bn = 256;
    {
        long long best = -1;
        static const int widths[4] = {256, 192, 128, 64};  // 192: not for SwiGLU (its halves must be whole 32-column groups)
        for (int wi = 0; wi < 4; ++wi) {
            const int cand = widths[wi];
            if (swiglu && cand == 192) continue;
            const int oc = swiglu ? cand / 2 : cand;
            const long long tiles = m_tiles * ((n_out + oc - 1) / oc);
            const long long cost = ((tiles + ctx->sm_count - 1) / ctx->sm_count) * (cand + 64);
            if (best < 0 || cost < best) {
                best = cost;
                bn = cand;
            }
        }
    }
    const int out_cols = swiglu ? bn / 2 : bn;
    p.bn = bn;
    p.y = y;
    p.bias = static_cast<const __nv_bfloat16*>(bias);
    p.seg_offsets = seg_offsets;
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.ld_res = ld_res;
    p.ldy = ldy;
    p.M = M; p.N = N; p.K = K;
    p.n_experts = n_experts;
    p.epilogue = epilogue;
    p.y_dtype = y_dtype;
    p.n_out = n_out;

    {
        const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        const uint64_t strides[1] = {static_cast<uint64_t>(ldx) * 2};
        const uint32_t box[2] = {GT_BK, GT_BM};
        const int rc = tma_encode(&p.tmap_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, dims, strides, box,
                                  CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != IZB_OK) return rc;
    }
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(n_experts)};
        const uint64_t strides[2] = {static_cast<uint64_t>(K) * 2, static_cast<uint64_t>(N) * static_cast<uint64_t>(K) * 2};
        const uint32_t box[3] = {GT_BK, static_cast<uint32_t>(swiglu ? bn / 2 : bn), 1};
        const int rc = tma_encode(&p.tmap_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, w, dims, strides, box,
                                  CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc != IZB_OK) return rc;
    }

    const int stage_bytes = (GT_BM + bn) * GT_BK * 2;
    const int staging = GT_EPI_WARPS * GT_STAGING_PER_WARP;
    int n_stages = std::min(GT_MAX_STAGES,
                            (ctx->max_smem_optin - 2048 - staging) / stage_bytes);  // 2048: static barriers + tile prefix, padded
    if (n_stages < 2) return IZB_ERR_UNSUPPORTED;
    static_assert(sizeof(GemmShared) <= 2048, "static shared memory budget");
    const int smem_bytes = n_stages * stage_bytes + staging;
    const int slot = ctx->device;
    void (*kernel)(GemmParams, int, int*) = nullptr;
#define IZB_GT_PICK(E)                                                                               \
    case E:                                                                                          \
        kernel = y_dtype == IZB_F32   ? gemm_tc_kernel<E, IZB_F32>                                   \
                 : y_dtype == IZB_F16 ? gemm_tc_kernel<E, IZB_F16>                                   \
                                      : gemm_tc_kernel<E, IZB_BF16>;                                 \
        break;
    switch (epilogue) {
        IZB_GT_PICK(GEMM_EPI_NONE)
        IZB_GT_PICK(GEMM_EPI_GELU)
        IZB_GT_PICK(GEMM_EPI_SILU)
        IZB_GT_PICK(GEMM_EPI_SWIGLU)
        IZB_GT_PICK(GEMM_EPI_GELU_TANH)
        default:
        IZB_GT_PICK(GEMM_EPI_GLU)
    }
#undef IZB_GT_PICK
    // the attribute is per kernel and per device: one record for each pair
    static std::atomic<int> smem_set[IZB_MAX_DEVICES][(GEMM_EPI_GLU + 1) * 3];
    const int which = epilogue * 3 + y_dtype;
    if (smem_set[slot][which].load(std::memory_order_relaxed) < smem_bytes) {
        IZB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        smem_set[slot][which].store(smem_bytes, std::memory_order_relaxed);
    }
    const long long tiles_bound = m_tiles * ((n_out + out_cols - 1) / out_cols);
    const int grid = static_cast<int>(std::min<long long>(tiles_bound, ctx->sm_count));
    IZB_CUDA_TRY(launch_chained(ctx, kernel, dim3(grid), dim3(GT_THREADS), smem_bytes, stream, p, n_stages, ctx->d_status + 1));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // namespace izb

