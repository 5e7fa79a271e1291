// Block-quantised linear layers for 1..4 tokens: integer dot products on the CUDA cores.
//
// Same plan, descriptors and TMA producer as the weight-streaming kernel (skinny.cu).  Lifting every
// int8 / 4-bit code to a floating-point tensor-core operand costs 3..4 instructions per weight, which
// bounds that kernel below the HBM rate.  Here the codes stay integers: one extra warp re-expresses
// each 32-value block of the activations as 16-bit fixed point (X = round(x * 2^(14-e)), e the
// exponent of the block maximum: exact for every bf16 value within 2^-7 of the maximum, absolute
// error <= 2^-15 of the maximum otherwise), split into a signed high byte and an unsigned low byte,
// and the consumers accumulate code * X with dp4a (four products per instruction, exact in int32).
// One conversion to fp32 and one multiply by (block scale * 2^(e-14)) per block and token finish the
// job: about one instruction per weight for one token.
//
// Tile = 64 weight rows; warps 0,1 take the first 128 k of every 256-k box for 32 rows each, warps
// 2,3 the second 128 k; one thread owns one row (16-byte loads, rows 272 or 144 bytes apart: no
// bank conflicts).  Warp 4 issues the copies, warp 5 converts the activations of each stage.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "gemv_dot.cuh"
#include "skinny.cuh"
#include "tma.cuh"

namespace izb {

constexpr int GV_CONSUMER_WARPS = 4;
constexpr int GV_PROD_WARP = GV_CONSUMER_WARPS, GV_CONV_WARP = GV_CONSUMER_WARPS + 1;
constexpr int GV_THREADS = 32 * (GV_CONSUMER_WARPS + 2);
constexpr int GV_TILE_ROWS = 64;

constexpr int GV_MAX_KSPLIT = 8;  // CTAs of a cluster sharing one row tile, each a slice of k

template <int MT, bool EX, bool KS>
struct GvShared {
    unsigned long long full[GV_MAX_STAGES];    // copies landed
    unsigned long long xready[GV_MAX_STAGES];  // activations of the stage converted
    unsigned long long empty[GV_MAX_STAGES];   // consumers done with the stage
    float red[2][GV_TILE_ROWS * MT];           // partial sums of the second k-half, double-buffered by tile parity
    // fused RmsNorm: every token's sum of squares over the k this CTA saw, left by the converter in the
    // slot of the tile's last stage
    float rs[EX ? GV_MAX_STAGES : 1][MT];
    // k split over a cluster: the other CTAs' sums (and sums of squares) land here in the first CTA
    float cl_red[KS ? (GV_MAX_KSPLIT - 1) * MT * GV_TILE_ROWS : 1];
    float cl_ss[KS ? (GV_MAX_KSPLIT - 1) * MT : 1];
    unsigned long long cl_bar;
    int abort_flag;
};

// EX: some problem of the launch carries a fused prologue (RmsNorm, silu(gate) * up) or a residual;
// the plain instantiation compiles none of that.
// KS: launched as clusters of `ksplit` CTAs along x; the CTAs of a cluster share one row tile and take
// consecutive slices of its k chunks, so a lone small projection spreads over the SMs instead of
// walking its k on a few of them.  One tile per cluster (grid = tiles * ksplit).
template <int FMT, int MT, bool EX, bool KS>
__global__ void __launch_bounds__(GV_THREADS)
    skinny_gemv_kernel(const SkinnyProblem* __restrict__ probs, const __grid_constant__ SkinnyProblem single, int n_probs,
                       int total_tiles, int n_stages, int stage_bytes, int xq_stage_bytes, int xq_bytes, int lite_bytes,
                       int y_dtype, int ksplit, int* status) {
    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    __shared__ GvShared<MT, EX, KS> sh;
    const int crank = KS ? static_cast<int>(blockIdx.x) % ksplit : 0;       // rank inside the cluster
    const int tile_first = KS ? static_cast<int>(blockIdx.x) / ksplit : static_cast<int>(blockIdx.x);
    const int tile_step = KS ? static_cast<int>(gridDim.x) / ksplit : static_cast<int>(gridDim.x);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const SkinnyProblem* plist = probs ? probs : &single;
    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.xready[s]), 1);
            mbar_init(smem_u32(&sh.empty[s]), GV_CONSUMER_WARPS);
        }
        if (KS) mbar_init(smem_u32(&sh.cl_bar), static_cast<uint32_t>((GV_TILE_ROWS) * (ksplit - 1)));
        sh.abort_flag = 0;
        mbar_fence_init();
    }
    // dynamic shared memory: [descriptor cache][converted activations per stage][stage ring]; stage = [weight boxes][activations]
    ProbLite* lite = reinterpret_cast<ProbLite*>(dyn_smem);
    const int n_cached = min(n_probs, lite_bytes / static_cast<int>(sizeof(ProbLite)));
    for (int i = threadIdx.x; i < n_cached; i += blockDim.x) lite[i] = lite_from(plist[i]);  // the plan: written by the host
    __syncthreads();
    if (KS) cluster_sync_all();  // every CTA's barriers exist before any CTA of the cluster signals one
    // Activations, residual and the output buffer belong to the kernels before this one: every role waits
    // for them (pdl_wait) before its first access.  The weights belong to nobody: the producer sends the
    // weight copies of its first ring-full of stages on their way first, so that they land while the
    // kernel in front is still finishing.

    volatile int* abort_flag = &sh.abort_flag;
    const uint32_t xq0 = smem_u32(dyn_smem) + static_cast<uint32_t>(lite_bytes);
    const uint32_t stage0 = xq0 + static_cast<uint32_t>(xq_bytes);

    if (warp == GV_PROD_WARP) {
        // ---------------- producer: one lane issues two tiled copies per stage ----------------
        if (lane != 0) return;
        int pre = 0;  // stages whose weight copy is already under way
        {
            int p = -1;
            for (int tile = tile_first; tile < total_tiles && pre < n_stages; tile += tile_step) {
                const int np = find_problem(lite, n_cached, plist, n_probs, tile);
                const SkinnyProblem* P = plist + np;
                if (np != p && probs) tma_fence_descriptor(&P->tmap_w);
                p = np;
                const ProbLite L = p < n_cached ? lite[p] : lite_from(*P);
                const int row0 = (tile - L.tile_start) * GV_TILE_ROWS;
                const int c0 = KS ? crank * L.n_chunks / ksplit : 0, c1 = KS ? (crank + 1) * L.n_chunks / ksplit : L.n_chunks;
                for (int c = c0; c < c1 && pre < n_stages; ++c, ++pre) {
                    const uint32_t fbar = smem_u32(&sh.full[pre]);
                    mbar_expect_tx(fbar, static_cast<uint32_t>(L.stage_tx));
                    tma_load_3d(stage0 + static_cast<uint32_t>(pre) * static_cast<uint32_t>(stage_bytes), &P->tmap_w, 0, row0, c * L.nb, fbar);
                }
            }
        }
        pdl_wait();
        int stage = 0, p = -1;
        uint32_t phase = 0;
        long long issued = 0;
        bool ok = true;
        for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step) {
            const int np = find_problem(lite, n_cached, plist, n_probs, tile);
            const bool moved = np != p;
            p = np;
            const SkinnyProblem* P = plist + p;
            if (moved && probs) {
                tma_fence_descriptor(&P->tmap_w);
                tma_fence_descriptor(&P->tmap_x);
            }
            const ProbLite L = p < n_cached ? lite[p] : lite_from(*P);
            const int row0 = (tile - L.tile_start) * GV_TILE_ROWS;
            const int xchunks = L.nb * 4;
            int up_chunk0 = 0, x_half = 0;
            if (EX && L.extras && P->prologue == IZB_PRO_SILU_MUL) {
                up_chunk0 = P->up_chunk0;
                x_half = P->x_half;
            }
            const int c0 = KS ? crank * L.n_chunks / ksplit : 0, c1 = KS ? (crank + 1) * L.n_chunks / ksplit : L.n_chunks;
            for (int c = c0; c < c1; ++c) {
                const uint32_t fbar = smem_u32(&sh.full[stage]);
                const uint32_t sbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                if (issued >= pre) {
                    if (!mbar_wait_bounded(smem_u32(&sh.empty[stage]), phase ^ 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(fbar, static_cast<uint32_t>(L.stage_tx));
                    tma_load_3d(sbase, &P->tmap_w, 0, row0, c * L.nb, fbar);
                }
                tma_load_3d(sbase + static_cast<uint32_t>(L.x_off), &P->tmap_x, 0, 0, c * xchunks, fbar);
                if (EX && up_chunk0)  // silu(gate) * up: the matching chunks of the second half of the rows
                    tma_load_3d(sbase + static_cast<uint32_t>(L.x_off + x_half), &P->tmap_x, 0, 0, up_chunk0 + c * xchunks, fbar);
                ++issued;
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
            atomicExch(status, 5);
        }
        return;
    }

    pdl_wait();
    if (warp == GV_CONV_WARP) {
        // ---------------- converter: bf16 activations of each stage -> 16-bit block fixed point ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step) {
            const int p = find_problem(lite, n_cached, plist, n_probs, tile);
            const ProbLite L = p < n_cached ? lite[p] : lite_from(plist[p]);
            const int M = min(L.M, MT);
            int pro = IZB_PRO_NONE, x_half = 0;
            const __nv_bfloat16* norm_w = nullptr;
            float ss[MT];  // fused RmsNorm: this lane's share of every token's sum of squares over the tile's k
#pragma unroll
            for (int m = 0; m < MT; ++m) ss[m] = 0.f;
            if (EX && L.extras) {
                const SkinnyProblem* P = plist + p;
                pro = P->prologue;
                x_half = P->x_half;
                norm_w = P->norm_w;
            }
            // norm weights of this lane's 8 values in the first two boxes of a chunk, fetched one chunk
            // ahead: a load from global memory inside the chunk loop would stall every stage by its latency
            const int klane = (lane >> 3) * 64 + (lane & 7) * 8;
            const int c0 = KS ? crank * L.n_chunks / ksplit : 0, c1 = KS ? (crank + 1) * L.n_chunks / ksplit : L.n_chunks;
            uint4 gnext[2] = {};
            if (EX && pro == IZB_PRO_RMSNORM) {
#pragma unroll
                for (int b = 0; b < 2; ++b)
                    if (b < L.nb) gnext[b] = __ldg(reinterpret_cast<const uint4*>(norm_w + (c0 * L.nb + b) * 256 + klane));
            }
            for (int c = c0; c < c1; ++c) {
                uint4 gcur[2] = {gnext[0], gnext[1]};
                if (EX && pro == IZB_PRO_RMSNORM && c + 1 < c1) {
#pragma unroll
                    for (int b = 0; b < 2; ++b)
                        if (b < L.nb) gnext[b] = __ldg(reinterpret_cast<const uint4*>(norm_w + ((c + 1) * L.nb + b) * 256 + klane));
                }
                if (!mbar_wait_bounded(smem_u32(&sh.full[stage]), phase, abort_flag)) {
                    ok = false;
                    break;
                }
                const uint32_t sbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                for (int b = 0; b < L.nb; ++b) {
                    uint4 gw = {};
                    if (EX && pro == IZB_PRO_RMSNORM)
                        gw = b == 0 ? gcur[0] : b == 1 ? gcur[1] : __ldg(reinterpret_cast<const uint4*>(norm_w + (c * L.nb + b) * 256 + klane));
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        if (m >= M) break;
                        // copied activations: [64-k chunk][token][128 bytes]; lane = chunk lane/8, 16-byte unit lane%8
                        const uint32_t xaddr = sbase + static_cast<uint32_t>(L.x_off) +
                                               static_cast<uint32_t>(((b * 4 + (lane >> 3)) * MT + m) * 128 + (lane & 7) * 16);
                        const uint32_t dst = xq0 + static_cast<uint32_t>(stage * xq_stage_bytes + (b * MT + m) * GV_XQ_BYTES);
                        const uint4 v = lds128(xaddr);
                        if (!EX || pro == IZB_PRO_NONE) {
                            gv_convert_unit(v, dst, lane);
                        } else {
                            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                            float f[8];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                f[2 * i] = __uint_as_float(w[i] << 16);
                                f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
                            }
                            uint4 o;  // the other factor of every value: norm weights, or the `up` half of the row
                            if (pro == IZB_PRO_RMSNORM) {
                                o = gw;
#pragma unroll
                                for (int i = 0; i < 8; ++i) ss[m] = fmaf(f[i], f[i], ss[m]);
                            } else {
                                o = lds128(xaddr + static_cast<uint32_t>(x_half));
#pragma unroll
                                for (int i = 0; i < 8; ++i) f[i] *= rcp_approx(1.0f + __expf(-f[i]));  // silu: x * sigmoid(x)
                            }
                            const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                f[2 * i] *= __uint_as_float(ow[i] << 16);
                                f[2 * i + 1] *= __uint_as_float(ow[i] & 0xFFFF0000u);
                            }
                            gv_convert_unit_f32(f, dst, lane);
                        }
                    }
                }
                if (EX && c == c1 - 1) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        float t = ss[m];
#pragma unroll
                        for (int d = 16; d > 0; d >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, d);
                        if (lane == 0) sh.rs[stage][m] = t;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sh.xready[stage]));
                if (++stage == n_stages) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        if (!ok && lane == 0) atomicExch(status, 5);
        return;
    }

    // ---------------- consumers ----------------
    const int kh = warp & 1;                  // which 128 k of every 256-k box
    const int row = (warp >> 1) * 32 + lane;  // row inside the tile
    int stage = 0, it = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = tile_first; tile < total_tiles; tile += tile_step, ++it) {
        const int p = find_problem(lite, n_cached, plist, n_probs, tile);
        const ProbLite L = p < n_cached ? lite[p] : lite_from(plist[p]);
        const int row0 = (tile - L.tile_start) * GV_TILE_ROWS;

        float acc[MT], rsv[MT];  // rsv: sum of squares of the token (fused RmsNorm), turned into 1 / rms at the end
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            acc[m] = 0.f;
            rsv[m] = 0.f;
        }
        float inv_k = 0.f, eps = 0.f;  // inv_k > 0: the problem carries a fused RmsNorm
        if (EX && L.extras && plist[p].prologue == IZB_PRO_RMSNORM) {
            inv_k = 1.0f / static_cast<float>(plist[p].K);
            eps = plist[p].eps;
        }
        // EX: bias and residual of this thread's row are fetched before the k loop, not at its end
        float addv[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) addv[m] = 0.f;
        if (EX && kh == 0 && row0 + row < L.N) {
            const float bias = L.bias ? __bfloat162float(L.bias[row0 + row]) : 0.f;
            const __nv_bfloat16* residual = L.extras ? plist[p].residual : nullptr;
            const int ld_res = residual ? plist[p].ld_res : 0;
#pragma unroll
            for (int m = 0; m < MT; ++m)
                addv[m] = bias + ((residual && m < L.M) ? __bfloat162float(residual[static_cast<long long>(m) * ld_res + row0 + row]) : 0.f);
        }

        const int c0 = KS ? crank * L.n_chunks / ksplit : 0, c1 = KS ? (crank + 1) * L.n_chunks / ksplit : L.n_chunks;
        for (int c = c0; c < c1; ++c) {
            if (ok && !mbar_wait_bounded(smem_u32(&sh.xready[stage]), phase, abort_flag)) ok = false;
            if (ok && !mbar_wait_bounded(smem_u32(&sh.full[stage]), phase, abort_flag)) ok = false;  // already complete
            if (ok) {
                const uint32_t sbase = stage0 + static_cast<uint32_t>(stage) * static_cast<uint32_t>(stage_bytes);
                for (int b = 0; b < L.nb; ++b) {
                    const uint32_t wrow = sbase + static_cast<uint32_t>(b * L.w_box_bytes + row * L.w_row_bytes);
                    const uint32_t xq = xq0 + static_cast<uint32_t>(stage * xq_stage_bytes + b * MT * GV_XQ_BYTES);
                    if constexpr (FMT == IZB_W_Q8_0) {
                        if (kh == 0) {
                            gv_pair_q8_0<0, MT>(acc, wrow, xq, GV_XQ_BYTES);
                            gv_pair_q8_0<1, MT>(acc, wrow, xq, GV_XQ_BYTES);
                        } else {
                            gv_pair_q8_0<2, MT>(acc, wrow, xq, GV_XQ_BYTES);
                            gv_pair_q8_0<3, MT>(acc, wrow, xq, GV_XQ_BYTES);
                        }
                    } else {
                        if (kh == 0) gv_half_q4_k<0, MT>(acc, wrow, xq, GV_XQ_BYTES);
                        else gv_half_q4_k<1, MT>(acc, wrow, xq, GV_XQ_BYTES);
                    }
                }
            }
            if (EX && ok && c == c1 - 1) {
#pragma unroll
                for (int m = 0; m < MT; ++m) rsv[m] = sh.rs[stage][m];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh.empty[stage]));
            if (++stage == n_stages) {
                stage = 0;
                phase ^= 1u;
            }
        }

        // the second k-half parks its sums in shared memory; the first adds them and stores the rows
        float* red = sh.red[it & 1];
        if (kh == 1) {
#pragma unroll
            for (int m = 0; m < MT; ++m) red[m * GV_TILE_ROWS + row] = acc[m];
        }
        named_bar_sync(1, GV_CONSUMER_WARPS * 32);
        if (kh == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[m] += red[m * GV_TILE_ROWS + row];
        }
        if (KS && kh == 0) {
            if (crank != 0) {
                // hand this CTA's share to the first CTA of the cluster and be done with the tile
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    st_cluster_f32(cluster_map_shared(smem_u32(&sh.cl_red[((crank - 1) * MT + m) * GV_TILE_ROWS + row]), 0), acc[m]);
                if (EX && row == 0) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) st_cluster_f32(cluster_map_shared(smem_u32(&sh.cl_ss[(crank - 1) * MT + m]), 0), rsv[m]);
                }
                mbar_arrive_cluster(cluster_map_shared(smem_u32(&sh.cl_bar), 0));
                continue;
            }
            // The other CTAs of the cluster store into this CTA's shared memory whatever became of their own
            // waits, and signal when done.  This CTA must stay resident until they have: it waits for them
            // even after giving up on its own pipeline (then on the clock alone, since the abort flag is
            // already up), and only uses their sums when everything went well.
            if (ok) {
                if (!mbar_wait_cluster_bounded(smem_u32(&sh.cl_bar), 0u, abort_flag)) ok = false;
            } else {
                (void)mbar_wait_cluster_clock_only(smem_u32(&sh.cl_bar), 0u, 2 * IZB_WAIT_LIMIT_CLOCKS);
            }
            if (ok) {
                for (int r = 0; r < ksplit - 1; ++r) {
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        acc[m] += sh.cl_red[(r * MT + m) * GV_TILE_ROWS + row];
                        if (EX) rsv[m] += sh.cl_ss[r * MT + m];
                    }
                }
            }
        }
        if (kh == 0 && ok) {
            const int grow = row0 + row;
            if (grow < L.N) {
                const float bias = (!EX && L.bias) ? __bfloat162float(L.bias[grow]) : 0.f;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m < L.M) {
                        float v = acc[m];
                        if (EX) v = fmaf(v, inv_k > 0.f ? rsqrtf(fmaf(rsv[m], inv_k, eps)) : 1.0f, addv[m]);
                        else v += bias;
                        const long long idx = static_cast<long long>(m) * L.ldy + grow;
                        store_typed(L.y, y_dtype, idx, v);
                    }
                }
            }
        }
    }
    if (!ok && lane == 0) atomicExch(status, 5);
}

template <int FMT, int MT, bool EX, bool KS>
static int gemv_prepare(const izb_ctx* ctx, const SkinnyPlanHeader& h) {
    auto kern = skinny_gemv_kernel<FMT, MT, EX, KS>;
    static std::atomic<int> smem_set[IZB_MAX_DEVICES];
    const int dev_slot = ctx->device;
    if (smem_set[dev_slot].load(std::memory_order_relaxed) < h.smem_bytes) {
        IZB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, h.smem_bytes));
        smem_set[dev_slot].store(h.smem_bytes, std::memory_order_relaxed);
    }
    return IZB_OK;
}

template <int FMT, int MT, bool EX, bool KS>
static int gemv_launch_one(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
                           const SkinnyProblem& single) {
    auto kern = skinny_gemv_kernel<FMT, MT, EX, KS>;
    const int rc = gemv_prepare<FMT, MT, EX, KS>(ctx, h);
    if (rc != IZB_OK) return rc;
    if (KS && (h.ksplit < 2 || h.ksplit > GV_MAX_KSPLIT || h.grid != h.total_tiles * h.ksplit)) return IZB_ERR_BAD_ARG;
    IZB_CUDA_TRY(launch_chained_cluster(ctx, KS ? h.ksplit : 1, kern, dim3(h.grid), dim3(GV_THREADS), h.smem_bytes, stream, dev,
                                        single, h.n_probs, h.total_tiles, h.n_stages, h.stage_bytes, h.xq_stage_bytes, h.red_bytes,
                                        h.lite_bytes, h.y_dtype, KS ? h.ksplit : 1, ctx->d_status + 4));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

template <int FMT, int MT>
static int gemv_launch_mt(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
                          const SkinnyProblem& single) {
    if constexpr (MT <= 2) {
        if (h.ksplit > 1)
            return h.extras ? gemv_launch_one<FMT, MT, true, true>(ctx, stream, h, dev, single)
                            : gemv_launch_one<FMT, MT, false, true>(ctx, stream, h, dev, single);
    }
    if (h.ksplit > 1) return IZB_ERR_BAD_ARG;
    return h.extras ? gemv_launch_one<FMT, MT, true, false>(ctx, stream, h, dev, single)
                    : gemv_launch_one<FMT, MT, false, false>(ctx, stream, h, dev, single);
}

template <int FMT>
static int gemv_launch_fmt(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev,
                           const SkinnyProblem& single) {
    switch (h.gemv) {
        case 1: return gemv_launch_mt<FMT, 1>(ctx, stream, h, dev, single);
        case 2: return gemv_launch_mt<FMT, 2>(ctx, stream, h, dev, single);
        case 4: return gemv_launch_mt<FMT, 4>(ctx, stream, h, dev, single);
        default: return IZB_ERR_BAD_ARG;
    }
}

int skinny_gemv_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& h, const SkinnyProblem* dev_probs,
                       const SkinnyProblem* single) {
    if (h.magic != SK_PLAN_MAGIC || !h.gemv) return IZB_ERR_BAD_ARG;
    if (!dev_probs && !single) return IZB_ERR_BAD_ARG;
    static const SkinnyProblem dummy = {};
    const SkinnyProblem& s = single ? *single : dummy;
    switch (h.fmt) {
        case IZB_W_Q8_0: return gemv_launch_fmt<IZB_W_Q8_0>(ctx, stream, h, dev_probs, s);
        case IZB_W_Q4_K: return gemv_launch_fmt<IZB_W_Q4_K>(ctx, stream, h, dev_probs, s);
        default: return IZB_ERR_BAD_ARG;
    }
}

// Can the device hold every cluster of the planned launch at once?  (Each cluster is one row tile and
// the kernel does not loop over tiles when k is split.)
template <int FMT, int MT, bool EX>
static bool gemv_clusters_fit(const izb_ctx* ctx, const SkinnyPlanHeader& h) {
    if (gemv_prepare<FMT, MT, EX, true>(ctx, h) != IZB_OK) return false;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(h.grid);
    cfg.blockDim = dim3(GV_THREADS);
    cfg.dynamicSmemBytes = h.smem_bytes;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(h.ksplit);
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, skinny_gemv_kernel<FMT, MT, EX, true>, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return clusters * h.ksplit >= h.grid;
}

bool skinny_gemv_clusters_fit(const izb_ctx* ctx, const SkinnyPlanHeader& h) {
    if (!ctx || h.ksplit < 2 || h.ksplit > GV_MAX_KSPLIT || h.gemv < 1 || h.gemv > 2) return false;
    // the answer depends on a handful of plan fields only: remember the last few (a decode step asks
    // the same four questions for every layer and token)
    struct Seen { int dev, fmt, gemv, extras, ksplit, smem, grid; bool fit; };
    static std::mutex mu;
    static std::vector<Seen> seen;
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const Seen& e : seen)
            if (e.dev == ctx->device && e.fmt == h.fmt && e.gemv == h.gemv && e.extras == h.extras && e.ksplit == h.ksplit &&
                e.smem == h.smem_bytes && e.grid == h.grid)
                return e.fit;
    }
    int prev = 0;
    if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(ctx->device) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    bool fit = false;
    if (h.fmt == IZB_W_Q8_0) {
        fit = h.gemv == 1 ? (h.extras ? gemv_clusters_fit<IZB_W_Q8_0, 1, true>(ctx, h) : gemv_clusters_fit<IZB_W_Q8_0, 1, false>(ctx, h))
                          : (h.extras ? gemv_clusters_fit<IZB_W_Q8_0, 2, true>(ctx, h) : gemv_clusters_fit<IZB_W_Q8_0, 2, false>(ctx, h));
    } else if (h.fmt == IZB_W_Q4_K) {
        fit = h.gemv == 1 ? (h.extras ? gemv_clusters_fit<IZB_W_Q4_K, 1, true>(ctx, h) : gemv_clusters_fit<IZB_W_Q4_K, 1, false>(ctx, h))
                          : (h.extras ? gemv_clusters_fit<IZB_W_Q4_K, 2, true>(ctx, h) : gemv_clusters_fit<IZB_W_Q4_K, 2, false>(ctx, h));
    }
    (void)cudaSetDevice(prev);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (seen.size() >= 64) seen.erase(seen.begin());
        seen.push_back({ctx->device, h.fmt, h.gemv, h.extras, h.ksplit, h.smem_bytes, h.grid, fit});
    }
    return fit;
}

}  // namespace izb
