// Small-M (decode) linear layers: persistent weight-streaming kernel.
//
// One CTA = 1 producer warp + 4 consumer warps.  The producer streams raw
// weight tiles (bf16, or GGML Q8_0 / Q4_K blocks exactly as stored) and the
// matching activation slice into a shared-memory ring with tiled TMA copies
// (one 3-D box per operand per stage) signalled on mbarriers; it runs ahead
// across tile and problem boundaries, so HBM stays busy while consumers finish
// a tile.  Consumers dequantise in registers and feed mma.sync m16n8k16 (bf16,
// fp32 accumulate) with 16 weight rows as the row operand and up to 8*NT tokens
// as the column operand.  The k order inside an mma step is permuted freely
// (the same permutation on both operands), which lets each lane build its
// fragment from the words it loaded without shuffles.
#pragma once

#include <cuda.h>

#include "izb_common.cuh"

namespace izb {

constexpr int SK_CONSUMER_WARPS = 4;
constexpr int SK_THREADS = 32 * (SK_CONSUMER_WARPS + 1);
constexpr int SK_MAX_STAGES = 8;
constexpr int GV_MAX_STAGES = 12;  // the integer-dot-product kernel alone on an SM runs a deeper ring
constexpr uint32_t SK_PLAN_MAGIC = 0x495A4232u;  // "IZB2"

struct alignas(64) SkinnyProblem {
    CUtensorMap tmap_w;  // weights viewed as [k-box][row][bytes of one k-box of a row]
    CUtensorMap tmap_x;  // activations viewed as [k/64][token][64 bf16], 128-byte swizzle
    void* y;
    const __nv_bfloat16* bias;
    int N, K, M, ldy;
    int tile_start;   // global id of this problem's first row tile
    int n_chunks;     // pipeline stages per row tile
    int nb;           // weight k-boxes per stage
    int kbox;         // k values per weight box
    int w_row_bytes;  // shared-memory bytes per weight row inside one box
    int w_box_bytes;  // TILE_ROWS * w_row_bytes
    int x_off;        // byte offset of the activation region inside a stage
    int stage_tx;     // bytes one full stage delivers (both boxes)
    // decode-step fusions (integer-dot-product kernel only)
    const __nv_bfloat16* norm_w;    // RmsNorm weight [K], or null
    const __nv_bfloat16* residual;  // [M, ld_res] added to the output, or null
    int ld_res;
    int prologue;    // izb_prologue
    float eps;
    int up_chunk0;   // SILU_MUL: 64-k chunk index where the `up` half of the activation rows starts
    int x_half;      // SILU_MUL: byte offset of the `up` chunks inside the stage's activation region
    // integer tensor-core kernel (skinny_imma.cu): its own copy of the activations, made by a kernel in front
    int ldx;
    uint8_t* xq;                    // converted activations in the caller's workspace
    const __nv_bfloat16* x_rows;    // the bf16 activation rows they are made from (ldx apart)
};
static_assert(sizeof(SkinnyProblem) == 384, "SkinnyProblem layout");

struct alignas(64) SkinnyPlanHeader {
    uint32_t magic;
    int fmt, nt, rt, ks;
    int n_probs, total_tiles;
    int n_stages, stage_bytes, red_bytes, smem_bytes;
    int grid, y_dtype;
    int lite_bytes;  // shared-memory bytes of the descriptor cache
    int tc;          // 1: the dequantise-into-tcgen05 kernel (17..64 tokens over block-quantised weights)
    int x_stages;    // tc: depth of the separate activation ring (n_stages / stage_bytes describe the raw weight ring)
    int gemv;        // 1, 2 or 4: the integer-dot-product kernel for that many tokens (block-quantised weights); 0: off
    int xq_stage_bytes;  // gemv: bytes of converted activations per stage (red_bytes holds all stages)
    int extras;          // gemv: some problem carries a prologue or a residual
    int ksplit;          // gemv: CTAs per cluster sharing a row tile, each a slice of its k chunks (1: no clusters)
    int imma;            // 1 or 2: the integer tensor-core kernel for that many groups of 8 tokens; 0: off
    int conv_grid;       // imma: blocks per problem of the activation-conversion launch
    int pad_[10];
};
static_assert(sizeof(SkinnyPlanHeader) == 128, "SkinnyPlanHeader layout");

#ifdef __CUDACC__
// The scalar fields of a problem descriptor, cached in shared memory at kernel start: a CTA meets
// a different problem on almost every tile, and walking the descriptors in global memory was a
// chain of dependent long-latency loads per tile.
struct alignas(16) ProbLite {
    void* y;
    const __nv_bfloat16* bias;
    int N, M, ldy, tile_start;
    int n_chunks, nb, kbox, w_row_bytes;
    int w_box_bytes, x_off, stage_tx;
    int extras;  // the problem carries a prologue or a residual: the roles read those fields from its descriptor
};
static_assert(sizeof(ProbLite) == 64, "ProbLite layout");
constexpr int SK_LITE_MAX = 160;  // problems cached; beyond that the descriptor is read from global memory

__device__ __forceinline__ ProbLite lite_from(const SkinnyProblem& q) {
    ProbLite l;
    l.y = q.y; l.bias = q.bias;
    l.N = q.N; l.M = q.M; l.ldy = q.ldy; l.tile_start = q.tile_start;
    l.n_chunks = q.n_chunks; l.nb = q.nb; l.kbox = q.kbox; l.w_row_bytes = q.w_row_bytes;
    l.w_box_bytes = q.w_box_bytes; l.x_off = q.x_off; l.stage_tx = q.stage_tx;
    l.extras = (q.prologue != 0 || q.residual != nullptr) ? 1 : 0;
    return l;
}

// Index of the problem that owns `tile`: last p with tile_start[p] <= tile (binary search).
__device__ __forceinline__ int find_problem(const ProbLite* lite, int n_cached, const SkinnyProblem* plist, int n_probs,
                                            int tile) {
    int lo = 0, hi = n_probs;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        const int start = mid < n_cached ? lite[mid].tile_start : plist[mid].tile_start;
        if (start <= tile) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ float half_bits_to_f32(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xFFFFu)));
}

// Four int8 in a word -> two f16x2 registers holding the exact integers.
// byte ^ 0x80 is q+128 as an unsigned byte; under the high byte 0x64 it reads as the fp16
// value 1024 + q + 128 (fp16 has a unit step from 1024 to 2048), and one packed subtraction
// of 1152 leaves q.
__device__ __forceinline__ void s8x4_to_f16x4(uint32_t w, uint32_t& p01, uint32_t& p23) {
    const uint32_t u = w ^ 0x80808080u;
    const uint32_t h01 = prmt(u, 0x64646464u, 0x5140), h23 = prmt(u, 0x64646464u, 0x7362);
    asm("sub.f16x2 %0, %1, %2;" : "=r"(p01) : "r"(h01), "r"(0x64806480u));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(p23) : "r"(h23), "r"(0x64806480u));
}

// A bf16 pair -> the same two values as an fp16 pair.  Exact for 2^-24 <= |x| <= 65504 (bf16
// carries 8 significant bits, fp16 11); larger magnitudes saturate to +-65504.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t b) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(b & 0xFFFF0000u)), "f"(__uint_as_float(b << 16)));
    return r;
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hfma2_bf16(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t bcast_bf16x2(float v) { return pack_bf16x2(v, v); }

#endif  // __CUDACC__

// Host side (skinny.cu)
int skinny_plan_build(const izb_ctx* ctx, const izb_linear_args* probs, int n, SkinnyPlanHeader* hdr,
                      SkinnyProblem* out);
int skinny_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& hdr, const SkinnyProblem* dev_probs,
                  const SkinnyProblem* single);
// skinny_tc.cu
int skinny_tc_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& hdr, const SkinnyProblem* dev_probs,
                     const SkinnyProblem* single);
// skinny_gemv.cu
bool skinny_gemv_clusters_fit(const izb_ctx* ctx, const SkinnyPlanHeader& hdr);  // all of hdr.grid / hdr.ksplit clusters resident at once
int skinny_gemv_max_tokens();  // widest token group the planner hands to the integer-dot-product kernel
int skinny_gemv_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& hdr, const SkinnyProblem* dev_probs,
                       const SkinnyProblem* single);
// skinny_imma.cu
bool skinny_imma_takes(const izb_linear_args* probs, int n);  // 3..16 tokens, block-quantised, every problem with room for its converted activations
size_t skinny_imma_xq_bytes(int64_t M, int64_t K);            // workspace bytes of one problem's converted activations (0: not eligible)
int skinny_imma_min_tokens();
int skinny_imma_max_tokens();
bool skinny_imma_format_ok(int fmt);
int skinny_imma_plan_build(const izb_ctx* ctx, const izb_linear_args* probs, int n, SkinnyPlanHeader* hdr, SkinnyProblem* out);
int skinny_imma_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& hdr, const SkinnyProblem* dev_probs,
                       const SkinnyProblem* single);

}  // namespace izb
