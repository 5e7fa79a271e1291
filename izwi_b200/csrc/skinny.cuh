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
};
static_assert(sizeof(SkinnyProblem) == 320, "SkinnyProblem layout");

struct alignas(64) SkinnyPlanHeader {
    uint32_t magic;
    int fmt, nt, rt, ks;
    int n_probs, total_tiles;
    int n_stages, stage_bytes, red_bytes, smem_bytes;
    int grid, y_dtype;
    int lite_bytes;  // shared-memory bytes of the descriptor cache
    int pad_[2];
};
static_assert(sizeof(SkinnyPlanHeader) == 64, "SkinnyPlanHeader layout");

// Host side (skinny.cu)
int skinny_plan_build(const izb_ctx* ctx, const izb_linear_args* probs, int n, SkinnyPlanHeader* hdr,
                      SkinnyProblem* out);
int skinny_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& hdr, const SkinnyProblem* dev_probs,
                  const SkinnyProblem* single);

}  // namespace izb
