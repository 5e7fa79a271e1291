// Small-M (decode) linear layers: persistent weight-streaming kernel.
//
// One CTA = 1 producer warp + 4 consumer warps.  The producer streams raw
// weight rows (bf16, or GGML Q8_0 / Q4_K blocks exactly as stored) and the
// matching activation slice into a shared-memory ring with 1-D bulk copies
// (TMA engine) signalled on mbarriers; it runs ahead across tile and problem
// boundaries, so HBM stays busy while consumers finish a tile.  Consumers
// dequantise in registers and feed mma.sync m16n8k16 (bf16, fp32 accumulate)
// with the weight rows as the 16-row operand and up to 8*NT tokens as the
// 8-column operand.  The k order inside an mma step is permuted freely (the
// same permutation on both operands), which is what lets each lane build its
// fragment from the words it loaded without any shuffles.
#pragma once

#include "izb_common.cuh"

namespace izb {

constexpr int SK_CONSUMER_WARPS = 4;
constexpr int SK_THREADS = 32 * (SK_CONSUMER_WARPS + 1);
constexpr int SK_MAX_STAGES = 8;
constexpr uint32_t SK_PLAN_MAGIC = 0x495A4231u;  // "IZB1"

struct alignas(16) SkinnyProblem {
    const uint8_t* w;
    const __nv_bfloat16* x;
    void* y;
    const __nv_bfloat16* bias;
    long long row_bytes;  // bytes of one weight row in global memory
    int N, K, M;
    int ldx, ldy;
    int tile_start;   // global id of this problem's first row tile
    int kc;           // k values per pipeline stage
    int n_chunks;     // ceil(K / kc)
    int chunk_bytes;  // bytes of a full k-chunk of one weight row
    int w_stride;     // shared-memory bytes between weight rows of a stage
    int x_stride;     // shared-memory bytes between activation rows of a stage
    int x_off;        // byte offset of the activation region inside a stage
    int pad_[3];
};
static_assert(sizeof(SkinnyProblem) == 112, "SkinnyProblem layout");

struct alignas(16) SkinnyPlanHeader {
    uint32_t magic;
    int fmt, nt, rt, ks;
    int n_probs, total_tiles;
    int n_stages, stage_bytes, red_bytes, smem_bytes;
    int grid, y_dtype;
    int pad_[3];
};
static_assert(sizeof(SkinnyPlanHeader) == 64, "SkinnyPlanHeader layout");

// Host side (skinny.cu)
int skinny_plan_build(const izb_ctx* ctx, const izb_linear_args* probs, int n, SkinnyPlanHeader* hdr,
                      SkinnyProblem* out);
int skinny_launch(izb_ctx* ctx, cudaStream_t stream, const SkinnyPlanHeader& hdr, const SkinnyProblem* dev_probs,
                  const SkinnyProblem* single);

}  // namespace izb
