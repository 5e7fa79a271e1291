// Dense bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), plain and grouped.
//
//   Y[M, N] = X[M, K] . W[N, K]^T (+ bias) with an optional fused epilogue.
//
// Persistent, warp-specialised, one CTA per SM:
//   warp 0      TMA producer: 128x64 tiles of X and BNx64 tiles of W into a shared-memory ring
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (128 x BN x 16) into one of two
//               TMEM accumulators, commits ring slots back to the producer and accumulators to
//               the epilogue through mbarriers
//   warps 2..9  epilogue: tcgen05.ld the accumulator (two warps per 32 TMEM lanes, half of the
//               columns each), bias / activation in fp32, bf16 or fp32 stores
// Both operands are K-major with the 128-byte swizzle; no cluster multicast anywhere.
#pragma once

#include <cuda.h>

#include "izb_common.cuh"

namespace izb {

enum GemmEpilogue : int {
    GEMM_EPI_NONE = 0,
    GEMM_EPI_GELU = 1,    // exact (erf) GELU
    GEMM_EPI_SILU = 2,    // x * sigmoid(x), FastConformer feed-forward
    GEMM_EPI_SWIGLU = 3,  // W = [gate ; up] rows: out[:, j] = silu(gate_j) * up_j, N_out = N / 2
    GEMM_EPI_GELU_TANH = 4,  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), Whisper fc1
    GEMM_EPI_GLU = 5,        // W = [a ; b] rows: out[:, j] = a_j * sigmoid(b_j), N_out = N / 2 (Conformer pointwise_conv1)
};

struct GemmParams {
    CUtensorMap tmap_a;  // X  viewed as [rows][K], box 64 x 128, 128-byte swizzle
    CUtensorMap tmap_b;  // W  viewed as [expert][N][K], box 64 x BN(/2) x 1, 128-byte swizzle
    void* y;
    const __nv_bfloat16* bias;  // [N] (per expert: [E][N]) or null
    const int* seg_offsets;     // grouped: [E + 1] row offsets of the expert segments, else null
    const __nv_bfloat16* residual;  // [M, ld_res] bf16 added to the finished (activated, rounded) output, or null
    long long ld_res;
    long long ldy;
    int M, N, K;                // grouped: M = total rows of X
    int n_experts;              // 1 when not grouped
    int epilogue;
    int y_dtype;
    int bn;                     // accumulator width in columns: 64, 128 or 256
    int n_out;                  // columns of Y
};

// residual (optional): bf16 [M, ld_res], added to the output after the bias and the epilogue function; the sum is
// what a separate add of two bf16 tensors gives (the product is rounded to the output type first).
int gemm_tc_launch(izb_ctx* ctx, cudaStream_t stream, const void* x, long long ldx, const void* w, const void* bias,
                   void* y, long long ldy, int y_dtype, int M, int N, int K, int epilogue, const int* seg_offsets,
                   int n_experts, const void* residual = nullptr, long long ld_res = 0);

}  // namespace izb
