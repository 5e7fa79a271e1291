/*
 * izwi_b200 — C ABI of the B200 (sm_100a) matrix-multiplication hot path of
 * izwi-core: decode/prefill linear layers over dense bf16 and GGML
 * block-quantised (Q8_0, Q4_K) weights, SwiGLU glue, block dequantisation,
 * and the top-k mixture-of-experts path.
 *
 * Conventions (identical to the reference's Candle `Linear`):
 *   - row-major; W is [N = out, K = in]; X is [M, K]; Y = X . W^T (+ bias).
 *   - every pointer is a DEVICE pointer unless the name starts with `host_`.
 *   - entry points never allocate or free device memory (izb_ctx_create /
 *     izb_ctx_destroy excepted); the caller owns x / w / y / workspace.
 *   - every launch goes to the caller's stream; entry points are re-entrant.
 *   - return value: IZB_OK (0) or a negative izb_status. No exceptions cross
 *     this boundary and there is no CPU fallback.
 *
 * File:line citations name the interface of the reference
 * (crates/izwi-core/src/...) that the entry point stands behind.
 */
#ifndef IZWI_B200_H
#define IZWI_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct izb_ctx izb_ctx;
typedef void* izb_stream; /* a cudaStream_t / CUstream */

typedef enum izb_status {
    IZB_OK = 0,
    IZB_ERR_BAD_ARG = -1,     /* null / misaligned pointer, negative size, shape mismatch */
    IZB_ERR_UNSUPPORTED = -2, /* shape or dtype outside what the kernels cover */
    IZB_ERR_LAUNCH = -3,      /* CUDA runtime refused the launch or the copy */
    IZB_ERR_TIMEOUT = -4,     /* a bounded device-side wait gave up */
    IZB_ERR_NO_DEVICE = -5,   /* no sm_100 device / driver entry point missing */
    IZB_ERR_SCRATCH_TOO_SMALL = -6 /* the problem needs more than the library's fixed scratch array */
} izb_status;

typedef enum izb_dtype { IZB_BF16 = 0, IZB_F32 = 1, IZB_F16 = 2 } izb_dtype;

/* Weight storage formats: dense bf16 (Candle `Linear` weight) or raw GGML
 * blocks exactly as they sit in a GGUF file (Candle `QTensor` data).
 * Q8_0 and Q4_K are multiplied in place by the streaming kernels.  Q6_K (some tensors of
 * Q4_K_M files; 210-byte super-blocks, so rows are not 16-byte aligned for tiled copies) is
 * supported by izb_dequantize and, in izb_linear, through the bf16 copy in `workspace`. */
typedef enum izb_wfmt { IZB_W_BF16 = 0, IZB_W_Q8_0 = 1, IZB_W_Q4_K = 2, IZB_W_Q6_K = 3 } izb_wfmt;

int32_t izb_version(void);
/* The gate of this library's kernels: the environment variable IZWI_B200_KERNELS, read once per
 * process with the rule the reference applies to IZWI_FUSED_KERNELS (`use_fused_kernels`,
 * kernels/mod.rs:46-57): unset means on; set, it is on only for 1 / true / yes / on (any case,
 * surrounding blanks ignored).  The entry points do not consult it: the host layer above does, and
 * takes its own path (the reference's Candle ops) when it returns 0. */
int32_t izb_kernels_enabled(void);
const char* izb_status_string(int32_t status);

/* One context per device and host thread group; owns a small device status
 * word that kernels use to report a bounded wait that ran out. */
int32_t izb_ctx_create(int32_t device, izb_ctx** out);
int32_t izb_ctx_destroy(izb_ctx* ctx);
/* Synchronises `stream`, then returns IZB_ERR_TIMEOUT if any kernel launched
 * through this context recorded a wait that gave up, or IZB_ERR_BAD_ARG if the embedding lookup met
 * a token id outside its table (and clears the record).  Call it with the context quiescent: a
 * record made by a kernel of another stream while this call runs may be cleared unseen. */
int32_t izb_ctx_check(izb_ctx* ctx, izb_stream stream);
/* Launches a one-warp kernel that waits on a barrier nothing completes, through the bounded wait all
 * pipeline kernels share: after the limit (about a second) it records the time-out and returns, so
 * the next izb_ctx_check reports IZB_ERR_TIMEOUT once and the context stays usable.  Lets a host
 * test its handling of that status without any kernel misbehaving.  No counterpart in the reference. */
int32_t izb_ctx_selftest_wait_timeout(izb_ctx* ctx, izb_stream stream);
/* Number of kernels this context has launched so far (diagnostic counter). */
int64_t izb_ctx_launch_count(const izb_ctx* ctx);

/* Byte size of `rows x cols` values in a block format; fails unless
 * rows*cols is a multiple of the block size (the reference's rule; a matrix that is to be
 * multiplied needs every row to be whole blocks, which izb_linear checks itself).
 * Replaces `quantized_storage_bytes` (models/architectures/qwen3/core.rs:891-909). */
int32_t izb_quantized_storage_bytes(int32_t wfmt, int64_t rows, int64_t cols, size_t* out_bytes);

/* Block dequantisation, bit-exact with GGML: Q8_0 `d*q`; Q4_K
 * `(d*sc)*q - (dmin*m)`; Q6_K `(d*sc)*q`; every product rounded separately.  `out_dtype` F32 is
 * exact; BF16 rounds the fp32 value to nearest-even.
 * Replaces `QTensor::dequantize` at models/shared/weights/gguf.rs:131 and
 * qwen3/core.rs:853-858. */
int32_t izb_dequantize(izb_ctx* ctx, izb_stream stream, int32_t wfmt, const void* raw,
                       int64_t n_elems, int32_t out_dtype, void* out);

/* Element-wise function fused into the output of a linear layer. */
typedef enum izb_epilogue {
    IZB_EPI_NONE = 0,
    IZB_EPI_GELU = 1,   /* exact erf GELU: the reference's `gelu_erf()` call sites
                           (granite_speech/asr/runtime.rs:1639, qwen3/tts/speech_tokenizer.rs:670,891) */
    IZB_EPI_SILU = 2,   /* x*sigmoid(x): FastConformer feed-forward (parakeet/asr/mod.rs:766-772) */
    IZB_EPI_SWIGLU = 3, /* W = [gate; up] rows: y[:, j] = silu(gate_j) * up_j, y has N/2 columns:
                           `Qwen3Mlp::forward` gate/up + silu-mul in one pass (qwen3/core.rs:1787-1795) */
    IZB_EPI_GELU_TANH = 4, /* 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))): the reference's `Tensor::gelu()` call
                           sites, Whisper `mlp_linear1` + GELU (whisper/model.rs:311-317) and the Qwen3-ASR audio
                           tower (qwen3/asr/audio.rs:385,667-668).  Evidence that `gelu()` is this form and not
                           the erf one: the reference keeps the two apart (it calls `gelu_erf()` where it wants
                           the exact form), and every GELU it writes out itself under that name is this formula
                           (audio/codec.rs:135-137, voxtral/realtime/audio.rs:73-88, lfm25_audio/conformer.rs:
                           1266-1280).  Candle's source is not part of the reference tree, so this is inferred. */
    IZB_EPI_GLU = 5     /* W = [a; b] rows: y[:, j] = a_j * sigmoid(b_j), y has N/2 columns: the gated linear unit
                           behind `pointwise_conv1` of the Conformer convolution module
                           (parakeet/asr/mod.rs:831-834) */
} izb_epilogue;

/* Function of the activations in front of a linear layer.  Inside the one- and two-token kernel both
 * skip the bf16 rounding of the intermediate the separate launches would store. */
typedef enum izb_prologue {
    IZB_PRO_NONE = 0,
    IZB_PRO_RMSNORM = 1,  /* y = W (x * rsqrt(mean(x^2) + eps) * norm_weight): the RmsNorm in front of the
                             QKV and gate/up projections (qwen3/core.rs:1868, 1874) */
    IZB_PRO_SILU_MUL = 2  /* x is [M, 2K] = [gate | up]; y = W (silu(gate) * up): the product in front of
                             `down_proj` (qwen3/core.rs:1787-1795) */
} izb_prologue;

/* One linear layer.  Replaces `impl Module for Qwen3Projection::forward`
 * (qwen3/core.rs:791-832): Dense -> `Linear::forward` (:794), Quantized ->
 * `QMatMul::forward` (:812) with the dtype casts around it folded away
 * (activations stay bf16, accumulation is fp32). */
typedef struct izb_linear_args {
    int32_t wfmt;      /* izb_wfmt */
    int32_t y_dtype;   /* izb_dtype of y: bf16, fp32 or fp16 */
    const void* x;     /* [M, ldx] in x_dtype (bf16 unless set otherwise below) */
    const void* w;     /* [N, K] in wfmt, rows contiguous */
    const void* bias;  /* [N] bf16 or NULL */
    void* y;           /* [M, ldy] */
    int64_t M, N, K;
    int64_t ldx, ldy;  /* row strides in elements */
    void* workspace;   /* NULL unless izb_linear_workspace_bytes_ex() > 0 for this call */
    size_t workspace_bytes;
    int32_t epilogue;  /* izb_epilogue fused after the bias add */
    int32_t prologue;  /* izb_prologue applied to x on its way into the product */
    /* What a decoder layer does around a projection (qwen3/core.rs:1863-1881), for every weight format
     * and token count.  `residual` is added by the epilogue of whichever kernel runs the product.
     * `prologue` is computed inside the one- and two-token block-format kernel (see
     * izb_linear_fusion_max_tokens: nothing is stored in between); on every other route izb_linear
     * itself launches the row norm or the SiLU-multiply into the tail of `workspace` (bf16, as the
     * reference's separate ops store it) and runs the product on that: size the workspace with
     * izb_linear_workspace_bytes_args.  The grouped launch (izb_linear_group_*) takes prologues only
     * for the in-kernel case. */
    const void* norm_weight; /* IZB_PRO_RMSNORM: bf16 [K], 16-byte aligned */
    const void* residual;    /* bf16 [M, ld_residual] added to the output after the bias; NULL = none */
    int64_t ld_residual;
    float norm_eps;
    /* izb_dtype of x.  IZB_BF16 (0, so a zeroed struct keeps its meaning) feeds the kernels directly.
     * IZB_F32 / IZB_F16 activations, the dtypes the reference's CUDA policy gives the QMatMul and Whisper
     * / Parakeet call sites (qwen3/core.rs:772-789, backends/device.rs:466-484), are rounded to bf16 once
     * by a cast launch into the tail of `workspace` (size it with izb_linear_workspace_bytes_args); not
     * together with `prologue`.  The arithmetic is bf16 x bf16 -> fp32 whatever the input type. */
    int32_t x_dtype;
} izb_linear_args;

/* M <= 32 (or <= 64 for the block formats) runs a weight-streaming kernel; larger M runs the
 * tcgen05/TMEM GEMM.  Block-quantised weights with M > 64 are first dequantised to bf16 into
 * `workspace` (N*K*2 bytes, see izb_linear_workspace_bytes); without a workspace they are
 * processed 64 token rows at a time by the streaming kernels instead.  Q6_K weights always go
 * through the workspace (any M; IZB_ERR_BAD_ARG without one).
 * Streaming kernels for the block formats: one or two tokens take integer dot products of the codes
 * with the activations re-expressed per 32-value block as 16-bit fixed point (absolute error at most
 * 2^-15 of the block's largest magnitude; a non-finite activation makes its token's outputs
 * non-finite); 3..16 tokens (Q8_0: ..32) lift the codes to fp16 / bf16 tensor-core operands in
 * registers; up to 64 tokens dequantise to bf16 in shared memory for tcgen05.  All accumulate in fp32. */
size_t izb_linear_workspace_bytes(int32_t wfmt, int64_t M, int64_t N, int64_t K);
/* The same query for a call that also fuses `epilogue`: over Q8_0 / Q4_K weights a fused epilogue
 * always runs on the GEMM and therefore needs the N*K*2-byte workspace, whatever M is (izb_linear
 * returns IZB_ERR_BAD_ARG without it).  Query with the epilogue the call will carry, allocate once,
 * pass it in `workspace`. */
size_t izb_linear_workspace_bytes_ex(int32_t wfmt, int64_t M, int64_t N, int64_t K, int32_t epilogue);
/* Row widths: K must be a whole number of blocks (32 for Q8_0, 256 for Q4_K / Q6_K; IZB_ERR_BAD_ARG
 * otherwise) and a multiple of 8 for bf16.  The streaming kernels walk 256 values of a block-format
 * row (64 of a bf16 row) at a time; other widths (a Q8_0 row of 384 values, say) run on the GEMM,
 * for which block formats need the workspace (the query above accounts for it; without one the
 * answer is IZB_ERR_UNSUPPORTED). */
/* The query for a whole call as it will be made (format, shape, epilogue, prologue AND x_dtype): bytes
 * of `workspace` izb_linear needs for exactly these arguments.  One case is a wish, not a need: 3..8
 * tokens over Q8_0 weights on the streaming route run on the int8 tensor-core kernel when the
 * workspace has room for the activations in its 16-bit block fixed point (K/32 * 72 * 16 bytes, what
 * this query returns then), and on the floating-point consumers, about 8 % slower, without it. */
size_t izb_linear_workspace_bytes_args(const izb_linear_args* args);
int32_t izb_linear(izb_ctx* ctx, izb_stream stream, const izb_linear_args* args);
/* Largest M for which the kernel itself computes `prologue` for weights in `wfmt` (0: never; the
 * call is still accepted above it, through the workspace). */
int32_t izb_linear_fusion_max_tokens(int32_t wfmt);

/* Thin typed forms of izb_linear (y is bf16, contiguous strides). */
int32_t izb_linear_bf16(izb_ctx* ctx, izb_stream stream, const void* x, const void* w,
                        const void* bias, void* y, int64_t M, int64_t N, int64_t K);
int32_t izb_linear_q8_0(izb_ctx* ctx, izb_stream stream, const void* x, const void* w,
                        void* y, int64_t M, int64_t N, int64_t K);
int32_t izb_linear_q4_k(izb_ctx* ctx, izb_stream stream, const void* x, const void* w,
                        void* y, int64_t M, int64_t N, int64_t K);

/* A group of independent small-M linear layers executed by ONE persistent
 * launch that streams all weights back to back (the projections of a decode
 * step that do not depend on one another, separate q/k/v or gate/up matrices,
 * the experts one token selects).  All problems share wfmt and y_dtype and
 * have M <= 64.  The plan is built on the host, copied by the caller to the
 * device (plain bytes), and can be launched any number of times.
 * No counterpart in the reference, which issues one Candle op per projection
 * (qwen3/core.rs:1599,1624,1787,1796). */
size_t izb_linear_group_plan_bytes(int32_t n_problems);
int32_t izb_linear_group_plan(izb_ctx* ctx, const izb_linear_args* problems, int32_t n_problems,
                              void* host_plan, size_t host_plan_bytes);
int32_t izb_linear_group_launch(izb_ctx* ctx, izb_stream stream, const void* host_plan,
                                const void* dev_plan);
/* One step of a planned group for a caller whose tensors live in host memory,
 * as the reference's CPU tensors do (its matmul reads and returns host
 * tensors: models/shared/weights/gguf.rs:75-85): copies `in_bytes` from
 * `host_in` to `dev_in` (the buffer the plan's x pointers lie in), launches
 * the group, copies `out_bytes` from `dev_out` (where the plan's y pointers
 * lie) to `host_out`, and returns when the results are in `host_out`.  Host
 * buffers should be page-locked; either byte count may be 0 to skip that
 * copy.  The y pointers of the planned problems may themselves lie in
 * page-locked host memory that the device can address (cudaHostAlloc /
 * cudaHostRegister under unified addressing): the kernels then store every
 * result straight into it while they run, and out_bytes = 0 (18 % less time
 * per step on the 112-projection decode stack than copying 0.7 MB back).  x
 * must stay in device memory: every CTA that works on a problem reads it. */
int32_t izb_linear_group_launch_host(izb_ctx* ctx, izb_stream stream, const void* host_plan,
                                     const void* dev_plan, const void* host_in, void* dev_in,
                                     size_t in_bytes, const void* dev_out, void* host_out,
                                     size_t out_bytes);

/* Size of the scratch array built into the library image (bytes). */
#define IZB_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
size_t izb_static_scratch_bytes(void);

/* Prefill-size linear layer over Q8_0 / Q4_K weights for callers that cannot hand over a
 * workspace and must not trigger a device allocation: host runtimes that gave the whole device to
 * their own memory pool at start-up, and latency-sensitive audio threads for which a cudaMalloc
 * (which can synchronise the whole device) in the middle of a request is not acceptable.
 * Same result as izb_linear with a workspace: the weights are dequantised to bf16 and multiplied
 * on the tensor cores; the bf16 copy goes into a fixed IZB_STATIC_SCRATCH_BYTES array that every
 * GPU loading this library holds until the process exits.  x is [M, K] bf16 contiguous, y is
 * [M, N] (N/2 columns with IZB_EPI_SWIGLU) contiguous.
 *   - N*K*2 bytes must fit the array, else IZB_ERR_SCRATCH_TOO_SMALL and nothing is launched.
 *   - calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - the first call on a device looks up the array's device address (a one-off host-side
 *     query); make that first call outside any stream capture.  The CUDA runtime loads a
 *     library's device code on first use, so it is also during this first call that the array
 *     becomes resident and the device's free memory drops by IZB_STATIC_SCRATCH_BYTES, once.
 *   - all calls on a device share the one array and it keeps the previous call's contents (each
 *     call rewrites the part it reads, so nothing needs clearing): two calls that may overlap
 *     on the GPU (different streams) race and must be ordered by the caller.
 * This entry point has no counterpart in the reference. */
int32_t izb_linear_quantized_static(izb_ctx* ctx, izb_stream stream, int32_t wfmt, const void* x,
                                    const void* w, const void* bias, void* y, int32_t y_dtype,
                                    int64_t M, int64_t N, int64_t K, int32_t epilogue);

/* out = silu(gate) * up, fp32 math, bf16 storage; gate/up/out are [rows, cols]
 * views with their own row strides so the two halves of a fused gate/up
 * output can be passed in place.
 * Replaces `try_fused_silu_mul_with_status` (kernels/mod.rs:94-108 ->
 * kernels/cuda.rs:51-62) as called by `Qwen3Mlp::forward` (qwen3/core.rs:1788). */
int32_t izb_silu_mul(izb_ctx* ctx, izb_stream stream, const void* gate, const void* up, void* out,
                     int64_t rows, int64_t cols, int64_t ld_gate, int64_t ld_up, int64_t ld_out);

/* ---- top-k mixture-of-experts feed-forward ------------------------------------------------
 * The reference has no MoE code (no counterpart to cite); the rules are this library's own:
 * experts are picked by router logit, equal logits resolve to the lowest expert id, the weights
 * are the softmax over the picked logits, permuted rows are ordered by expert and then by
 * ascending (token, slot), and the combine adds slots in ascending order in fp32. */

/* Router and expert choice in one launch: logits[T, E] = x[T, H] . w_router[E, H]^T (+ router_bias[E]),
 * fp32, written to logits_out; idx_out [T, k] int32 and weights_out [T, k] fp32 as izb_moe_topk gives them
 * for those logits.  x bf16 with rows ld_x apart, w_router and router_bias bf16.  Uses a small per-context
 * counter area: calls on one context must be ordered with respect to one another (one stream, or events).
 * H not a multiple of 32, unaligned operands or more than 16384 tokens run izb_linear + izb_moe_topk. */
int32_t izb_moe_route(izb_ctx* ctx, izb_stream stream, const void* x, int64_t ld_x, const void* w_router,
                      const void* router_bias, int64_t T, int64_t H, int64_t E, int32_t top_k,
                      void* logits_out, void* idx_out, void* weights_out);
/* logits [T, E] fp32 -> idx [T, k] int32 (descending logit) and weights [T, k] fp32. */
int32_t izb_moe_topk(izb_ctx* ctx, izb_stream stream, const void* logits, int64_t T, int64_t E,
                     int32_t top_k, void* idx_out, void* weights_out);
/* idx [pairs] int32 -> offsets [E + 1], perm [pairs] (pair id landing in each permuted row) and
 * inv [pairs] (permuted row of each pair); pair id = token * k + slot. */
int32_t izb_moe_permute(izb_ctx* ctx, izb_stream stream, const void* idx, int64_t pairs, int64_t E,
                        void* offsets_out, void* perm_out, void* inv_out);
/* x_perm[r, :] = x[perm[r] / k, :], bf16 rows of H values. */
int32_t izb_moe_gather(izb_ctx* ctx, izb_stream stream, const void* x, int64_t ldx, const void* perm,
                       int32_t top_k, int64_t rows, int64_t H, void* x_perm);
/* For every expert e: y[offsets[e]:offsets[e+1]] = epilogue(x_perm[same rows] . w[e]^T), w is
 * [E, N, K] bf16; tcgen05 GEMM over row tiles that never cross an expert boundary. */
int32_t izb_moe_grouped_gemm(izb_ctx* ctx, izb_stream stream, const void* x_perm, const void* w,
                             const void* offsets, void* y, int32_t y_dtype, int64_t rows, int64_t N,
                             int64_t K, int64_t E, int32_t epilogue);
/* y[t, :] = sum_slot weights[t, slot] * y_perm[inv[t*k + slot], :]  (bf16 in, fp32 sum, bf16 out). */
int32_t izb_moe_combine(izb_ctx* ctx, izb_stream stream, const void* y_perm, const void* inv,
                        const void* weights, int64_t T, int32_t top_k, int64_t H, void* y);

typedef struct izb_moe_args {
    const void* x;            /* [T, H] bf16 */
    const void* w_router;     /* [E, H] bf16 */
    const void* router_bias;  /* [E] bf16 or NULL */
    const void* w_gate_up;    /* [E, 2*I, H] bf16: gate rows then up rows of each expert */
    const void* w_down;       /* [E, H, I] bf16 */
    void* y;                  /* [T, H] bf16 */
    int64_t T, H, I, E;
    int32_t top_k;
    int32_t reserved_;
    void* workspace;          /* izb_moe_workspace_bytes(), 256-byte aligned */
    size_t workspace_bytes;
} izb_moe_args;

size_t izb_moe_workspace_bytes(int64_t T, int64_t H, int64_t I, int64_t E, int32_t top_k);
/* router + top-k (izb_moe_route) -> permute -> gather -> grouped gate/up GEMM with SwiGLU -> grouped down
 * GEMM -> combine, all on `stream`.  The workspace starts with logits [T,E] fp32, idx [T,k] int32 and
 * weights [T,k] fp32 (each region 256-byte aligned), which callers may read back. */
int32_t izb_moe_forward(izb_ctx* ctx, izb_stream stream, const izb_moe_args* args);

/* ---- sharded configurations: NCCL over NVLink --------------------------------------------
 * One process per GPU.  The reference is single-device (device ordinal fixed to 0,
 * backends/device.rs:632-636) and has no collective call site, so there is nothing to cite.
 * Rank 0 makes a 128-byte id, the host passes it to every rank by its own means, each rank calls
 * izb_comm_init.  All calls of a communicator must be issued in the same order on every rank. */
typedef struct izb_comm izb_comm;
int32_t izb_comm_unique_id(void* out_128_bytes);
int32_t izb_comm_init(izb_ctx* ctx, int32_t world, int32_t rank, const void* unique_id_128_bytes,
                      izb_comm** out);
int32_t izb_comm_destroy(izb_comm* comm);
/* Tensor parallel: in-place sum of `count` elements over all ranks (after a row-split O or down
 * projection). */
int32_t izb_tp_allreduce(izb_comm* comm, izb_stream stream, void* buf, int64_t count, int32_t dtype);
/* Every rank contributes bytes_per_rank bytes; recv holds world * bytes_per_rank (routing counts). */
int32_t izb_comm_allgather(izb_comm* comm, izb_stream stream, const void* send, void* recv,
                           int64_t bytes_per_rank);
/* Expert parallel: rows of row_bytes bytes; send holds the rows for rank 0, then rank 1, ...
 * (host_send_rows[p] of them), recv receives host_recv_rows[p] rows from each rank in rank
 * order.  The row counts are host arrays of `world` entries. */
int32_t izb_ep_alltoall(izb_comm* comm, izb_stream stream, const void* send,
                        const int64_t* host_send_rows, void* recv, const int64_t* host_recv_rows,
                        int64_t row_bytes);

/* One-shot all-reduce over NVLink peer memory for decode-size messages (a few KB to 1 MB): one
 * kernel pushes this rank's partial sums into every peer's buffer with plain stores, signals,
 * waits (bounded) for the peers and adds the contributions in rank order (deterministic).  Set-up:
 * every rank calls izb_ar_create (allocates its buffer), passes its 64-byte handle to all ranks,
 * and calls izb_ar_connect with the `world` handles in rank order.  izb_ar_allreduce is in place,
 * needs count*elem_size <= max_bytes, a 4-byte aligned buffer and a byte size that is a multiple
 * of 4; it can be replayed from a CUDA graph.
 * Messages above 1 MB (when max_bytes allows them: the sums after a row-split projection at
 * prefill sizes) take a two-shot bandwidth path instead: the operand sits in the rank's region, each
 * rank reduces 1/world of it with peer loads and stores the result chunk into every region, all in
 * ONE kernel that returns when the whole result has landed (16-byte aligned buffer,
 * IZB_ERR_UNSUPPORTED otherwise; a last 4, 8 or 12 bytes beyond whole 16-byte units go through the
 * one-shot kernel in a launch of their own).  izb_ar_allreduce copies the operand into the
 * region and the result out of it (three launches).  A caller that can place the operand itself
 * skips both copies: izb_ar_operand(which) is where the row-split projection writes its output
 * (a local device pointer of max_bytes bytes; which = 0 or 1: two buffers, so that the sum of one
 * projection can run on a second stream while the next projection writes the other),
 * izb_ar_allreduce_region(which, count, dtype) sums it over the ranks (one launch), and the sum is
 * read at izb_ar_result(which).  Calls on one buffer must be ordered by the caller (its operand is
 * rewritten only after the previous sum on that buffer has completed; every rank issues the same
 * calls in the same order); izb_ar_allreduce uses the same two buffers in turn, so do not interleave
 * it with region calls.  No counterpart in the reference (single device). */
typedef struct izb_ar izb_ar;
int32_t izb_ar_create(izb_ctx* ctx, int32_t world, int32_t rank, size_t max_bytes, izb_ar** out);
int32_t izb_ar_local_handle(izb_ar* ar, void* out_64_bytes);
int32_t izb_ar_connect(izb_ar* ar, const void* handles_world_x_64_bytes);
size_t izb_ar_max_bytes(const izb_ar* ar);
int32_t izb_ar_allreduce(izb_ar* ar, izb_stream stream, void* buf, int64_t count, int32_t dtype);
void* izb_ar_operand(izb_ar* ar, int32_t which);
const void* izb_ar_result(izb_ar* ar, int32_t which);
int32_t izb_ar_allreduce_region(izb_ar* ar, izb_stream stream, int32_t which, int64_t count, int32_t dtype);
int32_t izb_ar_destroy(izb_ar* ar);

/* Expert-parallel dispatch and return over NVLink peer memory (no host read per layer, no NCCL
 * launch): tokens are data-parallel, experts sit in contiguous blocks of n_experts / world per rank.
 * Set-up as for izb_ar_*: izb_ep_create on every rank (allocates the rank's receive and return
 * buffers for at most max_tokens_local tokens per rank and step), exchange the 64-byte handles,
 * izb_ep_connect.  Per layer, after the local routing (izb_moe_topk / permute / gather):
 *   izb_ep_dispatch(x, ld_x, perm, offsets, pairs): exchanges the per-expert counts, stores every row
 *     into its owner's receive buffer (rows grouped by local expert, then source rank) and, in the
 *     same kernel, waits for the rows of all ranks (two launches in all); with perm = NULL x holds the `pairs` rows already in expert-major order
 *     (izb_moe_gather's output), otherwise x is the token matrix [tokens, hidden] (rows ld_x apart)
 *     and row r is read from x[perm[r] / top_k]: the gather is fused into the dispatch; afterwards izb_ep_recv_rows() / izb_ep_recv_offsets() [local experts + 1]
 *     feed izb_moe_grouped_gemm with rows = izb_ep_recv_capacity_rows();
 *   izb_ep_return(y_rows): stores each result row back to the rank it came from, at the row it left
 *     from in that rank's permuted order, and waits for this rank's rows (one launch): izb_ep_returned_rows()
 *     then feeds izb_moe_combine.
 * All waits are bounded (izb_ctx_check reports IZB_ERR_TIMEOUT); the launches can be captured in a
 * CUDA graph.  No counterpart in the reference (single device). */
typedef struct izb_ep izb_ep;
int32_t izb_ep_create(izb_ctx* ctx, int32_t world, int32_t rank, int32_t n_experts, int32_t hidden,
                      int64_t max_tokens_local, int32_t top_k, izb_ep** out);
int32_t izb_ep_local_handle(izb_ep* ep, void* out_64_bytes);
int32_t izb_ep_connect(izb_ep* ep, const void* handles_world_x_64_bytes);
int64_t izb_ep_recv_capacity_rows(const izb_ep* ep);
void* izb_ep_recv_rows(const izb_ep* ep);
const void* izb_ep_recv_offsets(const izb_ep* ep);
const void* izb_ep_returned_rows(const izb_ep* ep);
int32_t izb_ep_dispatch(izb_ep* ep, izb_stream stream, const void* x, int64_t ld_x, const void* perm,
                        const void* offsets, int64_t pairs);
int32_t izb_ep_return(izb_ep* ep, izb_stream stream, const void* y_rows);
int32_t izb_ep_destroy(izb_ep* ep);

/* ---- glue around the projections of a decode step ---------------------------------------------
 * RMS normalisation of bf16 rows: out = h * rsqrt(mean(h^2) + eps) * weight, fp32 arithmetic, one
 * rounding; h = x, or x + residual rounded to bf16 (the reference adds the residual as a bf16
 * tensor first), in which case `sum_out` (may alias neither input) receives h when not NULL.
 * Serves the layer norms and, with rows = tokens * heads and cols = head_dim, the q/k norms.
 * Replaces try_fused_rms_norm (kernels/mod.rs:143-157, kernels/cuda.rs:78-84 -> candle_nn::ops::
 * rms_norm) and RmsNorm::forward at models/architectures/qwen3/core.rs:1446-1463. */
int32_t izb_rms_norm(izb_ctx* ctx, izb_stream stream, const void* x, const void* weight,
                     const void* residual, void* out, void* sum_out, int64_t rows, int64_t cols,
                     int64_t ld_x, int64_t ld_residual, int64_t ld_out, int64_t ld_sum, float eps);
/* Arg-max of every row of a bf16 / fp32 matrix (greedy token choice over the lm_head logits):
 * the lowest index among equal maxima; NaN is never selected (a row of only NaN gives 0, -inf).
 * `out_val` may be NULL.  A few long rows (16384 columns or more) are split across CTAs through a
 * small per-context scratch area, so such calls on one context must be ordered with respect to one
 * another (one stream, or events between streams).  Replaces `argmax`
 * (models/architectures/qwen3/chat.rs:574-601), which copies the logits row to the host and reduces
 * there. */
int32_t izb_argmax_rows(izb_ctx* ctx, izb_stream stream, const void* x, int32_t x_dtype, int64_t rows,
                        int64_t cols, int64_t ld_x, int32_t* out_idx, float* out_val);

/* Token choice beyond the arg-max, on the device, one draw per row of a bf16 / fp32 logits matrix, by the
 * rules of the reference's host-side samplers (`sample_from_logits`, models/architectures/lfm25_audio/
 * sampling.rs:65-160; `sample_semantic`, models/architectures/qwen3/tts/mod.rs:2293-2440):
 * temperature <= 1e-5 gives the arg-max; otherwise v = logit / temperature over the finite logits, the
 * top_k largest are kept (0: all; equal values keep the lowest indices), p = softmax(v) over those, the
 * smallest prefix in descending order of p whose mass reaches max(top_p, 1e-6) is kept (top_p >= 1: all),
 * and the candidates are walked (in descending order when top_k or top_p cut anything, in index order
 * otherwise) up to the first whose cumulative mass reaches uniform[row], a number in [0, 1) the caller
 * draws (device array, one per row; may be NULL for temperature <= 1e-5).  Masses are summed in 64-bit
 * fixed point, so the result is a pure function of its inputs.  out_idx [rows] int32 on the device. */
int32_t izb_sample_rows(izb_ctx* ctx, izb_stream stream, const void* logits, int32_t dtype, int64_t rows,
                        int64_t cols, int64_t ld, float temperature, int32_t top_k, float top_p,
                        const float* uniform, int32_t* out_idx);

/* Rotary position embedding of q [tokens, q_heads, head_dim] and k [tokens, k_heads, head_dim]
 * (bf16, in place, token rows ld_q / ld_k elements apart) with bf16 tables cos_half, sin_half
 * [tokens, head_dim / 2]: first half = x1 cos - x2 sin, second half = x1 sin + x2 cos, fp32
 * arithmetic, one rounding.  Replaces apply_rotary_emb (models/architectures/qwen3/core.rs:
 * 2402-2415) and try_fused_rope_pair_bshd (kernels/mod.rs:159-173; Metal only in the reference). */
int32_t izb_rope_pair(izb_ctx* ctx, izb_stream stream, void* q, void* k, const void* cos_half,
                      const void* sin_half, int64_t tokens, int32_t q_heads, int32_t k_heads,
                      int32_t head_dim, int64_t ld_q, int64_t ld_k);
/* Writes the new token's k and v [batch, kv_heads, head_dim] (rows ld_k / ld_v apart) at position
 * `pos` of the head-major caches [batch, kv_heads, kv_capacity, head_dim].  Replaces the cache
 * append inside Qwen3Attention::forward (models/architectures/qwen3/core.rs:1624-1732). */
int32_t izb_kv_append(izb_ctx* ctx, izb_stream stream, const void* k, const void* v, void* k_cache,
                      void* v_cache, int64_t batch, int32_t kv_heads, int32_t head_dim, int64_t pos,
                      int64_t kv_capacity, int64_t ld_k, int64_t ld_v);
/* The three steps above in one launch, for the fused QKV output [batch, (heads + 2 kv_heads) *
 * head_dim] of one decode token per sequence: q rows are RMS-normalised (q_norm_weight, may be NULL
 * together with k_norm_weight), rotated and written to q_out [batch, heads, head_dim]; k rows
 * likewise into position `pos` of the K cache; v rows are copied into the V cache.  fp32
 * arithmetic with a single rounding (the separate calls round after the norm and after the
 * rotation).  head_dim 64 or 128.  Replaces apply_qk_norm_pair + apply_rope_pair + the cache append
 * of Qwen3Attention::forward (qwen3/core.rs:1465-1575, 1624-1732), which the reference fuses only on
 * Metal (try_fused_qk_rms_norm, try_fused_rope_pair_bshd). */
int32_t izb_qk_norm_rope_append(izb_ctx* ctx, izb_stream stream, const void* qkv, int64_t ld_qkv,
                                const void* q_norm_weight, const void* k_norm_weight, float eps,
                                const void* cos_half, const void* sin_half, void* q_out,
                                int64_t ld_q_out, void* k_cache, void* v_cache, int64_t batch,
                                int32_t heads, int32_t kv_heads, int32_t head_dim, int64_t pos,
                                int64_t kv_capacity);
/* One query token per sequence against a head-major KV cache: q [batch, heads, head_dim] (rows ld_q
 * apart), k_cache / v_cache [batch, kv_heads, kv_capacity, head_dim] bf16 contiguous of which the
 * first kv_len positions are valid, out [batch, heads, head_dim] (rows ld_out apart);
 * out = softmax(q k^T * scale) v per head, query head h reading KV head h / (heads / kv_heads).
 * head_dim 64 or 128, heads / kv_heads <= 8.  The cache is split over CTAs; `workspace` holds
 * their partial results (izb_decode_gqa_attention_workspace_bytes; 0 for short caches).
 * Replaces dense_decode_attention (models/architectures/qwen3/core.rs:2189-2225) and
 * try_fused_decode_gqa_attention_with_kv_len (kernels/mod.rs:196-221; Metal only in the reference). */
size_t izb_decode_gqa_attention_workspace_bytes(const izb_ctx* ctx, int64_t batch, int32_t heads,
                                                int32_t kv_heads, int32_t head_dim, int64_t kv_len);
int32_t izb_decode_gqa_attention(izb_ctx* ctx, izb_stream stream, const void* q, const void* k_cache,
                                 const void* v_cache, void* out, int64_t batch, int32_t heads,
                                 int32_t kv_heads, int32_t head_dim, int64_t kv_len,
                                 int64_t kv_capacity, int64_t ld_q, int64_t ld_out, float scale,
                                 void* workspace, size_t workspace_bytes);

/* ---- paged KV cache (models/shared/attention/paged.rs) ------------------------------------------
 * A sequence's keys and values live in fixed-size pages of [page_size tokens, kv_heads, head_dim]
 * drawn from a pool the caller owns; page_table [batch, max_pages_per_seq] int32 (device) names the
 * pool pages of every sequence in order.  Storage follows the reference's KvPage (paged.rs:64-156):
 *   IZB_KV_NONE  bf16 values;
 *   IZB_KV_INT8  one byte per value, u8 = round(clamp(x / scale, -127, 127)) + 128, ONE fp32 scale per
 *                page, scale = max(max|x| / 127, 1e-8) or 1 for an all-zero page, with the reference's
 *                arithmetic in the cache dtype (every product rounded to bf16; quantize_tensor_int8 /
 *                dequantize_tensor_int8, paged.rs:158-199);
 *   IZB_KV_Q4_0  blocks of 32 consecutive values: fp32 scale = max|x| / 7 (1 if all zero), 4-bit codes
 *                clamp(round(x / scale), -7, 7) + 8, two per byte, low nibble first (quantize_tensor_q4_0
 *                / dequantize_tensor_q4_0, paged.rs:200-343).
 * values: pool_pages * izb_kv_page_bytes() bytes; scales: pool_pages * izb_kv_page_scales() floats
 * (NULL for IZB_KV_NONE).  The reference keeps one batch inside a page and so one Int8 scale for all
 * of its sequences; here every sequence has pages (and scales) of its own, which is the same for
 * batch 1, the case its decode path runs. */
typedef enum izb_kv_quantization { IZB_KV_NONE = 0, IZB_KV_INT8 = 1, IZB_KV_Q4_0 = 2 } izb_kv_quantization;
typedef struct izb_kv_pages {
    void* k_values;
    void* v_values;
    float* k_scales;
    float* v_scales;
    const int32_t* page_table;
    int32_t quantization; /* izb_kv_quantization */
    int32_t page_size;    /* tokens per page (the reference's DEFAULT_KV_PAGE_SIZE is 64) */
    int32_t kv_heads;
    int32_t head_dim;     /* 64 or 128 */
    int64_t max_pages_per_seq;
} izb_kv_pages;
size_t izb_kv_page_bytes(int32_t quantization, int32_t page_size, int32_t kv_heads, int32_t head_dim);
size_t izb_kv_page_scales(int32_t quantization, int32_t page_size, int32_t kv_heads, int32_t head_dim);
/* Appends n_new tokens to every sequence: k / v bf16, token i of sequence b at row b * n_new + i (rows
 * ld_k / ld_v apart, kv_heads * head_dim values each); seq_lens [batch] int32 on the device holds the
 * tokens already cached (the caller adds n_new afterwards).  A partly filled last page is rebuilt
 * from its dequantised contents plus the new rows and quantised anew, one page per call and page, as
 * `append_to_pages` does (paged.rs:345-388).  A sequence that outgrows max_pages_per_seq makes the
 * next izb_ctx_check return IZB_ERR_BAD_ARG. */
int32_t izb_kv_pages_append(izb_ctx* ctx, izb_stream stream, const izb_kv_pages* pages, const void* k,
                            const void* v, int64_t batch, int64_t n_new, int64_t ld_k, int64_t ld_v,
                            const int32_t* seq_lens);
/* The cached keys (which = 0) or values (1) of every sequence as dense bf16: out[b, t, :] for
 * t < seq_lens[b], rows ld_token apart, sequences ld_batch apart (`materialize_pages`, paged.rs:390-405). */
int32_t izb_kv_pages_materialize(izb_ctx* ctx, izb_stream stream, const izb_kv_pages* pages, int32_t which,
                                 int64_t batch, const int32_t* seq_lens, void* out, int64_t ld_token,
                                 int64_t ld_batch);
/* One query token per sequence over its pages: out = softmax(q k^T * scale) v per head with a running
 * maximum and sum over the pages, which are dequantised in registers and never materialised
 * (`paged_decode_attention`, paged.rs:486-628).  q / out [batch, heads, head_dim] bf16 (rows ld_q /
 * ld_out apart); seq_lens [batch] int32 on the device counts the cached tokens, the new one included;
 * max_seq_len bounds them (it sizes the split over CTAs and the workspace).  heads / kv_heads <= 8. */
size_t izb_paged_decode_gqa_attention_workspace_bytes(const izb_ctx* ctx, int64_t batch, int32_t heads,
                                                      int32_t kv_heads, int32_t head_dim,
                                                      int64_t max_seq_len);
int32_t izb_paged_decode_gqa_attention(izb_ctx* ctx, izb_stream stream, const void* q,
                                       const izb_kv_pages* pages, const int32_t* seq_lens, void* out,
                                       int64_t batch, int32_t heads, int64_t max_seq_len, int64_t ld_q,
                                       int64_t ld_out, float scale, void* workspace, size_t workspace_bytes);

/* ---- what a prompt needs before the first decode step -----------------------------------------
 * out[t, :] = table[ids[t], :]: the embedding lookup in front of the first layer (`embed_tokens`,
 * models/architectures/qwen3/core.rs:2099-2103).  table bf16 [vocab, hidden], ids int32 on the device
 * (a decode step passes the id izb_argmax_rows left there), out rows ld_out apart.  An id outside
 * [0, vocab) gives a zero row and makes the next izb_ctx_check return IZB_ERR_BAD_ARG. */
int32_t izb_embed_rows(izb_ctx* ctx, izb_stream stream, const void* table, int64_t vocab, int64_t hidden,
                       const int32_t* ids, int64_t tokens, void* out, int64_t ld_out);
/* izb_qk_norm_rope_append for a run of q_len consecutive tokens per sequence: token i of sequence b is
 * row b * q_len + i of qkv (rows ld_qkv apart) and of q_out, sits at cache position pos0 + i and is
 * rotated by row i of the tables [q_len, head_dim / 2].  With q_len = 1 it equals the decode call.
 * Replaces apply_qk_norm_pair + apply_rope_pair + the cache append of Qwen3Attention::forward for
 * seq_len > 1 (qwen3/core.rs:1465-1575, 1624-1732). */
int32_t izb_qk_norm_rope_append_seq(izb_ctx* ctx, izb_stream stream, const void* qkv, int64_t ld_qkv,
                                    const void* q_norm_weight, const void* k_norm_weight, float eps,
                                    const void* cos_half, const void* sin_half, void* q_out,
                                    int64_t ld_q_out, void* k_cache, void* v_cache, int64_t batch,
                                    int64_t q_len, int32_t heads, int32_t kv_heads, int32_t head_dim,
                                    int64_t pos0, int64_t kv_capacity);
/* Causal attention of those q_len new tokens over the cache they have just been appended to: token i
 * attends to positions 0 .. pos0 + i.  q / out rows as above ([batch * q_len, heads * head_dim], rows
 * ld_q / ld_out apart, q 16-byte aligned rows), caches head-major [batch, kv_heads, kv_capacity,
 * head_dim] bf16.  head_dim 64 or 128.  Replaces the seq_len > 1 branches of Qwen3Attention::forward
 * (qwen3/core.rs:1688-1732: causal mask + softmax + matmul). */
int32_t izb_prefill_gqa_attention(izb_ctx* ctx, izb_stream stream, const void* q, const void* k_cache,
                                  const void* v_cache, void* out, int64_t batch, int64_t q_len,
                                  int32_t heads, int32_t kv_heads, int32_t head_dim, int64_t pos0,
                                  int64_t kv_capacity, int64_t ld_q, int64_t ld_out, float scale);

/* ---- Conformer convolution module (parakeet/asr/mod.rs:775-864) ---------------------------------
 * Its two pointwise (1x1) convolutions are linear layers over [batch * frames, channels] rows:
 * izb_linear, the first with IZB_EPI_GLU.  Between them:
 * Load time: folds an inference-mode batch norm into the depthwise convolution before it
 * (`fold_depthwise_conv1d_batch_norm`, parakeet/asr/mod.rs:866-893): folded_weight[c, j] = conv_weight[c, j]
 * * scale[c], folded_bias[c] = bn_bias[c] - scale[c] * running_mean[c], scale = bn_weight / sqrt(running_var
 * + eps) (bn_weight / bn_bias NULL together: 1 and 0).  fp32 device inputs, conv_weight [channels, kernel];
 * bf16 outputs. */
int32_t izb_fold_depthwise_conv1d_batch_norm(izb_ctx* ctx, izb_stream stream, const float* conv_weight,
                                             const float* bn_weight, const float* bn_bias,
                                             const float* running_mean, const float* running_var, float eps,
                                             int64_t channels, int32_t kernel, void* folded_weight,
                                             void* folded_bias);
/* out[b, t, c] = swish(bias[c] + sum_j weight[c, j] * x[b, t + j - padding, c]) with zeros beyond each
 * utterance's ends (apply_swish = 0: without the swish).  x / out bf16 [batch * frames, channels] with
 * channels contiguous and rows ld_x / ld_out apart, weight bf16 [channels, kernel], bias bf16 [channels]
 * or NULL.  Odd kernel <= 31 with padding = (kernel - 1) / 2, stride and dilation 1, channels % 8 == 0.
 * Replaces try_depthwise_conv1d_bias_swish (Metal only in the reference) and the depthwise conv + batch
 * norm + swish sequence of ConformerConv::forward (parakeet/asr/mod.rs:836-858); the transposes to and
 * from [batch, channels, frames] (:829, :862) are not needed in this layout. */
int32_t izb_depthwise_conv1d_bias_swish(izb_ctx* ctx, izb_stream stream, const void* x, const void* weight,
                                        const void* bias, void* out, int64_t batch, int64_t frames,
                                        int64_t channels, int32_t kernel, int32_t padding, int64_t ld_x,
                                        int64_t ld_out, int32_t apply_swish);

/* ---- GGUF files -------------------------------------------------------------------------------
 * Read-only view of a GGUF v2 / v3 file (header, metadata, tensor directory; the file is mapped,
 * not copied).  Replaces the use of Candle's gguf_file::Content behind GgufLoader
 * (models/shared/weights/gguf.rs:36-143): from_path -> izb_gguf_open; has_tensor / tensor_shape ->
 * izb_gguf_find; tensor names -> izb_gguf_tensor_at; get_metadata_{string,u64} -> izb_gguf_meta_*;
 * load_qtensor -> izb_gguf_find + izb_gguf_upload (the kernels take the raw block bytes as they
 * are, no repacking); load_tensor -> the same followed by izb_dequantize.
 * Every length and offset in the file is validated against its size: a malformed file gives
 * IZB_ERR_BAD_ARG, an unknown GGUF version or tensor type IZB_ERR_UNSUPPORTED, a name or key that
 * is not present IZB_ERR_UNSUPPORTED. */
typedef struct izb_gguf izb_gguf;
typedef struct izb_gguf_tensor {
    const char* name;  /* owned by the izb_gguf */
    int32_t ggml_type; /* on-disk GGML type id (0 F32, 1 F16, 8 Q8_0, 12 Q4_K, 14 Q6_K, 30 BF16, ...) */
    int32_t wfmt;      /* izb_wfmt accepted by izb_linear / izb_dequantize for these bytes, or -1 */
    int32_t n_dims;
    int32_t reserved_;
    int64_t dims[4];   /* outermost first, as Candle reports shapes (the file stores them reversed) */
    int64_t rows;      /* product of all dims but the last */
    int64_t cols;      /* last dim: the contiguous one, K of a weight */
    const void* data;  /* host pointer into the mapping */
    size_t bytes;
} izb_gguf_tensor;
int32_t izb_gguf_open(const char* path, izb_gguf** out);
int32_t izb_gguf_close(izb_gguf* g);
int32_t izb_gguf_version(const izb_gguf* g);
int64_t izb_gguf_tensor_count(const izb_gguf* g);
int32_t izb_gguf_tensor_at(const izb_gguf* g, int64_t index, izb_gguf_tensor* out);
int32_t izb_gguf_find(const izb_gguf* g, const char* name, izb_gguf_tensor* out);
int64_t izb_gguf_meta_count(const izb_gguf* g);
const char* izb_gguf_meta_key(const izb_gguf* g, int64_t index);
/* Scalars of any integer / bool type as u64 (signed values sign-extended); any numeric type as f64;
 * strings as pointer + length into the mapping (not NUL-terminated). */
int32_t izb_gguf_meta_u64(const izb_gguf* g, const char* key, uint64_t* out);
int32_t izb_gguf_meta_f64(const izb_gguf* g, const char* key, double* out);
int32_t izb_gguf_meta_str(const izb_gguf* g, const char* key, const char** out, size_t* len);
/* Copies the tensor's bytes to device memory on `stream` (needs dst_bytes >= t->bytes). */
int32_t izb_gguf_upload(const izb_gguf* g, const izb_gguf_tensor* t, void* dev_dst, size_t dst_bytes,
                        izb_stream stream);

/* MLX affine-packed weights -> dense, the load-time expansion of `load_weight` for MLX-exported checkpoints
 * (models/shared/weights/mlx.rs:140-256): w[r][c] = q * scales[r][g] + biases[r][g] in fp32 (product and sum
 * rounded separately), q = (word[r][c / pack] >> ((c % pack) * bits)) & (2^bits - 1), pack = in_dim / packed_in,
 * bits = word_bits / pack (1..8), g = c / (in_dim / groups).  `packed` is [out_dim, packed_in] words of `word_bits`
 * (32 or 8) bits; `scales` / `biases` are fp32 [out_dim, groups], or [groups, out_dim] with params_transposed != 0
 * (the reference transposes those back, mlx.rs:66-74); biases may be NULL (zeros).  `out` is [out_dim, in_dim] in
 * out_dtype (fp32: the reference's vector bit for bit; bf16 / fp16: its `to_dtype` to the model's type).  Shapes the
 * reference rejects return IZB_ERR_BAD_ARG. */
int32_t izb_dequantize_mlx_affine(izb_ctx* ctx, izb_stream stream, const void* packed, int32_t word_bits, int64_t packed_in,
                                  const float* scales, const float* biases, int64_t groups, int32_t params_transposed,
                                  int64_t out_dim, int64_t in_dim, int32_t out_dtype, void* out);

/* ---- one decode token of a Qwen3 decoder in one launch -----------------------------------------------
 * Qwen3Model::forward for seq_len = 1 and one sequence, plus the greedy choice of the chat decode loop
 * (qwen3/core.rs:2099-2125, 1863-1881, 1624-1732; qwen3/chat.rs:574-601): embedding row, every decoder
 * layer with its cache append and attention, final norm, lm_head, arg-max.  The reference reaches the
 * same result through some ten tensor operations per layer; its FFI has no single call for it, so a
 * binding would put this behind decode_step (chat.rs:348-388) when the model qualifies: the four
 * projections of every layer in ONE of Q8_0 / Q4_K, lm_head in Q8_0 or Q4_K, head_dim 128, at most four
 * query heads per KV head, hidden and intermediate multiples of 256 (hidden <= 4096, intermediate and
 * heads * 128 <= 12288), vocab, hidden and 2 * intermediate multiples of 64; IZB_ERR_UNSUPPORTED
 * otherwise, and the caller keeps composing the step from izb_linear / izb_qk_norm_rope_append /
 * izb_decode_gqa_attention.  A cooperative launch of one CTA per SM; every device-side wait is bounded
 * (izb_ctx_check: IZB_ERR_TIMEOUT; a token id outside the vocabulary: IZB_ERR_BAD_ARG, nothing read). */
typedef struct izb_qwen3_layer_ptrs {
    /* every pointer 16-byte aligned */
    const void* input_norm; /* bf16 [hidden] */
    const void* post_norm;  /* bf16 [hidden] */
    const void* q_norm;     /* bf16 [head_dim], or NULL */
    const void* k_norm;
    const void* qkv;        /* raw blocks, rows q | k | v: [(heads + 2 kv_heads) * head_dim, hidden] */
    const void* o;          /* [hidden, heads * head_dim] */
    const void* gate_up;    /* rows gate | up: [2 * intermediate, hidden] */
    const void* down;       /* [hidden, intermediate] */
    void* k_cache;          /* bf16 [kv_heads, kv_capacity, head_dim]; position `pos` is written */
    void* v_cache;
} izb_qwen3_layer_ptrs;

typedef struct izb_qwen3_decode_args {
    int32_t wfmt;         /* izb_wfmt of the layers' projections */
    int32_t lm_head_fmt;  /* izb_wfmt of lm_head */
    int32_t n_layers, hidden, heads, kv_heads, head_dim, intermediate, vocab;
    int32_t pos;          /* position of this token = positions already in the caches */
    int64_t kv_capacity;
    float eps;
    int32_t reserved_;
    const izb_qwen3_layer_ptrs* layers; /* HOST array [n_layers <= 48] of device pointers: copied into the launch */
    const void* embed;      /* bf16 [vocab, hidden] */
    const void* final_norm; /* bf16 [hidden] */
    const void* lm_head;    /* raw blocks [vocab, hidden], 16-byte aligned */
    const int32_t* token;   /* device: the token to embed (the previous call's next_token chains without a host read) */
    const void* cos_half;   /* bf16 [head_dim / 2]: cos / sin of pos * inv_freq; 8-byte aligned */
    const void* sin_half;
    float* logits;          /* device fp32 [vocab], or NULL */
    int32_t* next_token;    /* device: arg-max of the logits, lowest index on ties */
    void* workspace;        /* izb_qwen3_decode_token_workspace_bytes, 256-byte aligned; partial sums between phases */
    size_t workspace_bytes;
} izb_qwen3_decode_args;

size_t izb_qwen3_decode_token_workspace_bytes(izb_ctx* ctx, const izb_qwen3_decode_args* args);
int32_t izb_qwen3_decode_token(izb_ctx* ctx, izb_stream stream, const izb_qwen3_decode_args* args);

#ifdef __cplusplus
}
#endif
#endif /* IZWI_B200_H */
