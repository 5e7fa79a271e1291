// One decode token of a Qwen3 decoder in ONE launch: embedding row, every layer (input norm, fused QKV,
// q/k norms, rotation, cache append, attention over the cache, O projection, residual, post-attention
// norm, gate/up, SiLU-multiply, down, residual), final norm, lm_head and the arg-max of the logits.
// Mirrors Qwen3Model::forward for seq_len = 1 plus the greedy choice of the chat decode loop
// (crates/izwi-core/src/models/architectures/qwen3/core.rs:2099-2125, 1863-1881, 1624-1732;
// qwen3/chat.rs:574-601) for one sequence over Q8_0 / Q4_K projections.
//
// Why one launch: at one token a 0.6B model is ~200 launches of 3..8 us each, every one of which reads
// its few megabytes in well under a microsecond; the token costs launches, not bytes.  Here a
// cooperative grid of one CTA per SM walks the phases of every layer and meets at a grid-wide barrier
// between phases (five per layer).  Inside a CTA a producer lane streams this CTA's share of the weight
// blocks through a shared-memory ring with tiled TMA copies (one per 64-row, 256-k box; the tensor maps
// travel as launch parameters) and runs AHEAD of the barriers (weights depend on nobody), so that after a
// barrier the consumers find their weights already on chip and the time of a phase is the barrier plus
// reading a few kilobytes of activations from L2, every load of which is asked for before the first is used.
//
// Work split of a projection [N, K]: units = (64-row tile, k slice); slices S per phase chosen by the
// host so that the units cover the SMs; unit u goes to CTA u mod G.  A unit writes 64 fp32 partial sums
// to part[slice][row]; the consumers of the NEXT phase add the S slices (fixed order: results do not
// depend on timing), apply what sits between the two projections (residual add and bf16 rounding of the
// stream, RmsNorm, SiLU-multiply, the merge of the attention splits) and convert to the 16-bit block
// fixed point that the integer dot products read (gemv_dot.cuh).
//
// Code size: the layer loop is straight-line code that every CTA fetches once per layer.  What several phases share
// (the per-unit consumer, the producer's walk, the norm prologue, the grid barrier, the attention unit) is a call
// (__noinline__, state passed by value) rather than an inline copy per phase: measured 4 % faster, and `no
// instruction` stalls halved.
//
// Every wait is bounded: ring barriers and the grid barrier give up after IZB_WAIT_LIMIT_CLOCKS, raise
// the workspace's abort word (which every other wait also watches) and a context status word, and
// the CTA leaves.
#include <algorithm>
#include <cstddef>
#include <cstdlib>
#include <cstring>

#include "gemv_dot.cuh"
#include "izb_common.cuh"
#include "tma.cuh"

namespace izb {

constexpr int DT_CONSUMER_WARPS = 8;
constexpr int DT_CONSUMERS = 32 * DT_CONSUMER_WARPS;
constexpr int DT_THREADS = DT_CONSUMERS + 32;
constexpr int DT_TILE_ROWS = 64;
constexpr int DT_SLOT_BYTES = DT_TILE_ROWS * 272;  // one 256-k box of 64 Q8_0 rows (Q4_K: 64 * 144 of it used)
constexpr int DT_MAX_SLOTS = 10;
constexpr int DT_MAX_BOXES = 48;    // K <= 12288
constexpr int DT_MAX_HIDDEN = 4096;
constexpr int DT_D = 128;           // head_dim
constexpr int DT_MAX_GQ = 4;        // query heads per kv head
constexpr int DT_MAX_LAYERS = 48;   // layer pointers and tensor maps travel as kernel parameters
constexpr int DT_MAX_SPLITS = 16;
constexpr int DT_REC = DT_D + 4;     // floats of one attention partial in global memory: D sums, max, sum of weights, padding to 16 bytes

struct DtParams {
    izb_qwen3_decode_args a;
    int s_qkv, s_o, s_gu, s_down, att_splits;
    int n_slots;
    // workspace carve-up
    float* part_qkv;   // [s_qkv][q_dim + 2 kv_dim]
    float* part_o;     // [s_o][hidden]
    float* part_gu;    // [s_gu][2 I]
    float* part_down;  // [s_down][hidden]
    float* att_part;   // [heads][att_splits][DT_REC]
    float* stream_a;   // [hidden] the layer's input stream (bf16 values)
    float* stream_b;   // [hidden] the stream behind the attention block
    unsigned long long* best;  // [G] packed (logit, ~index) of every CTA
    unsigned int* counter;     // grid barrier arrivals
    int* abort_word;
    int* status;        // context status word of a wait that gave up
    int* status_token;  // context status word of a token id outside the embedding table
    izb_qwen3_layer_ptrs layers[DT_MAX_LAYERS];
    // weights viewed as [k box][row][bytes of one 256-k box of a row]: qkv, o, gate_up, down of every layer, then lm_head
    CUtensorMap maps[4 * DT_MAX_LAYERS + 1];
};
static_assert(sizeof(DtParams) <= 32764, "kernel parameter space");

struct DtShared {
    unsigned long long full[DT_MAX_SLOTS];
    unsigned long long empty[DT_MAX_SLOTS];
    float red[4][DT_TILE_ROWS];
    float warp_red[DT_CONSUMER_WARPS];
    unsigned long long warp_best[DT_CONSUMER_WARPS];
    float inv_rms;
    int abort_flag;
};

__device__ __forceinline__ void consumer_sync() { named_bar_sync(1, DT_CONSUMERS); }
// Barrier over the consumers that also tells every one of them whether all of them passed `ok`: the
// consumers meet at named barriers, so they must leave a loop together or not at all.
__device__ __forceinline__ bool consumer_all(bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(static_cast<uint32_t>(ok)), "r"(DT_CONSUMERS)
        : "memory");
    return r != 0;
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// (value, index) -> one key whose unsigned order is value descending-last, lowest index winning ties.
__device__ __forceinline__ unsigned long long best_key(float v, int idx) {
    uint32_t b = __float_as_uint(v);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // monotone map of float order onto unsigned order
    return (static_cast<unsigned long long>(b) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(idx));
}

// ---------------------------------------------------------------------------------------------
// Grid barrier: arrival n of the kernel's k-th barrier makes the counter reach k * G.  Consumers only.
// ---------------------------------------------------------------------------------------------
__device__ __noinline__ bool grid_barrier_call(unsigned int* counter, int* abort_word, int* status, DtShared* shp, unsigned int target) {
    DtShared& sh = *shp;
    consumer_sync();  // this CTA's writes of the phase are done
    if (threadIdx.x == 0) {
        // release: the CTA's writes of the phase (ordered before this thread by the barrier above) are visible
        // to whoever reads the count with acquire
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
        const long long t0 = clock64();
        bool ok = true;
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if (v >= target) break;
            int ab;
            asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(ab) : "l"(abort_word) : "memory");
            if (ab != 0 || clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                ok = false;
                break;
            }
        }
        if (!ok) {
            atomicExch(abort_word, 1);
            atomicExch(status, 1);
            sh.abort_flag = 1;
        }
    }
    consumer_sync();
    return *reinterpret_cast<volatile int*>(&sh.abort_flag) == 0;
}

__device__ __forceinline__ bool grid_barrier(const DtParams& P, DtShared& sh, unsigned int target) {
    return grid_barrier_call(P.counter, P.abort_word, P.status, &sh, target);
}

// Units of a projection phase for this CTA: u = cta, cta + G, ...; unit -> (tile, slice) -> boxes [b0, b1).
struct DtUnit {
    int tile, slice, b0, b1;
};
__device__ __forceinline__ DtUnit dt_unit(int u, int S, int boxes) {
    DtUnit r;
    r.tile = u / S;
    r.slice = u - r.tile * S;
    r.b0 = r.slice * boxes / S;
    r.b1 = (r.slice + 1) * boxes / S;
    return r;
}

// ---------------------------------------------------------------------------------------------
// Producer warp: the weight boxes of this CTA's units of one projection, in unit order.
// ---------------------------------------------------------------------------------------------
struct DtRing {
    int slot;
    uint32_t phase;
    long long issued;
};

struct DtRingResult {
    DtRing ring;
    int ok;
};
// Shapes of the five kinds of projection phase, by value (a call cannot name the parameter space).
struct DtPhases {
    int tiles[5], boxes[5], S[5];  // qkv, o, gate/up, down of a layer; lm_head
    int n_layers;
};
// A position in this CTA's walk over every weight box of the token: layer, projection, unit, box.
struct DtCursor {
    int l, j, u, tile, b, b1;
    bool done;
};
__device__ __forceinline__ void dt_phase_dims(const DtPhases& ph, int j, int& tiles, int& boxes, int& S) {
    switch (j) {
        case 0: tiles = ph.tiles[0]; boxes = ph.boxes[0]; S = ph.S[0]; break;
        case 1: tiles = ph.tiles[1]; boxes = ph.boxes[1]; S = ph.S[1]; break;
        case 2: tiles = ph.tiles[2]; boxes = ph.boxes[2]; S = ph.S[2]; break;
        case 3: tiles = ph.tiles[3]; boxes = ph.boxes[3]; S = ph.S[3]; break;
        default: tiles = ph.tiles[4]; boxes = ph.boxes[4]; S = ph.S[4]; break;
    }
}
// Makes the cursor point at a box: skips phases in which this CTA has no unit (left).
__device__ __forceinline__ void dt_cursor_settle(const DtPhases& ph, DtCursor& c) {
    while (!c.done) {
        int tiles, boxes, S;
        dt_phase_dims(ph, c.j, tiles, boxes, S);
        if (c.u < tiles * S) {
            const DtUnit un = dt_unit(c.u, S, boxes);
            c.tile = un.tile;
            c.b = un.b0;
            c.b1 = un.b1;
            if (c.b < c.b1) return;
            c.u += static_cast<int>(gridDim.x);  // an empty slice (more slices than boxes): next unit
            continue;
        }
        // next phase: lm_head (j = 4) follows the last layer's down projection
        if (c.j == 4) {
            c.done = true;
        } else if (c.j == 3) {
            ++c.l;
            c.j = c.l == ph.n_layers ? 4 : 0;
        } else {
            ++c.j;
        }
        c.u = static_cast<int>(blockIdx.x);
    }
}
__device__ __forceinline__ void dt_cursor_next(const DtPhases& ph, DtCursor& c) {
    if (++c.b < c.b1) return;
    c.u += static_cast<int>(gridDim.x);
    dt_cursor_settle(ph, c);
}
__device__ __forceinline__ const CUtensorMap* dt_cursor_map(const CUtensorMap* maps, const DtCursor& c) {
    return maps + (c.j == 4 ? 4 * c.l : 4 * c.l + c.j);  // at lm_head l == n_layers
}
// The producer lane's whole job: every box of this CTA, in the consumers' order, into the ring.  (Asking boxes
// into L2 ahead of the ring with cp.async.bulk.prefetch.tensor, so that HBM streams on while the ring is full,
// was measured and is not here: 12 boxes ahead changed nothing, 24 and more cost 4 % at the 0.6B shape and 22 % at 8B.)
__device__ __noinline__ DtRingResult produce_all_call(DtShared* shp, uint32_t ring0, int n_slots, const CUtensorMap* maps,
                                                      const DtPhases ph, int w_row_bytes, int lm_row_bytes) {
    DtShared& sh = *shp;
    volatile int* abort_flag = &sh.abort_flag;
    const uint32_t full0 = smem_u32(&sh.full[0]), empty0 = smem_u32(&sh.empty[0]);
    DtRingResult out;
    out.ok = 1;
    DtRing R{0, 0u, 0};
    DtCursor cur{0, 0, static_cast<int>(blockIdx.x), 0, 0, 0, false};
    dt_cursor_settle(ph, cur);
    while (!cur.done) {
        if (R.issued >= n_slots && !mbar_wait_bounded_relaxed(empty0 + 8u * R.slot, R.phase ^ 1u, abort_flag)) {
            out.ok = 0;
            break;
        }
        const uint32_t fbar = full0 + 8u * R.slot;
        mbar_expect_tx(fbar, static_cast<uint32_t>(DT_TILE_ROWS * (cur.j == 4 ? lm_row_bytes : w_row_bytes)));
        tma_load_3d(ring0 + static_cast<uint32_t>(R.slot) * DT_SLOT_BYTES, dt_cursor_map(maps, cur), 0, cur.tile * DT_TILE_ROWS, cur.b, fbar);
        dt_cursor_next(ph, cur);
        ++R.issued;
        if (++R.slot == n_slots) {
            R.slot = 0;
            R.phase ^= 1u;
        }
    }
    out.ring = R;
    return out;
}

// ---------------------------------------------------------------------------------------------
// Consumers: the dot products of one unit (64 rows x boxes [b0, b1)) against the converted activations.
// Q8_0: thread = (row, pair of blocks) of every box; Q4_K: thread = (row, half of the super-block, box parity).
// Returns the row's sum in the threads with tid < 64.
// ---------------------------------------------------------------------------------------------
// One copy of this code per weight format serves the five projection phases: it is a call, not inline code, so that
// the layer loop stays small for the instruction cache.  Ring position in and out by value (registers).
struct DtUnitResult {
    float sum;
    int slot;
    uint32_t phase;
    int ok;
};
template <int FMT>
__device__ __noinline__ DtUnitResult consume_unit_call(DtShared* sh, uint32_t ring0, uint32_t xq0, int n_slots, int slot, uint32_t phase,
                                                       int b0, int b1) {
    const int tid = threadIdx.x, row = tid & 63, quarter = tid >> 6;
    const int w_row_bytes = FMT == IZB_W_Q8_0 ? 272 : 144;
    const uint32_t sh_addr = smem_u32(sh);
    volatile int* abort_flag = &sh->abort_flag;
    const uint32_t full0 = sh_addr + static_cast<uint32_t>(offsetof(DtShared, full));
    const uint32_t empty0 = sh_addr + static_cast<uint32_t>(offsetof(DtShared, empty));
    const uint32_t red0 = sh_addr + static_cast<uint32_t>(offsetof(DtShared, red));
    float acc[1] = {0.f};
    bool ok = true;
    for (int b = b0; b < b1; ++b) {
        if (ok && !mbar_wait_bounded(full0 + 8u * slot, phase, abort_flag)) ok = false;
        if (ok) {
            const uint32_t wrow = ring0 + static_cast<uint32_t>(slot) * DT_SLOT_BYTES + static_cast<uint32_t>(row * w_row_bytes);
            const uint32_t xq = xq0 + static_cast<uint32_t>(b * GV_XQ_BYTES);
            if constexpr (FMT == IZB_W_Q8_0) {
                switch (quarter) {
                    case 0: gv_pair_q8_0<0, 1>(acc, wrow, xq, GV_XQ_BYTES); break;
                    case 1: gv_pair_q8_0<1, 1>(acc, wrow, xq, GV_XQ_BYTES); break;
                    case 2: gv_pair_q8_0<2, 1>(acc, wrow, xq, GV_XQ_BYTES); break;
                    default: gv_pair_q8_0<3, 1>(acc, wrow, xq, GV_XQ_BYTES); break;
                }
            } else {
                // the two halves of a super-block go to quarters 0 / 1 for even boxes of the unit, 2 / 3 for odd ones
                if ((quarter >> 1) == ((b - b0) & 1)) {
                    if (quarter & 1) gv_half_q4_k<1, 1>(acc, wrow, xq, GV_XQ_BYTES);
                    else gv_half_q4_k<0, 1>(acc, wrow, xq, GV_XQ_BYTES);
                }
            }
        }
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(empty0 + 8u * slot);
        if (++slot == n_slots) {
            slot = 0;
            phase ^= 1u;
        }
    }
    ok = consumer_all(ok);  // also: the sums of the unit before this one have been read
    sts32f(red0 + 4u * static_cast<uint32_t>(quarter * DT_TILE_ROWS + row), acc[0]);
    consumer_sync();
    DtUnitResult r;
    r.sum = tid < 64 ? (lds32f(red0 + 4u * tid) + lds32f(red0 + 4u * (DT_TILE_ROWS + tid))) +
                           (lds32f(red0 + 4u * (2 * DT_TILE_ROWS + tid)) + lds32f(red0 + 4u * (3 * DT_TILE_ROWS + tid)))
                     : 0.f;
    r.slot = slot;
    r.phase = phase;
    r.ok = ok;
    return r;
}
template <int FMT>
__device__ __forceinline__ bool consume_unit(const DtParams& P, DtShared& sh, uint32_t ring0, uint32_t xq0, DtRing& R, const DtUnit& un,
                                             float& out) {
    const DtUnitResult r = consume_unit_call<FMT>(&sh, ring0, xq0, P.n_slots, R.slot, R.phase, un.b0, un.b1);
    R.slot = r.slot;
    R.phase = r.phase;
    out = r.sum;
    return r.ok != 0;
}

// Sums of four consecutive activation elements over the k slices of the projection that produced them,
// in slice order.  The loads of CH slices are issued before the first add: it is the number of L2 round
// trips, not of loads, that a phase pays for.
template <int CH>
__device__ __forceinline__ float4 part_sum4(const float* part, int S, int n, int i0) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < S; s0 += CH) {
        float4 t[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j)
            t[j] = s0 + j < S ? __ldcg(reinterpret_cast<const float4*>(part + static_cast<size_t>(s0 + j) * n + i0)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            acc.x += t[j].x; acc.y += t[j].y; acc.z += t[j].z; acc.w += t[j].w;
        }
    }
    return acc;
}

// xf[0 .. hidden) and 1 / rms over them, by all consumers; `value4(i0)` = elements i0 .. i0 + 3.
template <typename F>
__device__ __forceinline__ void stage_stream(DtShared& sh, float* xf, int hidden, float eps, F value4) {
    const int tid = threadIdx.x;
    float ss = 0.f;
    for (int i0 = tid * 4; i0 < hidden; i0 += DT_CONSUMERS * 4) {
        const float4 v = value4(i0);
        *reinterpret_cast<float4*>(xf + i0) = v;
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
    if ((tid & 31) == 0) sh.warp_red[tid >> 5] = ss;
    consumer_sync();
    if (tid == 0) {
        float t = 0.f;
        for (int w = 0; w < DT_CONSUMER_WARPS; ++w) t += sh.warp_red[w];
        sh.inv_rms = rsqrtf(t / static_cast<float>(hidden) + eps);
    }
    consumer_sync();
}

// stream + the k slices of the projection behind it, rounded to bf16 as the reference stores the stream
__device__ __forceinline__ float4 stream_plus(const float* stream, const float* part, int S, int n, int i0) {
    const float4 r = __ldcg(reinterpret_cast<const float4*>(stream + i0));
    const float4 p = part_sum4<8>(part, S, n, i0);
    return make_float4(bf16r(r.x + p.x), bf16r(r.y + p.y), bf16r(r.z + p.z), bf16r(r.w + p.w));
}

// The norm weights a warp needs for its boxes of a norm phase (boxes warp, warp + 8: hidden <= 4096), asked for
// BEFORE the stream is read so that both answers travel together.
struct DtNormW {
    uint4 w[2];
};
__device__ __forceinline__ DtNormW load_norm_weights(const __nv_bfloat16* nw, int boxes) {
    DtNormW r;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int b = warp + i * DT_CONSUMER_WARPS;
        r.w[i] = b < boxes ? __ldg(reinterpret_cast<const uint4*>(nw + b * 256 + lane * 8)) : make_uint4(0u, 0u, 0u, 0u);
    }
    return r;
}
// xq of every box of the normalised stream: x * (1 / rms) * weight
__device__ __forceinline__ void convert_normed(uint32_t xq0, const float* xf, float inv, const DtNormW& nw, int boxes) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int b = warp + i * DT_CONSUMER_WARPS;
        if (b >= boxes) break;
        const int k0 = b * 256 + lane * 8;
        const float4 x0 = *reinterpret_cast<const float4*>(xf + k0), x1 = *reinterpret_cast<const float4*>(xf + k0 + 4);
        const uint32_t ww[4] = {nw.w[i].x, nw.w[i].y, nw.w[i].z, nw.w[i].w};
        float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[2 * j] = v[2 * j] * inv * bf16_lo_to_f32(ww[j]);
            v[2 * j + 1] = v[2 * j + 1] * inv * bf16_hi_to_f32(ww[j]);
        }
        gv_convert_unit_f32(v, xq0 + static_cast<uint32_t>(b * GV_XQ_BYTES), lane);
    }
}

// The opening of a phase that reads the residual stream: stream = bf16(stream_in + the slices of the projection
// behind it), kept by CTA 0 in stream_out (when given); RmsNorm with norm_w; activations of every box converted.
// A call: three phases share the code.
__device__ __noinline__ void norm_prologue_call(DtShared* shp, float* xf, uint32_t xq0, const float* stream_in, const float* part, int S,
                                                int hidden, float eps, const __nv_bfloat16* norm_w, float* stream_out) {
    DtShared& sh = *shp;
    const int boxes = hidden / 256;
    const DtNormW nw = load_norm_weights(norm_w, boxes);
    stage_stream(sh, xf, hidden, eps, [&](int i0) { return stream_plus(stream_in, part, S, hidden, i0); });
    if (stream_out)
        for (int i = threadIdx.x; i < hidden; i += DT_CONSUMERS) stream_out[i] = xf[i];
    convert_normed(xq0, xf, sh.inv_rms, nw, boxes);
    consumer_sync();
}

// One warp converts one 256-k box: lane = 8 consecutive values.
template <typename F>
__device__ __forceinline__ void convert_boxes(uint32_t xq0, int b0, int b1, unsigned long long& done, F values) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int b = b0 + warp; b < b1; b += DT_CONSUMER_WARPS) {
        if ((done >> b) & 1ull) continue;
        float v[8];
        values(b * 256 + lane * 8, v);
        gv_convert_unit_f32(v, xq0 + static_cast<uint32_t>(b * GV_XQ_BYTES), lane);
    }
    for (int b = b0; b < b1; ++b) done |= 1ull << b;
}

// ---------------------------------------------------------------------------------------------
// Attention phase unit: kv head `kvh`, positions [t0, t1) of the cache (position `pos` = the new token).
// ---------------------------------------------------------------------------------------------
// What the unit reads of the launch parameters, by value: the unit is a call (one copy of the code per group size
// GQ = 1, 2, 4 query heads per kv head, of which a model runs one), and a call cannot name the parameter space.
struct DtAttArgs {
    const float* part_qkv;
    float* att_part;
    const void *cos_half, *sin_half, *q_norm, *k_norm;
    void *k_cache, *v_cache;
    int s_qkv, att_splits, heads, kv_heads, kv_capacity, pos, scratch_offset;
    float eps;
};
template <int GQ>
__device__ __noinline__ void attention_unit_call(const DtAttArgs A, int kvh, int split, int t0, int t1) {
    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    float* scratch = reinterpret_cast<float*>(dyn_smem + A.scratch_offset);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gq = A.heads / A.kv_heads, q_dim = A.heads * DT_D, kv_dim = A.kv_heads * DT_D, n_qkv = q_dim + 2 * kv_dim;
    float* qs = scratch;                  // [gq][D] rotated query heads (bf16 values)
    float* knew = qs + DT_MAX_GQ * DT_D;  // [D]
    float* vnew = knew + DT_D;            // [D]
    float* wpart = vnew + DT_D;           // [warps][gq][D + 2]
    const __nv_bfloat16* cosv = static_cast<const __nv_bfloat16*>(A.cos_half);
    const __nv_bfloat16* sinv = static_cast<const __nv_bfloat16*>(A.sin_half);
    __nv_bfloat16* kc = static_cast<__nv_bfloat16*>(A.k_cache) + static_cast<size_t>(kvh) * A.kv_capacity * DT_D;
    __nv_bfloat16* vc = static_cast<__nv_bfloat16*>(A.v_cache) + static_cast<size_t>(kvh) * A.kv_capacity * DT_D;
    const bool owns_new = A.pos >= t0 && A.pos < t1;

    // ---- the new token's rows of this kv head: warps 0 .. gq-1 a query head each, warp gq k, warp gq+1 v ----
    if (warp < gq + 2) {
        const int col0 = warp < gq ? (kvh * gq + warp) * DT_D : warp == gq ? q_dim + kvh * DT_D : q_dim + kv_dim + kvh * DT_D;
        // everything this warp's row needs from memory, asked for together
        const __nv_bfloat16* w = warp <= gq ? static_cast<const __nv_bfloat16*>(warp < gq ? A.q_norm : A.k_norm) : nullptr;
        const int jh = (lane & 15) * 4;  // lanes 0..15 hold the first half of the head, 16..31 the second
        uint2 wv = make_uint2(0u, 0u), cv = make_uint2(0u, 0u), sv = make_uint2(0u, 0u);
        if (w) wv = __ldg(reinterpret_cast<const uint2*>(w + lane * 4));
        if (warp <= gq) {
            cv = __ldg(reinterpret_cast<const uint2*>(cosv + jh));
            sv = __ldg(reinterpret_cast<const uint2*>(sinv + jh));
        }
        const float4 xs = part_sum4<4>(A.part_qkv, A.s_qkv, n_qkv, col0 + lane * 4);
        float x[4] = {bf16r(xs.x), bf16r(xs.y), bf16r(xs.z), bf16r(xs.w)};  // the QKV output as stored
        if (warp <= gq) {
            if (w) {
                const float wf[4] = {bf16_lo_to_f32(wv.x), bf16_hi_to_f32(wv.x), bf16_lo_to_f32(wv.y), bf16_hi_to_f32(wv.y)};
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) ss += x[j] * x[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o);
                const float scale = rsqrtf(ss / static_cast<float>(DT_D) + A.eps);
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] = x[j] * scale * wf[j];
            }
            const float cf[4] = {bf16_lo_to_f32(cv.x), bf16_hi_to_f32(cv.x), bf16_lo_to_f32(cv.y), bf16_hi_to_f32(cv.y)};
            const float sf[4] = {bf16_lo_to_f32(sv.x), bf16_hi_to_f32(sv.x), bf16_lo_to_f32(sv.y), bf16_hi_to_f32(sv.y)};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float other = __shfl_xor_sync(0xFFFFFFFFu, x[j], 16);
                x[j] = lane < 16 ? x[j] * cf[j] - other * sf[j] : other * sf[j] + x[j] * cf[j];
            }
        }
        float* dst = warp < gq ? qs + warp * DT_D : warp == gq ? knew : vnew;
#pragma unroll
        for (int j = 0; j < 4; ++j) dst[lane * 4 + j] = bf16r(x[j]);
        if (warp >= gq && owns_new) {
            __nv_bfloat16* row = (warp == gq ? kc : vc) + static_cast<size_t>(A.pos) * DT_D + lane * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) row[j] = __float2bfloat16_rn(x[j]);
        }
    }
    consumer_sync();

    // ---- every warp: positions t0 + warp, + 8, ...; lane owns 4 of the 128 values ----
    float q[GQ][4], acc[GQ][4], m[GQ], l[GQ];
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            q[g][j] = g < gq ? qs[g * DT_D + lane * 4 + j] : 0.f;
            acc[g][j] = 0.f;
        }
    }
    const float scale = rsqrtf(static_cast<float>(DT_D));
    // eight positions per trip to the cache: the loads of a position are a dependent chain otherwise
    constexpr int PT = 8;
    for (int tb = t0 + warp; tb < t1; tb += PT * DT_CONSUMER_WARPS) {
        uint2 kw[PT], vw[PT];
#pragma unroll
        for (int u = 0; u < PT; ++u) {
            const int t = tb + u * DT_CONSUMER_WARPS;
            kw[u] = vw[u] = make_uint2(0u, 0u);
            if (t < t1 && t != A.pos) {
                kw[u] = *reinterpret_cast<const uint2*>(kc + static_cast<size_t>(t) * DT_D + lane * 4);
                vw[u] = *reinterpret_cast<const uint2*>(vc + static_cast<size_t>(t) * DT_D + lane * 4);
            }
        }
        // the trip's scores first (independent chains), one running-max step for the trip, then the values
        float sc[GQ][PT];
#pragma unroll
        for (int u = 0; u < PT; ++u) {
            const int t = tb + u * DT_CONSUMER_WARPS;
            float kv[4];
            if (t == A.pos) {
#pragma unroll
                for (int j = 0; j < 4; ++j) kv[j] = knew[lane * 4 + j];
            } else {
                kv[0] = bf16_lo_to_f32(kw[u].x); kv[1] = bf16_hi_to_f32(kw[u].x); kv[2] = bf16_lo_to_f32(kw[u].y); kv[3] = bf16_hi_to_f32(kw[u].y);
            }
#pragma unroll
            for (int g = 0; g < GQ; ++g) {
                float d = 0.f;
                if (g < gq) d = q[g][0] * kv[0] + q[g][1] * kv[1] + q[g][2] * kv[2] + q[g][3] * kv[3];
                sc[g][u] = d;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int g = 0; g < GQ; ++g) {
                if (g >= gq) break;
#pragma unroll
                for (int u = 0; u < PT; ++u) sc[g][u] += __shfl_xor_sync(0xFFFFFFFFu, sc[g][u], o);
            }
        }
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
            if (g >= gq) break;
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < PT; ++u) {
                sc[g][u] = tb + u * DT_CONSUMER_WARPS < t1 ? sc[g][u] * scale : -INFINITY;
                mx = fmaxf(mx, sc[g][u]);
            }
            const float m_new = fmaxf(m[g], mx);   // finite: position tb is valid
            const float a = __expf(m[g] - m_new);  // first trip: exp(-inf) = 0
            m[g] = m_new;
            l[g] *= a;
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[g][j] *= a;
#pragma unroll
            for (int u = 0; u < PT; ++u) {
                sc[g][u] = __expf(sc[g][u] - m_new);  // past the end: exp(-inf) = 0
                l[g] += sc[g][u];
            }
        }
#pragma unroll
        for (int u = 0; u < PT; ++u) {
            const int t = tb + u * DT_CONSUMER_WARPS;
            float vv[4];
            if (t == A.pos) {
#pragma unroll
                for (int j = 0; j < 4; ++j) vv[j] = vnew[lane * 4 + j];
            } else {
                vv[0] = bf16_lo_to_f32(vw[u].x); vv[1] = bf16_hi_to_f32(vw[u].x); vv[2] = bf16_lo_to_f32(vw[u].y); vv[3] = bf16_hi_to_f32(vw[u].y);
            }
#pragma unroll
            for (int g = 0; g < GQ; ++g) {
                if (g >= gq) break;
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[g][j] = fmaf(sc[g][u], vv[j], acc[g][j]);
            }
        }
    }
    // ---- the eight warps' (max, sum, weighted values) -> one partial per query head and split ----
#pragma unroll
    for (int g = 0; g < GQ; ++g) {
        if (g >= gq) break;
        float* wp = wpart + (warp * DT_MAX_GQ + g) * (DT_D + 2);
#pragma unroll
        for (int j = 0; j < 4; ++j) wp[lane * 4 + j] = acc[g][j];
        if (lane == 0) {
            wp[DT_D] = m[g];
            wp[DT_D + 1] = l[g];
        }
    }
    consumer_sync();
    if (warp < gq) {
        const int g = warp;
        float mm = -INFINITY;
        for (int w = 0; w < DT_CONSUMER_WARPS; ++w) mm = fmaxf(mm, wpart[(w * DT_MAX_GQ + g) * (DT_D + 2) + DT_D]);
        float num[4] = {0.f, 0.f, 0.f, 0.f}, den = 0.f;
        for (int w = 0; w < DT_CONSUMER_WARPS; ++w) {
            const float* wp = wpart + (w * DT_MAX_GQ + g) * (DT_D + 2);
            const float wm = wp[DT_D];
            const float f = wm == -INFINITY ? 0.f : __expf(wm - mm);  // a warp without positions
#pragma unroll
            for (int j = 0; j < 4; ++j) num[j] = fmaf(f, wp[lane * 4 + j], num[j]);
            den = fmaf(f, wp[DT_D + 1], den);
        }
        float* out = A.att_part + (static_cast<size_t>(kvh * gq + g) * A.att_splits + split) * DT_REC;
#pragma unroll
        for (int j = 0; j < 4; ++j) out[lane * 4 + j] = num[j];
        if (lane == 0) {
            out[DT_D] = mm;
            out[DT_D + 1] = den;
        }
    }
    consumer_sync();  // scratch is reused by the CTA's next unit
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int FMT, int LM_FMT>
__global__ void __launch_bounds__(DT_THREADS, 1) qwen3_decode_token_kernel(const __grid_constant__ DtParams P) {
    extern __shared__ __align__(1024) uint8_t dyn_smem[];
    __shared__ DtShared sh;
    const izb_qwen3_decode_args& A = P.a;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
    const int q_dim = A.heads * DT_D, kv_dim = A.kv_heads * DT_D, n_qkv = q_dim + 2 * kv_dim;
    const int w_row = FMT == IZB_W_Q8_0 ? 272 : 144, lm_row = LM_FMT == IZB_W_Q8_0 ? 272 : 144;

    if (tid == 0) {
        for (int s = 0; s < P.n_slots; ++s) {
            mbar_init(smem_u32(&sh.full[s]), 1);
            mbar_init(smem_u32(&sh.empty[s]), DT_CONSUMER_WARPS);
        }
        sh.abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t ring0 = smem_u32(dyn_smem);
    uint8_t* scratch_gen = dyn_smem + static_cast<size_t>(P.n_slots) * DT_SLOT_BYTES;
    const uint32_t xq0 = ring0 + static_cast<uint32_t>(P.n_slots) * DT_SLOT_BYTES;            // [DT_MAX_BOXES][GV_XQ_BYTES]
    float* xf = reinterpret_cast<float*>(scratch_gen + DT_MAX_BOXES * GV_XQ_BYTES);           // [DT_MAX_HIDDEN]

    DtRing R{0, 0u, 0};

    if (warp == DT_CONSUMER_WARPS) {
        // ---------------- producer (one lane): every projection's boxes, in the consumers' order ----------------
        if (lane != 0) return;
        DtPhases ph;
        ph.tiles[0] = n_qkv / DT_TILE_ROWS; ph.boxes[0] = A.hidden / 256; ph.S[0] = P.s_qkv;
        ph.tiles[1] = A.hidden / DT_TILE_ROWS; ph.boxes[1] = q_dim / 256; ph.S[1] = P.s_o;
        ph.tiles[2] = 2 * A.intermediate / DT_TILE_ROWS; ph.boxes[2] = A.hidden / 256; ph.S[2] = P.s_gu;
        ph.tiles[3] = A.hidden / DT_TILE_ROWS; ph.boxes[3] = A.intermediate / 256; ph.S[3] = P.s_down;
        ph.tiles[4] = A.vocab / DT_TILE_ROWS; ph.boxes[4] = A.hidden / 256; ph.S[4] = 1;
        ph.n_layers = A.n_layers;
        const DtRingResult pr = produce_all_call(&sh, ring0, P.n_slots, P.maps, ph, w_row, lm_row);
        R = pr.ring;
        const bool ok = pr.ok != 0;
        // the copies still in flight land before the CTA's shared memory goes away
        {
            const long long first = R.issued > P.n_slots ? R.issued - P.n_slots : 0;
            for (long long f = first; f < R.issued; ++f) {
                const uint32_t bar = smem_u32(&sh.full[f % P.n_slots]);
                const uint32_t par = static_cast<uint32_t>((f / P.n_slots) & 1);
                const long long t0 = clock64();
                while (!mbar_try_wait(bar, par)) {
                    if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) break;
                }
            }
            if (!ok) {
                atomicExch(P.abort_word, 1);
                atomicExch(P.status, 1);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    unsigned int barriers = 0;
    bool ok = true;
    const int token = *A.token;
    const __nv_bfloat16* embed_row = static_cast<const __nv_bfloat16*>(A.embed) + static_cast<size_t>(token) * A.hidden;
    if (token < 0 || token >= A.vocab) {  // a token id outside the embedding table: nothing is read; the host sees a status word
        if (tid == 0) {
            atomicExch(P.abort_word, 1);
            atomicExch(P.status_token, 1);
        }
        ok = false;
    }

    for (int l = 0; l < A.n_layers && ok; ++l) {
        const izb_qwen3_layer_ptrs& Lp = P.layers[l];
        // ===== QKV: stream = previous stream + down partials (layer 0: the embedding row); input norm =====
        {
            const int boxes = A.hidden / 256, units = (n_qkv / DT_TILE_ROWS) * P.s_qkv;
            if (l == 0) {
                const DtNormW nw = load_norm_weights(static_cast<const __nv_bfloat16*>(Lp.input_norm), boxes);
                stage_stream(sh, xf, A.hidden, A.eps, [&](int i0) {
                    const uint2 w = *reinterpret_cast<const uint2*>(embed_row + i0);
                    return make_float4(bf16_lo_to_f32(w.x), bf16_hi_to_f32(w.x), bf16_lo_to_f32(w.y), bf16_hi_to_f32(w.y));
                });
                if (cta == 0) for (int i = tid; i < A.hidden; i += DT_CONSUMERS) P.stream_a[i] = xf[i];
                convert_normed(xq0, xf, sh.inv_rms, nw, boxes);
                consumer_sync();
            } else {
                norm_prologue_call(&sh, xf, xq0, P.stream_b, P.part_down, P.s_down, A.hidden, A.eps,
                                   static_cast<const __nv_bfloat16*>(Lp.input_norm), cta == 0 ? P.stream_a : nullptr);
            }
            for (int u = cta; u < units; u += G) {
                const DtUnit un = dt_unit(u, P.s_qkv, boxes);
                float y;
                ok = consume_unit<FMT>(P, sh, ring0, xq0, R, un, y) && ok;
                if (tid < 64) P.part_qkv[static_cast<size_t>(un.slice) * n_qkv + un.tile * DT_TILE_ROWS + tid] = y;
            }
        }
        ok = grid_barrier(P, sh, ++barriers * G) && ok;
        if (!ok) break;
        // ===== attention: q/k norms, rotation, cache append, softmax(q k) v per (kv head, split) =====
        {
            const int ctx_len = A.pos + 1;
            const int per = (ctx_len + P.att_splits - 1) / P.att_splits;
            const int units = A.kv_heads * P.att_splits;
            if (cta < units) {
                DtAttArgs aa;
                aa.part_qkv = P.part_qkv; aa.att_part = P.att_part;
                aa.cos_half = A.cos_half; aa.sin_half = A.sin_half; aa.q_norm = Lp.q_norm; aa.k_norm = Lp.k_norm;
                aa.k_cache = Lp.k_cache; aa.v_cache = Lp.v_cache;
                aa.s_qkv = P.s_qkv; aa.att_splits = P.att_splits; aa.heads = A.heads; aa.kv_heads = A.kv_heads;
                aa.kv_capacity = A.kv_capacity; aa.pos = A.pos; aa.scratch_offset = P.n_slots * DT_SLOT_BYTES;
                aa.eps = A.eps;
                const int gq = A.heads / A.kv_heads;
                for (int u = cta; u < units; u += G) {
                    const int kvh = u / P.att_splits, split = u - kvh * P.att_splits;
                    const int t0 = min(ctx_len, split * per), t1 = min(ctx_len, t0 + per);
                    if (gq == 1) attention_unit_call<1>(aa, kvh, split, t0, t1);
                    else if (gq == 2) attention_unit_call<2>(aa, kvh, split, t0, t1);
                    else attention_unit_call<4>(aa, kvh, split, t0, t1);
                }
            }
        }
        ok = grid_barrier(P, sh, ++barriers * G) && ok;
        if (!ok) break;
        // ===== O projection over the merged attention output =====
        {
            unsigned long long done = 0;
            const int boxes = q_dim / 256, units = (A.hidden / DT_TILE_ROWS) * P.s_o;
            for (int u = cta; u < units; u += G) {
                const DtUnit un = dt_unit(u, P.s_o, boxes);
                convert_boxes(xq0, un.b0, un.b1, done, [&](int k0, float (&v)[8]) {
                    // merge of the splits' (max, sum of weights, weighted values) for this lane's 8 values of one head;
                    // the records of the first eight splits and all the (max, sum) pairs are asked for in one go
                    const int head = k0 / DT_D, d0 = k0 - head * DT_D, S = P.att_splits;
                    const float* p = P.att_part + static_cast<size_t>(head) * S * DT_REC;
                    float2 ml[DT_MAX_SPLITS];
                    float4 t0[8], t1[8];
#pragma unroll
                    for (int j = 0; j < DT_MAX_SPLITS; ++j)
                        ml[j] = j < S ? __ldcg(reinterpret_cast<const float2*>(p + j * DT_REC + DT_D)) : make_float2(-INFINITY, 0.f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int sj = j < S ? j : 0;
                        t0[j] = __ldcg(reinterpret_cast<const float4*>(p + sj * DT_REC + d0));
                        t1[j] = __ldcg(reinterpret_cast<const float4*>(p + sj * DT_REC + d0 + 4));
                    }
                    float mm = -INFINITY;
#pragma unroll
                    for (int j = 0; j < DT_MAX_SPLITS; ++j) mm = fmaxf(mm, ml[j].x);
                    float f[DT_MAX_SPLITS], den = 0.f;
#pragma unroll
                    for (int j = 0; j < DT_MAX_SPLITS; ++j) {
                        f[j] = ml[j].x == -INFINITY ? 0.f : __expf(ml[j].x - mm);  // a split past the end of the cache
                        den = fmaf(f[j], ml[j].y, den);
                    }
                    float num[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int c = 0; c < DT_MAX_SPLITS / 8; ++c) {
                        if (c > 0) {
                            if (8 * c >= S) break;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const int sj = 8 * c + j < S ? 8 * c + j : 0;
                                t0[j] = __ldcg(reinterpret_cast<const float4*>(p + sj * DT_REC + d0));
                                t1[j] = __ldcg(reinterpret_cast<const float4*>(p + sj * DT_REC + d0 + 4));
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float cj = f[8 * c + j];  // 0 beyond the last split
                            num[0] = fmaf(cj, t0[j].x, num[0]); num[1] = fmaf(cj, t0[j].y, num[1]);
                            num[2] = fmaf(cj, t0[j].z, num[2]); num[3] = fmaf(cj, t0[j].w, num[3]);
                            num[4] = fmaf(cj, t1[j].x, num[4]); num[5] = fmaf(cj, t1[j].y, num[5]);
                            num[6] = fmaf(cj, t1[j].z, num[6]); num[7] = fmaf(cj, t1[j].w, num[7]);
                        }
                    }
                    const float r = 1.0f / den;
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = bf16r(num[j] * r);  // the attention output as stored
                });
                consumer_sync();
                float y;
                ok = consume_unit<FMT>(P, sh, ring0, xq0, R, un, y) && ok;
                if (tid < 64) P.part_o[static_cast<size_t>(un.slice) * A.hidden + un.tile * DT_TILE_ROWS + tid] = y;
            }
        }
        ok = grid_barrier(P, sh, ++barriers * G) && ok;
        if (!ok) break;
        // ===== gate / up: stream += O partials; post-attention norm =====
        {
            const int boxes = A.hidden / 256, units = (2 * A.intermediate / DT_TILE_ROWS) * P.s_gu;
            norm_prologue_call(&sh, xf, xq0, P.stream_a, P.part_o, P.s_o, A.hidden, A.eps, static_cast<const __nv_bfloat16*>(Lp.post_norm),
                               cta == 0 ? P.stream_b : nullptr);
            for (int u = cta; u < units; u += G) {
                const DtUnit un = dt_unit(u, P.s_gu, boxes);
                float y;
                ok = consume_unit<FMT>(P, sh, ring0, xq0, R, un, y) && ok;
                if (tid < 64) P.part_gu[static_cast<size_t>(un.slice) * 2 * A.intermediate + un.tile * DT_TILE_ROWS + tid] = y;
            }
        }
        ok = grid_barrier(P, sh, ++barriers * G) && ok;
        if (!ok) break;
        // ===== down over silu(gate) * up =====
        {
            unsigned long long done = 0;
            const int boxes = A.intermediate / 256, units = (A.hidden / DT_TILE_ROWS) * P.s_down;
            const int n_gu = 2 * A.intermediate;
            for (int u = cta; u < units; u += G) {
                const DtUnit un = dt_unit(u, P.s_down, boxes);
                convert_boxes(xq0, un.b0, un.b1, done, [&](int k0, float (&v)[8]) {
                    const float4 g0 = part_sum4<4>(P.part_gu, P.s_gu, n_gu, k0), g1 = part_sum4<4>(P.part_gu, P.s_gu, n_gu, k0 + 4);
                    const float4 u0 = part_sum4<4>(P.part_gu, P.s_gu, n_gu, A.intermediate + k0);
                    const float4 u1 = part_sum4<4>(P.part_gu, P.s_gu, n_gu, A.intermediate + k0 + 4);
                    const float gs[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                    const float us[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float g = bf16r(gs[j]), up = bf16r(us[j]);  // gate and up as the projection stores them
                        v[j] = g * rcp_approx(1.0f + __expf(-g)) * up;
                    }
                });
                consumer_sync();
                float y;
                ok = consume_unit<FMT>(P, sh, ring0, xq0, R, un, y) && ok;
                if (tid < 64) P.part_down[static_cast<size_t>(un.slice) * A.hidden + un.tile * DT_TILE_ROWS + tid] = y;
            }
        }
        ok = grid_barrier(P, sh, ++barriers * G) && ok;
    }

    // ===== final norm, lm_head, arg-max =====
    unsigned long long best = 0;
    if (ok) {
        const int boxes = A.hidden / 256, units = A.vocab / DT_TILE_ROWS;
        norm_prologue_call(&sh, xf, xq0, P.stream_b, P.part_down, P.s_down, A.hidden, A.eps, static_cast<const __nv_bfloat16*>(A.final_norm),
                           nullptr);
        for (int u = cta; u < units; u += G) {
            const DtUnit un = dt_unit(u, 1, boxes);
            float y;
            ok = consume_unit<LM_FMT>(P, sh, ring0, xq0, R, un, y) && ok;
            if (tid < 64) {
                const int row = un.tile * DT_TILE_ROWS + tid;
                if (A.logits) A.logits[row] = y;
                const unsigned long long key = best_key(y, row);
                best = key > best ? key : best;
            }
        }
        // the CTA's best row (only the first two warps hold candidates)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            best = other > best ? other : best;
        }
        if (lane == 0) sh.warp_best[warp] = best;
        consumer_sync();
        if (tid == 0) P.best[cta] = sh.warp_best[0] > sh.warp_best[1] ? sh.warp_best[0] : sh.warp_best[1];
        ok = grid_barrier(P, sh, ++barriers * G) && ok;
        if (ok && cta == 0 && warp == 0) {
            unsigned long long b = 0;
            for (int i = lane; i < G; i += 32) {
                const unsigned long long k = __ldcg(P.best + i);
                b = k > b ? k : b;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, b, o);
                b = other > b ? other : b;
            }
            if (lane == 0) *A.next_token = static_cast<int32_t>(~static_cast<uint32_t>(b & 0xFFFFFFFFull));
        }
    }
    if (!ok && tid == 0) {
        // the other CTAs' barrier waits and this CTA's producer see the failure at once
        atomicExch(P.abort_word, 1);
        if (token >= 0 && token < A.vocab) atomicExch(P.status, 1);
        sh.abort_flag = 1;
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
namespace {

size_t al256(size_t v) { return (v + 255) / 256 * 256; }

// k slices of a projection with `tiles` row tiles and `boxes` k boxes on G CTAs: the S (a divisor-free
// split into nearly equal box ranges) that minimises the boxes the busiest CTA walks, smallest S on ties.
int pick_slices(int tiles, int boxes, int G) {
    int best_s = 1;
    long long best_cost = -1;
    for (int s = 1; s <= boxes && s <= 16; ++s) {
        const long long rounds = (static_cast<long long>(tiles) * s + G - 1) / G;
        const long long per_unit = (boxes + s - 1) / s;
        const long long cost = rounds * per_unit * 8 + s;  // the next phase reads s partial vectors
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best_s = s;
        }
    }
    return best_s;
}

struct DtLayout {
    size_t part_qkv, part_o, part_gu, part_down, att_part, stream_a, stream_b, best, counter, total;
};

int dt_validate(const izb_qwen3_decode_args* a) {
    if (!a) return IZB_ERR_BAD_ARG;
    if (a->wfmt != IZB_W_Q8_0 && a->wfmt != IZB_W_Q4_K) return IZB_ERR_UNSUPPORTED;
    if (a->lm_head_fmt != IZB_W_Q8_0 && a->lm_head_fmt != IZB_W_Q4_K) return IZB_ERR_UNSUPPORTED;
    if (a->n_layers <= 0 || a->hidden <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->intermediate <= 0 || a->vocab <= 0) return IZB_ERR_BAD_ARG;
    if (a->head_dim != DT_D) return IZB_ERR_UNSUPPORTED;
    if (a->heads % a->kv_heads != 0 || a->heads / a->kv_heads > DT_MAX_GQ) return IZB_ERR_UNSUPPORTED;
    if (a->hidden % 256 != 0 || a->hidden > DT_MAX_HIDDEN || a->intermediate % 256 != 0 || a->intermediate > DT_MAX_BOXES * 256) return IZB_ERR_UNSUPPORTED;
    if (a->heads * DT_D > DT_MAX_BOXES * 256) return IZB_ERR_UNSUPPORTED;
    if (a->hidden % DT_TILE_ROWS != 0 || a->vocab % DT_TILE_ROWS != 0 || (2 * a->intermediate) % DT_TILE_ROWS != 0) return IZB_ERR_UNSUPPORTED;
    if (a->n_layers > DT_MAX_LAYERS) return IZB_ERR_UNSUPPORTED;
    if (a->pos < 0 || a->pos >= a->kv_capacity) return IZB_ERR_BAD_ARG;
    return IZB_OK;
}

// Weights [N, K] in GGML blocks as [K / 256 boxes][N rows][words of one box of a row]; one copy = 64 rows of one box.
int dt_weight_map(CUtensorMap* out, const void* w, int fmt, int N, int K) {
    const int w_row_bytes = fmt == IZB_W_Q8_0 ? 272 : 144;
    const uint64_t boxes = static_cast<uint64_t>(K) / 256, row_bytes = boxes * w_row_bytes;
    const uint32_t words = static_cast<uint32_t>(w_row_bytes / 4);
    const uint64_t dims[3] = {words, static_cast<uint64_t>(N), boxes};
    const uint64_t strides[2] = {row_bytes, static_cast<uint64_t>(w_row_bytes)};
    const uint32_t box[3] = {words, static_cast<uint32_t>(DT_TILE_ROWS), 1};
    return tma_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, w, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

void dt_plan(const izb_ctx* ctx, const izb_qwen3_decode_args* a, DtParams* p, DtLayout* lay) {
    const int G = ctx->sm_count;
    const int q_dim = a->heads * DT_D, kv_dim = a->kv_heads * DT_D, n_qkv = q_dim + 2 * kv_dim;
    p->s_qkv = pick_slices(n_qkv / DT_TILE_ROWS, a->hidden / 256, G);
    p->s_o = pick_slices(a->hidden / DT_TILE_ROWS, q_dim / 256, G);
    p->s_gu = pick_slices(2 * a->intermediate / DT_TILE_ROWS, a->hidden / 256, G);
    p->s_down = pick_slices(a->hidden / DT_TILE_ROWS, a->intermediate / 256, G);
    // splits of the cache per KV head: 64 positions each while eight splits cover the context (one trip for the
    // merge), 256 each beyond; the workspace is laid out for the most there can be
    const int max_splits = std::max(1, std::min(DT_MAX_SPLITS, G / a->kv_heads));
    const int ctx_len = a->pos + 1;
    const int want = ctx_len <= 8 * 64 * 4 ? std::min(8, (ctx_len + 63) / 64) : (ctx_len + 255) / 256;
    p->att_splits = std::max(1, std::min(max_splits, want));
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t at = off; off += al256(bytes); return at; };
    lay->part_qkv = take(sizeof(float) * p->s_qkv * n_qkv);
    lay->part_o = take(sizeof(float) * p->s_o * a->hidden);
    lay->part_gu = take(sizeof(float) * p->s_gu * 2 * a->intermediate);
    lay->part_down = take(sizeof(float) * p->s_down * a->hidden);
    lay->att_part = take(sizeof(float) * a->heads * max_splits * DT_REC);
    lay->stream_a = take(sizeof(float) * a->hidden);
    lay->stream_b = take(sizeof(float) * a->hidden);
    lay->best = take(sizeof(unsigned long long) * G);
    lay->counter = take(256);  // arrival counter, abort word
    lay->total = off;
}

constexpr int DT_SCRATCH_BYTES = DT_MAX_BOXES * GV_XQ_BYTES + DT_MAX_HIDDEN * 4;
static_assert(DT_SCRATCH_BYTES >= static_cast<int>(sizeof(float)) * ((DT_MAX_GQ + 2) * DT_D + DT_CONSUMER_WARPS * DT_MAX_GQ * (DT_D + 2)),
              "attention scratch fits the activation scratch");

template <int FMT, int LM>
int dt_launch(izb_ctx* ctx, cudaStream_t s, DtParams& p) {
    auto kern = qwen3_decode_token_kernel<FMT, LM>;
    int slots = (ctx->max_smem_optin - 2048 - static_cast<int>(sizeof(DtShared)) - DT_SCRATCH_BYTES - 1024) / DT_SLOT_BYTES;
    slots = std::min(slots, DT_MAX_SLOTS);
    if (slots < 2) return IZB_ERR_UNSUPPORTED;
    p.n_slots = slots;

    const int smem = slots * DT_SLOT_BYTES + DT_SCRATCH_BYTES + 1024;
    static std::atomic<int> smem_set[IZB_MAX_DEVICES];
    if (smem_set[ctx->device].load(std::memory_order_relaxed) < smem) {
        IZB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        smem_set[ctx->device].store(smem, std::memory_order_relaxed);
    }
    // the grid barrier needs every CTA resident at once: a cooperative launch checks exactly that
    IZB_CUDA_TRY(cudaMemsetAsync(p.counter, 0, 256, s));
    void* args[] = {&p};
    IZB_CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kern), dim3(ctx->sm_count), dim3(DT_THREADS), args,
                                             static_cast<size_t>(smem), s));
    ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

}  // namespace
}  // namespace izb

using namespace izb;

extern "C" {

size_t izb_qwen3_decode_token_workspace_bytes(izb_ctx* ctx, const izb_qwen3_decode_args* args) {
    if (!ctx || dt_validate(args) != IZB_OK) return 0;
    DtParams p;
    DtLayout lay;
    dt_plan(ctx, args, &p, &lay);
    return lay.total;
}

int32_t izb_qwen3_decode_token(izb_ctx* ctx, izb_stream stream, const izb_qwen3_decode_args* args) {
    if (!ctx) return IZB_ERR_BAD_ARG;
    const int rc = dt_validate(args);
    if (rc != IZB_OK) return rc;
    if (!args->layers || !args->embed || !args->final_norm || !args->lm_head || !args->token || !args->cos_half || !args->sin_half ||
        !args->next_token)
        return IZB_ERR_BAD_ARG;
    if (!izb_aligned(args->cos_half, 8) || !izb_aligned(args->sin_half, 8) || !izb_aligned(args->final_norm, 16)) return IZB_ERR_BAD_ARG;
    if (!izb_aligned(args->embed, 8) || !izb_aligned(args->lm_head, 16) || !izb_aligned(args->token, 4) || !izb_aligned(args->next_token, 4) ||
        (args->logits && !izb_aligned(args->logits, 4)))
        return IZB_ERR_BAD_ARG;
    DtParams p;
    std::memset(&p, 0, sizeof(p));
    DtLayout lay;
    dt_plan(ctx, args, &p, &lay);
    if (!args->workspace || !izb_aligned(args->workspace, 256) || args->workspace_bytes < lay.total) return IZB_ERR_BAD_ARG;
    p.a = *args;
    p.a.layers = nullptr;  // the kernel reads its own copy
    const int q_dim = args->heads * DT_D, n_qkv = q_dim + 2 * args->kv_heads * DT_D;
    for (int l = 0; l < args->n_layers; ++l) {
        const izb_qwen3_layer_ptrs& L = args->layers[l];
        if (!L.input_norm || !L.post_norm || !L.qkv || !L.o || !L.gate_up || !L.down || !L.k_cache || !L.v_cache) return IZB_ERR_BAD_ARG;
        if (!izb_aligned(L.input_norm, 16) || !izb_aligned(L.post_norm, 16) || (L.q_norm && !izb_aligned(L.q_norm, 16)) ||
            (L.k_norm && !izb_aligned(L.k_norm, 16)) || !izb_aligned(L.k_cache, 16) || !izb_aligned(L.v_cache, 16))
            return IZB_ERR_BAD_ARG;
        p.layers[l] = L;
        int rc2 = dt_weight_map(&p.maps[4 * l + 0], L.qkv, args->wfmt, n_qkv, args->hidden);
        if (rc2 == IZB_OK) rc2 = dt_weight_map(&p.maps[4 * l + 1], L.o, args->wfmt, args->hidden, q_dim);
        if (rc2 == IZB_OK) rc2 = dt_weight_map(&p.maps[4 * l + 2], L.gate_up, args->wfmt, 2 * args->intermediate, args->hidden);
        if (rc2 == IZB_OK) rc2 = dt_weight_map(&p.maps[4 * l + 3], L.down, args->wfmt, args->hidden, args->intermediate);
        if (rc2 != IZB_OK) return rc2;
    }
    {
        const int rc2 = dt_weight_map(&p.maps[4 * args->n_layers], args->lm_head, args->lm_head_fmt, args->vocab, args->hidden);
        if (rc2 != IZB_OK) return rc2;
    }
    uint8_t* ws = static_cast<uint8_t*>(args->workspace);
    p.part_qkv = reinterpret_cast<float*>(ws + lay.part_qkv);
    p.part_o = reinterpret_cast<float*>(ws + lay.part_o);
    p.part_gu = reinterpret_cast<float*>(ws + lay.part_gu);
    p.part_down = reinterpret_cast<float*>(ws + lay.part_down);
    p.att_part = reinterpret_cast<float*>(ws + lay.att_part);
    p.stream_a = reinterpret_cast<float*>(ws + lay.stream_a);
    p.stream_b = reinterpret_cast<float*>(ws + lay.stream_b);
    p.best = reinterpret_cast<unsigned long long*>(ws + lay.best);
    p.counter = reinterpret_cast<unsigned int*>(ws + lay.counter);
    p.abort_word = reinterpret_cast<int*>(ws + lay.counter + 64);
    p.status = ctx->d_status + 4;
    p.status_token = ctx->d_status + 6;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (args->wfmt == IZB_W_Q8_0)
        return args->lm_head_fmt == IZB_W_Q8_0 ? dt_launch<IZB_W_Q8_0, IZB_W_Q8_0>(ctx, s, p) : dt_launch<IZB_W_Q8_0, IZB_W_Q4_K>(ctx, s, p);
    return args->lm_head_fmt == IZB_W_Q8_0 ? dt_launch<IZB_W_Q4_K, IZB_W_Q8_0>(ctx, s, p) : dt_launch<IZB_W_Q4_K, IZB_W_Q4_K>(ctx, s, p);
}

}  // extern "C"
