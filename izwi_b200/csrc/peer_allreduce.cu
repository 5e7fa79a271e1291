// One-shot all-reduce over NVLink peer memory for decode-size messages (the sum after a row-split
// O or down projection: 8 KB .. 1 MB).  Every rank pushes its partial sums straight into a slot of
// every peer's buffer with plain 8-byte stores that carry the call's sequence number, polls
// (bounded) its own buffer for the words of all ranks and adds them in rank order.  One kernel, no
// NCCL launch, no multimem, no TMA on peer memory.  Slots are double-buffered by call parity; the
// call sequence number lives in device memory so the launch can be replayed from a CUDA graph.
#include <cstring>
#include <new>

#include "izb_common.cuh"

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_MAX_CTAS = 16;  // all CTAs must be resident at once (they wait on other GPUs)

struct ArDevState {
    unsigned int seq;   // calls completed so far on this rank (0 = none; slots start zeroed, so no stale word matches)
    unsigned int done;  // CTAs of the current call that finished reducing
};

struct ArPeers {
    unsigned char* base[AR_MAX_WORLD];  // every rank's region: [ArDevState (256 B)][2][world][slot_bytes]
};

struct izb_ar {
    izb_ctx* ctx;
    int world, rank;
    size_t slot_bytes;
    unsigned char* local;
    ArPeers peers;
    bool connected;
};

namespace {

constexpr size_t AR_HEADER = 256;

// Low-latency protocol: every 4 bytes of payload travel as one 8-byte store {payload, sequence
// number}.  An 8-byte store lands atomically, so a receiver that reads the expected sequence number
// in a word also has its payload: no fences, no separate flag, one NVLink store latency end to end.
// buf: count elements (bf16 or fp32), reduced in place, viewed as n_words 32-bit words.  CTA b owns
// words [b*per, (b+1)*per) for both the push and the reduction.
__device__ __forceinline__ void st_pair(uint2* p, uint32_t data, uint32_t seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

template <bool F32>
__global__ void __launch_bounds__(256) peer_allreduce_kernel(ArPeers peers, int world, int rank, size_t slot_bytes,
                                                             uint32_t* __restrict__ buf, long long n_words, int* status) {
    ArDevState* st = reinterpret_cast<ArDevState*>(peers.base[rank]);
    const unsigned int seq = st->seq + 1;  // written only by the previous call's last CTA
    const unsigned int parity = seq & 1u;
    const long long per = (n_words + gridDim.x - 1) / gridDim.x;
    const long long lo = static_cast<long long>(blockIdx.x) * per;
    const long long hi = lo + per < n_words ? lo + per : n_words;
    // slot [parity][src] of a rank's region holds n_words pairs written by rank src
    const size_t slot_off = AR_HEADER + (static_cast<size_t>(parity) * world) * slot_bytes;

    // 1. push {word, seq} into my slot on every rank (my own last)
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const uint32_t w = buf[i];
        for (int p = 1; p <= world; ++p) {
            uint2* dst = reinterpret_cast<uint2*>(peers.base[(rank + p) % world] + slot_off + rank * slot_bytes);
            st_pair(dst + i, w, seq);
        }
    }
    // 2. collect the same words from every rank's slot in my region, in rank order (bounded polling)
    bool ok = true;
    const long long t0 = clock64();
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float acc0 = 0.f, acc1 = 0.f;
        for (int r = 0; r < world; ++r) {
            const uint2* src = reinterpret_cast<const uint2*>(peers.base[rank] + slot_off + r * slot_bytes) + i;
            uint2 v = ld_pair(src);
            while (v.y != seq) {
                if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                    ok = false;
                    break;
                }
                v = ld_pair(src);
            }
            if (!ok) break;
            if (F32) {
                acc0 += __uint_as_float(v.x);
            } else {
                acc0 += izb::bf16_lo_to_f32(v.x);
                acc1 += izb::bf16_hi_to_f32(v.x);
            }
        }
        if (!ok) break;
        buf[i] = F32 ? __float_as_uint(acc0) : izb::pack_bf16x2(acc0, acc1);
    }
    if (!ok) atomicExch(status, 3);
    // 3. the last CTA out closes the call: the next call on this rank sees the new sequence number
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int prev = atomicAdd(&st->done, 1u);
        if (prev == gridDim.x - 1) {
            st->done = 0;
            __threadfence();
            st->seq = seq;
        }
    }
}

}  // namespace

extern "C" {

int32_t izb_ar_create(izb_ctx* ctx, int32_t world, int32_t rank, size_t max_bytes, izb_ar** out) {
    if (!ctx || !out || world <= 0 || world > AR_MAX_WORLD || rank < 0 || rank >= world || max_bytes == 0)
        return IZB_ERR_BAD_ARG;
    *out = nullptr;
    izb_ar* ar = new (std::nothrow) izb_ar();
    if (!ar) return IZB_ERR_LAUNCH;
    ar->ctx = ctx;
    ar->world = world;
    ar->rank = rank;
    ar->slot_bytes = (2 * max_bytes + 255) / 256 * 256;  // every 4 payload bytes travel as an 8-byte pair
    ar->connected = false;
    std::memset(&ar->peers, 0, sizeof(ar->peers));
    const size_t total = AR_HEADER + 2 * static_cast<size_t>(world) * ar->slot_bytes;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != ctx->device) cudaSetDevice(ctx->device);
    void* p = nullptr;
    const bool ok = cudaMalloc(&p, total) == cudaSuccess && cudaMemset(p, 0, total) == cudaSuccess &&
                    cudaDeviceSynchronize() == cudaSuccess;
    if (cur != ctx->device) cudaSetDevice(cur);
    if (!ok) {
        (void)cudaGetLastError();
        if (p) cudaFree(p);
        delete ar;
        return IZB_ERR_LAUNCH;
    }
    ar->local = static_cast<unsigned char*>(p);
    *out = ar;
    return IZB_OK;
}

int32_t izb_ar_local_handle(izb_ar* ar, void* out_64_bytes) {
    if (!ar || !out_64_bytes) return IZB_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    IZB_CUDA_TRY(cudaIpcGetMemHandle(&h, ar->local));
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t size");
    std::memcpy(out_64_bytes, &h, 64);
    return IZB_OK;
}

int32_t izb_ar_connect(izb_ar* ar, const void* handles_world_x_64_bytes) {
    if (!ar || !handles_world_x_64_bytes || ar->connected) return IZB_ERR_BAD_ARG;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != ar->ctx->device) cudaSetDevice(ar->ctx->device);
    int rc = IZB_OK;
    for (int r = 0; r < ar->world && rc == IZB_OK; ++r) {
        if (r == ar->rank) {
            ar->peers.base[r] = ar->local;
            continue;
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const unsigned char*>(handles_world_x_64_bytes) + 64 * r, 64);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            rc = IZB_ERR_LAUNCH;
        }
        ar->peers.base[r] = static_cast<unsigned char*>(p);
    }
    if (cur != ar->ctx->device) cudaSetDevice(cur);
    ar->connected = rc == IZB_OK;
    return rc;
}

size_t izb_ar_max_bytes(const izb_ar* ar) { return ar ? ar->slot_bytes / 2 : 0; }

int32_t izb_ar_allreduce(izb_ar* ar, izb_stream stream, void* buf, int64_t count, int32_t dtype) {
    if (!ar || count < 0 || (dtype != IZB_BF16 && dtype != IZB_F32)) return IZB_ERR_BAD_ARG;
    if (!ar->connected) return IZB_ERR_BAD_ARG;
    if (count == 0) return IZB_OK;
    const size_t bytes = static_cast<size_t>(count) * (dtype == IZB_F32 ? 4 : 2);
    if (!buf || !izb_aligned(buf, 4) || bytes % 4 != 0) return IZB_ERR_BAD_ARG;
    if (2 * bytes > ar->slot_bytes) return IZB_ERR_UNSUPPORTED;
    const long long n_words = static_cast<long long>(bytes / 4);
    // latency, not bandwidth: one word per thread while the CTA limit allows (an 8 KB message = 8 CTAs)
    int grid = static_cast<int>((n_words + 255) / 256);
    grid = grid < 1 ? 1 : (grid > AR_MAX_CTAS ? AR_MAX_CTAS : grid);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == IZB_F32)
        peer_allreduce_kernel<true><<<grid, 256, 0, s>>>(ar->peers, ar->world, ar->rank, ar->slot_bytes,
                                                         static_cast<uint32_t*>(buf), n_words, ar->ctx->d_status + 2);
    else
        peer_allreduce_kernel<false><<<grid, 256, 0, s>>>(ar->peers, ar->world, ar->rank, ar->slot_bytes,
                                                          static_cast<uint32_t*>(buf), n_words, ar->ctx->d_status + 2);
    IZB_CUDA_TRY(cudaGetLastError());
    ar->ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_ar_destroy(izb_ar* ar) {
    if (!ar) return IZB_ERR_BAD_ARG;
    for (int r = 0; r < ar->world; ++r)
        if (r != ar->rank && ar->peers.base[r]) (void)cudaIpcCloseMemHandle(ar->peers.base[r]);
    if (ar->local) (void)cudaFree(ar->local);
    delete ar;
    return IZB_OK;
}

}  // extern "C"
