// One-shot all-reduce over NVLink peer memory for decode-size messages (the sum after a row-split
// O or down projection: 8 KB .. 1 MB).  Every rank pushes its partial sums straight into a slot of
// every peer's buffer with plain 8-byte stores that carry the call's sequence number, polls
// (bounded) its own buffer for the words of all ranks and adds them in rank order.  One kernel, no
// NCCL launch, no multimem, no TMA on peer memory.  Slots are double-buffered by call parity; the
// call sequence number lives in device memory so the launch can be replayed from a CUDA graph.
#include <cstddef>
#include <cstring>
#include <new>

#include "izb_common.cuh"

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_MAX_CTAS = 16;
constexpr size_t AR_LL_MAX_BYTES = 1 << 20;  // above this the two-shot bandwidth path takes over  // all CTAs must be resident at once (they wait on other GPUs)

struct ArDevState {
    unsigned int seq;   // one-shot calls completed so far on this rank (0 = none; slots start zeroed, so no stale word matches)
    unsigned int done;  // CTAs of the current one-shot call that finished reducing
    // two-shot path (large messages)
    unsigned int big_seq;                  // two-shot calls completed on this rank
    unsigned int done_a, done_b, done_c;   // CTA counters of its three kernels
    unsigned int pad_[10];
    unsigned int flag_a[AR_MAX_WORLD];     // rank s has copied its operand into its region (value = call number)
    unsigned int pad2_[8];
    unsigned int flag_b[AR_MAX_WORLD];     // rank s has stored its reduced chunk into this region
};
static_assert(sizeof(ArDevState) <= 256, "ArDevState must fit the region header");

struct ArPeers {
    unsigned char* base[AR_MAX_WORLD];  // every rank's region: [ArDevState (256 B)][2][world][slot_bytes]
};

struct izb_ar {
    izb_ctx* ctx;
    int world, rank;
    size_t slot_bytes;
    size_t big_bytes;  // capacity of the two-shot operand / result buffers (0: path off)
    size_t big_in, big_res;  // their byte offsets inside a region
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

// ---------------------------------------------------------------------------------------------
// Two-shot all-reduce for large messages (the sums after a row-split projection at prefill sizes):
// bandwidth-bound, so every byte crosses NVLink once in each direction.  Three launches:
//   a. copy the operand into this rank's region, fence, raise flag_a on every rank;
//   b. wait for all flag_a; reduce this rank's 1/world chunk by loading it from every region (peer
//      loads), summing in fp32 in rank order, and storing the result chunk into every region;
//      fence, raise flag_b on every rank;
//   c. wait for all flag_b; copy the assembled result out.
// Stream order is the barrier inside a GPU; the flags (the call number) order the GPUs.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ar_st_flag(unsigned int* p, unsigned int v) {
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ar_ld_flag(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ar_ld_peer(const uint4* p) {  // not through L1: the line may be a previous call's
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// After a CTA's stores: system-scope fence, count the CTA in; the last one raises flag[rank] = value on every rank.
__device__ __forceinline__ void ar_signal_all(unsigned int* counter, const ArPeers& peers, size_t flag_field, int world, int rank,
                                              unsigned int value) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(counter, 1u);
        if (prev == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            for (int p = 0; p < world; ++p)
                ar_st_flag(reinterpret_cast<unsigned int*>(peers.base[(rank + p) % world] + flag_field) + rank, value);
        }
    }
}

// Threads 0 .. world-1 of the CTA wait (bounded) for flag[s] == value; returns false on time-out.
__device__ __forceinline__ bool ar_wait_all(const unsigned char* local, size_t flag_field, int world, unsigned int value, int* status) {
    __shared__ int timed_out;
    if (threadIdx.x == 0) timed_out = 0;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world) {
        const unsigned int* f = reinterpret_cast<const unsigned int*>(local + flag_field) + threadIdx.x;
        const long long t0 = clock64();
        while (ar_ld_flag(f) != value) {
            if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                timed_out = 1;
                atomicExch(status, 3);
                break;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    return timed_out == 0;
}

__global__ void __launch_bounds__(512)
    ar2_copy_in_kernel(ArPeers peers, int world, int rank, size_t big_in, const uint4* __restrict__ buf, long long n_units) {
    ArDevState* st = reinterpret_cast<ArDevState*>(peers.base[rank]);
    const unsigned int call = st->big_seq + 1;
    uint4* dst = reinterpret_cast<uint4*>(peers.base[rank] + big_in);
    for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < n_units;
         u += static_cast<long long>(gridDim.x) * blockDim.x)
        dst[u] = buf[u];
    ar_signal_all(&st->done_a, peers, offsetof(ArDevState, flag_a), world, rank, call);
}

template <bool F32>
__global__ void __launch_bounds__(512)
    ar2_reduce_kernel(ArPeers peers, int world, int rank, size_t big_in, size_t big_res, long long n_units, int* status) {
    ArDevState* st = reinterpret_cast<ArDevState*>(peers.base[rank]);
    const unsigned int call = st->big_seq + 1;
    const bool ok = ar_wait_all(peers.base[rank], offsetof(ArDevState, flag_a), world, call, status);
    if (ok) {
        const long long per = (n_units + world - 1) / world;
        const long long lo = per * rank, hi = lo + per < n_units ? lo + per : n_units;
        for (long long u = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < hi;
             u += static_cast<long long>(gridDim.x) * blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int r = 0; r < world; ++r) {
                const uint4 v = ar_ld_peer(reinterpret_cast<const uint4*>(peers.base[r] + big_in) + u);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (F32) {
                        acc[j] += __uint_as_float(w[j]);
                    } else {
                        acc[2 * j] += izb::bf16_lo_to_f32(w[j]);
                        acc[2 * j + 1] += izb::bf16_hi_to_f32(w[j]);
                    }
                }
            }
            uint4 o;
            if (F32) {
                o = make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]));
            } else {
                o = make_uint4(izb::pack_bf16x2(acc[0], acc[1]), izb::pack_bf16x2(acc[2], acc[3]), izb::pack_bf16x2(acc[4], acc[5]),
                               izb::pack_bf16x2(acc[6], acc[7]));
            }
            for (int p = 0; p < world; ++p) reinterpret_cast<uint4*>(peers.base[(rank + p) % world] + big_res)[u] = o;
        }
    }
    ar_signal_all(&st->done_b, peers, offsetof(ArDevState, flag_b), world, rank, call);
}

__global__ void __launch_bounds__(512)
    ar2_copy_out_kernel(ArPeers peers, int world, int rank, size_t big_res, uint4* __restrict__ buf, long long n_units, int* status) {
    ArDevState* st = reinterpret_cast<ArDevState*>(peers.base[rank]);
    const unsigned int call = st->big_seq + 1;
    if (ar_wait_all(peers.base[rank], offsetof(ArDevState, flag_b), world, call, status)) {
        const uint4* src = reinterpret_cast<const uint4*>(peers.base[rank] + big_res);
        for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < n_units;
             u += static_cast<long long>(gridDim.x) * blockDim.x)
            buf[u] = ar_ld_peer(src + u);
    }
    // the last CTA out closes the call
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&st->done_c, 1u) == gridDim.x - 1) {
            st->done_c = 0;
            __threadfence();
            st->big_seq = call;
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
    // messages up to 1 MB take the one-shot latency path; larger ones (up to max_bytes) the two-shot bandwidth path
    const size_t ll_max = max_bytes < AR_LL_MAX_BYTES ? max_bytes : AR_LL_MAX_BYTES;
    ar->slot_bytes = (2 * ll_max + 255) / 256 * 256;  // every 4 payload bytes travel as an 8-byte pair
    ar->big_bytes = max_bytes > AR_LL_MAX_BYTES ? (max_bytes + 255) / 256 * 256 : 0;
    ar->big_in = AR_HEADER + 2 * static_cast<size_t>(world) * ar->slot_bytes;
    ar->big_res = ar->big_in + ar->big_bytes;
    ar->connected = false;
    std::memset(&ar->peers, 0, sizeof(ar->peers));
    const size_t total = ar->big_res + ar->big_bytes;
    const size_t zeroed = ar->big_in;  // header and one-shot slots; the two-shot buffers are written before they are read
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != ctx->device) cudaSetDevice(ctx->device);
    void* p = nullptr;
    const bool ok = cudaMalloc(&p, total) == cudaSuccess && cudaMemset(p, 0, zeroed) == cudaSuccess &&
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

size_t izb_ar_max_bytes(const izb_ar* ar) { return ar ? (ar->big_bytes ? ar->big_bytes : ar->slot_bytes / 2) : 0; }

int32_t izb_ar_allreduce(izb_ar* ar, izb_stream stream, void* buf, int64_t count, int32_t dtype) {
    if (!ar || count < 0 || (dtype != IZB_BF16 && dtype != IZB_F32)) return IZB_ERR_BAD_ARG;
    if (!ar->connected) return IZB_ERR_BAD_ARG;
    if (count == 0) return IZB_OK;
    const size_t bytes = static_cast<size_t>(count) * (dtype == IZB_F32 ? 4 : 2);
    if (!buf || !izb_aligned(buf, 4) || bytes % 4 != 0) return IZB_ERR_BAD_ARG;
    if (2 * bytes > ar->slot_bytes) {
        // two-shot path: whole 16-byte units, operand 16-byte aligned
        if (bytes > ar->big_bytes) return IZB_ERR_UNSUPPORTED;
        if (bytes % 16 != 0 || !izb_aligned(buf, 16)) return IZB_ERR_UNSUPPORTED;
        const long long n_units = static_cast<long long>(bytes / 16);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        int* status = ar->ctx->d_status + 2;
        const int copy_grid = ar->ctx->sm_count * 2;
        const long long chunk = (n_units + ar->world - 1) / ar->world;
        long long rg = (chunk + 511) / 512;
        const int reduce_grid = static_cast<int>(rg < 1 ? 1 : (rg > ar->ctx->sm_count * 2 ? ar->ctx->sm_count * 2 : rg));
        ar2_copy_in_kernel<<<copy_grid, 512, 0, st>>>(ar->peers, ar->world, ar->rank, ar->big_in, static_cast<const uint4*>(buf),
                                                     n_units);
        IZB_CUDA_TRY(cudaGetLastError());
        if (dtype == IZB_F32)
            ar2_reduce_kernel<true><<<reduce_grid, 512, 0, st>>>(ar->peers, ar->world, ar->rank, ar->big_in, ar->big_res, n_units, status);
        else
            ar2_reduce_kernel<false><<<reduce_grid, 512, 0, st>>>(ar->peers, ar->world, ar->rank, ar->big_in, ar->big_res, n_units, status);
        IZB_CUDA_TRY(cudaGetLastError());
        ar2_copy_out_kernel<<<copy_grid, 512, 0, st>>>(ar->peers, ar->world, ar->rank, ar->big_res, static_cast<uint4*>(buf), n_units,
                                                      status);
        IZB_CUDA_TRY(cudaGetLastError());
        ar->ctx->launches.fetch_add(3, std::memory_order_relaxed);
        return IZB_OK;
    }
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
