// One-shot all-reduce over NVLink peer memory for decode-size messages (the sum after a row-split
// O or down projection: 8 KB .. 1 MB).  Every rank pushes its partial sums straight into a slot of
// every peer's buffer with plain 8-byte stores that carry the call's sequence number, polls
// (bounded) its own buffer for the words of all ranks and adds them in rank order.  One kernel, no
// NCCL launch, no multimem, no TMA on peer memory.  Slots are double-buffered by call parity; the
// call sequence number lives in device memory so the launch can be replayed from a CUDA graph.
#include <cstddef>
#include <cstdlib>
#include <cstring>
#include <new>

#include "izb_common.cuh"

constexpr int AR_MAX_WORLD = 8;
constexpr int AR_MAX_CTAS = 16;
constexpr size_t AR_LL_MAX_BYTES = 1 << 20;  // above this the two-shot bandwidth path takes over

struct ArDevState {
    unsigned int seq;   // one-shot calls completed so far on this rank (0 = none; slots start zeroed, so no stale word matches)
    unsigned int done;  // CTAs of the current one-shot call that finished reducing
    // two-shot path (large messages): two operand / result buffers, each with its own call number
    unsigned int big_seq[2];               // two-shot calls completed on this rank, per buffer
    unsigned int done_a[2], done_b[2], done_c[2];  // CTA counters of the kernel (chunks pushed / result stored / leaving)
    unsigned int pad_[6];
    unsigned int flag_a[2][AR_MAX_WORLD];  // rank s has its operand ready in its region (value = call number)
    unsigned int flag_b[2][AR_MAX_WORLD];  // rank s has stored its reduced chunk into this region
};
static_assert(sizeof(ArDevState) <= 256, "ArDevState must fit the region header");

struct ArPeers {
    unsigned char* base[AR_MAX_WORLD];  // every rank's region: [ArDevState (256 B)][2][world][slot_bytes]
};

struct izb_ar {
    izb_ctx* ctx;
    int world, rank;
    size_t slot_bytes;
    size_t big_bytes;  // capacity of each two-shot operand / result buffer (0: path off)
    size_t big_in[2], big_stage[2], big_res[2];  // byte offsets inside a region: operand, received chunks, result
    size_t cta_flags;  // pushing kernel: [buffer][phase][source rank][CTA] call numbers
    int push;          // 1: chunks are pushed to their owner (stores only cross NVLink); 0: the owner pulls them (peer loads)
    int next_buf;      // buffer the next izb_ar_allreduce of a large message uses
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
    izb::pdl_launch_dependents();
    izb::pdl_wait();  // buf holds the partial sums of the kernel before this one
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
// bandwidth-bound, so every byte crosses NVLink once in each direction.  The operand lives in this
// rank's region (the projection writes it there, or izb_ar_allreduce copies it in) and the result is
// assembled in the region too, so ONE kernel does the exchange:
//   1. CTA 0 raises flag_a[buf][rank] = call on every rank: "my operand is complete" (it is: the
//      kernel runs after its producer in stream order);
//   2. every CTA waits for all flag_a, then reduces its share of this rank's 1/world chunk: loads the
//      chunk from every region (peer loads), sums in fp32 in rank order (every rank gets the same
//      bits), stores the result into the result buffer of every region (peer stores);
//   3. system fence; the last CTA to finish raises flag_b[buf][rank] = call on every rank;
//   4. CTA 0 stays until all flag_b are up, so the kernel's completion means the whole result has
//      landed here; the last CTA out advances the buffer's call number.
// Two buffers (buf 0 / 1) let the sum of one projection overlap the next projection's writes.
// Stream order is the barrier inside a GPU; the flags (the call number) order the GPUs.  All waits
// are bounded.  CTAs never wait on sibling CTAs, so the grid need not be co-resident.
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

// Threads 0 .. world-1 of the CTA wait (bounded) for flag[s] == value; returns false on time-out.
__device__ __forceinline__ bool ar_wait_all(const unsigned int* flags, int world, unsigned int value, int* status) {
    __shared__ int timed_out;
    if (threadIdx.x == 0) timed_out = 0;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world) {
        const unsigned int* f = flags + threadIdx.x;
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

// 128 threads x 64 registers: small enough to share an SM with a CTA of the tcgen05 GEMM (320 threads x
// 166 registers, nearly all of the shared memory), so a sum on a second stream really runs beside it.
constexpr int AR2_THREADS = 128;
constexpr int AR2_UNROLL = 4;  // 16-byte units per thread and pass: world x 4 peer loads in flight per thread
constexpr int AR2_BATCH = 8;   // pushing kernel: 16-byte units copied per thread and pass

template <bool F32>
__global__ void __launch_bounds__(AR2_THREADS)
    ar2_region_kernel(ArPeers peers, int world, int rank, int buf, size_t big_in, size_t big_res, long long n_units, int* status) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();  // the operand was written by the kernel before this one
    ArDevState* st = reinterpret_cast<ArDevState*>(peers.base[rank]);
    const unsigned int call = st->big_seq[buf] + 1;
    const size_t flag_a = offsetof(ArDevState, flag_a) + sizeof(unsigned int) * AR_MAX_WORLD * buf;
    const size_t flag_b = offsetof(ArDevState, flag_b) + sizeof(unsigned int) * AR_MAX_WORLD * buf;
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < world) {
        __threadfence_system();
        ar_st_flag(reinterpret_cast<unsigned int*>(peers.base[threadIdx.x] + flag_a) + rank, call);
    }
    const bool ok = ar_wait_all(reinterpret_cast<const unsigned int*>(peers.base[rank] + flag_a), world, call, status);
    if (ok) {
        const long long per = (n_units + world - 1) / world;
        const long long lo = per * rank, hi = lo + per < n_units ? lo + per : n_units;
        const long long stride = static_cast<long long>(gridDim.x) * AR2_THREADS * AR2_UNROLL;
        for (long long u0 = lo + static_cast<long long>(blockIdx.x) * AR2_THREADS * AR2_UNROLL + threadIdx.x; u0 < hi; u0 += stride) {
            float acc[AR2_UNROLL][8];
#pragma unroll
            for (int j = 0; j < AR2_UNROLL; ++j)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
            for (int r = 0; r < world; ++r) {
                const uint4* src = reinterpret_cast<const uint4*>(peers.base[r] + big_in);
                uint4 v[AR2_UNROLL];
#pragma unroll
                for (int j = 0; j < AR2_UNROLL; ++j) {
                    const long long u = u0 + static_cast<long long>(j) * AR2_THREADS;
                    v[j] = u < hi ? ar_ld_peer(src + u) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int j = 0; j < AR2_UNROLL; ++j) {
                    const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (F32) {
                            acc[j][e] += __uint_as_float(w[e]);
                        } else {
                            acc[j][2 * e] += izb::bf16_lo_to_f32(w[e]);
                            acc[j][2 * e + 1] += izb::bf16_hi_to_f32(w[e]);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < AR2_UNROLL; ++j) {
                const long long u = u0 + static_cast<long long>(j) * AR2_THREADS;
                if (u >= hi) continue;
                uint4 o;
                if (F32) {
                    o = make_uint4(__float_as_uint(acc[j][0]), __float_as_uint(acc[j][1]), __float_as_uint(acc[j][2]),
                                   __float_as_uint(acc[j][3]));
                } else {
                    o = make_uint4(izb::pack_bf16x2(acc[j][0], acc[j][1]), izb::pack_bf16x2(acc[j][2], acc[j][3]),
                                   izb::pack_bf16x2(acc[j][4], acc[j][5]), izb::pack_bf16x2(acc[j][6], acc[j][7]));
                }
                for (int p = 0; p < world; ++p) reinterpret_cast<uint4*>(peers.base[(rank + p) % world] + big_res)[u] = o;
            }
        }
    }
    // this CTA's result stores are performed system-wide before it is counted in
    __threadfence_system();
    __syncthreads();
    __shared__ int last_to_store;
    if (threadIdx.x == 0) {
        last_to_store = atomicAdd(&st->done_b[buf], 1u) == gridDim.x - 1;
        if (last_to_store) st->done_b[buf] = 0;
    }
    __syncthreads();
    if (last_to_store && static_cast<int>(threadIdx.x) < world) {
        __threadfence_system();
        ar_st_flag(reinterpret_cast<unsigned int*>(peers.base[(rank + threadIdx.x) % world] + flag_b) + rank, call);
    }
    // CTA 0 holds the kernel open until every rank's chunk has landed in this region
    if (blockIdx.x == 0) (void)ar_wait_all(reinterpret_cast<const unsigned int*>(peers.base[rank] + flag_b), world, call, status);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&st->done_c[buf], 1u) == gridDim.x - 1) {
            st->done_c[buf] = 0;
            __threadfence();
            st->big_seq[buf] = call;
        }
    }
}

// The same exchange with stores only on the wire (posted writes do not wait a round trip the way peer
// loads do) and no grid-wide meeting.  CTA c of every rank works on the same set of 16-byte units of
// every chunk, so the exchange decomposes into independent per-CTA exchanges:
//   1. CTA c pushes its units of chunk j into a staging slot of rank j's region, for every other rank j
//      (peers visited in the order rank+1, rank+2, ... so that every receiver hears from one sender at
//      a time), fences, and raises its own flag (the call number) on each of them;
//   2. it waits for the same CTA's flag from every other rank, adds the staged copies of its units of
//      this rank's chunk in rank order (local reads; every rank gets the same bits), and stores the
//      result units into every region;
//   3. it fences, raises its second flag on every rank, and leaves once it holds every other rank's
//      second flag: when the kernel has completed, the whole result has landed here.
// A CTA waits only for CTAs of other GPUs, never for a sibling, so any number of CTAs per SM is safe,
// and CTAs proceed through the phases independently (no last-CTA tail, no atomics on the path).
constexpr int AR2_MAX_CTAS = 160;  // flag slots per (buffer, phase, source rank); the grid never exceeds it

__device__ __forceinline__ bool ar_wait_peers(const unsigned int* flags, int world, int rank, unsigned int value, int* status) {
    // flags: [source rank][AR2_MAX_CTAS] for this CTA's column; thread t waits for rank (rank + 1 + t) % world
    __shared__ int timed_out;
    if (threadIdx.x == 0) timed_out = 0;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world - 1) {
        const unsigned int* f = flags + ((rank + 1 + threadIdx.x) % world) * AR2_MAX_CTAS + blockIdx.x;
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

template <bool F32>
__global__ void __launch_bounds__(AR2_THREADS)
    ar2_push_kernel(ArPeers peers, int world, int rank, int buf, size_t big_in, size_t big_stage, size_t big_res, size_t cta_flags,
                    int n_units, int* status) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();  // the operand was written by the kernel before this one
    ArDevState* st = reinterpret_cast<ArDevState*>(peers.base[rank]);
    const unsigned int call = st->big_seq[buf] + 1;
    const size_t flags_a = cta_flags + sizeof(unsigned int) * AR2_MAX_CTAS * AR_MAX_WORLD * (2 * buf);
    const size_t flags_b = cta_flags + sizeof(unsigned int) * AR2_MAX_CTAS * AR_MAX_WORLD * (2 * buf + 1);
    const int per = (n_units + world - 1) / world;  // units per chunk; the last chunk may be shorter or empty
    const uint4* mine = reinterpret_cast<const uint4*>(peers.base[rank] + big_in);
    const int step = static_cast<int>(gridDim.x) * AR2_THREADS;
    const int first = static_cast<int>(blockIdx.x) * AR2_THREADS + static_cast<int>(threadIdx.x);

    // 1. push this CTA's units of the chunks other ranks own
    for (int p = 1; p < world; ++p) {
        const int j = (rank + p) % world;
        const int len = min(per, n_units - j * per);
        uint4* dst = reinterpret_cast<uint4*>(peers.base[j] + big_stage) + static_cast<size_t>(rank) * per;
        const uint4* src = mine + static_cast<size_t>(j) * per;
        // AR2_BATCH loads are issued before the first store: it is the number of 16-byte loads in
        // flight per thread that sets the rate
        for (int i0 = first; i0 < len; i0 += step * AR2_BATCH) {
            uint4 v[AR2_BATCH];
#pragma unroll
            for (int b = 0; b < AR2_BATCH; ++b) {
                const int i = i0 + b * step;
                if (i < len) v[b] = src[i];
            }
#pragma unroll
            for (int b = 0; b < AR2_BATCH; ++b) {
                const int i = i0 + b * step;
                if (i < len) dst[i] = v[b];
            }
        }
    }
    __threadfence_system();  // this thread's pushes are performed everywhere ...
    __syncthreads();         // ... and so are the whole CTA's before its flag goes out
    if (static_cast<int>(threadIdx.x) < world - 1)
        ar_st_flag(reinterpret_cast<unsigned int*>(peers.base[(rank + 1 + threadIdx.x) % world] + flags_a) + rank * AR2_MAX_CTAS + blockIdx.x,
                   call);
    // 2. the same CTA of every other rank has pushed: add in rank order, store the result everywhere
    const bool ok = ar_wait_peers(reinterpret_cast<const unsigned int*>(peers.base[rank] + flags_a), world, rank, call, status);
    if (ok) {
        const int lo = per * rank, len = min(per, n_units - lo);
        const uint4* stage = reinterpret_cast<const uint4*>(peers.base[rank] + big_stage);
        for (int i = first; i < len; i += step) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            uint4 in[AR_MAX_WORLD];
#pragma unroll
            for (int r = 0; r < AR_MAX_WORLD; ++r)
                if (r < world) in[r] = r == rank ? mine[lo + i] : ar_ld_peer(stage + static_cast<size_t>(r) * per + i);
#pragma unroll
            for (int r = 0; r < AR_MAX_WORLD; ++r) {
                if (r >= world) break;
                const uint4 v = in[r];
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (F32) {
                        acc[e] += __uint_as_float(w[e]);
                    } else {
                        acc[2 * e] += izb::bf16_lo_to_f32(w[e]);
                        acc[2 * e + 1] += izb::bf16_hi_to_f32(w[e]);
                    }
                }
            }
            const uint4 o = F32 ? make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]), __float_as_uint(acc[3]))
                                : make_uint4(izb::pack_bf16x2(acc[0], acc[1]), izb::pack_bf16x2(acc[2], acc[3]),
                                             izb::pack_bf16x2(acc[4], acc[5]), izb::pack_bf16x2(acc[6], acc[7]));
            for (int p = 0; p < world; ++p) reinterpret_cast<uint4*>(peers.base[(rank + p) % world] + big_res)[lo + i] = o;
        }
    }
    // 3. results performed everywhere, second flag out, wait for everyone else's
    __threadfence_system();
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < world - 1)
        ar_st_flag(reinterpret_cast<unsigned int*>(peers.base[(rank + 1 + threadIdx.x) % world] + flags_b) + rank * AR2_MAX_CTAS + blockIdx.x,
                   call);
    (void)ar_wait_peers(reinterpret_cast<const unsigned int*>(peers.base[rank] + flags_b), world, rank, call, status);
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&st->done_c[buf], 1u) == gridDim.x - 1) {
            st->done_c[buf] = 0;
            __threadfence();
            st->big_seq[buf] = call;
        }
    }
}

// Plain device-local copy in 16-byte units (operand into the region, result out of it).
__global__ void __launch_bounds__(512) ar2_copy_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n_units) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();
    for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < n_units;
         u += static_cast<long long>(gridDim.x) * blockDim.x)
        dst[u] = src[u];
}

int ar2_launch(izb_ar* ar, cudaStream_t st, int buf, size_t bytes, int dtype) {
    const long long n_units = static_cast<long long>(bytes / 16);
    int* status = ar->ctx->d_status + 2;
    if (ar->push) {
        // 128-thread CTAs, two per SM when the GPU is free, at most one beside a GEMM; every rank computes the
        // same grid (CTA c exchanges with CTA c of the other ranks)
        long long g = (n_units / ar->world + AR2_THREADS * 4 - 1) / (AR2_THREADS * 4);
        const int cap = ar->ctx->sm_count < AR2_MAX_CTAS ? ar->ctx->sm_count : AR2_MAX_CTAS;
        const int grid = static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
        if (dtype == IZB_F32)
            IZB_CUDA_TRY(izb::launch_chained(ar->ctx, ar2_push_kernel<true>, dim3(grid), dim3(AR2_THREADS), 0, st, ar->peers, ar->world,
                                             ar->rank, buf, ar->big_in[buf], ar->big_stage[buf], ar->big_res[buf], ar->cta_flags,
                                             static_cast<int>(n_units), status));
        else
            IZB_CUDA_TRY(izb::launch_chained(ar->ctx, ar2_push_kernel<false>, dim3(grid), dim3(AR2_THREADS), 0, st, ar->peers, ar->world,
                                             ar->rank, buf, ar->big_in[buf], ar->big_stage[buf], ar->big_res[buf], ar->cta_flags,
                                             static_cast<int>(n_units), status));
        ar->ctx->launches.fetch_add(1, std::memory_order_relaxed);
        return IZB_OK;
    }
    const long long chunk = (n_units + ar->world - 1) / ar->world;
    long long g = (chunk + AR2_THREADS * AR2_UNROLL - 1) / (AR2_THREADS * AR2_UNROLL);
    const int cap = ar->ctx->sm_count * 2;
    const int grid = static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
    if (dtype == IZB_F32)
        IZB_CUDA_TRY(izb::launch_chained(ar->ctx, ar2_region_kernel<true>, dim3(grid), dim3(AR2_THREADS), 0, st, ar->peers, ar->world,
                                         ar->rank, buf, ar->big_in[buf], ar->big_res[buf], n_units, status));
    else
        IZB_CUDA_TRY(izb::launch_chained(ar->ctx, ar2_region_kernel<false>, dim3(grid), dim3(AR2_THREADS), 0, st, ar->peers, ar->world,
                                         ar->rank, buf, ar->big_in[buf], ar->big_res[buf], n_units, status));
    ar->ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
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
    // staging holds `world` chunks of ceil(units / world) units each: up to world - 1 units more than the message
    const size_t stage_bytes = ar->big_bytes ? ar->big_bytes + 16 * static_cast<size_t>(world) + 256 : 0;
    size_t at = AR_HEADER + 2 * static_cast<size_t>(world) * ar->slot_bytes;
    ar->cta_flags = at;
    at += sizeof(unsigned int) * AR2_MAX_CTAS * AR_MAX_WORLD * 4;  // [2 buffers][2 phases][ranks][CTAs]
    at = (at + 255) / 256 * 256;
    for (int b = 0; b < 2; ++b) {
        ar->big_in[b] = at; at += ar->big_bytes;
        ar->big_stage[b] = at; at += (stage_bytes + 255) / 256 * 256;
        ar->big_res[b] = at; at += ar->big_bytes;
    }
    {
        const char* e = std::getenv("IZB_AR_PULL");
        ar->push = (e && e[0] == '1') ? 0 : 1;
    }
    ar->next_buf = 0;
    ar->connected = false;
    std::memset(&ar->peers, 0, sizeof(ar->peers));
    const size_t total = at;
    const size_t zeroed = ar->big_in[0];  // header and one-shot slots; the two-shot buffers are written before they are read
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
        // two-shot path: whole 16-byte units, operand 16-byte aligned; copy in, exchange, copy out.
        // A ragged end (4, 8 or 12 bytes) goes through the one-shot kernel afterwards.
        if (bytes > ar->big_bytes) return IZB_ERR_UNSUPPORTED;
        if (!izb_aligned(buf, 16)) return IZB_ERR_UNSUPPORTED;
        const size_t tail = bytes % 16;
        if (tail != 0) {
            const size_t whole = bytes - tail;
            const int64_t per = dtype == IZB_F32 ? 4 : 2;
            const int rc = izb_ar_allreduce(ar, stream, buf, static_cast<int64_t>(whole) / per, dtype);
            if (rc != IZB_OK) return rc;
            return izb_ar_allreduce(ar, stream, static_cast<unsigned char*>(buf) + whole, static_cast<int64_t>(tail) / per, dtype);
        }
        const long long n_units = static_cast<long long>(bytes / 16);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const int b = ar->next_buf;
        ar->next_buf ^= 1;
        const int copy_grid = ar->ctx->sm_count * 2;
        IZB_CUDA_TRY(izb::launch_chained(ar->ctx, ar2_copy_kernel, dim3(copy_grid), dim3(512), 0, st, static_cast<const uint4*>(buf),
                                         reinterpret_cast<uint4*>(ar->local + ar->big_in[b]), n_units));
        const int rc = ar2_launch(ar, st, b, bytes, dtype);
        if (rc != IZB_OK) return rc;
        IZB_CUDA_TRY(izb::launch_chained(ar->ctx, ar2_copy_kernel, dim3(copy_grid), dim3(512), 0, st,
                                         reinterpret_cast<const uint4*>(ar->local + ar->big_res[b]), static_cast<uint4*>(buf), n_units));
        ar->ctx->launches.fetch_add(2, std::memory_order_relaxed);
        return IZB_OK;
    }
    const long long n_words = static_cast<long long>(bytes / 4);
    // latency, not bandwidth: one word per thread.  Every CTA first pushes, then polls words that peers'
    // CTAs push, so all CTAs of all ranks must get to run: the grid is capped at one CTA per SM, which
    // is resident at once on a GPU this stream has to itself (a few dozen KB need 8 .. 32 CTAs).
    int grid = static_cast<int>((n_words + 255) / 256);
    const int cap = n_words <= 256 * AR_MAX_CTAS ? AR_MAX_CTAS : ar->ctx->sm_count;
    grid = grid < 1 ? 1 : (grid > cap ? cap : grid);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == IZB_F32)
        IZB_CUDA_TRY(izb::launch_chained(ar->ctx, peer_allreduce_kernel<true>, dim3(grid), dim3(256), 0, s, ar->peers, ar->world,
                                         ar->rank, ar->slot_bytes, static_cast<uint32_t*>(buf), n_words, ar->ctx->d_status + 2));
    else
        IZB_CUDA_TRY(izb::launch_chained(ar->ctx, peer_allreduce_kernel<false>, dim3(grid), dim3(256), 0, s, ar->peers, ar->world,
                                         ar->rank, ar->slot_bytes, static_cast<uint32_t*>(buf), n_words, ar->ctx->d_status + 2));
    ar->ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

void* izb_ar_operand(izb_ar* ar, int32_t which) {
    return (ar && ar->big_bytes && (which == 0 || which == 1)) ? ar->local + ar->big_in[which] : nullptr;
}

const void* izb_ar_result(izb_ar* ar, int32_t which) {
    return (ar && ar->big_bytes && (which == 0 || which == 1)) ? ar->local + ar->big_res[which] : nullptr;
}

int32_t izb_ar_allreduce_region(izb_ar* ar, izb_stream stream, int32_t which, int64_t count, int32_t dtype) {
    if (!ar || count < 0 || (dtype != IZB_BF16 && dtype != IZB_F32) || (which != 0 && which != 1)) return IZB_ERR_BAD_ARG;
    if (!ar->connected || !ar->big_bytes) return IZB_ERR_BAD_ARG;
    if (count == 0) return IZB_OK;
    const size_t bytes = static_cast<size_t>(count) * (dtype == IZB_F32 ? 4 : 2);
    if (bytes > ar->big_bytes) return IZB_ERR_UNSUPPORTED;
    if (bytes % 16 != 0) return IZB_ERR_UNSUPPORTED;
    return ar2_launch(ar, static_cast<cudaStream_t>(stream), which, bytes, dtype);
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
