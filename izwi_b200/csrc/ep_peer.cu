// Expert-parallel dispatch and return over NVLink peer memory, without the host in the loop.
//
// Tokens are data-parallel, experts live in contiguous blocks of E / world per rank.  After the local
// routing (top-k, stable permutation into expert-major rows) a rank has rows for every expert and
// their counts on the device.  Per layer:
//   1. counts: every rank pushes its E counts into every peer's region as 8-byte {count, sequence}
//      stores and polls its own region for the others (as in peer_allreduce.cu); from the full
//      [world][E] matrix each rank derives where its rows go on the owners, where the rows it
//      receives start per (local expert, source), the segment offsets of the grouped GEMM, and where
//      results return to;
//   2. dispatch: rows are stored straight into the owner's receive buffer at their final position
//      (grouped by local expert, then source rank, then source order); a system-scope fence, then the
//      last CTA raises this rank's flag on every peer;
//   3. the owner waits (bounded) for all flags, runs the grouped GEMMs on the receive buffer with the
//      device-side segment offsets;
//   4. return: result rows are stored into the source's buffer at the row they left from in its own
//      permuted order, flags again; the source waits and runs its ordered combine.
// Plain peer loads / stores only: no TMA on peer memory, no multimem.  Every wait is bounded and
// reports through the context's status word.  The step number lives in device memory, so the four
// launches can be replayed from a CUDA graph.
#include <cstddef>
#include <cstring>
#include <new>

#include "izb_common.cuh"

constexpr int EP_MAX_WORLD = 8;
constexpr int EP_MAX_EXPERTS = 256;

struct EpHeader {          // first 256 bytes of a rank's region
    unsigned int seq;      // steps completed on this rank
    unsigned int done_dispatch, done_return;  // CTA counters of the step in flight
};

struct EpPeers {
    unsigned char* base[EP_MAX_WORLD];
};

struct EpLayout {  // byte offsets inside a region
    size_t counts, flag_dispatch, flag_return, x_recv, y_ret, total;
};

struct EpTables {  // device-local tables rebuilt every step by the counts kernel
    int cnt[EP_MAX_WORLD][EP_MAX_EXPERTS];       // rows rank s has for expert e
    int dst_row[EP_MAX_EXPERTS];                 // first row, in the owner's receive buffer, of this rank's rows for expert e
    int recv_start[EP_MAX_EXPERTS * EP_MAX_WORLD / 2 + 1];  // [local expert][source] -> first received row; last = total
    int seg[EP_MAX_EXPERTS + 1];                 // grouped-GEMM offsets over local experts
    int ret_start[EP_MAX_WORLD][EP_MAX_EXPERTS]; // [source][local expert] -> row in the source's permuted order
    unsigned int step;                           // sequence number of the step in flight
};

struct izb_ep {
    izb_ctx* ctx;
    int world, rank, n_experts, e_local, hidden, top_k;
    long long max_pairs_local, recv_cap;
    EpLayout lay;
    unsigned char* local;
    EpPeers peers;
    EpTables* tables;
    bool connected;
};

namespace {

constexpr size_t EP_HEADER = 256;

__device__ __forceinline__ void ep_st_pair(uint2* p, uint32_t data, uint32_t seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(data), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ep_ld_pair(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void ep_st_flag(unsigned int* p, unsigned int v) {
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ep_ld_flag(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA.  offsets: this rank's [E + 1] expert offsets of the permuted rows.
__global__ void __launch_bounds__(256)
    ep_counts_kernel(EpPeers peers, EpLayout lay, EpTables* __restrict__ tb, const int* __restrict__ offsets, int world,
                     int rank, int n_experts, int e_local, long long recv_cap, int* status) {
    __shared__ int bad;
    __shared__ int s_cnt[EP_MAX_WORLD][EP_MAX_EXPERTS];
    __shared__ int s_pre[EP_MAX_WORLD + 1][EP_MAX_EXPERTS + 1];
    izb::pdl_launch_dependents();
    izb::pdl_wait();  // offsets come from the permutation kernel before this one
    EpHeader* hdr = reinterpret_cast<EpHeader*>(peers.base[rank]);
    const unsigned int seq = hdr->seq + 1;
    if (threadIdx.x == 0) {
        bad = 0;
        tb->step = seq;
    }
    __syncthreads();
    // push my counts to every rank (mine included)
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const unsigned int c = static_cast<unsigned int>(offsets[e + 1] - offsets[e]);
        for (int p = 0; p < world; ++p) {
            uint2* dst = reinterpret_cast<uint2*>(peers.base[(rank + p) % world] + lay.counts) + rank * n_experts + e;
            ep_st_pair(dst, c, seq);
        }
    }
    // collect everyone's into shared memory: every table below is sums over this [world][experts] matrix, and
    // walking it in global memory made this one-CTA kernel a third of the dispatch
    const long long t0 = clock64();
    bool ok = true;
    for (int i = threadIdx.x; i < world * n_experts && ok; i += blockDim.x) {
        const uint2* src = reinterpret_cast<const uint2*>(peers.base[rank] + lay.counts) + i;
        uint2 v = ep_ld_pair(src);
        while (v.y != seq) {
            if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                ok = false;
                break;
            }
            v = ep_ld_pair(src);
        }
        const int c = ok ? static_cast<int>(v.x) : 0;
        s_cnt[i / n_experts][i % n_experts] = c;
        tb->cnt[i / n_experts][i % n_experts] = c;
    }
    if (!ok) bad = 1;
    __syncthreads();
    if (bad) {
        if (threadIdx.x == 0) atomicExch(status, 6);
        // leave consistent (empty) tables so that the following kernels do nothing harmful
        for (int e = threadIdx.x; e <= e_local; e += blockDim.x) tb->seg[e] = 0;
        for (int i = threadIdx.x; i <= e_local * world; i += blockDim.x) tb->recv_start[i] = 0;
        for (int e = threadIdx.x; e < n_experts; e += blockDim.x) tb->dst_row[e] = -1;
        return;
    }
    // exclusive prefix sums over the experts, one warp per row: rows 0 .. world-1 = each source's counts,
    // row `world` = the totals over all sources; s_pre[r][n_experts] = the row's sum
    {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
        const int chunk = (n_experts + 31) / 32;
        for (int r = warp; r <= world; r += nwarps) {
            const int lo = min(lane * chunk, n_experts), hi = min(lo + chunk, n_experts);
            int sum = 0;
            for (int e = lo; e < hi; ++e) {
                int c = 0;
                if (r < world) c = s_cnt[r][e];
                else for (int s2 = 0; s2 < world; ++s2) c += s_cnt[s2][e];
                sum += c;
            }
            int incl = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += up;
            }
            int at = incl - sum;
            for (int e = lo; e < hi; ++e) {
                int c = 0;
                if (r < world) c = s_cnt[r][e];
                else for (int s2 = 0; s2 < world; ++s2) c += s_cnt[s2][e];
                s_pre[r][e] = at;
                at += c;
            }
            if (lane == 31) s_pre[r][n_experts] = incl;
        }
    }
    __syncthreads();
    const int* tot_pre = s_pre[world];
    // where my rows for expert e start on its owner: all rows of the owner's earlier experts, then the
    // rows of lower ranks for e
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const int first = e / e_local * e_local;
        long long at = tot_pre[e] - tot_pre[first];
        for (int s2 = 0; s2 < rank; ++s2) at += s_cnt[s2][e];
        tb->dst_row[e] = at + (offsets[e + 1] - offsets[e]) <= recv_cap ? static_cast<int>(at) : -1;
    }
    // rows I receive: [local expert][source] starts, and the GEMM's segment offsets
    const int mine0 = rank * e_local;
    for (int i = threadIdx.x; i < e_local * world; i += blockDim.x) {
        const int el = i / world, s2 = i - el * world;
        long long at = tot_pre[mine0 + el] - tot_pre[mine0];
        if (s2 == 0) tb->seg[el] = static_cast<int>(at < recv_cap ? at : recv_cap);
        for (int s3 = 0; s3 < s2; ++s3) at += s_cnt[s3][mine0 + el];
        tb->recv_start[i] = static_cast<int>(at < recv_cap ? at : recv_cap);
    }
    if (threadIdx.x == 0) {
        const long long at = tot_pre[mine0 + e_local] - tot_pre[mine0];
        const int total = static_cast<int>(at < recv_cap ? at : recv_cap);
        tb->seg[e_local] = total;
        tb->recv_start[e_local * world] = total;
        if (at > recv_cap) atomicExch(status, 7);  // more rows than the receive buffer holds: a rank exceeded its token limit
    }
    // where results go back: source s keeps its rows of expert e at its own offsets[e] = sum of its earlier counts
    for (int i = threadIdx.x; i < world * e_local; i += blockDim.x) {
        const int s2 = i / e_local, el = i % e_local;
        tb->ret_start[s2][el] = s_pre[s2][mine0 + el];
    }
}

// Copies one row of `row_units` 16-byte units with one warp: eight loads in flight per lane.
__device__ __forceinline__ void ep_copy_row(uint4* __restrict__ dst, const uint4* __restrict__ src, int row_units, int lane) {
    int u = lane;
    for (; u + 7 * 32 < row_units; u += 8 * 32) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = src[u + 32 * j];
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[u + 32 * j] = v[j];
    }
    for (; u < row_units; u += 32) dst[u] = src[u];
}

// After a CTA's stores: fence to system scope, count the CTA in; the last one raises this rank's
// flag (the step number) on every rank.
__device__ __forceinline__ void ep_signal(unsigned int* counter, EpPeers peers, size_t flag_off, int world, int rank,
                                          unsigned int seq) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(counter, 1u);
        if (prev == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            for (int p = 0; p < world; ++p)
                ep_st_flag(reinterpret_cast<unsigned int*>(peers.base[(rank + p) % world] + flag_off) + rank, seq);
        }
    }
}

// Threads 0 .. world-1 of the calling CTA wait (bounded) until every rank's flag shows this step.
__device__ __forceinline__ void ep_wait_flags(const unsigned char* local, size_t flag_off, unsigned int seq, int world, int* status) {
    const unsigned int* flags = reinterpret_cast<const unsigned int*>(local + flag_off);
    if (static_cast<int>(threadIdx.x) < world) {
        const long long t0 = clock64();
        while (ep_ld_flag(flags + threadIdx.x) != seq) {
            if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                atomicExch(status, 6);
                break;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
}

// Row r (expert-major order) of expert e goes to the owner's receive buffer at dst_row[e] +
// (r - offsets[e]).  Its source is x_perm[r], or, with `perm` given, x[perm[r] / top_k] (the gather
// of the routing fused into the dispatch).  One warp per row.
__global__ void __launch_bounds__(256)
    ep_dispatch_kernel(EpPeers peers, EpLayout lay, const EpTables* __restrict__ tb, const uint4* __restrict__ x,
                       const int* __restrict__ perm, int top_k, long long ld_units, const int* __restrict__ offsets,
                       long long pairs, int n_experts, int e_local, int row_units, int world, int rank, int* status) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();  // the tables come from the counts kernel, x and perm from the routing before it
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    for (long long r = static_cast<long long>(blockIdx.x) * wpb + warp; r < pairs; r += static_cast<long long>(gridDim.x) * wpb) {
        int e = 0, dst_row = -1;
        long long src_row = r;
        if (lane == 0) {
            int lo = 0, hi = n_experts;  // last e with offsets[e] <= r
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (offsets[mid] <= r) lo = mid; else hi = mid;
            }
            e = lo;
            dst_row = tb->dst_row[lo] < 0 ? -1 : tb->dst_row[lo] + static_cast<int>(r - offsets[lo]);
            if (perm) src_row = perm[r] / top_k;
        }
        e = __shfl_sync(0xFFFFFFFFu, e, 0);
        dst_row = __shfl_sync(0xFFFFFFFFu, dst_row, 0);
        src_row = __shfl_sync(0xFFFFFFFFu, src_row, 0);
        if (dst_row >= 0) {
            uint4* dst = reinterpret_cast<uint4*>(peers.base[e / e_local] + lay.x_recv) + static_cast<long long>(dst_row) * row_units;
            ep_copy_row(dst, x + src_row * ld_units, row_units, lane);
        }
    }
    EpHeader* hdr = reinterpret_cast<EpHeader*>(peers.base[rank]);
    ep_signal(&hdr->done_dispatch, peers, lay.flag_dispatch, world, rank, tb->step);
    // CTA 0 keeps the kernel open until every rank's rows have landed here, so what follows in the stream
    // (the grouped GEMM) needs no launch of its own to wait
    if (blockIdx.x == 0) ep_wait_flags(peers.base[rank], lay.flag_dispatch, tb->step, world, status);
}

// y: results for the received rows, same order.  Row i (local expert el, source s, position j) goes
// to the source's return buffer at ret_start[s][el] + j.  One warp per row.
__global__ void __launch_bounds__(256)
    ep_return_kernel(EpPeers peers, EpLayout lay, const EpTables* __restrict__ tb, const uint4* __restrict__ y, int e_local,
                     int row_units, int world, int rank, int* status) {
    izb::pdl_launch_dependents();
    izb::pdl_wait();  // y is the output of the grouped GEMM before this kernel
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpb = blockDim.x >> 5;
    const int groups = e_local * world;
    const int total = tb->recv_start[groups];
    for (int i = blockIdx.x * wpb + warp; i < total; i += gridDim.x * wpb) {
        int src = 0, dst_row = 0;
        if (lane == 0) {
            int lo = 0, hi = groups;  // last group whose start <= i (empty groups share a start: take the last)
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (tb->recv_start[mid] <= i) lo = mid; else hi = mid;
            }
            src = lo % world;
            dst_row = tb->ret_start[src][lo / world] + (i - tb->recv_start[lo]);
        }
        src = __shfl_sync(0xFFFFFFFFu, src, 0);
        dst_row = __shfl_sync(0xFFFFFFFFu, dst_row, 0);
        uint4* dst = reinterpret_cast<uint4*>(peers.base[src] + lay.y_ret) + static_cast<long long>(dst_row) * row_units;
        ep_copy_row(dst, y + static_cast<long long>(i) * row_units, row_units, lane);
    }
    EpHeader* hdr = reinterpret_cast<EpHeader*>(peers.base[rank]);
    ep_signal(&hdr->done_return, peers, lay.flag_return, world, rank, tb->step);
    // CTA 0 waits for this rank's own rows to come back from every rank, then closes the step
    if (blockIdx.x == 0) {
        ep_wait_flags(peers.base[rank], lay.flag_return, tb->step, world, status);
        if (threadIdx.x == 0) hdr->seq = tb->step;
    }
}

EpLayout ep_layout(int world, int n_experts, int hidden, long long recv_cap, long long max_pairs_local) {
    EpLayout l;
    size_t at = EP_HEADER;
    auto take = [&](size_t bytes) {
        const size_t start = at;
        at = (at + bytes + 255) / 256 * 256;
        return start;
    };
    l.counts = take(static_cast<size_t>(world) * n_experts * sizeof(uint2));
    l.flag_dispatch = take(static_cast<size_t>(world) * sizeof(unsigned int));
    l.flag_return = take(static_cast<size_t>(world) * sizeof(unsigned int));
    l.x_recv = take(static_cast<size_t>(recv_cap) * hidden * 2);
    l.y_ret = take(static_cast<size_t>(max_pairs_local) * hidden * 2);
    l.total = at;
    return l;
}

}  // namespace

extern "C" {

int32_t izb_ep_create(izb_ctx* ctx, int32_t world, int32_t rank, int32_t n_experts, int32_t hidden, int64_t max_tokens_local,
                      int32_t top_k, izb_ep** out) {
    if (!ctx || !out || world <= 0 || world > EP_MAX_WORLD || rank < 0 || rank >= world) return IZB_ERR_BAD_ARG;
    if (n_experts <= 0 || n_experts > EP_MAX_EXPERTS || n_experts % world != 0) return IZB_ERR_BAD_ARG;
    if (hidden <= 0 || hidden % 8 != 0 || max_tokens_local <= 0 || top_k <= 0 || top_k > n_experts) return IZB_ERR_BAD_ARG;
    if ((n_experts / world) * world > EP_MAX_EXPERTS * EP_MAX_WORLD / 2) return IZB_ERR_UNSUPPORTED;
    *out = nullptr;
    izb_ep* ep = new (std::nothrow) izb_ep();
    if (!ep) return IZB_ERR_LAUNCH;
    ep->ctx = ctx;
    ep->world = world; ep->rank = rank; ep->n_experts = n_experts; ep->e_local = n_experts / world;
    ep->hidden = hidden; ep->top_k = top_k;
    ep->max_pairs_local = max_tokens_local * top_k;
    ep->recv_cap = ep->max_pairs_local * world;  // every pair of every rank could choose this rank's experts
    if (ep->recv_cap > INT32_MAX / 2) {
        delete ep;
        return IZB_ERR_UNSUPPORTED;
    }
    ep->lay = ep_layout(world, n_experts, hidden, ep->recv_cap, ep->max_pairs_local);
    ep->connected = false;
    ep->tables = nullptr;
    std::memset(&ep->peers, 0, sizeof(ep->peers));
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != ctx->device) cudaSetDevice(ctx->device);
    void* p = nullptr;
    void* t = nullptr;
    // only the control words need a defined start; the row buffers are written before they are read
    const bool ok = cudaMalloc(&p, ep->lay.total) == cudaSuccess && cudaMemset(p, 0, ep->lay.x_recv) == cudaSuccess &&
                    cudaMalloc(&t, sizeof(EpTables)) == cudaSuccess && cudaMemset(t, 0, sizeof(EpTables)) == cudaSuccess &&
                    cudaDeviceSynchronize() == cudaSuccess;
    if (cur != ctx->device) cudaSetDevice(cur);
    if (!ok) {
        (void)cudaGetLastError();
        if (p) cudaFree(p);
        if (t) cudaFree(t);
        delete ep;
        return IZB_ERR_LAUNCH;
    }
    ep->local = static_cast<unsigned char*>(p);
    ep->tables = static_cast<EpTables*>(t);
    *out = ep;
    return IZB_OK;
}

int32_t izb_ep_local_handle(izb_ep* ep, void* out_64_bytes) {
    if (!ep || !out_64_bytes) return IZB_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    IZB_CUDA_TRY(cudaIpcGetMemHandle(&h, ep->local));
    std::memcpy(out_64_bytes, &h, 64);
    return IZB_OK;
}

int32_t izb_ep_connect(izb_ep* ep, const void* handles_world_x_64_bytes) {
    if (!ep || !handles_world_x_64_bytes || ep->connected) return IZB_ERR_BAD_ARG;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != ep->ctx->device) cudaSetDevice(ep->ctx->device);
    int rc = IZB_OK;
    for (int r = 0; r < ep->world && rc == IZB_OK; ++r) {
        if (r == ep->rank) {
            ep->peers.base[r] = ep->local;
            continue;
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const unsigned char*>(handles_world_x_64_bytes) + 64 * r, 64);
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            rc = IZB_ERR_LAUNCH;
        }
        ep->peers.base[r] = static_cast<unsigned char*>(p);
    }
    if (cur != ep->ctx->device) cudaSetDevice(cur);
    ep->connected = rc == IZB_OK;
    return rc;
}

int64_t izb_ep_recv_capacity_rows(const izb_ep* ep) { return ep ? ep->recv_cap : 0; }
void* izb_ep_recv_rows(const izb_ep* ep) { return ep ? ep->local + ep->lay.x_recv : nullptr; }
const void* izb_ep_recv_offsets(const izb_ep* ep) {
    return ep ? reinterpret_cast<const unsigned char*>(ep->tables) + offsetof(EpTables, seg) : nullptr;
}
const void* izb_ep_returned_rows(const izb_ep* ep) { return ep ? ep->local + ep->lay.y_ret : nullptr; }

int32_t izb_ep_dispatch(izb_ep* ep, izb_stream stream, const void* x, int64_t ld_x, const void* perm, const void* offsets,
                        int64_t pairs) {
    if (!ep || !ep->connected || pairs < 0 || pairs > ep->max_pairs_local) return IZB_ERR_BAD_ARG;
    if (!offsets || (pairs > 0 && !x) || !izb_aligned(x, 16) || !izb_aligned(offsets, 4) || !izb_aligned(perm, 4)) return IZB_ERR_BAD_ARG;
    if (ld_x < ep->hidden || ld_x % 8 != 0) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* status = ep->ctx->d_status + 5;
    IZB_CUDA_TRY(izb::launch_chained(ep->ctx, ep_counts_kernel, dim3(1), dim3(256), 0, s, ep->peers, ep->lay, ep->tables,
                                     static_cast<const int*>(offsets), ep->world, ep->rank, ep->n_experts, ep->e_local, ep->recv_cap,
                                     status));
    const long long cap = static_cast<long long>(ep->ctx->sm_count) * 4, blocks = (pairs + 7) / 8;
    const int grid = static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
    IZB_CUDA_TRY(izb::launch_chained(ep->ctx, ep_dispatch_kernel, dim3(grid), dim3(256), 0, s, ep->peers, ep->lay,
                                     static_cast<const EpTables*>(ep->tables), static_cast<const uint4*>(x),
                                     static_cast<const int*>(perm), ep->top_k, static_cast<long long>(ld_x / 8),
                                     static_cast<const int*>(offsets), static_cast<long long>(pairs), ep->n_experts, ep->e_local,
                                     ep->hidden / 8, ep->world, ep->rank, status));
    ep->ctx->launches.fetch_add(2, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_ep_return(izb_ep* ep, izb_stream stream, const void* y_rows) {
    if (!ep || !ep->connected || !y_rows || !izb_aligned(y_rows, 16)) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int* status = ep->ctx->d_status + 5;
    const int grid = ep->ctx->sm_count * 4;
    IZB_CUDA_TRY(izb::launch_chained(ep->ctx, ep_return_kernel, dim3(grid), dim3(256), 0, s, ep->peers, ep->lay,
                                     static_cast<const EpTables*>(ep->tables), static_cast<const uint4*>(y_rows), ep->e_local,
                                     ep->hidden / 8, ep->world, ep->rank, status));
    ep->ctx->launches.fetch_add(1, std::memory_order_relaxed);
    return IZB_OK;
}

int32_t izb_ep_destroy(izb_ep* ep) {
    if (!ep) return IZB_ERR_BAD_ARG;
    for (int r = 0; r < ep->world; ++r)
        if (r != ep->rank && ep->peers.base[r]) (void)cudaIpcCloseMemHandle(ep->peers.base[r]);
    if (ep->local) (void)cudaFree(ep->local);
    if (ep->tables) (void)cudaFree(ep->tables);
    delete ep;
    return IZB_OK;
}

}  // extern "C"
