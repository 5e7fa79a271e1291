// Shared device/host helpers for the izwi_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/izwi_b200.h"

struct izb_ctx {
    int device;
    int sm_count;
    int max_smem_optin;
    int* d_status;  // [IZB_STATUS_WORDS] device status words written by kernels on a failed wait
    std::atomic<int64_t> launches;
    // arg-max over a few very long rows, split across CTAs: one packed (value, index) key and one
    // arrival counter per row; the last CTA of a row writes the result and zeroes both again
    unsigned long long* d_argmax_keys;  // [IZB_ARGMAX_SPLIT_ROWS]
    unsigned int* d_argmax_done;        // [IZB_ARGMAX_SPLIT_ROWS]
    // fused router + top-k: one arrival counter per 16-token tile (zero between launches)
    unsigned int* d_route_done;         // [IZB_ROUTE_TILES]
    int pdl;  // launch the decode-step kernels with programmatic stream serialisation (IZB_PDL=0 turns it off)
};

constexpr int IZB_STATUS_WORDS = 8;
constexpr int IZB_MAX_DEVICES = 64;  // izb_ctx_create refuses device ordinals at or above this (per-device tables)
constexpr int IZB_ARGMAX_SPLIT_ROWS = 1024;
constexpr int IZB_ROUTE_TILES = 1024;
// Bounded device-side waits give up after this many clock64 ticks (~1 s).
constexpr long long IZB_WAIT_LIMIT_CLOCKS = 2000000000LL;

#define IZB_CUDA_TRY(expr)                                 \
    do {                                                   \
        cudaError_t _e = (expr);                           \
        if (_e != cudaSuccess) {                           \
            (void)cudaGetLastError();                      \
            return IZB_ERR_LAUNCH;                         \
        }                                                  \
    } while (0)

static inline bool izb_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

#ifdef __CUDACC__
namespace izb {

// Programmatic dependent launch.  The kernels of a decode step are a chain of short launches, each
// reading what the one before wrote.  Launched through launch_chained, a kernel may start while its
// predecessor in the stream still runs: its CTAs set up shared memory and barriers, then pdl_wait()
// blocks until the predecessor has completed and its writes are visible.  Every kernel launched this
// way calls pdl_wait() before its first access to global memory that another kernel writes, and
// before its own first write; pdl_launch_dependents() at its top lets the successor do the same.
// Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// `cluster_x` > 1 launches thread-block clusters of that many CTAs along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained_cluster(const izb_ctx* ctx, int cluster_x, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                          size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2] = {};
    unsigned n = 0;
    if (ctx && ctx->pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(const izb_ctx* ctx, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                  cudaStream_t stream, Args... args) {
    return launch_chained_cluster(ctx, 1, kernel, grid, block, smem, stream, args...);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for the phase with the given parity; gives up after
// IZB_WAIT_LIMIT_CLOCKS and returns false. `abort_flag` (shared memory) lets
// the first thread that gives up release every other waiter of the CTA at once.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 0x3FFu) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Same, for waiters that can afford to wake late (copy producers several stages ahead): sleeps
// between polls instead of competing with the computing warps for issue slots.
__device__ __forceinline__ bool mbar_wait_bounded_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        __nanosleep(64);
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 0xFFu) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// 1-D bulk copy global -> shared (TMA engine), completion counted on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// Thread-block clusters: address of a shared-memory location in another CTA of the cluster, a store
// and an mbarrier arrival there (release at cluster scope, so the stores before it are visible to a
// waiter that acquires at cluster scope), and the barrier over all threads of the cluster.
__device__ __forceinline__ uint32_t cluster_map_shared(uint32_t addr, uint32_t cta_rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((++spins & 0x3FFu) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > IZB_WAIT_LIMIT_CLOCKS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}
// Waits on the clock alone (no abort flag): for a CTA that has already given up on its own work but
// must outlive the stores its cluster peers still make into its shared memory.
__device__ __forceinline__ bool mbar_wait_cluster_clock_only(uint32_t bar, uint32_t parity, long long limit_clocks) {
    const long long t0 = clock64();
    while (!mbar_try_wait_cluster(bar, parity)) {
        if (clock64() - t0 > limit_clocks) return false;
    }
    return true;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

template <int IMM>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(IMM));
    return r;
}

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
// One output element in the caller's type (izb_dtype): fp32, bf16 or fp16, round to nearest even.
__device__ __forceinline__ void store_typed(void* y, int y_dtype, long long idx, float v) {
    if (y_dtype == IZB_F32) static_cast<float*>(y)[idx] = v;
    else if (y_dtype == IZB_F16) static_cast<__half*>(y)[idx] = __float2half_rn(v);
    else static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float bf16_lo_to_f32(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi_to_f32(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

}  // namespace izb
#endif  // __CUDACC__
