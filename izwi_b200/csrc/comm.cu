// NCCL plumbing for the sharded configurations: tensor-parallel all-reduce, expert-parallel
// all-to-all, all-gather of routing counts.  NCCL is opened with dlopen (the copy a host process
// already loaded, e.g. torch's, is reused), so the library has no link-time dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <new>

#include "izb_common.cuh"

struct izb_comm {
    ncclComm_t comm;
    int world, rank, device;
};

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    bool ok;
};
NcclApi g_nccl = {};
std::once_flag g_nccl_once;

void load_nccl() {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    bool ok = true;
    auto sym = [&](const char* name) {
        void* p = dlsym(h, name);
        if (!p) ok = false;
        return p;
    };
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
    g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(sym("ncclCommInitRank"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(sym("ncclCommDestroy"));
    g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(sym("ncclAllReduce"));
    g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(sym("ncclAllGather"));
    g_nccl.Send = reinterpret_cast<decltype(g_nccl.Send)>(sym("ncclSend"));
    g_nccl.Recv = reinterpret_cast<decltype(g_nccl.Recv)>(sym("ncclRecv"));
    g_nccl.GroupStart = reinterpret_cast<decltype(g_nccl.GroupStart)>(sym("ncclGroupStart"));
    g_nccl.GroupEnd = reinterpret_cast<decltype(g_nccl.GroupEnd)>(sym("ncclGroupEnd"));
    g_nccl.ok = ok;
}

const NcclApi* nccl() {
    std::call_once(g_nccl_once, load_nccl);
    return g_nccl.ok ? &g_nccl : nullptr;
}

int nccl_dtype(int32_t dtype, ncclDataType_t* out) {
    switch (dtype) {
        case IZB_BF16: *out = ncclBfloat16; return IZB_OK;
        case IZB_F32: *out = ncclFloat32; return IZB_OK;
        default: return IZB_ERR_BAD_ARG;
    }
}

}  // namespace

extern "C" {

int32_t izb_comm_unique_id(void* out_128_bytes) {
    if (!out_128_bytes) return IZB_ERR_BAD_ARG;
    const NcclApi* n = nccl();
    if (!n) return IZB_ERR_NO_DEVICE;
    ncclUniqueId id;
    if (n->GetUniqueId(&id) != ncclSuccess) return IZB_ERR_LAUNCH;
    static_assert(sizeof(id) == 128, "ncclUniqueId size");
    memcpy(out_128_bytes, &id, 128);
    return IZB_OK;
}

int32_t izb_comm_init(izb_ctx* ctx, int32_t world, int32_t rank, const void* unique_id_128_bytes, izb_comm** out) {
    if (!ctx || !unique_id_128_bytes || !out || world <= 0 || rank < 0 || rank >= world) return IZB_ERR_BAD_ARG;
    *out = nullptr;
    const NcclApi* n = nccl();
    if (!n) return IZB_ERR_NO_DEVICE;
    int cur = -1;
    IZB_CUDA_TRY(cudaGetDevice(&cur));
    if (cur != ctx->device) IZB_CUDA_TRY(cudaSetDevice(ctx->device));
    ncclUniqueId id;
    memcpy(&id, unique_id_128_bytes, 128);
    ncclComm_t c = nullptr;
    const ncclResult_t r = n->CommInitRank(&c, world, id, rank);
    if (cur != ctx->device) (void)cudaSetDevice(cur);
    if (r != ncclSuccess || !c) return IZB_ERR_LAUNCH;
    izb_comm* h = new (std::nothrow) izb_comm{c, world, rank, ctx->device};
    if (!h) {
        n->CommDestroy(c);
        return IZB_ERR_LAUNCH;
    }
    *out = h;
    return IZB_OK;
}

int32_t izb_comm_destroy(izb_comm* comm) {
    if (!comm) return IZB_ERR_BAD_ARG;
    const NcclApi* n = nccl();
    if (n && comm->comm) n->CommDestroy(comm->comm);
    delete comm;
    return IZB_OK;
}

int32_t izb_tp_allreduce(izb_comm* comm, izb_stream stream, void* buf, int64_t count, int32_t dtype) {
    if (!comm || count < 0) return IZB_ERR_BAD_ARG;
    if (count == 0 || comm->world == 1) return IZB_OK;
    if (!buf) return IZB_ERR_BAD_ARG;
    ncclDataType_t dt;
    if (nccl_dtype(dtype, &dt) != IZB_OK) return IZB_ERR_BAD_ARG;
    const NcclApi* n = nccl();
    if (!n) return IZB_ERR_NO_DEVICE;
    return n->AllReduce(buf, buf, static_cast<size_t>(count), dt, ncclSum, comm->comm, static_cast<cudaStream_t>(stream)) ==
                   ncclSuccess
               ? IZB_OK
               : IZB_ERR_LAUNCH;
}

int32_t izb_comm_allgather(izb_comm* comm, izb_stream stream, const void* send, void* recv, int64_t bytes_per_rank) {
    if (!comm || bytes_per_rank < 0) return IZB_ERR_BAD_ARG;
    if (bytes_per_rank == 0) return IZB_OK;
    if (!send || !recv) return IZB_ERR_BAD_ARG;
    const NcclApi* n = nccl();
    if (!n) return IZB_ERR_NO_DEVICE;
    return n->AllGather(send, recv, static_cast<size_t>(bytes_per_rank), ncclUint8, comm->comm,
                        static_cast<cudaStream_t>(stream)) == ncclSuccess
               ? IZB_OK
               : IZB_ERR_LAUNCH;
}

int32_t izb_ep_alltoall(izb_comm* comm, izb_stream stream, const void* send, const int64_t* host_send_rows, void* recv,
                        const int64_t* host_recv_rows, int64_t row_bytes) {
    if (!comm || !host_send_rows || !host_recv_rows || row_bytes <= 0) return IZB_ERR_BAD_ARG;
    const NcclApi* n = nccl();
    if (!n) return IZB_ERR_NO_DEVICE;
    int64_t s_total = 0, r_total = 0;
    for (int p = 0; p < comm->world; ++p) {
        if (host_send_rows[p] < 0 || host_recv_rows[p] < 0) return IZB_ERR_BAD_ARG;
        s_total += host_send_rows[p];
        r_total += host_recv_rows[p];
    }
    if ((s_total > 0 && !send) || (r_total > 0 && !recv)) return IZB_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint8_t* sp = static_cast<const uint8_t*>(send);
    uint8_t* rp = static_cast<uint8_t*>(recv);
    bool ok = n->GroupStart() == ncclSuccess;
    for (int p = 0; p < comm->world && ok; ++p) {
        const size_t sb = static_cast<size_t>(host_send_rows[p]) * row_bytes, rb = static_cast<size_t>(host_recv_rows[p]) * row_bytes;
        if (p == comm->rank) {
            // own block: a device-to-device copy on the same stream
            if (sb != rb) { ok = false; break; }
            if (sb && cudaMemcpyAsync(rp, sp, sb, cudaMemcpyDeviceToDevice, s) != cudaSuccess) ok = false;
        } else {
            if (sb) ok = ok && n->Send(sp, sb, ncclUint8, p, comm->comm, s) == ncclSuccess;
            if (rb) ok = ok && n->Recv(rp, rb, ncclUint8, p, comm->comm, s) == ncclSuccess;
        }
        sp += sb;
        rp += rb;
    }
    const bool ended = n->GroupEnd() == ncclSuccess;
    return ok && ended ? IZB_OK : IZB_ERR_LAUNCH;
}

}  // extern "C"
