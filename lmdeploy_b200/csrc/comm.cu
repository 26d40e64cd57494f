// Tensor-parallel communicator: thin NCCL wrapper, one process per GPU.  Collectives go on the
// caller's stream and are never followed by a host synchronisation (the reference's NcclGuard,
// src/turbomind/models/llama/LlamaNcclGuard.h:36-79, syncs the stream after every collective when
// several groups share a process; one process per GPU makes that unnecessary).
#include "comm.h"
#include "tm_b200.h"

#include <cstring>
#include <new>

#if TM_B200_WITH_NCCL

extern "C" int tm_comm_unique_id(void* id128)
{
    if (!id128) return TM_ERR_INVALID_ARG;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    ncclUniqueId id;
    if (ncclGetUniqueId(&id) != ncclSuccess) return TM_ERR_NCCL;
    std::memcpy(id128, &id, sizeof(id));
    return TM_OK;
}

extern "C" int tm_comm_create(tm_comm** out, int world_size, int rank, const void* id128, int device)
{
    if (!out || !id128 || world_size < 1 || rank < 0 || rank >= world_size) return TM_ERR_INVALID_ARG;
    *out = nullptr;
    int prev = 0;
    cudaGetDevice(&prev);
    if (cudaSetDevice(device) != cudaSuccess) return TM_ERR_CUDA;
    tm_comm* c = new (std::nothrow) tm_comm();
    if (!c) return TM_ERR_CUDA;
    ncclUniqueId id;
    std::memcpy(&id, id128, sizeof(id));
    ncclResult_t r = ncclCommInitRank(&c->comm, world_size, id, rank);
    cudaSetDevice(prev);
    if (r != ncclSuccess) {
        delete c;
        return TM_ERR_NCCL;
    }
    c->world  = world_size;
    c->rank   = rank;
    c->device = device;
    *out      = c;
    return TM_OK;
}

extern "C" int tm_comm_destroy(tm_comm* c)
{
    if (!c) return TM_OK;
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    for (int j = 0; j < tmb::kMaxP2pRanks; ++j) {
        if (c->p2p_peer[j]) cudaIpcCloseMemHandle(c->p2p_peer[j]);
    }
    if (c->p2p_local) cudaFree(c->p2p_local);
    cudaSetDevice(prev);
    if (c->comm) ncclCommDestroy(c->comm);
    delete c;
    return TM_OK;
}

extern "C" int tm_allreduce_sum_f16(tm_comm* c, void* buf, size_t count, void* stream)
{
    if (!c || !buf) return TM_ERR_INVALID_ARG;
    if (c->world == 1 || count == 0) return TM_OK;
    // in place, as src/turbomind/utils/nccl_utils.cc:57-69
    return ncclAllReduce(buf, buf, count, ncclHalf, ncclSum, c->comm, (cudaStream_t)stream) == ncclSuccess ? TM_OK :
                                                                                                               TM_ERR_NCCL;
}

extern "C" int tm_allgather(tm_comm* c, const void* send, void* recv, size_t bytes_per_rank, void* stream)
{
    if (!c || !send || !recv) return TM_ERR_INVALID_ARG;
    if (bytes_per_rank == 0) return TM_OK;
    return ncclAllGather(send, recv, bytes_per_rank, ncclInt8, c->comm, (cudaStream_t)stream) == ncclSuccess ? TM_OK :
                                                                                                                TM_ERR_NCCL;
}

#else  // built without NCCL

extern "C" int tm_comm_unique_id(void*) { return TM_ERR_NOT_BUILT; }
extern "C" int tm_comm_create(tm_comm**, int, int, const void*, int) { return TM_ERR_NOT_BUILT; }
extern "C" int tm_comm_destroy(tm_comm*) { return TM_OK; }
extern "C" int tm_allreduce_sum_f16(tm_comm*, void*, size_t, void*) { return TM_ERR_NOT_BUILT; }
extern "C" int tm_allgather(tm_comm*, const void*, void*, size_t, void*) { return TM_ERR_NOT_BUILT; }

#endif
