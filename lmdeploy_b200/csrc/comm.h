// State behind the opaque tm_comm of the C ABI.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#if TM_B200_WITH_NCCL
#include <nccl.h>
#endif

namespace tmb {
constexpr int kMaxP2pRanks = 8;
}

struct tm_comm {
#if TM_B200_WITH_NCCL
    ncclComm_t comm = nullptr;
#endif
    int world  = 1;
    int rank   = 0;
    int device = 0;
    // peer-memory all-reduce (allreduce.cu): this rank's exported region and the peers' mappings of theirs
    void*     p2p_local = nullptr;
    void*     p2p_peer[tmb::kMaxP2pRanks] = {};
    size_t    p2p_slot_bytes  = 0;
    int       p2p_ready       = 0;
    long long p2p_wait_cycles = 0;  // 0 = the default bound of the wait for the peers
    int       p2p_mode        = 0;  // 0 automatic; 1 every rank reads every slot; 2 rows dealt to owners
    int       p2p_bulk        = -1; // peers' rows fetched by bulk copies into shared memory: 1 yes, 0 16-byte loads, -1 by world size (beyond two ranks)
};

namespace tmb {
cudaError_t allreduce_add_rmsnorm_launch(tm_comm* c, int slot, __half* residual, __half* out, const __half* scale, float eps, int m,
                                         int n, unsigned* status, cudaStream_t st, bool pdl);
}
