// State behind the opaque tm_comm of the C ABI.
#pragma once

#include <cuda_runtime.h>

#if TM_B200_WITH_NCCL
#include <nccl.h>
#endif

struct tm_comm {
#if TM_B200_WITH_NCCL
    ncclComm_t comm = nullptr;
#endif
    int world  = 1;
    int rank   = 0;
    int device = 0;
};
