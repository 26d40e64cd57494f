// Per-device state behind the opaque tm_handle of the C ABI.
#pragma once
#include <cuda_fp16.h>

#include "gemm_s4_f16.h"
#include "mmha.h"

struct tm_handle {
    int                device          = 0;
    int                sm_count        = 0;
    int                max_smem        = 0;
    int                l2_bytes        = 0;
    void*              scratch         = nullptr;  // split-K / split-KV partials
    size_t             scratch_bytes   = 0;
    int*               counters        = nullptr;  // self-resetting arrival tickets
    size_t             counter_ints    = 0;
    void*              attn_scratch    = nullptr;  // split-KV partials of the attention kernel
    size_t             attn_scratch_bytes = 0;
    int*               attn_counters   = nullptr;
    size_t             attn_counter_ints = 0;
    unsigned*          status          = nullptr;  // device status word (bounded waits)
    int                last_cuda_error = 0;
    unsigned long long launches        = 0;
    int                mmha_chunk      = 0;  // 0 = automatic; TM_B200_MMHA_CHUNK overrides
    int                mmha_warps      = 0;  // 0 = automatic; TM_B200_MMHA_WARPS (1, 2 or 4) overrides
    int                gemm_tc_min_n   = 17; // token count from which the tcgen05 kernel is used; TM_B200_GEMM_TC_MIN overrides
    int                gemm_wait_cycles = 0; // 0 = default bound of the split-tile wait of the tcgen05 GEMM (option "gemm_wait_cycles")
    int                pdl_direct      = 0;  // option "pdl_direct": direct GEMM / attention calls launch with programmatic serialization too
    int                p2p_allreduce   = 1;  // TM_B200_P2P_ALLREDUCE / option "p2p_allreduce": peer-memory all-reduce + norm in the decode step
    int                fold_norm       = 1;  // TM_B200_FOLD_NORM=0 / option "fold_norm": the decode step keeps residual add + RMSNorm as kernels of their own
    int                lm_head_cublas  = 0;  // TM_B200_LM_HEAD_CUBLAS=1 / option "lm_head_cublas": the decode step's lm-head through cuBLAS (comparison only)
    int                gemv_cols       = 1;  // TM_B200_GEMV_COLS / option "gemv_cols": 0 = the small-token GEMM never uses its column-owner kernel,
                                             // 1 = 32-column strips, 2 = 64-column strips
    int                pdl             = 1;  // TM_B200_PDL=0: the decode driver launches its kernels without programmatic dependent launch
};

namespace tmb {
// lm_head.cu: logits[tokens][ld] (fp32) = x[tokens][hidden] . w[vocab][hidden]^T, fp16 operands, tcgen05
cudaError_t lm_head_prepare(int max_smem);
cudaError_t sampling_prepare(int max_smem);  // sampling.cu
int lm_head_launch(float* logits, int ld, const __half* x, const __half* w, int tokens, int vocab, int hidden, unsigned* status,
                   long long max_wait_cycles, int max_smem, cudaStream_t st, bool pdl, unsigned long long* launches);
// Set by the decode driver around its launches (per host thread): the kernel launches made through
// the C ABI on this thread carry the programmatic-dependent-launch attribute.  Off for direct callers,
// who may put any kernel in front of ours.
extern thread_local int g_pdl;
// Set by the decode driver around ONE tm_gemm_s4_f16 call whose launch should carry a GemmNormFusion (gemm_s4_f16.h);
// the driver has checked with gemm_can_fuse_norm that the call is a single tensor-core launch with every tile split.
struct GemmNormFusion;
extern thread_local const GemmNormFusion* g_gemm_fusion;
bool gemm_can_fuse_norm(const tm_handle* h, int m, int n, int k);
}  // namespace tmb

