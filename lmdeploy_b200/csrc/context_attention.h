// Shared between the two prefill attention kernels (context_attention.cu: mma.sync; context_attention_tc.cu: tcgen05).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace tmb {

struct CtxParams {
    __half*       out;
    const __half* q;  // [B, H, max_q_len, 128]
    void* const*  k_cache;
    void* const*  v_cache;
    size_t        offset;  // elements
    const int*    cu_seqlens;
    const int*    context_length;
    int           max_q_len, max_seq_len, H, n_rep;
    float         scale_log2;  // softmax scale * log2(e)
    float         k_scale, k_zp, v_scale, v_zp;
    unsigned*     status;           // bounded waits of the tcgen05 kernel record here
    long long     max_wait_cycles;
};

// context_attention_tc.cu
cudaError_t context_attention_tc_launch(const CtxParams& p, bool int8, int batch, cudaStream_t st);

}  // namespace tmb
