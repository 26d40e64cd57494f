// Internal interface between the C ABI and the decode attention kernel.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>

namespace tmb {

// What the kernel needs to know about the sequence of grid row z, gathered into one 32-byte record by the decode
// driver (two 16-byte loads instead of a chain of dependent ones through order -> lengths / pointers).
struct MmhaSeqDesc {
    const void* k_cache;   // per-sequence base pointers (before the layer offset)
    const void* v_cache;
    int         length;    // tokens already cached
    int         seq;       // index of the sequence in the batch
    int         finished;
    int         reserved;
};

struct MmhaParams {
    __half*              out;       // [B, H*128]
    const __half*        qkv;       // [B, stride]: q heads | k heads | v heads
    const __half*        bias;      // [(H + 2 Hkv) * 128] or null
    void* const*         k_cache;   // device array [B] of per-sequence base pointers
    void* const*         v_cache;
    size_t               cache_offset;  // elements, added to every base pointer (layer offset)
    const int*           lengths;   // [B] tokens already cached
    const unsigned char* finished;  // [B] or null
    const int*           padding;   // [B] or null (total_padding_tokens)
    const int*           order;     // [B] or null: sequence handled by grid row z (longest first evens out the tail)
    const MmhaSeqDesc*   desc;      // [B] or null: the same in launch order with lengths, pointers and flags gathered
    const float2*        rope_table;  // [B][64] {cos, sin} of every sequence's position, in the order of `desc` (launch order), or null (computed in the kernel)
    int                  B, H, Hkv, stride, S_max, timestep, rot_dim, max_pos, use_dynamic_ntk, use_logn;
    int                  pos_from_length;  // RoPE position = cached length (the decode driver; lets a CUDA graph be replayed)
    float                rope_base, inv_sqrt_dh, k_scale, k_zp, v_scale, v_zp;
    float*               ws;        // split partials
    int*                 counters;  // self-resetting tickets
    unsigned*            status;
    int                  chunk, max_splits;  // filled from the plan
};

struct MmhaPlan {
    int    head_blocks;   // CTAs per KV head along the query-head axis (8 heads each)
    int    chunk;         // cached tokens per split (multiple of 64)
    int    max_splits;
    int    warps;         // warps per CTA: 4, 2 or 1
    size_t ws_floats;
    size_t counter_ints;
};

cudaError_t mmha_prepare();
MmhaPlan    mmha_plan(int B, int H, int Hkv, int max_len, int sm_count, int want_chunk, int want_warps = 0);
cudaError_t mmha_launch(const MmhaPlan& plan, MmhaParams p, bool int8, cudaStream_t st, bool pdl = false);

// RMSNorm kernels (norm.cu)
cudaError_t rmsnorm_launch(__half* out, const __half* in, const __half* scale, float eps, int m, int n, cudaStream_t st, bool pdl = false);
cudaError_t add_residual_rmsnorm_launch(
    __half* residual, __half* in_out, const __half* bias, const __half* scale, float eps, int m, int n, cudaStream_t st,
    bool pdl = false);

}  // namespace tmb
