// Test infrastructure: a flat C entry layer over the REFERENCE's own CUDA kernels for this path
// (lmdeploy v0.0.9), so that the GPU tests can run the reference and this library on the same
// inputs.  Nothing here is shipped and nothing under lmdeploy_b200/ links or loads it.
//
// The reference sources are compiled where they lie (see build_ref.py next to this file):
//   src/turbomind/kernels/gemm_s_f16/format.cu                      format converters
//   src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.cu                 GemmS4F16 (mma.sync tiles)
//   src/turbomind/kernels/decoder_masked_multihead_attention.cu     dispatcher
//   src/turbomind/kernels/decoder_masked_multihead_attention/decoder_masked_multihead_attention_128.cu
//   src/turbomind/models/llama/llama_decoder_kernels.cu             invokeFusedAddBiasResidualRMSNorm
// They build for sm_100a as they are (mma.sync / ldmatrix / cp.async).
#include "src/turbomind/kernels/decoder_masked_multihead_attention.h"
#include "src/turbomind/kernels/gemm_s_f16/format.h"
#include "src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h"
#include "src/turbomind/models/llama/llama_decoder_kernels.h"

#include <cmath>
#include <cstdio>
#include <exception>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
bool g_sync = true;
int  finish(cudaStream_t st)
{
    cudaError_t e = g_sync ? cudaStreamSynchronize(st) : cudaSuccess;
    if (e == cudaSuccess) e = cudaGetLastError();
    return (int)e;
}
}  // namespace

// 1 (default): every entry point waits for its kernels; 0: launches only (timing loops, graph capture)
REF_API void ref_set_sync(int on)
{
    g_sync = on != 0;
}

// src/turbomind/kernels/gemm_s_f16/format.h:11-30
REF_API int ref_reformat_s4_k_m8(void* dst, const void* src, int m, int k, void* stream)
{
    turbomind::reformat_s4_k_m8((uint32_t*)dst, (const uint32_t*)src, m, k, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

REF_API int ref_convert_s4_k_m8(void* A_dst, void* Q_dst, void* workspace, const void* A_src, const void* scales,
                                const void* qzeros, int m, int k, int group_size, void* stream)
{
    turbomind::convert_s4_k_m8((uint32_t*)A_dst, (half2*)Q_dst, (half*)workspace, (const uint32_t*)A_src, (const half*)scales,
                               (const uint32_t*)qzeros, m, k, group_size, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

REF_API int ref_transpose_qk_s4_k_m8_hf(void* dst, const void* src, int m, int k, int size_per_head, void* stream)
{
    turbomind::transpose_qk_s4_k_m8_hf((uint32_t*)dst, (const uint32_t*)src, m, k, size_per_head, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

REF_API int ref_fuse_w1_w3_s4_k_m8(void* dst, const void* src, int m, int k, void* stream)
{
    turbomind::fuse_w1_w3_s4_k_m8((uint32_t*)dst, (const uint32_t*)src, m, k, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

REF_API int ref_dequantize_s4(void* dst, const void* src, size_t count, void* stream)
{
    turbomind::dequantize_s4((uint4*)dst, (const uint32_t*)src, count, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

// GemmS4F16::Run (src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h:41-51), kernel chosen by the
// reference's own estimate (algo_id = -1).  type: 0 = kGemm, 1 = kFusedSiluFfn.
REF_API int ref_gemm_s4_f16(void* C, const void* A, const void* B, const void* Q, int m, int n, int k, int group_size, int type,
                            void* stream)
{
    static turbomind::GemmS4F16 gemm;
    try {
        gemm.Run((half*)C, (const uint*)A, (const half*)B, (const half2*)Q, m, n, k, group_size,
                 type ? turbomind::GemmS4F16::kFusedSiluFfn : turbomind::GemmS4F16::kGemm, -1, (cudaStream_t)stream);
    }
    catch (const std::exception& e) {
        std::fprintf(stderr, "ref_gemm_s4_f16: %s\n", e.what());
        return -1;
    }
    return finish((cudaStream_t)stream);
}

// masked_multihead_attention for fp16 (src/turbomind/kernels/decoder_masked_multihead_attention.h:50-133), with the
// members LlamaDecoderSelfAttentionLayer.cc:44-166 sets for LLaMA.
REF_API int ref_mmha_decode(void* out, const void* q, const void* k, const void* v, const void* q_bias, const void* k_bias,
                            const void* v_bias, int stride, int batch_size, int memory_max_len, int num_heads, int num_kv_heads,
                            int rotary_embedding_dim, float rotary_embedding_base, int timestep, const int* total_padding_tokens,
                            const unsigned char* finished, const int* length_per_sample, void** k_cache_per_sample,
                            void** v_cache_per_sample, size_t kv_cache_per_sample_offset, int int8_mode, float k_scale, float k_zp,
                            float v_scale, float v_zp, int max_position_embeddings, int use_dynamic_ntk, int use_logn_attn,
                            void* stream)
{
    Masked_multihead_attention_params<uint16_t> p{};
    p.out                        = (uint16_t*)out;
    p.q                          = (const uint16_t*)q;
    p.k                          = (const uint16_t*)k;
    p.v                          = (const uint16_t*)v;
    p.q_bias                     = (const uint16_t*)q_bias;
    p.k_bias                     = (const uint16_t*)k_bias;
    p.v_bias                     = (const uint16_t*)v_bias;
    p.stride                     = stride;
    p.finished                   = (bool*)finished;
    p.k_cache_per_sample         = (uint16_t**)k_cache_per_sample;
    p.v_cache_per_sample         = (uint16_t**)v_cache_per_sample;
    p.kv_cache_per_sample_offset = kv_cache_per_sample_offset;
    p.batch_size                 = batch_size;
    p.beam_width                 = 1;
    p.memory_max_len             = memory_max_len;
    p.length_per_sample          = length_per_sample;
    p.timestep                   = timestep;
    p.num_heads                  = num_heads;
    p.num_kv_heads               = num_kv_heads;
    p.hidden_size_per_head       = 128;
    p.rotary_embedding_dim       = rotary_embedding_dim;
    p.rotary_embedding_base      = rotary_embedding_base;
    p.max_position_embeddings    = max_position_embeddings;
    p.use_dynamic_ntk            = use_dynamic_ntk != 0;
    p.use_logn_attn              = use_logn_attn != 0;
    p.inv_sqrt_dh                = 1.f / std::sqrt(128.f);
    p.total_padding_tokens       = total_padding_tokens;
    p.int8_mode                  = int8_mode;
    p.attention_k_scale          = k_scale;
    p.attention_k_zp             = k_zp;
    p.attention_v_scale          = v_scale;
    p.attention_v_zp             = v_zp;
    masked_multihead_attention(p, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

// llama_decoder_kernels.h:8-9 (llama_kernels.cu, which holds the plain RMSNorm, drags in the
// reference's flash-attention sources and is left out)
REF_API int ref_add_residual_rmsnorm(void* residual, void* in_out, const void* bias, const void* scale, float eps, int batch_size,
                                     int n_dims, void* stream)
{
    turbomind::invokeFusedAddBiasResidualRMSNorm((half*)residual, (half*)in_out, (const half*)bias, (const half*)scale, eps,
                                                 batch_size, n_dims, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}
