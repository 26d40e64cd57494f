/* Drop-in for src/turbomind/kernels/decoder_masked_multihead_attention.h of lmdeploy v0.0.9 (:50-133).
 *
 * With `-I <this repo>/include/compat -I <this repo>/include` ahead of the TurboMind source root,
 * fusedQKV_masked_attention_dispatch (src/turbomind/models/llama/LlamaDecoderSelfAttentionLayer.cc:44-166)
 * compiles unchanged: it fills a Masked_multihead_attention_params<uint16_t> and calls
 * masked_multihead_attention(params, stream), which here hands the fields LLaMA uses to tm_mmha_decode.
 * The reference's decoder_masked_multihead_attention*.cu are then not compiled.
 *
 * The parameter structs keep the reference's member names, types and defaults, because the call site
 * assigns them by name (and memsets the whole struct first).  Members the LLaMA path never sets to
 * anything but zero / null are carried for source compatibility only; a call that does set one of them
 * (beams, prefix prompts, relative or linear position bias, int8 activations) is refused with an
 * exception instead of being computed wrongly. */
#pragma once

#include "tm_b200.h"

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <stdexcept>
#include <string>

#if defined(__has_include)
#if __has_include("src/turbomind/utils/cuda_bf16_wrapper.h")
#include "src/turbomind/utils/cuda_bf16_wrapper.h"
#endif
#endif

#ifndef CHECK_CUDA
#define CHECK_CUDA(call)                                                                                               \
    do {                                                                                                               \
        cudaError_t tm_b200_status_ = (call);                                                                          \
        if (tm_b200_status_ != cudaSuccess) {                                                                          \
            fprintf(stderr, "CUDA error (%s:%d): %s\n", __FILE__, __LINE__, cudaGetErrorString(tm_b200_status_));      \
            exit(1);                                                                                                   \
        }                                                                                                              \
    } while (0)
#endif

/* B sequences, H query heads, Dh = 128 values per head.  Members are grouped by kind here (the call site assigns them
 * by name after a memset of the whole struct, so their order is free). */
template<typename T>
struct Multihead_attention_params_base {
    // ---- tensors the LLaMA path uses
    T*       out = nullptr;                                      // [B, H * Dh]
    const T *q = nullptr, *k = nullptr, *v = nullptr;            // new token; one fused buffer for LLaMA, `stride` apart per sequence
    const T *q_bias = nullptr, *k_bias = nullptr, *v_bias = nullptr;
    const int* total_padding_tokens = nullptr;                   // rotary position of sequence b = timestep - total_padding_tokens[b]

    // ---- sizes and scalars the LLaMA path uses
    int   stride = 0, batch_size = 0, num_heads = 0, hidden_size_per_head = 0, rotary_embedding_dim = 0;
    int   memory_max_len = 0;                                    // rows of every sequence's cache (a ring once the sequence is longer)
    int   timestep = 0;                                          // >= every length_per_sample[b]
    int   max_input_length = 0;
    float inv_sqrt_dh = 0.0f;
    int   int8_mode = 0;                                         // bit 2 (QuantPolicy::kCacheKVInt8): the cache holds int8
    float attention_k_scale = 0.f, attention_k_zp = 0.f, attention_v_scale = 0.f, attention_v_zp = 0.f;

    // ---- carried for source compatibility: must stay 0 / null (a call that sets one is refused), except masked_tokens,
    // ---- which the reference's LLaMA kernel ignores as well
    int          beam_width = 0;                                 // 0 or 1 only
    const bool*  masked_tokens = nullptr;
    const int*   prefix_prompt_lengths = nullptr;
    int          max_prefix_prompt_length = 0;
    const T*     relative_attention_bias = nullptr;
    int          relative_attention_bias_stride = 0;
    const T*     linear_bias_slopes = nullptr;
    const float *query_weight_output_scale = nullptr, *attention_qk_scale = nullptr, *attention_output_weight_input_scale_inv = nullptr;
    const float *qkv_scale_out = nullptr, *attention_out_scale = nullptr;
};

template<typename T>
struct Multihead_attention_params: public Multihead_attention_params_base<T> {
    T **       k_cache_per_sample = nullptr, **v_cache_per_sample = nullptr;  // [B] base pointers
    size_t     kv_cache_per_sample_offset = 0;                                // elements from a base pointer to this layer
    const int* length_per_sample = nullptr;                                   // [B] tokens already cached
    bool*      finished = nullptr;                                            // [B] or null: finished sequences are skipped
    int        num_kv_heads = 0, max_position_embeddings = 0;
    float      rotary_embedding_base = 10000.0f;
    bool       use_dynamic_ntk = false, use_logn_attn = false;
};

template<class T>
using Masked_multihead_attention_params = Multihead_attention_params<T>;

/* half data travels as uint16_t in this interface (SATypeConverter, LlamaDecoderSelfAttentionLayer.cc:35-43) */
inline void masked_multihead_attention(const Masked_multihead_attention_params<uint16_t>& params, const cudaStream_t& stream)
{
    if (params.beam_width > 1 || params.prefix_prompt_lengths || params.max_prefix_prompt_length || params.relative_attention_bias
        || params.linear_bias_slopes || params.qkv_scale_out || params.attention_out_scale || params.query_weight_output_scale
        || params.attention_qk_scale || params.attention_output_weight_input_scale_inv) {
        throw std::runtime_error("[TM][b200] masked_multihead_attention: a feature outside the LLaMA decode path was requested");
    }
    tm_mmha_params a{};
    a.out                        = params.out;
    a.q                          = params.q;
    a.q_bias                     = params.q_bias;
    a.k                          = params.k;
    a.k_bias                     = params.k_bias;
    a.v                          = params.v;
    a.v_bias                     = params.v_bias;
    a.stride                     = params.stride;
    a.batch_size                 = params.batch_size;
    a.memory_max_len             = params.memory_max_len;
    a.num_heads                  = params.num_heads;
    a.num_kv_heads               = params.num_kv_heads;
    a.hidden_size_per_head       = params.hidden_size_per_head;
    a.rotary_embedding_dim       = params.rotary_embedding_dim;
    a.timestep                   = params.timestep;
    a.inv_sqrt_dh                = params.inv_sqrt_dh;
    a.total_padding_tokens       = params.total_padding_tokens;
    a.int8_mode                  = params.int8_mode;
    a.attention_k_scale          = params.attention_k_scale;
    a.attention_k_zp             = params.attention_k_zp;
    a.attention_v_scale          = params.attention_v_scale;
    a.attention_v_zp             = params.attention_v_zp;
    a.finished                   = reinterpret_cast<const unsigned char*>(params.finished);
    a.length_per_sample          = params.length_per_sample;
    a.k_cache_per_sample         = reinterpret_cast<void**>(params.k_cache_per_sample);
    a.v_cache_per_sample         = reinterpret_cast<void**>(params.v_cache_per_sample);
    a.kv_cache_per_sample_offset = params.kv_cache_per_sample_offset;
    a.max_position_embeddings    = params.max_position_embeddings;
    a.use_dynamic_ntk            = params.use_dynamic_ntk ? 1 : 0;
    a.use_logn_attn              = params.use_logn_attn ? 1 : 0;
    a.rotary_embedding_base      = params.rotary_embedding_base;
    tm_handle* h = tm_handle_of_current_device();
    if (!h) throw std::runtime_error("[TM][b200] no handle for the current CUDA device");
    const int rc = tm_mmha_decode(h, &a, (void*)stream);
    if (rc != TM_OK) throw std::runtime_error(std::string("[TM][b200] tm_mmha_decode: ") + tm_status_string(rc));
}

/* LlamaDecoderSelfAttentionLayer is instantiated for float as well (LlamaDecoderSelfAttentionLayer.cc:306-307),
 * so the overload must exist; the W4A16 path is half-only (LlamaLinear.h:64,78-80 says the same of its GEMM). */
inline void masked_multihead_attention(const Masked_multihead_attention_params<float>& params, const cudaStream_t& stream)
{
    (void)params, (void)stream;
    throw std::runtime_error("[TM][b200] masked_multihead_attention<float>: only half is built");
}
#ifdef ENABLE_BF16
inline void masked_multihead_attention(const Masked_multihead_attention_params<__nv_bfloat16>& params, const cudaStream_t& stream)
{
    (void)params, (void)stream;
    throw std::runtime_error("[TM][b200] masked_multihead_attention<bf16>: only half is built");
}
#endif
