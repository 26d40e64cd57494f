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
//   src/turbomind/models/llama/llama_kernels.cu                     invokeRootMeanSquareNorm, invokeExtendKVCache,
//                                                                   invokeTransposeKVCache
//   src/turbomind/kernels/unfused_attention_kernels.cu              invokeAddFusedQKVBiasTranspose
//   src/turbomind/utils/logger.cc, src/turbomind/utils/Tensor.cc    (needed by the file above)
//   src/turbomind/models/llama/LlamaCacheManager.cc                 KV slab manager (host code; entry layer at the end)
// They build for sm_100a as they are (mma.sync / ldmatrix / cp.async).  llama_kernels.cu also holds the
// FlashAttentionOp front end, whose implementation needs CUTLASS and is not built: the empty
// FlashAttentionOpImpl below only satisfies the linker and aborts if it is ever called.
#include "src/turbomind/kernels/decoder_masked_multihead_attention.h"
#include "src/turbomind/kernels/gemm_s_f16/format.h"
#include "src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h"
#include "src/turbomind/kernels/unfused_attention_kernels.h"
#include "src/turbomind/models/llama/llama_decoder_kernels.h"
#include "src/turbomind/models/llama/llama_kernels.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <exception>

#define REF_API extern "C" __attribute__((visibility("default")))

namespace turbomind {
template<typename T, int V>
class FlashAttentionOpImpl<T, V>::impl {};
template<typename T, int V>
FlashAttentionOpImpl<T, V>::FlashAttentionOpImpl(int, int, int, int, int)
{
}
template<typename T, int V>
FlashAttentionOpImpl<T, V>::~FlashAttentionOpImpl()
{
}
template<typename T, int V>
int FlashAttentionOpImpl<T, V>::get_workspace_size() const
{
    return 0;
}
template<typename T, int V>
void FlashAttentionOpImpl<T, V>::operator()(Params&, cudaStream_t) const
{
    std::fprintf(stderr, "FlashAttentionOpImpl is not built in this test library\n");
    std::abort();
}
template class FlashAttentionOpImpl<half, 1>;
template class FlashAttentionOpImpl<half, 2>;
template class FlashAttentionOpImpl<float, 1>;
template class FlashAttentionOpImpl<float, 2>;
}  // namespace turbomind

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

// The same with the tile configuration named by the caller: algo_id indexes the list of
// src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.cu:72-93 (0 = 256x128x32 ... 15 = 64x16x256, 16 = 64x8x256).
REF_API int ref_gemm_s4_f16_algo(void* C, const void* A, const void* B, const void* Q, int m, int n, int k, int group_size, int type,
                                 int algo_id, void* stream)
{
    static turbomind::GemmS4F16 gemm;
    try {
        gemm.Run((half*)C, (const uint*)A, (const half*)B, (const half2*)Q, m, n, k, group_size,
                 type ? turbomind::GemmS4F16::kFusedSiluFfn : turbomind::GemmS4F16::kGemm, algo_id, (cudaStream_t)stream);
    }
    catch (const std::exception& e) {
        std::fprintf(stderr, "ref_gemm_s4_f16_algo: %s\n", e.what());
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

// llama_decoder_kernels.h:8-9
REF_API int ref_add_residual_rmsnorm(void* residual, void* in_out, const void* bias, const void* scale, float eps, int batch_size,
                                     int n_dims, void* stream)
{
    turbomind::invokeFusedAddBiasResidualRMSNorm((half*)residual, (half*)in_out, (const half*)bias, (const half*)scale, eps,
                                                 batch_size, n_dims, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

// llama_kernels.h:15-16
REF_API int ref_rmsnorm(void* out, const void* input, const void* scale, float eps, int m, int n, void* stream)
{
    turbomind::invokeRootMeanSquareNorm((half*)out, (const half*)input, (const half*)scale, eps, m, n, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

// unfused_attention_kernels.h:66-86
REF_API int ref_add_fused_qkv_bias_transpose(void* q_buf, void* k_buf, void* v_buf, void* QKV, const void* qkv_bias,
                                             const int* padding_offset, const int* history_length, const int* input_length,
                                             int batch_size, int seq_len, int token_num, int head_num, int kv_head_num,
                                             int size_per_head, int rotary_embedding_dim, float rotary_embedding_base,
                                             int max_position_embeddings, int use_dynamic_ntk, int use_logn_attn, void* stream)
{
    turbomind::invokeAddFusedQKVBiasTranspose((half*)q_buf, (half*)k_buf, (half*)v_buf, (half*)QKV, (const half*)qkv_bias,
                                              padding_offset, history_length, input_length, batch_size, seq_len, token_num,
                                              head_num, kv_head_num, size_per_head, rotary_embedding_dim, rotary_embedding_base,
                                              max_position_embeddings, use_dynamic_ntk != 0, use_logn_attn != 0,
                                              (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

// llama_kernels.h:36-51
REF_API int ref_extend_kv_cache(void** k_dst, void** v_dst, size_t dst_offset, const void* k_src, const void* v_src,
                                int local_batch_size, const int* query_length, int max_q_len, const int* history_length,
                                int max_seq_len, int size_per_head, int local_head_num, void* stream, int quant,
                                const float* kv_scale)
{
    turbomind::invokeExtendKVCache((half**)k_dst, (half**)v_dst, dst_offset, (const half*)k_src, (const half*)v_src,
                                   local_batch_size, query_length, max_q_len, history_length, max_seq_len, size_per_head,
                                   local_head_num, (cudaStream_t)stream, quant, kv_scale);
    return finish((cudaStream_t)stream);
}

// llama_kernels.h:53-68
REF_API int ref_transpose_kv_cache(void* key_cache_trans, void* val_cache_trans, const void** key_cache, const void** val_cache,
                                   size_t src_offset, int batch_size, const int* key_length, int max_kv_len, int max_seq_len,
                                   int size_per_head, int head_num, int head_n_rep, void* stream, int quant,
                                   const float* kv_scale)
{
    turbomind::invokeTransposeKVCache((half*)key_cache_trans, (half*)val_cache_trans, (const half**)key_cache,
                                      (const half**)val_cache, src_offset, batch_size, key_length, max_kv_len, max_seq_len,
                                      size_per_head, head_num, head_n_rep, (cudaStream_t)stream, quant, kv_scale);
    return finish((cudaStream_t)stream);
}

// llama_kernels.h:32-34: mask half [batch, max_q_len, max_k_len], 1 = visible
REF_API int ref_create_causal_masks(void* mask, const int* q_lens, const int* k_lens, int max_q_len, int max_k_len, int batch_size,
                                    void* stream)
{
    turbomind::invokeCreateCausalMasks((half*)mask, q_lens, k_lens, max_q_len, max_k_len, batch_size, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

// unfused_attention_kernels.h:22-40 as LlamaContextAttentionLayer.cc:372-382 fills it (half in, half out, in place allowed)
REF_API int ref_masked_softmax(void* attention_score, const void* qk, const void* attention_mask, int batch_size, int q_length,
                               int k_length, int num_heads, float qk_scale, void* stream)
{
    turbomind::MaskedSoftmaxParam<half, half> param{};
    param.attention_score    = (half*)attention_score;
    param.qk                 = (const half*)qk;
    param.attention_mask     = (const half*)attention_mask;
    param.batch_size         = batch_size;
    param.q_length           = q_length;
    param.k_length           = k_length;
    param.num_heads          = num_heads;
    param.qk_scale           = (half)qk_scale;
    param.linear_bias_slopes = nullptr;
    turbomind::invokeMaskedSoftmax(param, (cudaStream_t)stream);
    return finish((cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// LlamaCacheManager (src/turbomind/models/llama/LlamaCacheManager.{h,cc}), the reference's KV slab manager,
// compiled unmodified and driven through a flat C layer.  The engine's allocator is replaced by the few
// lines below (plain cudaMalloc / cudaFree): the manager only calls malloc(size, false) and free(&ptr).
#include "src/turbomind/models/llama/LlamaCacheManager.h"

#include <cstring>

namespace {

class PlainCudaAllocator: public turbomind::IAllocator {
public:
    void* malloc(size_t size, const bool is_set_zero = true, bool is_host = false) override
    {
        void* p = nullptr;
        if (cudaMalloc(&p, size) != cudaSuccess) return nullptr;
        if (is_set_zero) cudaMemset(p, 0, size);
        return p;
    }
    void free(void** ptr, bool is_host = false) const override
    {
        if (ptr && *ptr) cudaFree(*ptr);
        if (ptr) *ptr = nullptr;
    }
    void         setStream(cudaStream_t) override {}
    cudaStream_t returnStream() override { return nullptr; }
    void         memSet(void* ptr, const int val, const size_t size) override { cudaMemset(ptr, val, size); }

protected:
    bool                   isExist(void*) const override { return false; }
    turbomind::ReallocType isReMalloc(void*, size_t) const override { return turbomind::ReallocType::INCREASE; }
};

struct RefCacheManager {
    PlainCudaAllocator            alloc;
    turbomind::LlamaCacheManager* mgr = nullptr;
};

void fill(const turbomind::LlamaCacheManager::Sequence& s, unsigned long long* out)
{
    // id, max_seq_len, cache_len, token_count, k_cache, v_cache, timestamp
    out[0] = s.id, out[1] = s.max_seq_len, out[2] = s.cache_len, out[3] = s.token_ids.size();
    out[4] = (unsigned long long)(uintptr_t)s.k_cache, out[5] = (unsigned long long)(uintptr_t)s.v_cache, out[6] = s.timestamp;
}

}  // namespace

REF_API void* ref_cache_manager_create(size_t layer_num, size_t head_num, size_t size_per_head, size_t max_seq_len, size_t elem_bits,
                                       size_t max_entry_count, size_t chunk_size)
{
    auto* m = new RefCacheManager();
    try {
        m->mgr = new turbomind::LlamaCacheManager(layer_num, head_num, size_per_head, max_seq_len, elem_bits, max_entry_count,
                                                  chunk_size, /*rank*/ 1, &m->alloc);
    }
    catch (const std::exception& e) {
        std::fprintf(stderr, "ref_cache_manager_create: %s\n", e.what());
        delete m;
        return nullptr;
    }
    return m;
}

REF_API void ref_cache_manager_destroy(void* h)
{
    auto* m = (RefCacheManager*)h;
    if (!m) return;
    delete m->mgr;
    delete m;
}

// op: 0 create, 1 fetch.  out[7] as in fill().  Returns 0, or -1 when the reference throws (unknown id, every slab pinned).
REF_API int ref_cache_get(void* h, int op, unsigned long long id, unsigned long long* out, int* tokens, size_t capacity)
{
    auto* m = (RefCacheManager*)h;
    try {
        const auto s = op == 0 ? m->mgr->create(id, nullptr) : m->mgr->fetch(id, nullptr);
        fill(s, out);
        for (size_t i = 0; i < s.token_ids.size() && i < capacity; ++i) tokens[i] = s.token_ids[i];
    }
    catch (const std::exception&) {
        return -1;
    }
    return cudaDeviceSynchronize() == cudaSuccess ? 0 : -2;
}

// update(seq): the caller hands back what create / fetch returned, with new tokens and cache_len
REF_API int ref_cache_update(void* h, const unsigned long long* seq, const int* tokens, size_t token_count)
{
    auto* m = (RefCacheManager*)h;
    turbomind::LlamaCacheManager::Sequence s{};
    s.id = seq[0], s.max_seq_len = seq[1], s.cache_len = seq[2];
    s.k_cache = (void*)(uintptr_t)seq[4], s.v_cache = (void*)(uintptr_t)seq[5], s.timestamp = seq[6];
    s.token_ids.assign(tokens, tokens + token_count);
    try {
        m->mgr->update(s, nullptr);
    }
    catch (const std::exception&) {
        return -1;
    }
    return 0;
}

REF_API int ref_cache_erase(void* h, unsigned long long id)
{
    try {
        ((RefCacheManager*)h)->mgr->erase(id);
    }
    catch (const std::exception&) {
        return -1;
    }
    return 0;
}

REF_API int ref_cache_contains(void* h, unsigned long long id)
{
    return ((RefCacheManager*)h)->mgr->contains(id) ? 1 : 0;
}

// ---- token sampling: the reference's penalty and top-k sampling kernels, as BaseSamplingLayer::forward and
// ---- TopKSamplingLayer::runSampling call them (fp32 logits)
#include "src/turbomind/kernels/sampling_penalty_kernels.h"
#include "src/turbomind/kernels/sampling_topk_kernels.h"

REF_API size_t ref_curand_state_bytes()
{
    return sizeof(curandState_t);
}

REF_API int ref_curand_batch_init(void* states, int batch, const unsigned long long* seeds, cudaStream_t st)
{
    turbomind::invokeCurandBatchInitialize((curandState_t*)states, (size_t)batch, seeds, st);
    return finish(st);
}

// temperature -> repetition penalty (multiplicative) -> minimum length; any of the three pointers may be null
REF_API int ref_sampling_penalties(float* logits, int batch, int vocab, const float* temperatures, const float* rep_penalties,
                                   const int* output_ids, const int* input_lengths, int max_input_length, int step,
                                   const int* min_lengths, const int* end_ids, const int* sequence_lengths, cudaStream_t st)
{
    if (temperatures) turbomind::invokeBatchApplyTemperaturePenalty(logits, (const float*)nullptr, temperatures, batch, vocab, vocab, st);
    if (rep_penalties && step > 0) {
        turbomind::invokeBatchApplyRepetitionPenalty(logits, rep_penalties, output_ids, batch, batch, vocab, input_lengths,
                                                     max_input_length, step, turbomind::RepetitionPenaltyType::Multiplicative, st);
    }
    if (min_lengths) turbomind::invokeMinLengthPenalty(logits, min_lengths, end_ids, sequence_lengths, max_input_length, batch, vocab, st);
    return finish(st);
}

// workspace == null: returns the bytes needed in *workspace_bytes
REF_API int ref_batch_topk_sampling(void* workspace, size_t* workspace_bytes, const float* logits, int* ids, int* sequence_length,
                                    bool* finished, void* curand_states, int max_top_k, const int* top_ks, const float* top_ps,
                                    int vocab, const int* end_ids, int batch, const bool* skip_decode, cudaStream_t st)
{
    size_t ws = *workspace_bytes;
    turbomind::invokeBatchTopKSampling(workspace, ws, logits, ids, sequence_length, finished, (float*)nullptr, (float*)nullptr,
                                       (curandState_t*)curand_states, max_top_k, top_ks, 1.0f, top_ps, vocab, end_ids, st, batch,
                                       skip_decode);
    *workspace_bytes = ws;
    return workspace ? finish(st) : 0;
}

// ---- top-p sampling as TopPSamplingLayer<float>::runSampling drives it (src/turbomind/layers/sampling_layers/
// ---- TopPSamplingLayer.cu:254-346): invokeTopPInitialize, invokeAddBiasSoftMax (the logits become probabilities in
// ---- place), invokeBatchTopPSampling, invokeComputeToppDecay.  Scratch is allocated and freed here.
#include "src/turbomind/kernels/sampling_topp_kernels.h"

REF_API int ref_batch_topp_sampling(float* logits, int* ids, int* sequence_length, bool* finished, void* curand_states, float max_top_p,
                                    const float* top_ps, int vocab, const int* end_ids, int batch, const bool* skip_decode, cudaStream_t st)
{
    int *id_vals = nullptr, *offsets = nullptr, *begin_offsets = nullptr;
    if (cudaMalloc(&id_vals, sizeof(int) * (size_t)batch * vocab) != cudaSuccess) return -2;
    if (cudaMalloc(&offsets, sizeof(int) * (batch + 1)) != cudaSuccess) return -2;
    if (cudaMalloc(&begin_offsets, sizeof(int) * (batch + 1)) != cudaSuccess) return -2;
    turbomind::invokeTopPInitialize(id_vals, offsets, begin_offsets, (size_t)batch, vocab, st);
    turbomind::invokeAddBiasSoftMax(logits, (float*)nullptr, end_ids, finished, batch, vocab, vocab, st);
    size_t ws = 0, cub = 0;
    turbomind::invokeBatchTopPSampling<float>(nullptr, ws, cub, ids, sequence_length, finished, nullptr, nullptr, logits, id_vals, offsets,
                                              begin_offsets, (curandState_t*)curand_states, batch, (size_t)vocab, end_ids, max_top_p, top_ps,
                                              st, nullptr, skip_decode);
    void* work = nullptr;
    if (cudaMalloc(&work, ws) != cudaSuccess) return -2;
    turbomind::invokeBatchTopPSampling<float>(work, ws, cub, ids, sequence_length, finished, nullptr, nullptr, logits, id_vals, offsets,
                                              begin_offsets, (curandState_t*)curand_states, batch, (size_t)vocab, end_ids, max_top_p, top_ps,
                                              st, nullptr, skip_decode);
    const int rc = finish(st);
    cudaFree(work), cudaFree(id_vals), cudaFree(offsets), cudaFree(begin_offsets);
    return rc;
}

REF_API int ref_compute_topp_decay(float* runtime_top_p, const float* initial_top_p, const int* output_ids, const float* decay,
                                   const float* top_p_min, const int* reset_ids, int batch, cudaStream_t st)
{
    turbomind::invokeComputeToppDecay(runtime_top_p, initial_top_p, output_ids, decay, top_p_min, reset_ids, batch, st);
    return finish(st);
}

// ---- word lists and stopping: the reference's kernels as DynamicDecodeLayer::forward calls them (beam width 1)
#include "src/turbomind/kernels/ban_bad_words.h"
#include "src/turbomind/kernels/stop_criteria_kernels.h"

REF_API int ref_ban_bad_words(float* logits, const int* output_ids, int batch, const int* bad_words, int share_words, int bad_words_len,
                              int vocab, int step, cudaStream_t st)
{
    turbomind::invokeBanBadWords(logits, output_ids, (const int*)nullptr, batch, batch, 1, bad_words, share_words != 0,
                                 (size_t)bad_words_len, 0, vocab, (size_t)step, st);
    return finish(st);
}

REF_API int ref_stop_words_criterion(const int* output_ids, const int* stop_words, bool* finished, int stop_words_len, int batch, int step,
                                     cudaStream_t st)
{
    turbomind::invokeStopWordsCriterion(output_ids, (const int*)nullptr, stop_words, finished, 0, (size_t)stop_words_len, batch, 1, step, st);
    return finish(st);
}
