// Prefill driver: runs the new tokens of a batch of sequences through every layer and leaves their keys /
// values in the cache, as LlamaContextDecoder<T>::forward does around LlamaContextAttentionLayer<T>::forward
// (src/turbomind/models/llama/LlamaContextDecoder.cc:173-290, LlamaContextAttentionLayer.cc:119-247) for the
// int4 path: per layer { qkv GEMM, bias + RoPE + transpose, cache extend, causal attention over the cache,
// o GEMM, [allreduce], add + norm, w1|w3 GEMM with SiLU, w2 GEMM, [allreduce], add + norm }.  Tokens are
// packed ([token_num, hidden] activations, no padding rows reach a GEMM).  Asynchronous on `stream`.
#include "common.cuh"
#include "llama.h"
#include "tm_b200.h"

using namespace tmb;

namespace {

// per packed token: offset to its padded index b * max_q_len + s (what invokeGetPaddingOffsetAndCuSeqLens yields,
// src/turbomind/kernels/bert_preprocess_kernels.cu:54); per sequence: its length
__global__ void prefill_prepare_kernel(const int* cu_seqlens, int B, int max_q_len, int* padding_offset, int* input_length,
                                       const int* history, const int* context, int session_len, unsigned* status)
{
    const int b = blockIdx.x;
    const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
    if (threadIdx.x == 0) {
        input_length[b] = n;
        // The writers drop rows that do not fit (they never write outside a cache head), the attention clamps: the
        // result is then wrong without a fault, so the caller's mistake is recorded in the device status word.
        if (n > max_q_len || history[b] + n > session_len || context[b] != history[b] + n) atomicOr(status, kStatusPrefillOverflow);
    }
    for (int s = threadIdx.x; s < n; s += blockDim.x) padding_offset[t0 + s] = b * max_q_len + s - (t0 + s);
}

__global__ void prefill_embedding_kernel(__half* x, const __half* table, const int* ids, int hidden, int vocab)
{
    int id = ids[blockIdx.x];
    id     = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * hidden);
    uint4*       dst = reinterpret_cast<uint4*>(x + (size_t)blockIdx.x * hidden);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

bool grow(tm_llama* m, void** p, size_t* have, size_t need)
{
    if (*have >= need) return true;
    if (*p) cudaFree(*p);
    *p    = nullptr;
    *have = 0;
    if (cudaMalloc(p, need) != cudaSuccess) return false;
    *have = need;
    return true;
}

}  // namespace

extern "C" int tm_llama_prefill(tm_llama* m, const tm_llama_prefill_state* st, void* stream)
{
    if (!m || !st) return TM_ERR_INVALID_ARG;
    if (!st->input_ids || !st->cu_seqlens || !st->history_lengths || !st->context_lengths || !st->k_cache_ptrs || !st->v_cache_ptrs) {
        return TM_ERR_INVALID_ARG;
    }
    if (st->batch_size < 0 || st->token_num < 0 || st->max_q_len < 0) return TM_ERR_INVALID_ARG;
    if (st->batch_size == 0 || st->token_num == 0 || st->max_q_len == 0) return TM_OK;
    if (!m->tok_embeddings || !m->output_norm) return TM_ERR_INVALID_ARG;
    for (const auto& l : m->layers) {
        if (!l.set) return TM_ERR_INVALID_ARG;
    }
    const tm_llama_config& cfg = m->cfg;
    const int    B = st->batch_size, T = st->token_num, S = st->max_q_len;
    const int    H = m->local_heads, Hkv = m->local_kv_heads;
    const size_t hid = (size_t)m->hidden;
    cudaStream_t s   = (cudaStream_t)stream;
    int          prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(m->h->device);

    // ---- activations of this call (kept and reused; grown when a larger call comes)
    tm_llama::PrefillBuffers& pb = m->prefill;
    const size_t qkv_cols = (size_t)(H + 2 * Hkv) * 128;
    bool ok = grow(m, (void**)&pb.x, &pb.x_bytes, T * hid * 2) && grow(m, (void**)&pb.h, &pb.h_bytes, T * hid * 2)
              && grow(m, (void**)&pb.qkv, &pb.qkv_bytes, T * qkv_cols * 2)
              && grow(m, (void**)&pb.q, &pb.q_bytes, (size_t)B * H * S * 128 * 2)
              && grow(m, (void**)&pb.k, &pb.k_bytes, (size_t)B * Hkv * S * 128 * 2)
              && grow(m, (void**)&pb.v, &pb.v_bytes, (size_t)B * Hkv * S * 128 * 2)
              && grow(m, (void**)&pb.ctx, &pb.ctx_bytes, (size_t)T * H * 128 * 2)
              && grow(m, (void**)&pb.ffn, &pb.ffn_bytes, (size_t)T * m->local_inter * 2)
              && grow(m, (void**)&pb.pad, &pb.pad_bytes, (size_t)T * 4) && grow(m, (void**)&pb.len, &pb.len_bytes, (size_t)B * 4);
    int rc = ok ? TM_OK : TM_ERR_CUDA;
    auto step = [&](int r) {
        if (rc == TM_OK && r != TM_OK) rc = r;
        return rc == TM_OK;
    };
    auto launched = [&]() { return step(cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA); };
    LlamaLinear linear(m->h);

    if (rc == TM_OK) {
        prefill_prepare_kernel<<<B, 256, 0, s>>>(st->cu_seqlens, B, S, pb.pad, pb.len, st->history_lengths, st->context_lengths,
                                                 cfg.session_len, m->h->status);
        launched();
    }
    if (rc == TM_OK) {
        prefill_embedding_kernel<<<T, 128, 0, s>>>(pb.x, (const __half*)m->tok_embeddings, st->input_ids, m->hidden, cfg.vocab_size);
        launched();
    }
    // LlamaContextDecoder.cc:238-244
    if (rc == TM_OK) step(tm_rmsnorm(pb.h, pb.x, m->layers[0].self_attn_norm_weights, cfg.norm_eps, T, m->hidden, s));

    for (int l = 0; l < cfg.num_layer && rc == TM_OK; ++l) {
        const LlamaDecoderLayerWeight& w = m->layers[l];
        const size_t layer_offset = (size_t)l * Hkv * cfg.session_len * 128;  // LlamaContextAttentionLayer.cc:185
        // ---- LlamaContextAttentionLayer.cc:155-238
        if (!step(linear.forward(pb.qkv, pb.h, T, w.qkv, LlamaLinear::kGemm, s))) break;
        if (!step(tm_add_fused_qkv_bias_transpose(pb.q, pb.k, pb.v, pb.qkv, w.qkv.bias, pb.pad, st->history_lengths, pb.len, B, S, T,
                                                  H, Hkv, cfg.size_per_head, cfg.size_per_head, cfg.rope_theta, cfg.session_len, 0, 0,
                                                  s))) {
            break;
        }
        if (!step(tm_extend_kv_cache(st->k_cache_ptrs, st->v_cache_ptrs, layer_offset, pb.k, pb.v, B, pb.len, S, st->history_lengths,
                                     cfg.session_len, cfg.size_per_head, Hkv, s, cfg.quant_policy, w.past_kv_scale))) {
            break;
        }
        tm_context_attention_params a{};
        a.attn_out = pb.ctx, a.query = pb.q;
        a.key_cache = st->k_cache_ptrs, a.val_cache = st->v_cache_ptrs, a.cache_layer_offset = layer_offset;
        a.cu_seqlens = st->cu_seqlens, a.context_lengths = st->context_lengths;
        a.batch_size = B, a.head_num = H, a.kv_head_num = Hkv, a.size_per_head = cfg.size_per_head;
        a.max_q_len = S, a.max_seq_len = cfg.session_len, a.quant_policy = cfg.quant_policy;
        for (int i = 0; i < 4; ++i) a.kv_scale[i] = w.past_kv_scale[i];
        a.status_word = m->h->status;
        if (!step(tm_context_attention(&a, s))) break;
        if (!step(linear.forward(pb.h, pb.ctx, T, w.output, LlamaLinear::kGemm, s))) break;
        if (m->comm && m->comm->world > 1) {
            if (!step(tm_allreduce_sum_f16(m->comm, pb.h, (size_t)T * hid, s))) break;  // :244-248
        }
        // ---- LlamaContextDecoder.cc:252-279
        if (!step(tm_add_residual_rmsnorm(pb.x, pb.h, nullptr, w.ffn_norm_weights, cfg.norm_eps, T, m->hidden, s))) break;
        if (!step(linear.forward(pb.ffn, pb.h, T, w.fused_gating_intermediate, LlamaLinear::kFusedSiluFfn, s))) break;
        if (!step(linear.forward(pb.h, pb.ffn, T, w.ffn_output, LlamaLinear::kGemm, s))) break;
        if (m->comm && m->comm->world > 1) {
            if (!step(tm_allreduce_sum_f16(m->comm, pb.h, (size_t)T * hid, s))) break;
        }
        const void* next_norm = l + 1 < cfg.num_layer ? m->layers[l + 1].self_attn_norm_weights : m->output_norm;
        if (!step(tm_add_residual_rmsnorm(pb.x, pb.h, nullptr, next_norm, cfg.norm_eps, T, m->hidden, s))) break;
    }
    if (rc == TM_OK && st->hidden_out) {
        step(cudaMemcpyAsync(st->hidden_out, pb.h, (size_t)T * hid * 2, cudaMemcpyDeviceToDevice, s) == cudaSuccess ? TM_OK : TM_ERR_CUDA);
    }
    cudaSetDevice(prev);
    return rc;
}
