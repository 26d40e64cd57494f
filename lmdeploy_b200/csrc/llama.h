// Host-side decode driver: weight descriptors and the per-step layer loop, mirroring the
// reference's LlamaDenseWeight / LlamaDecoderLayerWeight / LlamaLinear / LlamaDecoder types
// (src/turbomind/models/llama/ of lmdeploy v0.0.9) for the int4 path.
#pragma once

#include "comm.h"
#include "handle.h"
#include "tm_b200.h"

#include <cublas_v2.h>
#include <vector>

namespace tmb {

enum class WeightType : int { kFP32, kFP16, kFP8, kINT8, kINT4 };  // LlamaDenseWeight.h:28-35

struct LlamaDenseWeight {  // LlamaDenseWeight.h:54-63
    size_t      input_dims       = 0;
    size_t      output_dims      = 0;
    const void* kernel           = nullptr;
    WeightType  type             = WeightType::kINT4;
    const void* bias             = nullptr;
    const void* scales_and_zeros = nullptr;
    int         group_size       = 128;
};

struct LlamaDecoderLayerWeight {  // LlamaDecoderLayerWeight.h / .cc:30-79 (per tensor-parallel rank)
    const void*      self_attn_norm_weights = nullptr;
    const void*      ffn_norm_weights       = nullptr;
    LlamaDenseWeight qkv, output, fused_gating_intermediate, ffn_output;
    float            past_kv_scale[4] = {1.f, 0.f, 1.f, 0.f};
    bool             set              = false;

    void init_dims(const tm_llama_config& c);
};

// LlamaLinear<half>::forward for int4 weights (LlamaLinear.h:28-42, 62-81)
class LlamaLinear {
public:
    enum Type { kGemm, kFusedSiluFfn };
    explicit LlamaLinear(tm_handle* h): h_(h) {}
    int forward(void* out, const void* in, int batch_size, const LlamaDenseWeight& w, Type type, cudaStream_t st) const;

private:
    tm_handle* h_;
};

}  // namespace tmb

struct tm_llama {
    tm_handle*      h    = nullptr;
    tm_comm*        comm = nullptr;
    tm_llama_config cfg{};
    int             hidden = 0, local_heads = 0, local_kv_heads = 0, local_inter = 0, local_vocab = 0;

    std::vector<tmb::LlamaDecoderLayerWeight> layers;
    const void* tok_embeddings = nullptr;
    const void* output_norm    = nullptr;
    const void* output_weight  = nullptr;
    std::vector<void*> owned;  // device copies made by tm_llama_load_workspace

    // activations, sized for max_batch_size
    __half *x = nullptr, *hbuf = nullptr, *qkv = nullptr, *ctx = nullptr, *ffn = nullptr;
    float * logits_local = nullptr, *logits = nullptr;
    int *   ids_in = nullptr, *picked = nullptr;
    int*    order = nullptr;  // sequences by cached length, longest first (attention launch order)
    tmb::MmhaSeqDesc* seq_desc   = nullptr;  // the same order, with lengths, cache pointers and flags gathered per sequence
    float2*           rope_table = nullptr;  // [batch][64] {cos, sin} of every sequence's position in this step
    unsigned long long* ssq      = nullptr;  // [2 * num_layer][max batch]: per-token sums of squares of the folded norms (fixed point)
    unsigned char* inactive = nullptr;

    // activations of tm_llama_prefill, sized by the largest call so far
    struct PrefillBuffers {
        __half *x = nullptr, *h = nullptr, *qkv = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *ctx = nullptr, *ffn = nullptr;
        int *   pad = nullptr, *len = nullptr;
        size_t  x_bytes = 0, h_bytes = 0, qkv_bytes = 0, q_bytes = 0, k_bytes = 0, v_bytes = 0, ctx_bytes = 0, ffn_bytes = 0,
               pad_bytes = 0, len_bytes = 0;
    } prefill;

    cublasHandle_t cublas    = nullptr;
    void*          cublas_ws = nullptr;

    // one captured step, keyed by the state it was captured for
    cudaGraphExec_t       graph_exec = nullptr;
    tm_llama_decode_state graph_key{};
    unsigned long long    launches_per_step = 0;
    unsigned long long    last_launches     = 0;
};
