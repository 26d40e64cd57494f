// LLaMA decode driver (host C++): per-step layer loop over the W4A16 GEMM, the decode attention
// and the RMSNorm kernels, embedding lookup, lm-head and greedy pick; one CUDA graph per step.
// Sequencing follows LlamaDecoder::forward (src/turbomind/models/llama/LlamaDecoder.cc:158-242),
// LlamaDecoderSelfAttentionLayer::forward (LlamaDecoderSelfAttentionLayer.cc:193-304),
// LlamaFfnLayer::forward (LlamaFfnLayer.cc:66-116), LlamaV2::embeddingLookup / postDecodeEmbedding
// (LlamaV2.cc:184-201, 312-372) of lmdeploy v0.0.9.
#include "llama.h"

#include <cstdlib>
#include <cstring>
#include <new>
#include <nvtx3/nvToolsExt.h>

int tm_mmha_decode_impl(tm_handle* h, const tm_mmha_params* a, void* stream, int pos_from_length, const int* order,
                        const tmb::MmhaSeqDesc* desc = nullptr, const float2* rope_table = nullptr);

namespace tmb {

void LlamaDecoderLayerWeight::init_dims(const tm_llama_config& c)
{
    // LlamaDecoderLayerWeight.cc:49-77
    const size_t hidden = (size_t)c.head_num * c.size_per_head;
    const size_t tp     = c.tensor_para_size;
    qkv.input_dims      = hidden;
    qkv.output_dims     = (size_t)(c.head_num + 2 * c.kv_head_num) * c.size_per_head / tp;
    output.input_dims   = hidden / tp;
    output.output_dims  = hidden;
    fused_gating_intermediate.input_dims  = hidden;
    fused_gating_intermediate.output_dims = (size_t)c.inter_size / tp * 2;
    ffn_output.input_dims                 = (size_t)c.inter_size / tp;
    ffn_output.output_dims                = hidden;
    for (LlamaDenseWeight* w : {&qkv, &output, &fused_gating_intermediate, &ffn_output}) {
        w->type       = WeightType::kINT4;
        w->group_size = c.group_size;
    }
}

int LlamaLinear::forward(void* out, const void* in, int batch_size, const LlamaDenseWeight& w, Type type, cudaStream_t st) const
{
    if (w.type != WeightType::kINT4) return TM_ERR_UNSUPPORTED;  // only the W4A16 path is built
    return tm_gemm_s4_f16(h_, out, w.kernel, in, w.scales_and_zeros, (int)w.output_dims, batch_size, (int)w.input_dims,
                          w.group_size, type == kFusedSiluFfn ? TM_GEMM_FUSED_SILU_FFN : TM_GEMM_PLAIN, nullptr, 0, st);
}

namespace {

// Per step, one block of 64 threads per sequence: input token and activity, the attention's launch order (longest
// cached sequence first) with everything the attention needs to know about the sequence gathered into one record,
// and the rotation coefficients of the sequence's position (the same for every layer and head: computed here once
// with the calls the attention kernel would make, decoder_masked_multihead_attention_utils.h:885-897).
__global__ void prepare_step_kernel(const int* step, const int* start_step, const int* forced_ids, const int* picked,
                                    int* ids_in, unsigned char* inactive, int B, int max_steps, int vocab, const int* lengths,
                                    int* order, MmhaSeqDesc* desc, void* const* k_ptrs, void* const* v_ptrs, float2* rope_table,
                                    float rope_base, int rot_dim)
{
    const int b    = blockIdx.x;
    const int mine = lengths[b];
    // attention launch order: longest cached sequence first (rank by length, ties by index)
    __shared__ int s_rank;
    if (threadIdx.x == 0) {
        int rank = 0;
        for (int j = 0; j < B; ++j) {
            const int l = lengths[j];
            rank += (l > mine || (l == mine && j < b)) ? 1 : 0;
        }
        s_rank = rank;
    }
    __syncthreads();
    const int rank = s_rank;
    // the rotation coefficients sit at the sequence's place in the launch order, like its record: the attention CTA
    // asks for both at once, without first learning which sequence it has
    if (threadIdx.x < 64 && 2 * (int)threadIdx.x < rot_dim) {
        const float inv_freq = (float)mine / powf(rope_base, (float)(2 * threadIdx.x) / (float)rot_dim);
        float       sn, cs;
        sincosf(inv_freq, &sn, &cs);
        rope_table[(size_t)rank * 64 + threadIdx.x] = make_float2(cs, sn);
    }
    if (threadIdx.x != 0) return;
    const int  s   = *step;
    const bool off = s >= max_steps || (start_step != nullptr && s < start_step[b]);
    inactive[b]    = off ? 1 : 0;
    int id         = picked[b];
    if (!off && forced_ids != nullptr) {
        const int f = forced_ids[(size_t)s * B + b];
        if (f >= 0) id = f;
    }
    ids_in[b] = min(max(id, 0), vocab - 1);
    order[rank] = b;
    MmhaSeqDesc d;
    d.k_cache = k_ptrs[b], d.v_cache = v_ptrs[b], d.length = mine, d.seq = b, d.finished = off ? 1 : 0, d.reserved = 0;
    desc[rank] = d;
}

// x[b, :] = table[ids[b], :]   (kernels/decoding_kernels.cu:69-106)
__global__ void embedding_lookup_kernel(__half* x, const __half* table, const int* ids, int hidden)
{
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)ids[blockIdx.x] * hidden);
    uint4*       dst = reinterpret_cast<uint4*>(x + (size_t)blockIdx.x * hidden);
    for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// greedy pick over logits laid out [tp][B][vocab / tp]; ties go to the lowest token id
__global__ void argmax_kernel(const float* logits, int* picked, int* output_ids, const int* step,
                              const unsigned char* inactive, int B, int local_vocab, int tp, int max_steps)
{
    __shared__ float s_val[1024];
    __shared__ int   s_idx[1024];
    const int b    = blockIdx.x;
    float     best = -INFINITY;
    int       idx  = 0x7fffffff;
    auto take = [&](float x, int i) {
        if (x > best || (x == best && i < idx)) {
            best = x;
            idx  = i;
        }
    };
    for (int r = 0; r < tp; ++r) {
        const float* row = logits + ((size_t)r * B + b) * local_vocab;
        if ((local_vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
            // four logits per load, several loads in flight per thread
            const float4* row4 = reinterpret_cast<const float4*>(row);
            for (int v = threadIdx.x; v < local_vocab / 4; v += blockDim.x) {
                const float4 x = row4[v];
                const int    i = r * local_vocab + 4 * v;
                take(x.x, i);
                take(x.y, i + 1);
                take(x.z, i + 2);
                take(x.w, i + 3);
            }
        }
        else {
            for (int v = threadIdx.x; v < local_vocab; v += blockDim.x) take(row[v], r * local_vocab + v);
        }
    }
    s_val[threadIdx.x] = best;
    s_idx[threadIdx.x] = idx;
    __syncthreads();
    for (int off = blockDim.x / 2; off > 0; off >>= 1) {
        if (threadIdx.x < off) {
            const float x = s_val[threadIdx.x + off];
            const int   i = s_idx[threadIdx.x + off];
            if (x > s_val[threadIdx.x] || (x == s_val[threadIdx.x] && i < s_idx[threadIdx.x])) {
                s_val[threadIdx.x] = x;
                s_idx[threadIdx.x] = i;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const int s = *step;
        if (!inactive[b]) {
            picked[b] = s_idx[0];
        }
        if (s < max_steps) {
            output_ids[(size_t)s * B + b] = inactive[b] ? -1 : s_idx[0];
        }
    }
}

__global__ void advance_kernel(int* step, int* lengths, const unsigned char* inactive, int B)
{
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B && !inactive[b]) lengths[b] += 1;
    if (b == 0) *step += 1;
}

// [tp][B][vocab/tp] -> [B][vocab]
__global__ void gather_logits_kernel(float* out, const float* in, int B, int local_vocab, int tp)
{
    const size_t total = (size_t)tp * B * local_vocab;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int    v = i % local_vocab;
        const size_t t = i / local_vocab;
        const int    b = t % B;
        const int    r = t / B;
        out[(size_t)b * local_vocab * tp + (size_t)r * local_vocab + v] = in[i];
    }
}

// Named ranges for timeline tools, off unless TM_B200_NVTX=1 (the reference: PUSH_RANGE / POP_RANGE,
// src/turbomind/utils/nvtx_utils.h:37-49, at LlamaDecoderSelfAttentionLayer.cc:163,239 and LlamaFfnLayer.cc:87).
// Header-only NVTX: without a tool attached a push is a null call.  Ranges mark host-side enqueue order; inside a
// replayed CUDA graph they are not re-emitted.
struct NvtxRange {
    static bool enabled()
    {
        static const bool on = [] {
            const char* e = std::getenv("TM_B200_NVTX");
            return e && e[0] == '1';
        }();
        return on;
    }
    explicit NvtxRange(const char* name)
    {
        if (enabled()) nvtxRangePushA(name);
    }
    ~NvtxRange()
    {
        if (enabled()) nvtxRangePop();
    }
};

struct StepCtx {
    tm_llama*                    m;
    const tm_llama_decode_state* st;
    cudaStream_t                 stream;
    unsigned long long           launches = 0;
    int                          rc       = TM_OK;

    bool ok(int r)
    {
        if (rc == TM_OK && r != TM_OK) rc = r;
        return rc == TM_OK;
    }
    bool ok_cuda()
    {
        ++launches;
        return ok(cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA);
    }
};

// one decode step for the whole batch
int run_step(StepCtx& c)
{
    tm_llama&                    m   = *c.m;
    const tm_llama_config&       cfg = m.cfg;
    const tm_llama_decode_state& st  = *c.st;
    const int                    B   = st.batch_size;
    cudaStream_t                 s   = c.stream;
    LlamaLinear                  linear(m.h);
    const unsigned long long     l0 = m.h->launches;
    // kernels of this step overlap their prologues with the tail of the kernel before them
    struct PdlScope {
        explicit PdlScope(int on) { g_pdl = on; }
        ~PdlScope() { g_pdl = 0; }
    } pdl_scope(m.h->pdl);

    prepare_step_kernel<<<B, 64, 0, s>>>(st.step, st.start_step, st.forced_ids, m.picked, m.ids_in, m.inactive, B, st.max_steps,
                                         cfg.vocab_size, st.sequence_lengths, m.order, m.seq_desc, st.k_cache_ptrs, st.v_cache_ptrs,
                                         m.rope_table, cfg.rope_theta, cfg.size_per_head);
    if (!c.ok_cuda()) return c.rc;
    embedding_lookup_kernel<<<B, 128, 0, s>>>(m.x, (const __half*)m.tok_embeddings, m.ids_in, m.hidden);
    if (!c.ok_cuda()) return c.rc;

    // LlamaDecoder.cc:198-206
    if (!c.ok(tm_rmsnorm(m.hbuf, m.x, m.layers[0].self_attn_norm_weights, cfg.norm_eps, B, m.hidden, s))) return c.rc;
    ++c.launches;

    // Tensor parallel: the row-split GEMMs write their partial sums into a slot that the peers have mapped, and one
    // kernel sums the ranks, adds the residual and normalises (allreduce.cu); otherwise NCCL + the plain fused norm.
    const bool tp_on  = m.comm && m.comm->world > 1;
    const bool p2p    = tp_on && m.comm->p2p_ready && m.h->p2p_allreduce && (size_t)B * m.hidden * 2 <= m.comm->p2p_slot_bytes;
    __half*    part_o = p2p ? (__half*)tm_comm_p2p_slot(m.comm, 0) : m.hbuf;
    __half*    part_f = p2p ? (__half*)tm_comm_p2p_slot(m.comm, 1) : m.hbuf;
    auto reduce_add_norm = [&](int slot, const void* norm_w) {
        if (p2p) {
            ++c.launches;
            return c.ok(allreduce_add_rmsnorm_launch(m.comm, slot, m.x, m.hbuf, (const __half*)norm_w, cfg.norm_eps, B, m.hidden,
                                                     m.h->status, s, g_pdl != 0)
                                == cudaSuccess ?
                            TM_OK :
                            TM_ERR_CUDA);
        }
        if (tp_on) {
            if (!c.ok(tm_allreduce_sum_f16(m.comm, m.hbuf, (size_t)B * m.hidden, s))) return false;  // :292-297, LlamaFfnLayer.cc:106-110
            ++c.launches;
        }
        ++c.launches;
        return c.ok(tm_add_residual_rmsnorm(m.x, m.hbuf, nullptr, norm_w, cfg.norm_eps, B, m.hidden, s));
    };

    // Residual add + RMSNorm folded into the GEMMs on either side (gemm_s4_f16.h, GemmNormFusion): single GPU, a batch
    // the tensor-core kernel takes in one launch with every output tile split.  The first norm of the step and the
    // last one (in front of the lm-head) stay kernels of their own.
    const LlamaDecoderLayerWeight& w0 = m.layers[0];
    const bool fold = !tp_on && m.h->fold_norm && gemm_can_fuse_norm(m.h, (int)w0.qkv.output_dims, B, (int)w0.qkv.input_dims)
                      && gemm_can_fuse_norm(m.h, (int)w0.output.output_dims, B, (int)w0.output.input_dims)
                      && gemm_can_fuse_norm(m.h, (int)w0.fused_gating_intermediate.output_dims, B, (int)w0.fused_gating_intermediate.input_dims)
                      && gemm_can_fuse_norm(m.h, (int)w0.ffn_output.output_dims, B, (int)w0.ffn_output.input_dims);
    if (fold) {
        if (!c.ok(cudaMemsetAsync(m.ssq, 0, (size_t)2 * cfg.num_layer * cfg.max_batch_size * sizeof(unsigned long long), s) == cudaSuccess ?
                      TM_OK :
                      TM_ERR_CUDA)) {
            return c.rc;
        }
    }
    struct FusionScope {
        explicit FusionScope(const GemmNormFusion* f) { g_gemm_fusion = f; }
        ~FusionScope() { g_gemm_fusion = nullptr; }
    };
    auto ssq_of = [&](int idx) { return m.ssq + (size_t)idx * cfg.max_batch_size; };
    // consumer: scale rows by the 1 / rms that the sums of squares `idx` give; producer: fold the add + norm-weight in
    auto consumer = [&](int idx) {
        GemmNormFusion f;
        f.ssq_in = ssq_of(idx), f.inv_n = 1.f / (float)m.hidden, f.eps = cfg.norm_eps;
        return f;
    };
    auto producer = [&](int idx, const void* norm_w) {
        GemmNormFusion f;
        f.residual = m.x, f.norm_weight = (const __half*)norm_w, f.ssq_out = ssq_of(idx);
        return f;
    };

    for (int l = 0; l < cfg.num_layer; ++l) {
        const LlamaDecoderLayerWeight& w = m.layers[l];
        // ---- self attention (LlamaDecoderSelfAttentionLayer.cc:193-304)
        {
            NvtxRange r("qkv_gemm");
            const GemmNormFusion f = consumer(2 * l - 1);
            FusionScope          fs(fold && l > 0 ? &f : nullptr);
            if (!c.ok(linear.forward(m.qkv, m.hbuf, B, w.qkv, LlamaLinear::kGemm, s))) return c.rc;
        }
        tm_mmha_params a;
        std::memset(&a, 0, sizeof(a));
        a.out    = m.ctx;
        a.q      = m.qkv;
        a.k      = m.qkv + (size_t)m.local_heads * 128;
        a.v      = m.qkv + (size_t)(m.local_heads + m.local_kv_heads) * 128;
        if (w.qkv.bias) {
            a.q_bias = w.qkv.bias;
            a.k_bias = (const __half*)w.qkv.bias + (size_t)m.local_heads * 128;
            a.v_bias = (const __half*)w.qkv.bias + (size_t)(m.local_heads + m.local_kv_heads) * 128;
        }
        a.stride                     = (m.local_heads + 2 * m.local_kv_heads) * 128;
        a.batch_size                 = B;
        a.memory_max_len             = cfg.session_len;
        a.num_heads                  = m.local_heads;
        a.num_kv_heads               = m.local_kv_heads;
        a.hidden_size_per_head       = cfg.size_per_head;
        a.rotary_embedding_dim       = cfg.size_per_head;
        a.rotary_embedding_base      = cfg.rope_theta;
        a.timestep                   = cfg.session_len;  // upper bound on every cached length
        a.inv_sqrt_dh                = 1.f / sqrtf((float)cfg.size_per_head);
        a.finished                   = m.inactive;
        a.length_per_sample          = st.sequence_lengths;
        a.k_cache_per_sample         = st.k_cache_ptrs;
        a.v_cache_per_sample         = st.v_cache_ptrs;
        a.kv_cache_per_sample_offset = (size_t)l * m.local_kv_heads * cfg.session_len * 128;  // :243
        a.int8_mode                  = cfg.quant_policy;
        a.attention_k_scale          = w.past_kv_scale[0];
        a.attention_k_zp             = w.past_kv_scale[1];
        a.attention_v_scale          = w.past_kv_scale[2];
        a.attention_v_zp             = w.past_kv_scale[3];
        {
            NvtxRange r("scaled dot-product fusion");
            if (!c.ok(tm_mmha_decode_impl(m.h, &a, s, 1, m.order, m.seq_desc, m.rope_table))) return c.rc;
        }
        {
            NvtxRange r("o_gemm");
            const GemmNormFusion f = producer(2 * l, w.ffn_norm_weights);
            FusionScope          fs(fold ? &f : nullptr);
            if (!c.ok(linear.forward(part_o, m.ctx, B, w.output, LlamaLinear::kGemm, s))) return c.rc;
        }
        // ---- [sum over ranks] ; x += attn ; h = RMSNorm(x) * ffn_norm   (LlamaDecoder.cc:212-220)
        if (!fold && !reduce_add_norm(0, w.ffn_norm_weights)) return c.rc;
        // ---- feed forward (LlamaFfnLayer.cc:66-116): fused w1|w3 GEMM with the SiLU epilogue, then w2
        const bool  last      = l + 1 == cfg.num_layer;
        const void* next_norm = !last ? m.layers[l + 1].self_attn_norm_weights : m.output_norm;
        {
            NvtxRange r("ffn");
            {
                const GemmNormFusion f = consumer(2 * l);
                FusionScope          fs(fold ? &f : nullptr);
                if (!c.ok(linear.forward(m.ffn, m.hbuf, B, w.fused_gating_intermediate, LlamaLinear::kFusedSiluFfn, s))) return c.rc;
            }
            const GemmNormFusion f = producer(2 * l + 1, next_norm);
            FusionScope          fs(fold && !last ? &f : nullptr);
            if (!c.ok(linear.forward(part_f, m.ffn, B, w.ffn_output, LlamaLinear::kGemm, s))) return c.rc;
        }
        if ((!fold || last) && !reduce_add_norm(1, next_norm)) return c.rc;
    }
    if (st.hidden_out) {
        c.ok(cudaMemcpyAsync(st.hidden_out, m.hbuf, (size_t)B * m.hidden * 2, cudaMemcpyDeviceToDevice, s) == cudaSuccess ?
                 TM_OK :
                 TM_ERR_CUDA);
    }

    // ---- lm-head (LlamaV2.cc:312-372): fp16 weights, fp32 logits, vocab split + all-gather
    const float one = 1.f, zero = 0.f;
    const int   tp  = cfg.tensor_para_size;
    cublasSetStream(m.cublas, s);
    float* dst = tp > 1 ? m.logits_local : m.logits;
    if (m.h->lm_head_cublas) {
        // comparison only: the library GEMM the reference uses
        if (cublasGemmEx(m.cublas, CUBLAS_OP_T, CUBLAS_OP_N, m.local_vocab, B, m.hidden, &one, m.output_weight, CUDA_R_16F,
                         m.hidden, m.hbuf, CUDA_R_16F, m.hidden, &zero, dst, CUDA_R_32F, m.local_vocab, CUBLAS_COMPUTE_32F,
                         CUBLAS_GEMM_DEFAULT)
            != CUBLAS_STATUS_SUCCESS) {
            return c.rc = TM_ERR_CUDA;
        }
        ++c.launches;
    }
    else if (!c.ok(lm_head_launch(dst, m.local_vocab, m.hbuf, (const __half*)m.output_weight, B, m.local_vocab, m.hidden, m.h->status,
                                  m.h->gemm_wait_cycles, m.h->max_smem, s, g_pdl != 0, &c.launches))) {
        return c.rc;
    }
    if (tp > 1) {
        if (!c.ok(tm_allgather(m.comm, m.logits_local, m.logits, (size_t)B * m.local_vocab * sizeof(float), s))) return c.rc;
        ++c.launches;
    }
    if (st.logits_out) {
        gather_logits_kernel<<<m.h->sm_count * 4, 256, 0, s>>>(st.logits_out, m.logits, B, m.local_vocab, tp);
        if (!c.ok_cuda()) return c.rc;
    }
    argmax_kernel<<<B, 1024, 0, s>>>(m.logits, m.picked, st.output_ids, st.step, m.inactive, B, m.local_vocab, tp, st.max_steps);
    if (!c.ok_cuda()) return c.rc;
    advance_kernel<<<(B + 127) / 128, 128, 0, s>>>(st.step, st.sequence_lengths, m.inactive, B);
    if (!c.ok_cuda()) return c.rc;
    c.launches += m.h->launches - l0;
    return c.rc;
}

}  // namespace
}  // namespace tmb

using namespace tmb;

extern "C" int tm_llama_create(tm_llama** out, tm_handle* h, tm_comm* comm, const tm_llama_config* cfg)
{
    if (!out || !h || !cfg) return TM_ERR_INVALID_ARG;
    *out = nullptr;
    const tm_llama_config& c = *cfg;
    if (c.head_num <= 0 || c.kv_head_num <= 0 || c.inter_size <= 0 || c.num_layer <= 0 || c.vocab_size <= 0
        || c.max_batch_size <= 0 || c.session_len <= 0 || c.tensor_para_size <= 0 || c.tensor_para_rank < 0
        || c.tensor_para_rank >= c.tensor_para_size) {
        return TM_ERR_INVALID_ARG;
    }
    if (c.size_per_head != 128 || c.group_size != 128 || (c.quant_policy != 0 && c.quant_policy != 4)) return TM_ERR_UNSUPPORTED;
    const int tp = c.tensor_para_size;
    if (c.head_num % c.kv_head_num || c.head_num % tp || c.kv_head_num % tp || c.inter_size % tp || c.vocab_size % tp
        || (c.head_num * 128 / tp) % 128 || (c.inter_size / tp) % 128) {
        return TM_ERR_UNSUPPORTED;
    }
    if (tp > 1 && (!comm || comm->world != tp || comm->rank != c.tensor_para_rank)) return TM_ERR_INVALID_ARG;

    tm_llama* m = new (std::nothrow) tm_llama();
    if (!m) return TM_ERR_CUDA;
    m->h              = h;
    m->comm           = comm;
    m->cfg            = c;
    m->hidden         = c.head_num * 128;
    m->local_heads    = c.head_num / tp;
    m->local_kv_heads = c.kv_head_num / tp;
    m->local_inter    = c.inter_size / tp;
    m->local_vocab    = c.vocab_size / tp;
    m->layers.resize(c.num_layer);
    for (auto& l : m->layers) l.init_dims(c);

    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(h->device);
    const size_t B = c.max_batch_size;
    cudaError_t  e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) {
        if (e == cudaSuccess) e = cudaMalloc(p, bytes);
    };
    alloc((void**)&m->x, B * m->hidden * 2);
    alloc((void**)&m->hbuf, B * m->hidden * 2);
    alloc((void**)&m->qkv, B * (m->local_heads + 2 * m->local_kv_heads) * 128 * 2);
    alloc((void**)&m->ctx, B * m->local_heads * 128 * 2);
    alloc((void**)&m->ffn, B * m->local_inter * 2);
    alloc((void**)&m->logits_local, B * m->local_vocab * 4);
    alloc((void**)&m->logits, B * c.vocab_size * 4);
    alloc((void**)&m->ids_in, B * 4);
    alloc((void**)&m->picked, B * 4);
    alloc((void**)&m->inactive, B);
    alloc((void**)&m->order, (size_t)B * sizeof(int));
    alloc((void**)&m->seq_desc, (size_t)B * sizeof(MmhaSeqDesc));
    alloc((void**)&m->rope_table, (size_t)B * 64 * sizeof(float2));
    alloc((void**)&m->ssq, (size_t)2 * c.num_layer * B * sizeof(unsigned long long));
    alloc(&m->cublas_ws, 32u << 20);
    if (e == cudaSuccess) e = cudaMemset(m->picked, 0, B * 4);
    bool ok = e == cudaSuccess;
    if (ok) ok = cublasCreate(&m->cublas) == CUBLAS_STATUS_SUCCESS;
    if (ok) ok = cublasSetWorkspace(m->cublas, m->cublas_ws, 32u << 20) == CUBLAS_STATUS_SUCCESS;
    cudaSetDevice(prev);
    if (!ok) {
        h->last_cuda_error = (int)e;
        tm_llama_destroy(m);
        return TM_ERR_CUDA;
    }
    *out = m;
    return TM_OK;
}

extern "C" int tm_llama_destroy(tm_llama* m)
{
    if (!m) return TM_OK;
    if (m->graph_exec) cudaGraphExecDestroy(m->graph_exec);
    if (m->cublas) cublasDestroy(m->cublas);
    for (void* p : {(void*)m->x, (void*)m->hbuf, (void*)m->qkv, (void*)m->ctx, (void*)m->ffn, (void*)m->logits_local,
                    (void*)m->logits, (void*)m->ids_in, (void*)m->picked, (void*)m->inactive, (void*)m->order, (void*)m->seq_desc, (void*)m->rope_table, (void*)m->ssq, m->cublas_ws}) {
        if (p) cudaFree(p);
    }
    for (void* p : m->owned) cudaFree(p);
    for (void* p : {(void*)m->prefill.x, (void*)m->prefill.h, (void*)m->prefill.qkv, (void*)m->prefill.q, (void*)m->prefill.k,
                    (void*)m->prefill.v, (void*)m->prefill.ctx, (void*)m->prefill.ffn, (void*)m->prefill.pad, (void*)m->prefill.len}) {
        if (p) cudaFree(p);
    }
    delete m;
    return TM_OK;
}

extern "C" int tm_llama_set_layer(tm_llama* m, int layer, const tm_llama_layer_weights* w)
{
    if (!m || !w || layer < 0 || layer >= m->cfg.num_layer) return TM_ERR_INVALID_ARG;
    if (!w->self_attn_norm || !w->ffn_norm || !w->qkv_qweight || !w->qkv_scales_zeros || !w->o_qweight || !w->o_scales_zeros
        || !w->w13_qweight || !w->w13_scales_zeros || !w->w2_qweight || !w->w2_scales_zeros) {
        return TM_ERR_INVALID_ARG;
    }
    LlamaDecoderLayerWeight& l = m->layers[layer];
    l.self_attn_norm_weights   = w->self_attn_norm;
    l.ffn_norm_weights         = w->ffn_norm;
    l.qkv.kernel               = w->qkv_qweight;
    l.qkv.scales_and_zeros     = w->qkv_scales_zeros;
    l.qkv.bias                 = w->qkv_bias;
    l.output.kernel            = w->o_qweight;
    l.output.scales_and_zeros  = w->o_scales_zeros;
    l.fused_gating_intermediate.kernel           = w->w13_qweight;
    l.fused_gating_intermediate.scales_and_zeros = w->w13_scales_zeros;
    l.ffn_output.kernel                          = w->w2_qweight;
    l.ffn_output.scales_and_zeros                = w->w2_scales_zeros;
    std::memcpy(l.past_kv_scale, w->past_kv_scale, sizeof(l.past_kv_scale));
    l.set = true;
    if (m->graph_exec) {  // pointers are baked into the captured step
        cudaGraphExecDestroy(m->graph_exec);
        m->graph_exec = nullptr;
    }
    return TM_OK;
}

extern "C" int tm_llama_set_globals(tm_llama* m, const void* tok_embeddings, const void* output_norm, const void* output_weight)
{
    if (!m || !tok_embeddings || !output_norm || !output_weight) return TM_ERR_INVALID_ARG;
    m->tok_embeddings = tok_embeddings;
    m->output_norm    = output_norm;
    m->output_weight  = output_weight;
    if (m->graph_exec) {
        cudaGraphExecDestroy(m->graph_exec);
        m->graph_exec = nullptr;
    }
    return TM_OK;
}

extern "C" int tm_llama_check_status(tm_llama* m, void* stream, unsigned* word)
{
    if (!m) return TM_ERR_INVALID_ARG;
    return tm_check_device_status(m->h, stream, word);
}

extern "C" unsigned long long tm_llama_last_launches(const tm_llama* m)
{
    return m ? m->last_launches : 0ull;
}

extern "C" int tm_llama_decode(tm_llama* m, const tm_llama_decode_state* st, int n_steps, int use_graph, void* stream)
{
    if (!m || !st || n_steps < 0) return TM_ERR_INVALID_ARG;
    if (st->batch_size <= 0 || st->batch_size > m->cfg.max_batch_size || st->max_steps <= 0) return TM_ERR_INVALID_ARG;
    if (!st->k_cache_ptrs || !st->v_cache_ptrs || !st->sequence_lengths || !st->output_ids || !st->step) return TM_ERR_INVALID_ARG;
    if (!m->tok_embeddings) return TM_ERR_INVALID_ARG;
    for (const auto& l : m->layers) {
        if (!l.set) return TM_ERR_INVALID_ARG;
    }
    cudaStream_t s   = (cudaStream_t)stream;
    m->last_launches = 0;
    if (!use_graph) {
        for (int i = 0; i < n_steps; ++i) {
            StepCtx c{m, st, s};
            if (run_step(c) != TM_OK) return c.rc;
            m->last_launches += c.launches;
        }
        return TM_OK;
    }
    if (!m->graph_exec || std::memcmp(&m->graph_key, st, sizeof(*st)) != 0) {
        if (m->graph_exec) {
            cudaGraphExecDestroy(m->graph_exec);
            m->graph_exec = nullptr;
        }
        if (s == nullptr) return TM_ERR_INVALID_ARG;  // the legacy stream cannot be captured
        cudaGraph_t g = nullptr;
        if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return TM_ERR_CUDA;
        StepCtx c{m, st, s};
        run_step(c);
        const cudaError_t e = cudaStreamEndCapture(s, &g);
        if (c.rc != TM_OK || e != cudaSuccess || !g) {
            if (g) cudaGraphDestroy(g);
            m->h->last_cuda_error = (int)e;
            return c.rc != TM_OK ? c.rc : TM_ERR_CUDA;
        }
        const cudaError_t ei = cudaGraphInstantiate(&m->graph_exec, g, 0);
        cudaGraphDestroy(g);
        if (ei != cudaSuccess) {
            m->graph_exec         = nullptr;
            m->h->last_cuda_error = (int)ei;
            return TM_ERR_CUDA;
        }
        m->graph_key         = *st;
        m->launches_per_step = c.launches;
    }
    for (int i = 0; i < n_steps; ++i) {
        if (cudaGraphLaunch(m->graph_exec, s) != cudaSuccess) return TM_ERR_CUDA;
    }
    m->last_launches = m->launches_per_step * (unsigned long long)n_steps;
    return TM_OK;
}
