/*
 * tm_b200 — C ABI of a B200 (sm_100a) implementation of TurboMind's quantized decode path.
 *
 * Every entry point takes plain pointers and sizes.  Device pointers are caller-owned,
 * 16-byte aligned CUDA allocations of the device the handle was created on; `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).  All work is asynchronous
 * on `stream`.  Functions return TM_OK (0) or a negative tm_status; they never throw, abort or
 * exit.  Citations name the interface of lmdeploy v0.0.9 (TurboMind) that each entry replaces,
 * by the file's path inside that project.
 *
 * Naming trap kept from the reference GEMM: `m` is the number of OUTPUT FEATURES, `n` the
 * number of TOKENS (batch), `k` the number of input features.
 */
#ifndef TM_B200_H_
#define TM_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TM_API __attribute__((visibility("default")))
#else
#define TM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tm_status {
    TM_OK                 = 0,
    TM_ERR_INVALID_ARG    = -1, /* null pointer, misaligned pointer, negative size            */
    TM_ERR_UNSUPPORTED    = -2, /* group_size != 128, k % 128, m % 32, head_dim != 128 ...    */
    TM_ERR_WORKSPACE      = -3, /* caller workspace too small                                 */
    TM_ERR_CUDA           = -4, /* a CUDA runtime call failed (see tm_last_cuda_error)        */
    TM_ERR_DEVICE_TIMEOUT = -5, /* a bounded device-side wait gave up (status word non-zero)  */
    TM_ERR_NCCL           = -6,
    TM_ERR_NOT_BUILT      = -7, /* feature compiled out (e.g. NCCL missing)                   */
    TM_ERR_IO             = -8  /* a weight file is missing or has the wrong size            */
} tm_status;

typedef struct tm_handle tm_handle;

/* Per-device state: SM count, split-K scratch, split-KV scratch, device status word.
 * One handle is used by one host thread at a time (the reference runs one engine thread per
 * GPU: src/turbomind/models/llama/LlamaV2.cc:435-438); handles of different devices may be
 * used concurrently.  No process-global mutable state, with three exceptions: the per-device table behind
 * tm_gemm_s4_f16_noalloc (guarded by a mutex), the shared handles of tm_handle_of_current_device and a thread-local switch the decode driver sets around its
 * own launches. */
TM_API int tm_create(tm_handle** out, int device);
TM_API int tm_destroy(tm_handle* h);
/* A handle shared by everything in the process that runs on the current CUDA device, created on first use and kept
 * until the process exits (NULL if it cannot be created).  For callers that must keep a signature of the reference
 * and so cannot carry a handle: the header shims under include/compat.  A third piece of process-global state, guarded
 * by a mutex; the one-host-thread-at-a-time rule above applies to everyone who shares it. */
TM_API tm_handle* tm_handle_of_current_device(void);
TM_API const char* tm_status_string(int status);
/* cudaError_t of the most recent failing CUDA call made through this handle (0 if none). */
TM_API int tm_last_cuda_error(const tm_handle* h);
/* Synchronises `stream`, then reads and clears the device status word written by bounded
 * waits inside the kernels.  *word == 0 means no kernel gave up. */
TM_API int tm_check_device_status(tm_handle* h, void* stream, unsigned* word);
/* Number of kernel launches issued through this handle since creation. */
TM_API unsigned long long tm_launch_count(const tm_handle* h);
/* Tuning knobs of this handle (no reference counterpart; the same knobs are read from the environment
 * at tm_create).  `name`: "gemm_tc_min_n" (token count from which the tcgen05 GEMM is used),
 * "pdl_direct" (1: GEMM / attention calls made directly through the handle launch with programmatic stream
 * serialization, as the decode driver's do; only where no kernel ahead in the stream writes weights or cached rows),
 * "gemm_wait_cycles" (bound of the tcgen05 GEMM's wait for the partners of a split tile, 0 = default; tests),
 * "fold_norm" (0: the single-GPU decode step keeps residual add + RMSNorm as kernels of their own instead of folding
 * them into the tensor-core GEMMs on either side),
 * "lm_head_cublas" (1: the decode driver computes the lm-head with cuBLAS, as the reference does, instead of this
 * library's kernel; for comparison),
 * "gemv_cols" (the GEMM for 1..8 tokens: 0 = always the stream-K kernel, 1 = the column-owner kernel on 32-column strips
 * where the weight has a strip for every SM, 2 = on 64-column strips),
 * "mmha_chunk" (cached tokens per KV split, 0 = automatic), "mmha_warps" (warps per attention CTA: 1, 2,
 * 4 or 0 = automatic), "pdl" (1 = tm_llama_decode launches with programmatic dependent launch).
 * Returns TM_ERR_INVALID_ARG for an unknown name or value. */
TM_API int tm_set_option(tm_handle* h, const char* name, int value);

/* ------------------------------------------------------------------------------------------
 * AWQ W4A16 GEMM.  Replaces GemmS4F16::Run
 *   (src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h:41-51), called by
 *   LlamaLinear<half>::forwardInt4 (src/turbomind/models/llama/LlamaLinear.h:62-81).
 *
 *   C  half  [n, m]        (type 0)  or  [n, m/2]  (type 1: silu(C[:,2j]) * C[:,2j+1])
 *   A  uint  [k/32][m/32][32] uint4  — the runtime int4 layout written by tm_convert_s4_k_m8
 *   B  half  [n, k]        activations, row major
 *   Q  half2 [k/128, m]    {64 + zero, scale}
 * Requirements: group_size == 128, k % 128 == 0, m % 32 == 0 (type 1: m % 64 == 0), n >= 1.
 * `workspace` may be NULL (the handle's own scratch is used); otherwise it must hold
 * tm_gemm_s4_f16_workspace_bytes(m, n, k) bytes, zero-filled once before first use.
 */
enum { TM_GEMM_PLAIN = 0, TM_GEMM_FUSED_SILU_FFN = 1 };
TM_API size_t tm_gemm_s4_f16_workspace_bytes(int m, int n, int k);
TM_API int tm_gemm_s4_f16(tm_handle* h, void* C, const void* A, const void* B, const void* Q, int m, int n, int k,
                   int group_size, int type, void* workspace, size_t workspace_bytes, void* stream);

/* The same GEMM for callers that cannot allocate device memory — a server plugin whose memory is
 * owned by the server, a process that gave every free byte to its KV-cache pool, a loop that must
 * not meet cudaMalloc's device-wide synchronisation.  No counterpart in the reference (its GEMM
 * needs no scratch).  It takes no handle and calls no allocator: the split-K scratch is an 8 MB
 * array built into the library image (every GPU that loads the library holds it until exit).
 * Limits: n <= 16 tokens, and a shape whose partial tiles fit the 8 MB: every Llama-2-7B projection
 * and every tensor-parallel shard of Llama-2-70B does at all n <= 16; the un-sharded 70B gate_up
 * (m = 57344) does up to 8 tokens only.  Anything larger returns TM_ERR_WORKSPACE.  Runs on the CURRENT device, asynchronously on
 * `stream`.  The first call on a device resolves the array's device address and sets kernel
 * attributes: make that call before any stream capture.  All calls share the one array, so two
 * calls that overlap on the GPU (different streams) race; calls on one stream are safe.  A
 * bounded wait that gives up leaves the output incomplete and is not reported by this entry. */
TM_API int tm_gemm_s4_f16_noalloc(void* C, const void* A, const void* B, const void* Q, int m, int n, int k,
                           int group_size, int type, void* stream);

/* ------------------------------------------------------------------------------------------
 * int4 format helpers.  Replace the functions of
 *   src/turbomind/kernels/gemm_s_f16/format.h:11-30 that src/turbomind/python/bind.cpp:414-465
 *   exports to lmdeploy/serve/turbomind/deploy.py.  Same argument order.  `dst` is fully
 *   overwritten and must not alias `src`.
 */
TM_API int tm_reformat_s4_k_m8(uint32_t* dst, const uint32_t* src, int m, int k, void* stream);
TM_API int tm_convert_s4_k_m8(uint32_t* A_dst, void* Q_dst, void* workspace, const uint32_t* A_src, const void* scales,
                       const uint32_t* qzeros, int m, int k, int group_size, void* stream);
TM_API int tm_transpose_qk_s4_k_m8_hf(uint32_t* dst, const uint32_t* src, int m, int k, int size_per_head, void* stream);
TM_API int tm_fuse_w1_w3_s4_k_m8(uint32_t* dst, const uint32_t* src, int m, int k, void* stream);
/* dst: 8 halves per source word, nibble order [0,4,1,5,2,6,3,7], plain values 0..15. */
TM_API int tm_dequantize_s4(void* dst, const uint32_t* src, size_t count, void* stream);

/* ------------------------------------------------------------------------------------------
 * Decode-step masked multi-head attention with fused RoPE, KV append and (optionally) an int8
 * KV cache.  Replaces masked_multihead_attention(const Masked_multihead_attention_params<
 * uint16_t>&, const cudaStream_t&)
 *   (src/turbomind/kernels/decoder_masked_multihead_attention.h:50-133) as LLaMA drives it
 *   (fusedQKV_masked_attention_dispatch, src/turbomind/models/llama/
 *   LlamaDecoderSelfAttentionLayer.cc:44-166).  The struct mirrors the fields that call site
 *   sets, with the reference's names and meaning; zero-initialise it and fill what you use.
 *
 *   q/k/v              one fused buffer half [batch, stride]; q heads | k heads | v heads
 *   out                half [batch, num_heads * 128]
 *   k/v_cache_per_sample  device array [batch] of base pointers; sequence b's cache for this
 *                      layer starts kv_cache_per_sample_offset ELEMENTS in and is laid out
 *                      [num_kv_heads][memory_max_len][128] (element = half, or int8 when
 *                      int8_mode & 4)
 *   length_per_sample  device int [batch]: tokens already cached; the new token is written to
 *                      slot length % memory_max_len and attends to the last
 *                      min(length, memory_max_len - 1) cached tokens plus itself
 *   timestep           >= every length_per_sample[b]; RoPE position of sequence b is
 *                      timestep - total_padding_tokens[b] (0 padding if the pointer is NULL)
 *   finished           device bool [batch] or NULL: finished sequences are skipped entirely
 * Only hidden_size_per_head == 128 is supported (as in the reference build).
 */
typedef struct tm_mmha_params {
    void*       out;
    const void* q;
    const void* q_bias;
    const void* k;
    const void* k_bias;
    const void* v;
    const void* v_bias;
    int         stride;
    int         batch_size;
    int         memory_max_len;
    int         num_heads;
    int         num_kv_heads;
    int         hidden_size_per_head;
    int         rotary_embedding_dim;
    int         timestep;
    float       inv_sqrt_dh;
    const int*  total_padding_tokens;
    int         int8_mode; /* bit 2 (value 4, QuantPolicy::kCacheKVInt8): int8 KV cache */
    float       attention_k_scale;
    float       attention_k_zp;
    float       attention_v_scale;
    float       attention_v_zp;
    const unsigned char* finished;
    const int*  length_per_sample;
    void**      k_cache_per_sample;
    void**      v_cache_per_sample;
    size_t      kv_cache_per_sample_offset;
    int         max_position_embeddings;
    int         use_dynamic_ntk;
    int         use_logn_attn;
    float       rotary_embedding_base;
} tm_mmha_params;

TM_API int tm_mmha_decode(tm_handle* h, const tm_mmha_params* params, void* stream);

/* ------------------------------------------------------------------------------------------
 * lm-head: logits[tokens][ld] (fp32) = x[tokens][hidden] (half) . w[vocab][hidden]^T (half), ld >= vocab.
 * Replaces the cublas_wrapper_->Gemm call of LlamaV2::postDecodeEmbedding
 *   (src/turbomind/models/llama/LlamaV2.cc:312-372) for one rank's slice of the vocabulary (its
 *   all-gather and transpose stay with the caller: tm_allgather, and the decode driver's own gather).
 * hidden % 64 == 0; x and w 16-byte aligned.  A tcgen05 kernel of this library, no cuBLAS.
 */
TM_API int tm_lm_head_f16(tm_handle* h, float* logits, int ld, const void* x, const void* w, int tokens, int vocab, int hidden,
                   void* stream);

/* ------------------------------------------------------------------------------------------
 * Sampling of the next token from fp32 logits: temperature, repetition penalty, minimum length, then top-k
 * sampling with the top-p cut inside the k candidates - one kernel in place of the reference's
 *   invokeBatchApplyTemperaturePenalty / invokeBatchApplyRepetitionPenalty / invokeMinLengthPenalty
 *       (src/turbomind/kernels/sampling_penalty_kernels.cu:118-146, 386-465, 486-517), in the order of
 *       BaseSamplingLayer<T>::forward (src/turbomind/layers/sampling_layers/BaseSamplingLayer.cc:300-353), and
 *   invokeBatchTopKSampling (src/turbomind/kernels/sampling_topk_kernels.cu:380-441)
 * with the same draw: u = curand_uniform(state of the sequence); target = u * top_p * sum of exp(l_i - l_max) over
 * the k candidates; candidates are walked in descending order.  Pointers are device pointers; optional ones may be
 * NULL (that step is then skipped).  The logits are rewritten with the penalised values, as the reference's kernels do.
 *   logits [batch][ld] fp32, vocab_size <= ld; the row must fit shared memory (vocab_size up to about 55 000)
 *   output_ids [step][batch]: the tokens so far (prompt and generated), rows input_lengths[b] .. max_input_length - 1
 *       of sequence b are padding and not penalised; repetition penalty is multiplicative (l < 0 ? l * p : l / p),
 *       applied once per distinct token
 *   min_lengths / sequence_lengths: the end id is masked while sequence_lengths[b] + 1 - max_input_length < min_lengths[b]
 *   top_ks [batch] (else max_top_k for all), 1..1024; top_ps [batch] (else top_p), in (0, 1]
 *   rng_states: curandState_t per sequence (tm_sampling_rng_state_bytes each, set by tm_sampling_rng_init, which is
 *       curand_init(seed, 0, 0) as invokeCurandBatchInitialize does); or uniforms [batch] in (0, 1] supplied by the caller
 *   finished [batch] (bytes): a finished sequence gets end_ids[b]; with sequence_lengths_out also set, both are
 *       updated after the draw as topk_stage2_sampling does (length + 1, finished = drew the end id)
 *   skip_decode [batch] (bytes): sequences left alone (the reference's per-request top_k == 0)
 */
typedef struct tm_sampling_params {
    float*               logits;
    int                  ld;
    int                  vocab_size;
    int                  batch_size;
    const int*           output_ids;
    int                  step;
    const int*           input_lengths;
    int                  max_input_length;
    const float*         temperatures;
    const float*         repetition_penalties;
    const int*           min_lengths;
    const int*           sequence_lengths;
    const int*           end_ids;
    const int*           top_ks;
    int                  max_top_k;
    const float*         top_ps;
    float                top_p;
    void*                rng_states;
    const float*         uniforms;
    int*                 ids;
    int*                 sequence_lengths_out;
    unsigned char*       finished;
    const unsigned char* skip_decode;
    int                  output_ids_stride; /* ints between the rows of output_ids; 0 = batch_size */
} tm_sampling_params;
TM_API size_t tm_sampling_rng_state_bytes(void);
/* seeds [batch] on the device, or NULL: every sequence starts from `seed` */
TM_API int tm_sampling_rng_init(void* states, int batch_size, const unsigned long long* seeds, unsigned long long seed, void* stream);
TM_API int tm_sample_topk(tm_handle* h, const tm_sampling_params* params, void* stream);
/* Top-p sampling over the whole vocabulary, for the sequences the reference hands to its TopPSamplingLayer (per-request
 * top_k == 0; mark the others in skip_decode, and the other way round for tm_sample_topk).  Same parameter block
 * (top_ks / max_top_k are not read) and the same penalties first.  Replaces, in one kernel and without sorting,
 *   invokeAddBiasSoftMax       (src/turbomind/kernels/sampling_topp_kernels.cu:1295-1361)  p = exp(l - max) / (sum + 1e-6)
 *   invokeBatchTopPSampling    (sampling_topp_kernels.cu:1007-1161; topp_beam_topk_kernel :802-858, topp_sampling :878-1004)
 * as TopPSamplingLayer<T>::runSampling calls them (src/turbomind/layers/sampling_layers/TopPSamplingLayer.cu:254-346):
 * u = curand_uniform(state of the sequence) is drawn for every sequence that is not skipped; when the largest
 * probability alone reaches top_p that token is taken; otherwise the tokens are walked by descending probability
 * (equal ones in token order) until the running sum reaches u * top_p (the most probable token if it never does).
 * Unlike the reference the logits keep the penalised values, not the probabilities.
 * tm_top_p_decay is invokeComputeToppDecay (sampling_topp_kernels.cu:1381-1426), run by the layer after every draw:
 *   top_p[b] = output_ids[b] == reset_ids[b] ? initial[b] : max(top_p[b] * decay[b], min[b]). */
TM_API int tm_sample_topp(tm_handle* h, const tm_sampling_params* params, void* stream);
TM_API int tm_top_p_decay(float* runtime_top_p, const float* initial_top_p, const int* output_ids, const float* top_p_decay,
                   const float* top_p_min, const int* top_p_reset_ids, int batch_size, void* stream);
/* Word lists and stopping, beam width 1.  Replace invokeBanBadWords (src/turbomind/kernels/ban_bad_words.h),
 * invokeStopWordsCriterion and invokeLengthCriterion (src/turbomind/kernels/stop_criteria_kernels.h) as
 * DynamicDecodeLayer<T>::forward calls them (src/turbomind/layers/DynamicDecodeLayer.cc:214-236, 303-337).
 * A word list is the reference's int tensor [2][len] per sequence (or one shared list): row 0 the tokens of all items
 * back to back, row 1 the exclusive end offset of every item, padded with -1.  output_ids[s * stride + b] is the token of
 * sequence b at step s (stride 0 = batch_size).
 *   tm_ban_bad_words         logits[b][last token of an item] = -inf when the item's other tokens are the last ones generated
 *                            (steps step - size + 1 .. step - 1); single-token items are always banned
 *   tm_stop_words_criterion  finished[b] = 1 when the tokens up to and including step `step` end with an item
 *   tm_length_criterion      finished[b] |= step >= sequence_limit_length[b]; *finished_count (device, optional) = how many */
TM_API int tm_ban_bad_words(float* logits, int ld, int vocab_size, int batch_size, const int* output_ids, int output_ids_stride,
                     const int* bad_words, int bad_words_len, int share_words, int step, void* stream);
TM_API int tm_stop_words_criterion(const int* output_ids, int output_ids_stride, const int* stop_words, int stop_words_len,
                            unsigned char* finished, int batch_size, int step, void* stream);
TM_API int tm_length_criterion(unsigned char* finished, const unsigned* sequence_limit_length, int batch_size, int step,
                        int* finished_count, void* stream);

/* ------------------------------------------------------------------------------------------
 * RMSNorm of the decoder loop (half data, fp32 math).  Replace
 *   invokeRootMeanSquareNorm            (src/turbomind/models/llama/llama_kernels.cu:69-79)
 *   invokeFusedAddBiasResidualRMSNorm   (src/turbomind/models/llama/llama_decoder_kernels.cu:147-160)
 * tm_rmsnorm: out[m, n] = in * rsqrt(mean(in^2) + eps) * scale   (out may alias in).
 * tm_add_residual_rmsnorm: residual += in_out (+ bias); in_out = RMSNorm(residual) * scale.
 * n % 8 == 0, n <= 16384.
 */
TM_API int tm_rmsnorm(void* out, const void* in, const void* scale, float eps, int m, int n, void* stream);
TM_API int tm_add_residual_rmsnorm(void* residual, void* in_out, const void* bias, const void* scale, float eps, int m,
                            int n, void* stream);

/* ------------------------------------------------------------------------------------------
 * Prefill-side writers around the KV cache (half data, size_per_head == 128).  Replace, with the
 * same argument order and meaning,
 *   invokeAddFusedQKVBiasTranspose  (src/turbomind/kernels/unfused_attention_kernels.h:66-86, definition
 *                                    unfused_attention_kernels.cu:999-1027; caller
 *                                    src/turbomind/models/llama/LlamaContextAttentionLayer.cc:163-182)
 *   invokeExtendKVCache             (src/turbomind/models/llama/llama_kernels.h:36-51, llama_kernels.cu:400-464;
 *                                    caller LlamaContextAttentionLayer.cc:195-209)
 *   invokeTransposeKVCache          (llama_kernels.h:53-68, llama_kernels.cu:586-660; caller
 *                                    LlamaContextAttentionLayer.cc:332-346)
 *
 * tm_add_fused_qkv_bias_transpose: QKV [token_num, (head_num + 2 kv_head_num) * 128] (+ bias), interleaved-pair
 *   RoPE of q and k at position history_length[b] + s, optional log-n scaling of q, written to
 *   q_buf [B, head_num, seq_len, 128], k_buf / v_buf [B, kv_head_num, seq_len, 128].  padding_offset
 *   (may be NULL) maps a packed token to its padded index b * seq_len + s.  QKV itself is not modified.
 * tm_extend_kv_cache: k_src / v_src [B, heads, max_q_len, 128] rows [0, query_length[b]) -> cache rows
 *   history_length[b] + s of k_dst[b] / v_dst[b] (device arrays of device pointers) at element offset
 *   dst_offset, cache layout [heads, max_seq_len, 128]; quant & 4: int8 cache,
 *   q = sat_s8(rint((x - zp) / scale)), kv_scale = HOST pointer to {k_scale, k_zp, v_scale, v_zp}.
 * tm_transpose_kv_cache: cache rows [0, key_length[b]) -> [B, head_num, max_kv_len, 128], query head h
 *   reading cached head h / head_n_rep; int8 rows dequantised as half(q * scale + zp).
 * K and V are moved by one launch each call; all launches are asynchronous on `stream`.
 */
TM_API int tm_add_fused_qkv_bias_transpose(void* q_buf, void* k_buf, void* v_buf, const void* QKV, const void* qkv_bias,
                                           const int* padding_offset, const int* history_length, const int* input_length,
                                           int batch_size, int seq_len, int token_num, int head_num, int kv_head_num,
                                           int size_per_head, int rotary_embedding_dim, float rotary_embedding_base,
                                           int max_position_embeddings, int use_dynamic_ntk, int use_logn_attn, void* stream);
TM_API int tm_extend_kv_cache(void** k_dst, void** v_dst, size_t dst_offset, const void* k_src, const void* v_src,
                              int local_batch_size, const int* query_length, int max_q_len, const int* history_length,
                              int max_seq_len, int size_per_head, int local_head_num, void* stream, int quant,
                              const float* kv_scale);
TM_API int tm_transpose_kv_cache(void* key_cache_trans, void* val_cache_trans, const void** key_cache, const void** val_cache,
                                 size_t src_offset, int batch_size, const int* key_length, int max_kv_len, int max_seq_len,
                                 int size_per_head, int head_num, int head_n_rep, void* stream, int quant,
                                 const float* kv_scale);

/* ------------------------------------------------------------------------------------------
 * Prefill (context) attention over the KV cache: causal softmax(q k^T / sqrt(128)) v for the new tokens of
 * every sequence, keys / values read in place from the per-sequence cache (fp16, or int8 dequantised as
 * half(q * scale + zp) on the fly), grouped-query heads.  Replaces what
 *   LlamaContextAttentionLayer<T>::fusedMultiHeadAttention  (src/turbomind/models/llama/
 *   LlamaContextAttentionLayer.cc:257-313) asks of FlashAttentionOp<T>::operator()
 *   (src/turbomind/models/llama/llama_kernels.h:129-150): query = q_buf_2_, key / val = the cache pointers
 *   with the layer offset, cu_seqlens for the packed output, actual_seqlen_k = context_lengths,
 * and, for an int8 cache, the unfused route (:316-420) without its dequantised copy of the cache.
 * Query i of sequence b sits at position context_lengths[b] - q_len[b] + i and sees keys [0, position];
 * q_len[b] = cu_seqlens[b + 1] - cu_seqlens[b]; its output row is cu_seqlens[b] + i.
 * The new tokens' keys / values must already be in the cache (tm_extend_kv_cache).
 * Runs on the tcgen05 tensor core (scores and output accumulate in TMEM); TM_B200_CTX_ATTN_LEGACY=1 selects the
 * earlier mma.sync kernel for comparison.
 */
typedef struct tm_context_attention_params {
    void*        attn_out;           /* half [token_num, head_num * 128]                           */
    const void*  query;              /* half [batch, head_num, max_q_len, 128]                     */
    void**       key_cache;          /* device array [batch] of per-sequence cache base pointers   */
    void**       val_cache;
    size_t       cache_layer_offset; /* elements: layer * kv_head_num * max_seq_len * 128          */
    const int*   cu_seqlens;         /* device int [batch + 1], prefix sums of the query lengths   */
    const int*   context_lengths;    /* device int [batch], history + query length                 */
    int          batch_size;
    int          head_num;
    int          kv_head_num;
    int          size_per_head;      /* 128 */
    int          max_q_len;
    int          max_seq_len;        /* rows per head of the cache                                 */
    int          quant_policy;       /* & 4: int8 cache                                            */
    float        kv_scale[4];        /* k_scale, k_zp, v_scale, v_zp                               */
    unsigned*    status_word;        /* optional device word (a handle's): a bounded wait inside the
                                        kernel that gives up sets a bit there; NULL = a word kept by
                                        the library, read with tm_context_attention_last_status      */
} tm_context_attention_params;
TM_API int tm_context_attention(const tm_context_attention_params* params, void* stream);
/* Synchronises the device, then reads and clears the status word the library keeps for calls that passed no
 * status_word of their own (current device).  0 = no wait gave up. */
TM_API int tm_context_attention_last_status(unsigned* word);

/* ------------------------------------------------------------------------------------------
 * Tensor-parallel communicator (one process per GPU; NCCL over NVLink).  Replaces
 *   ftNcclAllReduceSum<half> / ftNcclAllGather (src/turbomind/utils/nccl_utils.h:94-99) and the
 *   NcclParam set-up of src/turbomind/triton_backend/transformer_triton_backend.cpp:24-82.
 * Rank 0 calls tm_comm_unique_id and hands the 128 bytes to the other ranks by any host channel.
 * Collectives are issued on the caller's stream with no host synchronisation.
 */
typedef struct tm_comm tm_comm;
TM_API int tm_comm_unique_id(void* id128);
TM_API int tm_comm_create(tm_comm** out, int world_size, int rank, const void* id128, int device);
TM_API int tm_comm_destroy(tm_comm* c);
TM_API int tm_allreduce_sum_f16(tm_comm* c, void* buf, size_t count, void* stream);
/* Peer-memory all-reduce for the decode step (no counterpart in the reference, whose custom all-reduce,
 * src/turbomind/kernels/custom_ar_kernels.cu:138-199, is not used by the LLaMA layers): the sum over the tensor-parallel
 * ranks fused with the residual add and RMSNorm that follow it (LlamaDecoder.cc:212-236).
 *   tm_comm_p2p_export   allocates this rank's region (three buffers of slot_bytes each + counters) and returns its CUDA IPC
 *                        handle (64 bytes); every rank passes the handles of all ranks, in rank order, to
 *   tm_comm_p2p_import   which maps the peers' regions.  One process per GPU, all on one node, world <= 8.
 *   tm_comm_p2p_slot     device address of slot 0 / 1 of THIS rank: the row-split GEMM writes its partial sums there.
 *   tm_allreduce_add_residual_rmsnorm   residual[m, n] += sum over ranks of slot rows (rounded to fp16 first, as an fp16
 *                        all-reduce delivers it); out[m, n] = RMSNorm(residual) * scale.  Ranks are read in rank order.
 *                        With token rows dealt to owner ranks ("p2p_mode" below; rank r owns rows
 *                        [r * ceil(m / world), (r + 1) * ceil(m / world))) every rank gets all of `out`, but `residual`
 *                        is updated for the rank's own rows only: it must be fed back to this call alone, as the
 *                        decode step does.  The region then holds a third buffer of slot_bytes for the handed-on rows.
 *                        Calls must alternate between the two slots on every rank alike.  `status_word` is a device
 *                        word (a handle's): a peer that does not show up within the bound sets a bit there and the
 *                        kernel finishes on what it has, it never hangs. */
TM_API int tm_comm_p2p_export(tm_comm* c, size_t slot_bytes, void* handle64);
/* "p2p_wait_cycles": bound, in SM clock cycles, of the wait for the peers' slots (0 = default, about a quarter of a second);
 * "p2p_bulk": 1 a peer's rows come to shared memory with one bulk copy per rank and row (no multicast), 0 with 16-byte
 * loads of the threads, -1 (default) bulk copies beyond two ranks (environment: TM_B200_P2P_BULK);
 * "p2p_mode": 1 every rank reads every rank's whole slot, 2 token rows dealt to owner ranks, which finish them and
 * hand them on, 0 (default) picks 1 up to four ranks and 2 beyond (environment: TM_B200_P2P_MODE, read by
 * tm_comm_p2p_export). */
TM_API int tm_comm_set_option(tm_comm* c, const char* name, long long value);
TM_API int tm_comm_p2p_import(tm_comm* c, const void* handles);
TM_API void* tm_comm_p2p_slot(tm_comm* c, int slot);
TM_API size_t tm_comm_p2p_slot_bytes(const tm_comm* c);
TM_API int tm_allreduce_add_residual_rmsnorm(tm_comm* c, int slot, void* residual, void* out, const void* scale, float eps, int m,
                                             int n, unsigned* status_word, void* stream);
TM_API int tm_allgather(tm_comm* c, const void* send, void* recv, size_t bytes_per_rank, void* stream);

/* ------------------------------------------------------------------------------------------
 * LLaMA decode driver: the per-step layer loop of LlamaDecoder::forward
 *   (src/turbomind/models/llama/LlamaDecoder.cc:158-242) with
 *   LlamaDecoderSelfAttentionLayer::forward (LlamaDecoderSelfAttentionLayer.cc:193-304),
 *   LlamaFfnLayer::forward (LlamaFfnLayer.cc:66-116), the embedding lookup, lm-head and greedy
 *   pick of LlamaV2 (LlamaV2.cc:184-201, 312-372), for int4 (W4A16) weights.
 * Dimensions are GLOBAL; with tensor_para_size > 1 every rank holds the slices of
 *   LlamaDecoderLayerWeight (LlamaDecoderLayerWeight.cc:30-79): qkv and w13 column-split
 *   (this rank's q heads | k heads | v heads; gate/up interleaved), wo and w2 row-split, norms
 *   and embeddings replicated, lm-head vocab-split.
 * All weight pointers are caller-owned device memory that must outlive the model.
 */
typedef struct tm_llama_config {
    int   head_num;
    int   kv_head_num;
    int   size_per_head; /* 128 */
    int   inter_size;
    int   num_layer;
    int   vocab_size;
    float norm_eps;
    float rope_theta;
    int   quant_policy; /* 4 = int8 KV cache, 0 = fp16 */
    int   group_size;   /* 128 */
    int   tensor_para_size;
    int   tensor_para_rank;
    int   max_batch_size;
    int   session_len;  /* slots per sequence in the KV cache (memory_max_len) */
} tm_llama_config;

/* One decoder layer: the fields of LlamaDecoderLayerWeight (LlamaDecoderLayerWeight.h:60-64) that
 * the int4 path uses.  qweight = runtime int4 layout, scales_zeros = half2 {64 + z, s}. */
typedef struct tm_llama_layer_weights {
    const void* self_attn_norm; /* half [hidden] */
    const void* ffn_norm;       /* half [hidden] */
    const void* qkv_qweight;
    const void* qkv_scales_zeros;
    const void* qkv_bias;       /* half [(H + 2 Hkv) * 128 / tp] or NULL */
    const void* o_qweight;
    const void* o_scales_zeros;
    const void* w13_qweight;
    const void* w13_scales_zeros;
    const void* w2_qweight;
    const void* w2_scales_zeros;
    float       past_kv_scale[4]; /* k_scale, k_zp, v_scale, v_zp (LlamaDecoderLayerWeight.cc:296-306) */
} tm_llama_layer_weights;

typedef struct tm_llama tm_llama;
TM_API int tm_llama_create(tm_llama** out, tm_handle* h, tm_comm* comm, const tm_llama_config* cfg);
TM_API int tm_llama_destroy(tm_llama* m);
TM_API int tm_llama_set_layer(tm_llama* m, int layer, const tm_llama_layer_weights* w);
/* tok_embeddings half [vocab, hidden]; output_norm half [hidden]; output_weight half
 * [vocab / tp (this rank's rows), hidden]. */
TM_API int tm_llama_set_globals(tm_llama* m, const void* tok_embeddings, const void* output_norm, const void* output_weight);
/* Loads every weight of this rank from a TurboMind workspace directory: the binary files that
 * LlamaWeight::loadModel (src/turbomind/models/llama/LlamaWeight.cc:86-106) and
 * LlamaDecoderLayerWeight::loadModel (LlamaDecoderLayerWeight.cc:261-307; int4 branch of loadWeights,
 * :206-220) read, i.e. what lmdeploy's deploy.py exports for W4A16: tok_embeddings.weight, norm.weight,
 * output.weight, layers.<l>.{attention_norm,ffn_norm}.weight, layers.<l>.{attention.w_qkv,attention.wo,
 * feed_forward.w13,feed_forward.w2}.<rank>.{qweight,scales_zeros}, optional ...w_qkv.<rank>.bias and
 * layers.<l>.past_kv_scale.<rank>.weight.  The model owns the device copies.  TM_ERR_IO when a file is
 * missing or its size does not match the configuration. */
TM_API int tm_llama_load_workspace(tm_llama* m, const char* dir);

/* ------------------------------------------------------------------------------------------
 * KV slab manager: sequence id -> cache slab with least-recently-used eviction.  Replaces LlamaCacheManager
 *   (src/turbomind/models/llama/LlamaCacheManager.h:13-100, LlamaCacheManager.cc:16-183): create / fetch /
 *   update / erase / contains with the same policy.  A slab holds keys then values of one sequence,
 *   2 x layer_num x head_num x max_seq_len x size_per_head x elem_bits / 8 bytes; slabs come from chunks of
 *   `chunk_size` slabs allocated on demand up to `max_entry_count` (the first chunk at creation).  fetch / create
 *   pin the sequence (timestamp = UINT64_MAX); update stamps it and makes it evictable; when no slab is free the
 *   sequence with the smallest stamp loses its slab and its cache_len becomes 0.
 *   Errors: unknown id -> TM_ERR_INVALID_ARG (the reference aborts); every slab pinned -> TM_ERR_WORKSPACE
 *   ("No enough cache entries."); allocation failure -> TM_ERR_CUDA.
 *   device >= 0: slabs in that GPU's memory, zero-filled with cudaMemsetAsync on `stream`;
 *   device == -1: slabs in host memory (for tests of the policy without a GPU).
 *   One manager is used by one host thread at a time, like a handle.
 */
typedef struct tm_cache_manager tm_cache_manager;
typedef struct tm_cache_sequence { /* LlamaCacheManager::Sequence, LlamaCacheManager.h:45-61 */
    uint64_t id;
    size_t   max_seq_len;
    size_t   cache_len;    /* 0 = cache miss                                              */
    size_t   token_count;  /* tokens stored by the last update (read them with tm_cache_tokens) */
    void*    k_cache;
    void*    v_cache;
    uint64_t timestamp;
} tm_cache_sequence;
TM_API int tm_cache_manager_create(tm_cache_manager** out, size_t layer_num, size_t head_num, size_t size_per_head,
                                   size_t max_seq_len, size_t elem_bits, size_t max_entry_count, size_t chunk_size, int device);
TM_API int tm_cache_manager_destroy(tm_cache_manager* m);
TM_API int tm_cache_create(tm_cache_manager* m, uint64_t id, void* stream, tm_cache_sequence* out);
TM_API int tm_cache_fetch(tm_cache_manager* m, uint64_t id, void* stream, tm_cache_sequence* out);
TM_API int tm_cache_update(tm_cache_manager* m, const tm_cache_sequence* seq, const int* token_ids, size_t token_count);
TM_API int tm_cache_tokens(const tm_cache_manager* m, uint64_t id, int* token_ids, size_t capacity, size_t* token_count);
TM_API int tm_cache_erase(tm_cache_manager* m, uint64_t id);
TM_API int tm_cache_contains(const tm_cache_manager* m, uint64_t id);

/* Prefill: runs the new tokens of `batch_size` sequences (packed, `token_num` in all) through every layer and
 * leaves their keys / values in the cache — what LlamaContextDecoder<T>::forward
 * (src/turbomind/models/llama/LlamaContextDecoder.cc:173-290) does around
 * LlamaContextAttentionLayer<T>::forward (LlamaContextAttentionLayer.cc:119-247), int4 weights.  The reference
 * discards the last layer's output (LlamaV2::contextDecode, LlamaV2.cc:204: the prompt's last token goes
 * through the decoder step instead); `hidden_out` (may be NULL) receives it after the final norm for tests.
 * All pointers are device memory of the caller; activations live in the model and grow to the largest call.
 * Not captured into a CUDA graph (shapes change per call); asynchronous on `stream`. */
typedef struct tm_llama_prefill_state {
    int        batch_size;
    int        token_num;        /* sum of the new-token counts                                   */
    int        max_q_len;        /* largest new-token count                                       */
    const int* input_ids;        /* [token_num], packed sequence after sequence                   */
    const int* cu_seqlens;       /* [batch + 1] prefix sums of the new-token counts               */
    const int* history_lengths;  /* [batch] tokens already cached per sequence                    */
    const int* context_lengths;  /* [batch] history + new                                         */
    void**     k_cache_ptrs;     /* as in tm_llama_decode_state                                   */
    void**     v_cache_ptrs;
    void*      hidden_out;       /* optional half [token_num, hidden]                             */
} tm_llama_prefill_state;
TM_API int tm_llama_prefill(tm_llama* m, const tm_llama_prefill_state* st, void* stream);

/* config.ini of a TurboMind workspace (`dir`/config.ini, section [llama]: written by
 * lmdeploy/serve/turbomind/deploy.py:209-239, read by LlamaTritonModel's constructor,
 * src/turbomind/triton_backend/llama/LlamaTritonModel.cc:118-143) -> tm_llama_config, with the defaults of
 * handleMissingParams (:59-98).  tensor_para_rank is set to 0: the caller fills in its own rank.  The keys the decode
 * driver has no use for land in `info` (may be NULL).  TM_ERR_IO: no file or no [llama] section; TM_ERR_INVALID_ARG: a
 * required key is missing or a value does not parse. */
typedef struct tm_llama_workspace_info {
    char model_name[64];
    char weight_type[16];           /* "int4" for the W4A16 workspaces this library loads */
    int  start_id, end_id;
    int  rotary_embedding_dim;
    int  max_context_token_num;     /* already multiplied by session_len when <= max_batch_size (:146-148) */
    int  step_length;
    int  cache_max_entry_count, cache_chunk_size;
    int  use_context_fmha;
    int  attn_bias;
    int  max_position_embeddings, use_dynamic_ntk, use_logn_attn;
} tm_llama_workspace_info;
TM_API int tm_llama_read_config(const char* dir, tm_llama_config* cfg, tm_llama_workspace_info* info);

/* Decode state, all device memory owned by the caller:
 *   k_cache_ptrs/v_cache_ptrs  [batch] base pointers; sequence b's cache is
 *                              [num_layer][kv_head_num / tp][session_len][128]
 *   sequence_lengths  int [batch]   tokens cached so far (updated by every step)
 *   start_step        int [batch]   sequence b is inactive (skipped like a finished one) while
 *                                   step < start_step[b]
 *   forced_ids        int [max_steps][batch] or NULL: >= 0 forces the step's input token
 *                                   (prompt tokens, teacher forcing), < 0 takes the previous pick
 *   output_ids        int [max_steps][batch]  the token picked at every step (step major, as
 *                                   src/turbomind/kernels/decoding_kernels.cu:69-106 stores ids)
 *   step              int [1]       current step counter (updated by every step)
 *   hidden_out        half [batch, hidden] or NULL: copy of the last normed hidden state
 *   logits_out        float [batch, vocab] or NULL: copy of the logits (after the all-gather)
 */
typedef struct tm_llama_decode_state {
    int         batch_size;
    int         max_steps;
    void**      k_cache_ptrs;
    void**      v_cache_ptrs;
    int*        sequence_lengths;
    const int*  start_step;
    const int*  forced_ids;
    int*        output_ids;
    int*        step;
    void*       hidden_out;
    float*      logits_out;
} tm_llama_decode_state;

/* Runs n_steps decode steps on `stream`.  With use_graph != 0 one step is captured into a CUDA
 * graph on first use (per state/batch size) and replayed; the stream must not be capturing. */
TM_API int tm_llama_decode(tm_llama* m, const tm_llama_decode_state* st, int n_steps, int use_graph, void* stream);
/* Kernels (own + library) launched by the most recent tm_llama_decode call. */
TM_API unsigned long long tm_llama_last_launches(const tm_llama* m);
/* tm_llama_decode and tm_llama_prefill only enqueue work.  What goes wrong on the device afterwards — a bounded
 * wait inside a kernel that gave up, a prefill whose history + new tokens exceed session_len (the surplus rows
 * are dropped, never written outside a cache head) — is recorded in the status word of the model's handle.
 * This call synchronises `stream`, reads and clears that word: TM_OK, or TM_ERR_DEVICE_TIMEOUT with the bits in
 * *word (tm_check_device_status on the model's handle).  Call it wherever the host synchronises anyway. */
TM_API int tm_llama_check_status(tm_llama* m, void* stream, unsigned* word);

/* ------------------------------------------------------------------------------------------
 * Persistent-batch scheduler over tm_cache_*, tm_llama_prefill, tm_llama_decode, tm_sample_topk / tm_sample_topp and
 * tm_ban_bad_words: the part of
 * LlamaBatch<T> (src/turbomind/models/llama/LlamaBatch.cc: initialize :562-763, contextDecode :765-877, generate
 * :471-559, finish / finishRequest :930-970, 1056-1118) that decides who runs.  Requests wait in a queue; every
 * tm_batch_step admits as many as there are free slots (their session's cached tokens come back from the cache
 * manager, everything without keys / values except the last token is context-decoded, at most
 * max_context_token_num new tokens per prefill call), runs ONE decoder step for all live sequences, draws one
 * token for each, and retires the sequences that drew `end_id` or reached their length: their tokens and cache
 * length go back to the cache manager (tm_cache_update), or the slab is released when end_flag was set.
 * Live sequences are kept dense in the batch; nothing is padded.  Not thread-safe: one host thread per scheduler.
 * Sampling fields of a request: top_k 0 and top_p 0 mean greedy, top_p 0 means 1, temperature / repetition_penalty 0
 * mean 1 (TopKSamplingLayer<T>::setup, src/turbomind/layers/sampling_layers/TopKSamplingLayer.cu:60-112); a request
 * with a top_p and no top_k is drawn over the whole vocabulary by tm_sample_topp, the others by tm_sample_topk, as the
 * reference's two layers share a batch (src/turbomind/layers/DynamicDecodeLayer.cc:305-312).
 * With tensor parallelism every rank runs its own scheduler on the same requests and seeds and draws the same tokens.
 */
typedef struct tm_batch tm_batch;
typedef struct tm_request {
    uint64_t           id;                 /* session id: the key of the cache manager                      */
    int                start_flag;         /* first request of the session: a new cache slab               */
    int                end_flag;           /* last request of the session: the slab is released at the end */
    const int*         input_ids;          /* host memory, copied by tm_batch_submit                        */
    int                input_length;
    int                request_output_len; /* new tokens wanted (cut so that the sequence fits session_len) */
    int                top_k;
    float              top_p;
    float              temperature;
    float              repetition_penalty;
    unsigned long long random_seed;
    int                ignore_eos;
    const int*         stop_ids;           /* host memory, copied: drawing one of these tokens ends the request too (the   */
    int                stop_count;         /* single-token stop words, the only kind LlamaBatch takes: LlamaBatch.cc:513-514) */
    const int*         bad_ids;            /* host memory, copied: tokens the request never draws (single-token bad words,    */
    int                bad_count;          /* at most 32; their logits are set to -inf before every draw)                     */
    int                rewind;             /* 1: a continued session first goes back to its first `step` tokens (the "step"   */
    int                step;               /* input of the reference's requests, LlamaBatch.cc:587-596); 0: history kept     */
} tm_request;
enum { TM_REQUEST_QUEUED = 0, TM_REQUEST_RUNNING = 1, TM_REQUEST_FINISHED = 2, TM_REQUEST_FAILED = 3 };
TM_API int tm_batch_create(tm_batch** out, tm_llama* model, tm_cache_manager* cache, int max_batch_size, int session_len,
                           int start_id, int end_id, int max_context_token_num);
TM_API int tm_batch_destroy(tm_batch* b);
TM_API int tm_batch_submit(tm_batch* b, const tm_request* r);
TM_API int tm_batch_step(tm_batch* b, void* stream, int use_graph);
/* tokens generated so far for the session's latest request (first min(capacity, *count) of them) and its state */
TM_API int tm_batch_output(const tm_batch* b, uint64_t id, int* tokens, size_t capacity, size_t* count, int* state);
/* forget the output of a finished / failed request (they are kept until then, or until the id is submitted again) */
TM_API int tm_batch_forget(tm_batch* b, uint64_t id);
TM_API int tm_batch_counts(const tm_batch* b, int* active, int* pending, unsigned long long* steps, unsigned long long* prefill_tokens);

#ifdef __cplusplus
}
#endif
#endif /* TM_B200_H_ */
