// Token sampling of the decode step: temperature, repetition penalty, minimum length, then either top-k sampling with
// a top-p cut inside the k candidates or top-p sampling over the whole vocabulary.  One kernel each, one CTA per
// sequence, the logits row held in shared memory.
//
// Restates, for fp32 logits, what the reference runs as five launches per step
//   batchApplyTemperaturePenalty   src/turbomind/kernels/sampling_penalty_kernels.cu:118-146   logit *= 1 / (T + 1e-6)
//   batchApplyRepetitionPenalty    sampling_penalty_kernels.cu:386-430   multiplicative, every distinct token once
//   batchApplyMinLengthPenalty     sampling_penalty_kernels.cu:486-500   end id masked while too short
//   topk_stage1 / topk_stage2_sampling   src/turbomind/kernels/sampling_topk_kernels.cu:125-312
// in the order of BaseSamplingLayer<T>::forward (src/turbomind/layers/sampling_layers/BaseSamplingLayer.cc:300-353).
// The draw is the reference's: u = curand_uniform(state of the sequence), target = u * top_p * sum_k exp(l_i - l_max),
// walk the candidates in descending order until the running sum reaches the target.  Equal logits are ordered by
// token id (the reference leaves that to the reduction tree).
#include "common.cuh"
#include "handle.h"
#include "tm_b200.h"

#include <algorithm>
#include <cfloat>
#include <curand_kernel.h>

namespace tmb {
namespace {

constexpr int kSampleThreads = 512;
constexpr int kSampleMaxK    = 1024;  // TopKSamplingLayer.cu clamps top_k to 1024 as well

struct Best {
    float v;
    int   i;
};

__device__ __forceinline__ Best better(Best a, Best b)
{
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// The penalised logits of sequence b -> s_row (and back to the logits, as the reference's penalty kernels rewrite them):
// temperature, repetition penalty, minimum length.  Every thread of the CTA calls this; ends with a barrier.
__device__ __forceinline__ void penalised_row(const tm_sampling_params& p, int b, float* s_row, unsigned* s_seen)
{
    const int   tid   = threadIdx.x;
    const int   V     = p.vocab_size;
    float*      row   = p.logits + (size_t)b * p.ld;
    const float inv_t = p.temperatures ? 1.0f / (p.temperatures[b] + 1e-6f) : 1.0f;
    const bool  scale = p.temperatures != nullptr;
    for (int v = tid; v < V; v += kSampleThreads) s_row[v] = scale ? row[v] * inv_t : row[v];
    const bool rep = p.repetition_penalties && p.output_ids && p.step > 0;
    if (rep) {
        for (int w = tid; w < (V + 31) / 32; w += kSampleThreads) s_seen[w] = 0u;
    }
    __syncthreads();
    if (rep) {
        const int in_len = p.input_lengths ? p.input_lengths[b] : p.max_input_length;
        for (int s = tid; s < p.step; s += kSampleThreads) {
            if (s >= in_len && s < p.max_input_length) continue;  // padding rows of the prompt block
            const int tok = p.output_ids[(size_t)s * (p.output_ids_stride > 0 ? p.output_ids_stride : p.batch_size) + b];
            if (tok >= 0 && tok < V) atomicOr(&s_seen[tok >> 5], 1u << (tok & 31));
        }
        __syncthreads();
        const float pen = p.repetition_penalties[b];
        for (int v = tid; v < V; v += kSampleThreads) {
            if (s_seen[v >> 5] >> (v & 31) & 1u) {
                const float l = s_row[v];
                s_row[v]      = l < 0.f ? l * pen : l / pen;
            }
        }
        __syncthreads();
    }
    if (tid == 0 && p.min_lengths && p.sequence_lengths && p.sequence_lengths[b] + 1 - p.max_input_length < p.min_lengths[b]) {
        const int e = p.end_ids[b];
        if (e >= 0 && e < V) s_row[e] = -FLT_MAX;
    }
    __syncthreads();
    if (scale || rep || p.min_lengths) {
        for (int v = tid; v < V; v += kSampleThreads) row[v] = s_row[v];
    }
}

__global__ void __launch_bounds__(kSampleThreads) sample_topk_kernel(tm_sampling_params p)
{
    extern __shared__ float s_dyn[];
    float*    s_row  = s_dyn;                                             // [vocab]
    unsigned* s_seen = reinterpret_cast<unsigned*>(s_row + p.vocab_size); // bitmap of tokens to penalise
    float*    s_cand = reinterpret_cast<float*>(s_seen + (p.vocab_size + 31) / 32);  // [k] exp(l_i - l_max)
    int*      s_cid  = reinterpret_cast<int*>(s_cand + kSampleMaxK);                 // [k] token ids
    __shared__ Best s_warp[kSampleThreads / 32];
    __shared__ Best s_pick;

    const int b   = blockIdx.x;
    const int tid = threadIdx.x;
    if (p.skip_decode && p.skip_decode[b]) return;
    const int V = p.vocab_size;
    if (p.finished && p.finished[b]) {
        // topk_stage2_sampling: a finished sequence keeps emitting its end id and nothing else changes
        if (tid == 0) p.ids[b] = p.end_ids[b];
        return;
    }
    penalised_row(p, b, s_row, s_seen);

    int k = p.top_ks ? p.top_ks[b] : p.max_top_k;
    k     = max(1, min(k, min(kSampleMaxK, V)));
    // every thread keeps the best of the elements it owns; an iteration takes the best of those, and only the owner
    // of the element taken looks through its elements again
    auto scan = [&]() {
        Best m{-FLT_MAX, 0x7fffffff};
        for (int v = tid; v < V; v += kSampleThreads) m = better(m, Best{s_row[v], v});
        return m;
    };
    Best mine = scan();
    for (int it = 0; it < k; ++it) {
        Best w = mine;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            Best other{__shfl_xor_sync(0xffffffffu, w.v, o), __shfl_xor_sync(0xffffffffu, w.i, o)};
            w = better(w, other);
        }
        if ((tid & 31) == 0) s_warp[tid >> 5] = w;
        __syncthreads();
        if (tid < 32) {
            Best t = tid < kSampleThreads / 32 ? s_warp[tid] : Best{-FLT_MAX, 0x7fffffff};
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                Best other{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
                t = better(t, other);
            }
            if (tid == 0) {
                s_pick     = t;
                s_cand[it] = t.v;
                s_cid[it]  = t.i;
            }
        }
        __syncthreads();
        const int taken = s_pick.i;
        if (taken < V && (taken % kSampleThreads) == tid) {
            s_row[taken] = -FLT_MAX;
            mine         = scan();
        }
    }
    if (tid == 0) {
        const float l_max = s_cand[0];
        float       sum   = 0.f;
        for (int i = 0; i < k; ++i) {
            const float e = __expf(s_cand[i] - l_max);
            s_cand[i]     = e;
            sum += e;
        }
        const float top_p = p.top_ps ? p.top_ps[b] : p.top_p;
        float       u;
        if (p.uniforms) {
            u = p.uniforms[b];
        }
        else {
            curandState_t* st = reinterpret_cast<curandState_t*>(p.rng_states) + b;
            u                 = curand_uniform(st);
        }
        float r    = u * top_p * sum;
        int   pick = s_cid[k - 1];
        for (int i = 0; i < k; ++i) {
            r -= s_cand[i];
            if (r <= 0.f || i == k - 1) {
                pick = s_cid[i];
                break;
            }
        }
        if (pick < 0 || pick >= V) pick = s_cid[0];
        p.ids[b] = pick;
        if (p.sequence_lengths_out && p.finished) {
            p.sequence_lengths_out[b] += 1;
            p.finished[b] = pick == p.end_ids[b] ? 1 : 0;
        }
    }
}

// ---- top-p sampling over the whole vocabulary -------------------------------------------------------------------
// The reference softmaxes the row, sorts all of it by probability (cub segmented radix sort, descending, equal values
// in token order) and walks the sorted row until the running sum reaches u * top_p; when the largest probability alone
// reaches top_p it takes that token without sorting (sampling_topp_kernels.cu:802-858, 878-1004, 1295-1346).  Here
// nothing is sorted: the probability at which the walk stops is found by a radix select over the bits of the
// probabilities, eight bits a pass, with the probability mass of every bucket in 2^-40 fixed point (integer sums:
// the same answer in any order of arrival).  What is left is which of the tokens with exactly that probability, in
// token order.
constexpr float kMassScale = 1099511627776.f;  // 2^40

__device__ __forceinline__ float block_reduce_max(float v, float* s_red)
{
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();  // s_red may still be read from an earlier reduction
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = s_red[0];
    for (int w = 1; w < kSampleThreads / 32; ++w) r = fmaxf(r, s_red[w]);
    return r;
}

__device__ __forceinline__ float block_reduce_sum(float v, float* s_red)
{
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
    for (int w = 0; w < kSampleThreads / 32; ++w) r += s_red[w];  // fixed order: every thread gets the same sum
    return r;
}

__global__ void __launch_bounds__(kSampleThreads) sample_topp_kernel(tm_sampling_params p)
{
    extern __shared__ float s_dyn[];
    float*              s_row  = s_dyn;                                              // [vocab] logits, then probabilities
    unsigned*           s_seen = reinterpret_cast<unsigned*>(s_row + p.vocab_size);  // bitmap of tokens to penalise
    unsigned long long* s_hist = reinterpret_cast<unsigned long long*>(
        (reinterpret_cast<uintptr_t>(s_seen + (p.vocab_size + 31) / 32) + 7) & ~uintptr_t(7));  // [256] mass per bucket
    __shared__ float              s_red[kSampleThreads / 32];
    __shared__ int                s_cnt[kSampleThreads / 32];
    __shared__ unsigned           s_prefix;   // bits of the stopping probability found so far
    __shared__ unsigned long long s_above;    // mass of everything above the buckets still in play
    __shared__ int                s_found;    // 0: the whole row is lighter than the target
    __shared__ float              s_u;

    const int b   = blockIdx.x;
    const int tid = threadIdx.x;
    if (p.skip_decode && p.skip_decode[b]) return;
    const int V = p.vocab_size;
    // topp_sampling draws before it looks at anything else, finished sequences included
    if (tid == 0) s_u = p.uniforms ? p.uniforms[b] : curand_uniform(reinterpret_cast<curandState_t*>(p.rng_states) + b);
    if (p.finished && p.finished[b]) {
        // addBiasSoftMax turns the row of a finished sequence into a one-hot of its end id: that id comes out, the
        // length stays and the sequence stays finished (topp_sampling's bookkeeping, sampling_topp_kernels.cu:996-1000)
        if (tid == 0) p.ids[b] = p.end_ids[b];
        return;
    }
    penalised_row(p, b, s_row, s_seen);

    // softmax as addBiasSoftMax: exp(l - max) / (sum + 1e-6)
    float m = -FLT_MAX;
    for (int v = tid; v < V; v += kSampleThreads) m = fmaxf(m, s_row[v]);
    m = block_reduce_max(m, s_red);
    float part = 0.f;
    for (int v = tid; v < V; v += kSampleThreads) {
        const float e = __expf(s_row[v] - m);
        s_row[v]      = e;
        part += e;
    }
    const float denom = block_reduce_sum(part, s_red) + 1e-6f;
    Best        top{-1.f, 0x7fffffff};
    for (int v = tid; v < V; v += kSampleThreads) {
        const float q = s_row[v] / denom;
        s_row[v]      = q;
        top           = better(top, Best{q, v});
    }
    // the most probable token (the lowest id among equals)
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        Best other{__shfl_xor_sync(0xffffffffu, top.v, o), __shfl_xor_sync(0xffffffffu, top.i, o)};
        top = better(top, other);
    }
    __shared__ Best s_top[kSampleThreads / 32];
    if ((tid & 31) == 0) s_top[tid >> 5] = top;
    __syncthreads();
    top = s_top[0];
    for (int w = 1; w < kSampleThreads / 32; ++w) top = better(top, s_top[w]);

    const float top_p = p.top_ps ? p.top_ps[b] : p.top_p;
    int         pick  = top.i;
    if (!(top.v >= top_p)) {
        // target of the walk, in fixed point (at least one unit: a bucket without mass never stops the walk)
        const float              r_f    = s_u * top_p;
        const unsigned long long target = max(1ull, (unsigned long long)(r_f * kMassScale));
        if (tid == 0) {
            s_prefix = 0u;
            s_above  = 0ull;
            s_found  = 1;
        }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < 256; i += kSampleThreads) s_hist[i] = 0ull;
            __syncthreads();
            const unsigned prefix = s_prefix;
            for (int v = tid; v < V; v += kSampleThreads) {
                const unsigned key = __float_as_uint(s_row[v]);
                if (pass == 0 || (key >> (shift + 8)) == prefix) {
                    const unsigned long long w = (unsigned long long)(s_row[v] * kMassScale);
                    if (w) atomicAdd(&s_hist[(key >> shift) & 255u], w);
                }
            }
            __syncthreads();
            if (tid == 0 && s_found) {
                unsigned long long acc = s_above;
                int                d   = 255;
                for (; d >= 0; --d) {
                    const unsigned long long h = s_hist[d];
                    if (h && acc + h >= target) break;
                    acc += h;
                }
                if (d < 0) {
                    s_found = 0;  // only in the first pass: the row sums to less than the target
                }
                else {
                    s_prefix = (prefix << 8) | (unsigned)d;
                    s_above  = acc;
                }
            }
            __syncthreads();
        }
        if (s_found) {
            // all tokens whose probability has exactly these bits weigh the same; the walk passes them in token order
            const unsigned           key  = s_prefix;
            const unsigned long long w    = (unsigned long long)(__uint_as_float(key) * kMassScale);
            const unsigned long long need = target > s_above ? target - s_above : 1ull;
            const long long          nth  = (long long)((need + w - 1) / w);  // w > 0: its bucket had mass
            const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
            const int v0 = tid * chunk, v1 = min(V, v0 + chunk);
            int       mine = 0;
            for (int v = v0; v < v1; ++v) mine += __float_as_uint(s_row[v]) == key;
            // exclusive prefix of the counts over the threads (thread order = token order)
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if ((tid & 31) >= o) incl += t;
            }
            if ((tid & 31) == 31) s_cnt[tid >> 5] = incl;
            __syncthreads();
            int before = incl - mine;
            for (int w2 = 0; w2 < (tid >> 5); ++w2) before += s_cnt[w2];
            int total = 0;
            for (int w2 = 0; w2 < kSampleThreads / 32; ++w2) total += s_cnt[w2];
            const long long want = nth < 1 ? 1 : (nth > total ? total : nth);  // 1-based rank among the equals
            __shared__ int s_pick_id;
            if (tid == 0) s_pick_id = top.i;
            __syncthreads();
            if (want > before && want <= before + mine) {
                int seen = before;
                for (int v = v0; v < v1; ++v) {
                    if (__float_as_uint(s_row[v]) == key && ++seen == want) {
                        s_pick_id = v;
                        break;
                    }
                }
            }
            __syncthreads();
            pick = s_pick_id;
        }
    }
    if (tid == 0) {
        p.ids[b] = pick;
        if (p.sequence_lengths_out && p.finished) {
            p.sequence_lengths_out[b] += 1;
            p.finished[b] = pick == p.end_ids[b] ? 1 : 0;
        }
    }
}

// invokeComputeToppDecay (sampling_topp_kernels.cu:1381-1426): top_p = token == reset id ? initial : max(top_p * decay, min)
__global__ void topp_decay_kernel(float* top_p, const float* initial, const int* ids, const float* decay, const float* top_p_min,
                                  const int* reset_ids, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    top_p[i] = ids[i] == reset_ids[i] ? initial[i] : fmaxf(top_p[i] * decay[i], top_p_min[i]);
}

__global__ void rng_init_kernel(curandState_t* states, int n, const unsigned long long* seeds, unsigned long long seed)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) curand_init(seeds ? seeds[i] : seed, 0, 0, &states[i]);  // sampling_topk_kernels.cu:32-58
}

}  // namespace

cudaError_t sampling_prepare(int max_smem)
{
    // the kernel also has a few static words: leave room for them
    cudaError_t e = cudaFuncSetAttribute(sample_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem - 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(sample_topp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem - 1024);
}

}  // namespace tmb

using namespace tmb;

extern "C" size_t tm_sampling_rng_state_bytes(void)
{
    return sizeof(curandState_t);
}

extern "C" int tm_sampling_rng_init(void* states, int batch_size, const unsigned long long* seeds, unsigned long long seed, void* stream)
{
    if (!states || batch_size <= 0) return TM_ERR_INVALID_ARG;
    rng_init_kernel<<<(batch_size + 255) / 256, 256, 0, (cudaStream_t)stream>>>((curandState_t*)states, batch_size, seeds, seed);
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}

extern "C" int tm_sample_topk(tm_handle* h, const tm_sampling_params* params, void* stream)
{
    if (!h || !params) return TM_ERR_INVALID_ARG;
    const tm_sampling_params& p = *params;
    if (!p.logits || !p.ids || p.batch_size <= 0 || p.vocab_size <= 0 || p.ld < p.vocab_size) return TM_ERR_INVALID_ARG;
    if (!p.uniforms && !p.rng_states) return TM_ERR_INVALID_ARG;
    if ((p.finished || p.min_lengths) && !p.end_ids) return TM_ERR_INVALID_ARG;
    if (!p.top_ks && (p.max_top_k < 1 || p.max_top_k > kSampleMaxK)) return TM_ERR_INVALID_ARG;
    if (!p.top_ps && !(p.top_p > 0.f && p.top_p <= 1.f)) return TM_ERR_INVALID_ARG;
    const size_t smem = (size_t)p.vocab_size * 4 + (size_t)((p.vocab_size + 31) / 32) * 4 + (size_t)kSampleMaxK * 8;
    if (smem > (size_t)h->max_smem - 1024) return TM_ERR_UNSUPPORTED;  // the row must fit shared memory (about 55 000 tokens)
    sample_topk_kernel<<<p.batch_size, kSampleThreads, smem, (cudaStream_t)stream>>>(p);
    ++h->launches;
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}

extern "C" int tm_sample_topp(tm_handle* h, const tm_sampling_params* params, void* stream)
{
    if (!h || !params) return TM_ERR_INVALID_ARG;
    const tm_sampling_params& p = *params;
    if (!p.logits || !p.ids || p.batch_size <= 0 || p.vocab_size <= 0 || p.ld < p.vocab_size) return TM_ERR_INVALID_ARG;
    if (!p.uniforms && !p.rng_states) return TM_ERR_INVALID_ARG;
    if ((p.finished || p.min_lengths) && !p.end_ids) return TM_ERR_INVALID_ARG;
    if (!p.top_ps && !(p.top_p > 0.f && p.top_p <= 1.f)) return TM_ERR_INVALID_ARG;
    const size_t smem = (size_t)p.vocab_size * 4 + (size_t)((p.vocab_size + 31) / 32) * 4 + 8 + 256 * 8;
    if (smem > (size_t)h->max_smem - 1024) return TM_ERR_UNSUPPORTED;
    sample_topp_kernel<<<p.batch_size, kSampleThreads, smem, (cudaStream_t)stream>>>(p);
    ++h->launches;
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}

extern "C" int tm_top_p_decay(float* runtime_top_p, const float* initial_top_p, const int* output_ids, const float* top_p_decay,
                              const float* top_p_min, const int* top_p_reset_ids, int batch_size, void* stream)
{
    if (!runtime_top_p || !initial_top_p || !output_ids || !top_p_decay || !top_p_min || !top_p_reset_ids || batch_size <= 0) {
        return TM_ERR_INVALID_ARG;
    }
    topp_decay_kernel<<<(batch_size + 255) / 256, 256, 0, (cudaStream_t)stream>>>(runtime_top_p, initial_top_p, output_ids, top_p_decay,
                                                                                   top_p_min, top_p_reset_ids, batch_size);
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}

// ---- word lists and stopping (beam width 1): ban_bad_words (src/turbomind/kernels/ban_bad_words.cu:22-84),
// ---- stop_words_criterion and length_criterion (src/turbomind/kernels/stop_criteria_kernels.cu:25-132), as
// ---- DynamicDecodeLayer<T>::forward drives them (src/turbomind/layers/DynamicDecodeLayer.cc:214-236, 303-337).
// A word list is the reference's tensor [2][len]: row 0 the tokens of all items back to back, row 1 the exclusive
// end offset of every item (-1 pads the row).  History: ids[s * stride + b] for steps s < step (+ the token of `step`
// itself for the stop check).
namespace tmb {
namespace {

__global__ void ban_bad_words_kernel(float* logits, int ld, int vocab, const int* ids, int stride, const int* words, int len,
                                     int share, int step)
{
    const int id = blockIdx.x * blockDim.x + threadIdx.x;
    const int b  = blockIdx.y;
    const int* w   = share ? words : words + (size_t)b * 2 * len;
    const int* off = w + len;
    if (id >= len || off[id] < 0) return;
    const int end = off[id], start = id > 0 ? off[id - 1] : 0, size = end - start;
    bool ban = size == 1;  // a single token is banned whatever came before
    if (size > 1 && step >= size - 1) {
        ban = true;  // the item's first size - 1 tokens must be the last ones generated
        for (int k = size - 2; k >= 0; --k) {
            if (ids[(size_t)(step - (size - 1) + k) * stride + b] != w[start + k]) {
                ban = false;
                break;
            }
        }
    }
    if (ban) {
        const int t = w[end - 1];
        if (0 < t && t < vocab) logits[(size_t)b * ld + t] = -INFINITY;
    }
}

__global__ void stop_words_kernel(const int* ids, int stride, const int* words, int len, unsigned char* finished, int step)
{
    const int id = blockIdx.x * blockDim.x + threadIdx.x;
    const int b  = blockIdx.y;
    const int* w   = words + (size_t)b * 2 * len;
    const int* off = w + len;
    if (id >= len || off[id] < 0) return;
    const int end = off[id], start = id > 0 ? off[id - 1] : 0, size = end - start;
    if (step + 1 < size) return;  // not enough tokens yet
    for (int k = size - 1; k >= 0; --k) {
        if (ids[(size_t)(step - (size - 1) + k) * stride + b] != w[start + k]) return;
    }
    finished[b] = 1;
}

__global__ void length_criterion_kernel(unsigned char* finished, const unsigned* limit, int batch, int step, int* finished_count)
{
    __shared__ int s_count;
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    int mine = 0;
    for (int b = threadIdx.x; b < batch; b += blockDim.x) {
        if ((unsigned)step >= limit[b]) finished[b] = 1;
        mine += finished[b] ? 1 : 0;
    }
    if (mine) atomicAdd(&s_count, mine);
    __syncthreads();
    if (threadIdx.x == 0 && finished_count) *finished_count = s_count;
}

}  // namespace
}  // namespace tmb

extern "C" int tm_ban_bad_words(float* logits, int ld, int vocab_size, int batch_size, const int* output_ids, int output_ids_stride,
                                const int* bad_words, int bad_words_len, int share_words, int step, void* stream)
{
    if (!logits || !bad_words || batch_size <= 0 || vocab_size <= 0 || ld < vocab_size || bad_words_len < 0 || step < 0) return TM_ERR_INVALID_ARG;
    if (bad_words_len == 0) return TM_OK;
    if (!output_ids && step > 0) return TM_ERR_INVALID_ARG;
    const int threads = std::min(256, (bad_words_len + 31) / 32 * 32);
    const dim3 grid((bad_words_len + threads - 1) / threads, batch_size);
    ban_bad_words_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(logits, ld, vocab_size, output_ids,
                                                                     output_ids_stride > 0 ? output_ids_stride : batch_size, bad_words,
                                                                     bad_words_len, share_words, step);
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}

extern "C" int tm_stop_words_criterion(const int* output_ids, int output_ids_stride, const int* stop_words, int stop_words_len,
                                       unsigned char* finished, int batch_size, int step, void* stream)
{
    if (!output_ids || !stop_words || !finished || batch_size <= 0 || stop_words_len < 0 || step < 0) return TM_ERR_INVALID_ARG;
    if (stop_words_len == 0) return TM_OK;
    const int threads = std::min(256, (stop_words_len + 31) / 32 * 32);
    const dim3 grid((stop_words_len + threads - 1) / threads, batch_size);
    stop_words_kernel<<<grid, threads, 0, (cudaStream_t)stream>>>(output_ids, output_ids_stride > 0 ? output_ids_stride : batch_size,
                                                                  stop_words, stop_words_len, finished, step);
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}

extern "C" int tm_length_criterion(unsigned char* finished, const unsigned* sequence_limit_length, int batch_size, int step,
                                   int* finished_count, void* stream)
{
    if (!finished || !sequence_limit_length || batch_size <= 0 || step < 0) return TM_ERR_INVALID_ARG;
    length_criterion_kernel<<<1, std::min(512, (batch_size + 31) / 32 * 32), 0, (cudaStream_t)stream>>>(finished, sequence_limit_length,
                                                                                                       batch_size, step, finished_count);
    return cudaGetLastError() == cudaSuccess ? TM_OK : TM_ERR_CUDA;
}
