// Persistent-batch scheduler: requests come and go while the decode loop keeps running on whoever is active.
//
// The host-side counterpart of LlamaBatch<T> (src/turbomind/models/llama/LlamaBatch.cc): request intake with the
// sequence's cached history (initialize, :562-763), context decode of everything but the last prompt token
// (contextDecode, :765-877), one decoder step + sampling per call (generate, :471-559), finish bookkeeping
// (finish / finishRequest, :930-970, 1056-1118: a sequence that ends keeps its tokens and cache length in the cache
// manager unless the request was the session's last, in which case the slab is released).
// Re-designed around this library's decode state instead of the reference's padded step counter: every sequence
// carries its own length, so there is no padding count to keep; the active slots are kept dense (a slot that ends is
// filled with the last one), which is all "persistent batch" means at this level.
// One scheduler is driven by one host thread; every call works on the stream it is given.
#include "common.cuh"
#include "handle.h"
#include "llama.h"
#include "tm_b200.h"

#include <algorithm>
#include <cstring>
#include <deque>
#include <new>
#include <unordered_map>
#include <vector>

namespace tmb {
namespace {

constexpr int kMaxBadWords = 32;  // banned tokens per request (LlamaBatch.h:132 keeps 32 ints per list)

struct Slot {
    tm_request        req{};
    std::vector<int>  stop_ids;      // tokens that end the request besides the end id
    std::vector<int>  bad_ids;       // tokens the request must never draw
    tm_cache_sequence seq{};
    std::vector<int>  tokens;        // everything the sequence holds: cached history, prompt, generated
    int               prompt_end = 0;  // tokens.size() when generation started
    int               limit      = 0;  // generation stops when tokens.size() reaches this (LlamaBatch.cc:708-722)
};

struct Result {
    std::vector<int> generated;
    int              state = TM_REQUEST_QUEUED;
};

// hist[len[b]][b] = ids[b]: the token just drawn joins the history the repetition penalty reads
__global__ void append_history_kernel(int* hist, const int* ids, const int* lens_after, int B, int max_batch, int session_len)
{
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int row = lens_after[b];  // index of the new token = tokens before it
    if (row >= 0 && row < session_len) hist[(size_t)row * max_batch + b] = ids[b];
}

}  // namespace
}  // namespace tmb

struct tm_batch {
    tm_llama*         model   = nullptr;
    tm_cache_manager* cache   = nullptr;
    int               max_batch = 0, session_len = 0, vocab = 0, start_id = 0, end_id = 0, max_context_tokens = 0;
    int               device = 0;

    std::deque<tm_request>                       pending;
    std::deque<std::vector<int>>                 pending_ids;  // the prompt of pending[i]
    std::deque<std::vector<int>>                 pending_stop; // its stop tokens
    std::deque<std::vector<int>>                 pending_bad;  // its banned tokens
    std::vector<tmb::Slot>                       slots;        // [0, active) are live
    int                                          active = 0;
    std::unordered_map<uint64_t, tmb::Result>    results;

    // device
    void **d_k = nullptr, **d_v = nullptr;
    int *  d_len = nullptr, *d_forced = nullptr, *d_out = nullptr, *d_step = nullptr, *d_ids = nullptr, *d_hist = nullptr;
    int *  d_topk = nullptr, *d_hist_len = nullptr;
    float *d_logits = nullptr, *d_topp = nullptr, *d_temp = nullptr, *d_rep = nullptr;
    void*  d_rng = nullptr;
    int*                d_bad  = nullptr;  // [max batch][2][kMaxBadWords]: the live requests' banned tokens as word lists
    unsigned char*      d_skip = nullptr;  // [2][max batch]: rows the top-k draw leaves alone | rows the top-p draw leaves alone
    unsigned long long* d_seed = nullptr;
    // prefill staging (grown on demand)
    int*   d_pf_ids = nullptr;
    size_t pf_capacity = 0;
    int *  d_pf_cu = nullptr, *d_pf_hist = nullptr, *d_pf_ctx = nullptr;
    void **d_pf_k = nullptr, **d_pf_v = nullptr;
    // pinned host
    int* h_ids = nullptr;

    unsigned long long steps = 0, prefill_tokens = 0;
};

using namespace tmb;

namespace {

template<typename T>
bool dev_alloc(T** p, size_t count)
{
    return cudaMalloc((void**)p, count * sizeof(T)) == cudaSuccess;
}

void batch_free(tm_batch* b)
{
    void* ptrs[] = {b->d_k,    b->d_v,    b->d_len,  b->d_forced, b->d_out,    b->d_step,  b->d_ids,   b->d_hist, b->d_topk, b->d_hist_len,
                    b->d_logits, b->d_topp, b->d_temp, b->d_rep,    b->d_rng,    b->d_seed,  b->d_pf_ids, b->d_pf_cu, b->d_pf_hist, b->d_pf_ctx,
                    b->d_pf_k, b->d_pf_v, b->d_skip, b->d_bad};
    for (void* p : ptrs) {
        if (p) cudaFree(p);
    }
    if (b->h_ids) cudaFreeHost(b->h_ids);
    delete b;
}

}  // namespace

extern "C" int tm_batch_create(tm_batch** out, tm_llama* model, tm_cache_manager* cache, int max_batch_size, int session_len,
                               int start_id, int end_id, int max_context_token_num)
{
    if (!out || !model || !cache || max_batch_size <= 0 || session_len <= 1) return TM_ERR_INVALID_ARG;
    if (max_batch_size > model->cfg.max_batch_size || session_len > model->cfg.session_len) return TM_ERR_INVALID_ARG;
    *out        = nullptr;
    tm_batch* b = new (std::nothrow) tm_batch();
    if (!b) return TM_ERR_CUDA;
    b->model              = model;
    b->cache              = cache;
    b->max_batch          = max_batch_size;
    b->session_len        = session_len;
    b->vocab              = model->cfg.vocab_size;
    b->start_id           = start_id;
    b->end_id             = end_id;
    b->max_context_tokens = max_context_token_num > 0 ? max_context_token_num : session_len;
    b->device             = model->h->device;
    b->slots.resize(max_batch_size);
    const size_t B = (size_t)max_batch_size;
    bool ok = dev_alloc(&b->d_k, B) && dev_alloc(&b->d_v, B) && dev_alloc(&b->d_len, B) && dev_alloc(&b->d_forced, B)
              && dev_alloc(&b->d_out, B) && dev_alloc(&b->d_step, 1) && dev_alloc(&b->d_ids, B)
              && dev_alloc(&b->d_hist, B * session_len) && dev_alloc(&b->d_topk, B) && dev_alloc(&b->d_hist_len, B)
              && dev_alloc(&b->d_logits, B * b->vocab) && dev_alloc(&b->d_topp, B) && dev_alloc(&b->d_temp, B) && dev_alloc(&b->d_rep, B)
              && dev_alloc(&b->d_seed, B) && dev_alloc(&b->d_pf_cu, B + 1) && dev_alloc(&b->d_pf_hist, B) && dev_alloc(&b->d_pf_ctx, B)
              && dev_alloc(&b->d_pf_k, B) && dev_alloc(&b->d_pf_v, B) && dev_alloc(&b->d_skip, 2 * B) && dev_alloc(&b->d_bad, B * 2 * kMaxBadWords);
    ok = ok && cudaMalloc(&b->d_rng, B * tm_sampling_rng_state_bytes()) == cudaSuccess;
    ok = ok && cudaMallocHost((void**)&b->h_ids, B * sizeof(int)) == cudaSuccess;
    ok = ok && cudaMemset(b->d_hist, 0, B * session_len * sizeof(int)) == cudaSuccess;
    if (!ok) {
        batch_free(b);
        return TM_ERR_CUDA;
    }
    *out = b;
    return TM_OK;
}

extern "C" int tm_batch_destroy(tm_batch* b)
{
    if (!b) return TM_ERR_INVALID_ARG;
    batch_free(b);
    return TM_OK;
}

// The request is copied (the prompt too); it waits until a slot is free.
extern "C" int tm_batch_submit(tm_batch* b, const tm_request* r)
{
    if (!b || !r || r->input_length < 0 || (r->input_length > 0 && !r->input_ids) || r->request_output_len < 0) return TM_ERR_INVALID_ARG;
    if (r->top_k < 0 || r->top_k > 1024 || r->top_p < 0.f || r->top_p > 1.f) return TM_ERR_INVALID_ARG;
    if (r->stop_count < 0 || (r->stop_count > 0 && !r->stop_ids)) return TM_ERR_INVALID_ARG;
    if (r->bad_count < 0 || r->bad_count > tmb::kMaxBadWords || (r->bad_count > 0 && !r->bad_ids)) return TM_ERR_INVALID_ARG;
    for (int i = 0; i < r->input_length; ++i) {
        if (r->input_ids[i] < 0 || r->input_ids[i] >= b->vocab) return TM_ERR_INVALID_ARG;
    }
    auto it = b->results.find(r->id);
    if (it != b->results.end() && it->second.state != TM_REQUEST_FINISHED && it->second.state != TM_REQUEST_FAILED) {
        return TM_ERR_INVALID_ARG;  // one request per session at a time (LlamaBatch.cc:20-113 rejects duplicates)
    }
    if (!r->start_flag && !tm_cache_contains(b->cache, r->id)) return TM_ERR_INVALID_ARG;  // continuing an unknown session
    b->pending.push_back(*r);
    b->pending_ids.emplace_back(r->input_ids, r->input_ids + r->input_length);
    b->pending_stop.emplace_back(r->stop_ids, r->stop_ids + r->stop_count);
    b->pending_bad.emplace_back(r->bad_ids, r->bad_ids + r->bad_count);
    b->pending.back().input_ids = nullptr;
    b->pending.back().stop_ids  = nullptr;
    b->pending.back().bad_ids   = nullptr;
    b->results[r->id]           = Result{};
    return TM_OK;
}

extern "C" int tm_batch_output(const tm_batch* b, uint64_t id, int* tokens, size_t capacity, size_t* count, int* state)
{
    if (!b) return TM_ERR_INVALID_ARG;
    auto it = b->results.find(id);
    if (it == b->results.end()) return TM_ERR_INVALID_ARG;
    const auto& g = it->second.generated;
    if (count) *count = g.size();
    if (state) *state = it->second.state;
    if (tokens && !g.empty()) std::memcpy(tokens, g.data(), std::min(capacity, g.size()) * sizeof(int));
    return TM_OK;
}

// Drops what the scheduler remembers of a finished (or failed) request; its session's cache entry is not touched.
extern "C" int tm_batch_forget(tm_batch* b, uint64_t id)
{
    if (!b) return TM_ERR_INVALID_ARG;
    auto it = b->results.find(id);
    if (it == b->results.end()) return TM_ERR_INVALID_ARG;
    if (it->second.state != TM_REQUEST_FINISHED && it->second.state != TM_REQUEST_FAILED) return TM_ERR_INVALID_ARG;
    b->results.erase(it);
    return TM_OK;
}

extern "C" int tm_batch_counts(const tm_batch* b, int* active, int* pending, unsigned long long* steps, unsigned long long* prefill_tokens)
{
    if (!b) return TM_ERR_INVALID_ARG;
    if (active) *active = b->active;
    if (pending) *pending = (int)b->pending.size();
    if (steps) *steps = b->steps;
    if (prefill_tokens) *prefill_tokens = b->prefill_tokens;
    return TM_OK;
}

namespace {

// Context decode of the newly admitted sequences `group` (slot indices): every token that has no keys / values yet,
// except the last one, which goes through the decoder step (LlamaV2::contextDecode, LlamaV2.cc:204).
int prefill_group(tm_batch* b, const std::vector<int>& group, const std::vector<int>& cached, cudaStream_t s)
{
    std::vector<int>   ids, cu{0}, hist, ctx;
    std::vector<void*> kp, vp;
    int                max_q = 0;
    for (size_t g = 0; g < group.size(); ++g) {
        const Slot& sl = b->slots[group[g]];
        const int   n  = (int)sl.tokens.size() - 1 - cached[g];
        if (n <= 0) continue;
        ids.insert(ids.end(), sl.tokens.begin() + cached[g], sl.tokens.end() - 1);
        cu.push_back((int)ids.size());
        hist.push_back(cached[g]);
        ctx.push_back(cached[g] + n);
        kp.push_back(sl.seq.k_cache);
        vp.push_back(sl.seq.v_cache);
        max_q = std::max(max_q, n);
    }
    if (ids.empty()) return TM_OK;
    if (ids.size() > b->pf_capacity) {
        if (b->d_pf_ids) cudaFree(b->d_pf_ids);
        b->d_pf_ids    = nullptr;
        b->pf_capacity = 0;
        if (cudaMalloc((void**)&b->d_pf_ids, ids.size() * sizeof(int)) != cudaSuccess) return TM_ERR_CUDA;
        b->pf_capacity = ids.size();
    }
    const size_t n = hist.size();
    bool ok = cudaMemcpyAsync(b->d_pf_ids, ids.data(), ids.size() * sizeof(int), cudaMemcpyHostToDevice, s) == cudaSuccess
              && cudaMemcpyAsync(b->d_pf_cu, cu.data(), cu.size() * sizeof(int), cudaMemcpyHostToDevice, s) == cudaSuccess
              && cudaMemcpyAsync(b->d_pf_hist, hist.data(), n * sizeof(int), cudaMemcpyHostToDevice, s) == cudaSuccess
              && cudaMemcpyAsync(b->d_pf_ctx, ctx.data(), n * sizeof(int), cudaMemcpyHostToDevice, s) == cudaSuccess
              && cudaMemcpyAsync(b->d_pf_k, kp.data(), n * sizeof(void*), cudaMemcpyHostToDevice, s) == cudaSuccess
              && cudaMemcpyAsync(b->d_pf_v, vp.data(), n * sizeof(void*), cudaMemcpyHostToDevice, s) == cudaSuccess;
    if (!ok) return TM_ERR_CUDA;
    tm_llama_prefill_state st{};
    st.batch_size      = (int)n;
    st.token_num       = (int)ids.size();
    st.max_q_len       = max_q;
    st.input_ids       = b->d_pf_ids;
    st.cu_seqlens      = b->d_pf_cu;
    st.history_lengths = b->d_pf_hist;
    st.context_lengths = b->d_pf_ctx;
    st.k_cache_ptrs    = b->d_pf_k;
    st.v_cache_ptrs    = b->d_pf_v;
    const int rc       = tm_llama_prefill(b->model, &st, s);
    // the staging vectors above are pageable: their copies were staged before cudaMemcpyAsync returned
    if (rc == TM_OK) b->prefill_tokens += ids.size();
    return rc;
}

// The sequence in `slot` is done: its tokens and cache length go back to the cache manager, or the slab is released
// when this was the session's last request (finishRequest, LlamaBatch.cc:1056-1118).
void finish_slot(tm_batch* b, int slot, int state)
{
    Slot& sl = b->slots[slot];
    if (sl.req.end_flag || state == TM_REQUEST_FAILED) {
        tm_cache_erase(b->cache, sl.req.id);
    }
    else {
        // the token drawn last has no keys / values yet: it is fed again when the session continues
        sl.seq.cache_len = sl.tokens.size() - 1;
        tm_cache_update(b->cache, &sl.seq, sl.tokens.data(), sl.tokens.size());
    }
    b->results[sl.req.id].state = state;
}

// Fill the hole at `slot` with the last live slot (host record, history column, random state).
int compact(tm_batch* b, int slot, cudaStream_t s)
{
    const int last = b->active - 1;
    if (slot != last) {
        b->slots[slot] = std::move(b->slots[last]);
        const size_t pitch = (size_t)b->max_batch * sizeof(int);
        const size_t rng_b = tm_sampling_rng_state_bytes();
        if (cudaMemcpy2DAsync(b->d_hist + slot, pitch, b->d_hist + last, pitch, sizeof(int), b->session_len, cudaMemcpyDeviceToDevice, s)
                != cudaSuccess
            || cudaMemcpyAsync((char*)b->d_rng + slot * rng_b, (char*)b->d_rng + last * rng_b, rng_b, cudaMemcpyDeviceToDevice, s)
                   != cudaSuccess) {
            return TM_ERR_CUDA;
        }
    }
    b->slots[last] = Slot{};
    --b->active;
    return TM_OK;
}

}  // namespace

// One scheduling round: admit waiting requests into free slots (cache slab, history, context decode), one decoder
// step for every live sequence, one draw per sequence, then the bookkeeping of whoever finished.  Synchronises
// `stream` once (the host must see the drawn tokens, as LlamaBatch::finish does every step).
extern "C" int tm_batch_step(tm_batch* b, void* stream, int use_graph)
{
    if (!b) return TM_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int          rc;

    // ---- 1. intake (LlamaBatch::initialize)
    std::vector<int> fresh, fresh_cached;
    while (!b->pending.empty() && b->active < b->max_batch) {
        tm_request       r   = b->pending.front();
        std::vector<int> ids = std::move(b->pending_ids.front());
        Slot sl{};
        sl.stop_ids = std::move(b->pending_stop.front());
        sl.bad_ids  = std::move(b->pending_bad.front());
        b->pending.pop_front();
        b->pending_ids.pop_front();
        b->pending_stop.pop_front();
        b->pending_bad.pop_front();
        sl.req = r;
        rc     = r.start_flag ? tm_cache_create(b->cache, r.id, s, &sl.seq) : tm_cache_fetch(b->cache, r.id, s, &sl.seq);
        if (rc != TM_OK) {
            b->results[r.id].state = TM_REQUEST_FAILED;
            continue;
        }
        sl.tokens.resize(sl.seq.token_count);
        size_t got = 0;
        if (sl.seq.token_count) tm_cache_tokens(b->cache, r.id, sl.tokens.data(), sl.tokens.size(), &got);
        sl.tokens.resize(got);
        int cached = (int)std::min(sl.seq.cache_len, sl.tokens.size());  // a swapped-out slab comes back with 0
        if (r.rewind && !r.start_flag && r.step >= 0 && r.step <= (int)sl.tokens.size()) {
            // the session goes back to its first `step` tokens (LlamaBatch.cc:587-596; a step beyond the history is
            // ignored there with a warning, here silently); rows of the slab beyond them are overwritten as needed
            sl.tokens.resize(r.step);
            cached = std::min(cached, r.step);
        }
        sl.tokens.insert(sl.tokens.end(), ids.begin(), ids.end());
        if (sl.tokens.empty()) sl.tokens.push_back(b->start_id);  // LlamaBatch.cc:599-604
        const int context_len = (int)sl.tokens.size();
        if (context_len >= b->session_len) {
            // no room for even one new token: refuse (the reference truncates request_output_len to nothing and warns)
            tm_cache_erase(b->cache, r.id);
            b->results[r.id].state = TM_REQUEST_FAILED;
            continue;
        }
        sl.prompt_end = context_len;
        sl.limit      = std::min(context_len + r.request_output_len, b->session_len);
        const int slot = b->active++;
        const size_t pitch = (size_t)b->max_batch * sizeof(int);
        if (cudaMemcpy2DAsync(b->d_hist + slot, pitch, sl.tokens.data(), sizeof(int), sizeof(int), context_len, cudaMemcpyHostToDevice, s)
            != cudaSuccess) {
            return TM_ERR_CUDA;
        }
        rc = tm_sampling_rng_init((char*)b->d_rng + slot * tm_sampling_rng_state_bytes(), 1, nullptr, r.random_seed, s);
        if (rc != TM_OK) return rc;
        b->slots[slot]         = std::move(sl);
        b->results[r.id].state = TM_REQUEST_RUNNING;
        fresh.push_back(slot);
        fresh_cached.push_back(cached);
    }

    // ---- 2. context decode of the newcomers, at most max_context_tokens new tokens per call (contextDecode :765-877)
    {
        std::vector<int> group, group_cached;
        int              sum = 0;
        for (size_t i = 0; i <= fresh.size(); ++i) {
            const int n = i < fresh.size() ? std::max(0, (int)b->slots[fresh[i]].tokens.size() - 1 - fresh_cached[i]) : 0;
            if (i == fresh.size() || (!group.empty() && sum + n > b->max_context_tokens)) {
                if ((rc = prefill_group(b, group, group_cached, s)) != TM_OK) {
                    // the newcomers have no usable context: give their slots and slabs back before reporting
                    cudaStreamSynchronize(s);
                    std::sort(fresh.begin(), fresh.end());
                    for (int k = (int)fresh.size() - 1; k >= 0; --k) {
                        finish_slot(b, fresh[k], TM_REQUEST_FAILED);
                        compact(b, fresh[k], s);
                    }
                    return rc;
                }
                group.clear();
                group_cached.clear();
                sum = 0;
            }
            if (i < fresh.size()) {
                group.push_back(fresh[i]);
                group_cached.push_back(fresh_cached[i]);
                sum += n;
            }
        }
    }
    // a request that asked for no new tokens is done once its context is cached
    for (int slot = b->active - 1; slot >= 0; --slot) {
        if ((int)b->slots[slot].tokens.size() >= b->slots[slot].limit) {
            if (cudaStreamSynchronize(s) != cudaSuccess) return TM_ERR_CUDA;
            // nothing was drawn: every token but the last has keys / values
            finish_slot(b, slot, TM_REQUEST_FINISHED);
            if ((rc = compact(b, slot, s)) != TM_OK) return rc;
        }
    }
    const int B = b->active;
    if (B == 0) return TM_OK;

    // ---- 3. one decoder step + one draw (generate :471-559)
    std::vector<void*> kp(B), vp(B);
    std::vector<int>   len(B), last(B), hist_len(B), topk(B);
    std::vector<float> topp(B), temp(B), rep(B);
    std::vector<unsigned char> skip(2 * (size_t)b->max_batch, 0);
    int                longest = 0, n_topk = 0;
    bool               any_rep = false;
    for (int i = 0; i < B; ++i) {
        const Slot& sl = b->slots[i];
        kp[i] = sl.seq.k_cache, vp[i] = sl.seq.v_cache;
        len[i]      = (int)sl.tokens.size() - 1;  // tokens that have keys / values
        last[i]     = sl.tokens.back();
        hist_len[i] = (int)sl.tokens.size();
        longest     = std::max(longest, hist_len[i]);
        // The reference's two sampling layers share the batch (DynamicDecodeLayer.cc:305-312): a request with a top_k is
        // drawn by the top-k layer (top_p 0 there means 1: TopKSamplingLayer.cu:60-76), one with only a top_p by the
        // top-p layer (TopPSamplingLayer.cu:70-81), one with neither is greedy (k = 1).
        const bool only_p = sl.req.top_k == 0 && sl.req.top_p > 0.f;
        topk[i] = sl.req.top_k > 0 ? sl.req.top_k : 1;
        topp[i] = sl.req.top_p > 0.f ? sl.req.top_p : 1.f;
        skip[i]                = only_p ? 1 : 0;
        skip[b->max_batch + i] = only_p ? 0 : 1;
        n_topk += only_p ? 0 : 1;
        temp[i] = sl.req.temperature > 0.f ? sl.req.temperature : 1.f;
        rep[i]  = sl.req.repetition_penalty > 0.f ? sl.req.repetition_penalty : 1.f;
        any_rep = any_rep || rep[i] != 1.f;
    }
    auto up = [&](void* dst, const void* src, size_t bytes) { return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, s) == cudaSuccess; };
    if (!(up(b->d_k, kp.data(), B * sizeof(void*)) && up(b->d_v, vp.data(), B * sizeof(void*)) && up(b->d_len, len.data(), B * 4)
          && up(b->d_forced, last.data(), B * 4) && up(b->d_hist_len, hist_len.data(), B * 4) && up(b->d_topk, topk.data(), B * 4)
          && up(b->d_topp, topp.data(), B * 4) && up(b->d_temp, temp.data(), B * 4) && up(b->d_rep, rep.data(), B * 4)
          && up(b->d_skip, skip.data(), skip.size())
          && cudaMemsetAsync(b->d_step, 0, sizeof(int), s) == cudaSuccess)) {
        return TM_ERR_CUDA;
    }
    tm_llama_decode_state st{};
    st.batch_size       = B;
    st.max_steps        = 1;
    st.k_cache_ptrs     = b->d_k;
    st.v_cache_ptrs     = b->d_v;
    st.sequence_lengths = b->d_len;
    st.forced_ids       = b->d_forced;
    st.output_ids       = b->d_out;
    st.step             = b->d_step;
    st.logits_out       = b->d_logits;
    if ((rc = tm_llama_decode(b->model, &st, 1, use_graph, s)) != TM_OK) return rc;

    // bad_words_list of the requests (DynamicDecodeLayer.cc:214-236): single tokens, as the reference's scheduler takes
    // them, banned through the word-list kernel (an item of one token is banned whatever came before it)
    size_t n_bad = 0;
    for (int i = 0; i < B; ++i) n_bad = std::max(n_bad, b->slots[i].bad_ids.size());
    if (n_bad > 0) {
        std::vector<int> words((size_t)B * 2 * n_bad, -1);
        for (int i = 0; i < B; ++i) {
            const auto& bad = b->slots[i].bad_ids;
            for (size_t k = 0; k < n_bad; ++k) {
                words[((size_t)i * 2 + 0) * n_bad + k] = k < bad.size() ? bad[k] : 0;
                words[((size_t)i * 2 + 1) * n_bad + k] = k < bad.size() ? (int)k + 1 : -1;
            }
        }
        if (!up(b->d_bad, words.data(), words.size() * sizeof(int))) return TM_ERR_CUDA;
        if ((rc = tm_ban_bad_words(b->d_logits, b->vocab, b->vocab, B, nullptr, 0, b->d_bad, (int)n_bad, 0, 0, s)) != TM_OK) return rc;
    }

    tm_sampling_params sp{};
    sp.logits       = b->d_logits;
    sp.ld           = b->vocab;
    sp.vocab_size   = b->vocab;
    sp.batch_size   = B;
    sp.temperatures = b->d_temp;
    if (any_rep) {
        // history rows of sequence i: [0, hist_len[i]); the rows up to the longest history are padding for it
        sp.repetition_penalties = b->d_rep;
        sp.output_ids           = b->d_hist;
        sp.output_ids_stride    = b->max_batch;
        sp.step                 = longest;
        sp.input_lengths        = b->d_hist_len;
        sp.max_input_length     = longest;
    }
    sp.top_ks     = b->d_topk;
    sp.top_ps     = b->d_topp;
    sp.rng_states = b->d_rng;
    sp.ids        = b->d_ids;
    if (n_topk > 0) {
        sp.skip_decode = n_topk < B ? b->d_skip : nullptr;
        if ((rc = tm_sample_topk(b->model->h, &sp, s)) != TM_OK) return rc;
    }
    if (n_topk < B) {
        sp.skip_decode = n_topk > 0 ? b->d_skip + b->max_batch : nullptr;
        if ((rc = tm_sample_topp(b->model->h, &sp, s)) != TM_OK) return rc;
    }
    append_history_kernel<<<(B + 127) / 128, 128, 0, s>>>(b->d_hist, b->d_ids, b->d_hist_len, B, b->max_batch, b->session_len);
    if (cudaGetLastError() != cudaSuccess) return TM_ERR_CUDA;
    if (cudaMemcpyAsync(b->h_ids, b->d_ids, B * sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess
        || cudaStreamSynchronize(s) != cudaSuccess) {
        return TM_ERR_CUDA;
    }
    ++b->steps;

    // ---- 4. what the step produced (finish :930-970)
    for (int i = B - 1; i >= 0; --i) {
        Slot&     sl  = b->slots[i];
        const int tok = b->h_ids[i];
        sl.tokens.push_back(tok);
        b->results[sl.req.id].generated.push_back(tok);
        const bool stop = (tok == b->end_id && !sl.req.ignore_eos) || (int)sl.tokens.size() >= sl.limit
                          || std::find(sl.stop_ids.begin(), sl.stop_ids.end(), tok) != sl.stop_ids.end();
        if (stop) {
            finish_slot(b, i, TM_REQUEST_FINISHED);
            if ((rc = compact(b, i, s)) != TM_OK) return rc;
        }
    }
    return TM_OK;
}
