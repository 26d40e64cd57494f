// KV slab manager: sequences -> fixed-size cache slabs with least-recently-used eviction, the policy of
// LlamaCacheManager (src/turbomind/models/llama/LlamaCacheManager.h:13-100, LlamaCacheManager.cc:16-183 of
// lmdeploy v0.0.9): slabs of 2 x layers x heads x max_seq_len x size_per_head elements (keys then values) are
// carved out of chunks of `chunk_size` slabs allocated on demand up to `max_entry_count`; a sequence that is
// being used carries the timestamp -1 and cannot be evicted; `update` stamps it with a running counter; when no
// slab is free the sequence with the smallest stamp loses its slab (it stays known, with cache_len 0) and
// `fetch` gives it a zeroed slab again.
//
// Host-side differences from the reference, none of them visible in results: sequences are found through a
// hash map instead of a linear scan (thousands of resident sequences fit 180 GB), errors come back as status
// codes instead of FT_CHECK aborts, and device == -1 keeps the slabs in host memory so that the policy can be
// tested without a GPU (the reference injects an IAllocator for the same purpose).
#include "tm_b200.h"

#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <deque>
#include <unordered_map>
#include <vector>

struct tm_cache_manager {
    size_t cache_bytes = 0;  // one of k / v
    size_t max_entries = 0, chunk_size = 0, max_seq_len = 0;
    int    device      = 0;

    struct Entry {
        uint64_t         id;
        std::vector<int> token_ids;
        size_t           cache_len = 0;
        void*            k_cache   = nullptr;
        uint64_t         timestamp = ~0ull;
        uint64_t         order;  // creation order: ties between equal stamps go to the oldest entry, as a scan would
    };
    std::unordered_map<uint64_t, Entry> entries;
    std::deque<void*>                   free_slabs;
    std::vector<void*>                  chunks;
    size_t                              entry_count = 0;
    uint64_t                            clock = 0, created = 0;

    void* raw_alloc(size_t bytes) const
    {
        if (device < 0) return std::malloc(bytes);
        void* p = nullptr;
        return cudaMalloc(&p, bytes) == cudaSuccess ? p : nullptr;
    }
    void raw_free(void* p) const
    {
        if (device < 0) {
            std::free(p);
        }
        else {
            cudaFree(p);
        }
    }
    int zero(void* p, cudaStream_t st) const
    {
        if (device < 0) {
            std::memset(p, 0, 2 * cache_bytes);
            return TM_OK;
        }
        return cudaMemsetAsync(p, 0, 2 * cache_bytes, st) == cudaSuccess ? TM_OK : TM_ERR_CUDA;
    }

    // LlamaCacheManager.cc:103-125
    void* evict()
    {
        Entry* best = nullptr;
        for (auto& kv : entries) {
            Entry& e = kv.second;
            if (!best || e.timestamp < best->timestamp || (e.timestamp == best->timestamp && e.order < best->order)) best = &e;
        }
        if (!best || best->timestamp == ~0ull || !best->k_cache) return nullptr;  // everything is in use
        void* p         = best->k_cache;
        best->k_cache   = nullptr;
        best->cache_len = 0;
        best->timestamp = ~0ull;
        return p;
    }

    // LlamaCacheManager.cc:16-57; *rc = TM_ERR_WORKSPACE when every slab is in use, TM_ERR_CUDA when memory ran out
    void* allocate(bool preallocate, int* rc)
    {
        *rc = TM_OK;
        if (!free_slabs.empty()) {
            if (preallocate) return nullptr;
            void* p = free_slabs.front();
            free_slabs.pop_front();
            return p;
        }
        if (entry_count < max_entries) {
            const size_t n     = chunk_size < max_entries - entry_count ? chunk_size : max_entries - entry_count;
            void*        chunk = raw_alloc(n * 2 * cache_bytes);
            if (!chunk) {
                *rc = TM_ERR_CUDA;
                return nullptr;
            }
            chunks.push_back(chunk);
            entry_count += n;
            for (size_t i = 0; i < n; ++i) free_slabs.push_back(static_cast<unsigned char*>(chunk) + i * 2 * cache_bytes);
            if (preallocate) return nullptr;
            void* p = free_slabs.front();
            free_slabs.pop_front();
            return p;
        }
        void* p = evict();
        if (!p) *rc = TM_ERR_WORKSPACE;  // "No enough cache entries."
        return p;
    }

    void fill(const Entry& e, tm_cache_sequence* out) const
    {
        out->id          = e.id;
        out->max_seq_len = max_seq_len;
        out->cache_len   = e.cache_len;
        out->token_count = e.token_ids.size();
        out->k_cache     = e.k_cache;
        out->v_cache     = e.k_cache ? static_cast<unsigned char*>(e.k_cache) + cache_bytes : nullptr;
        out->timestamp   = e.timestamp;
    }
};

extern "C" int tm_cache_manager_create(tm_cache_manager** out, size_t layer_num, size_t head_num, size_t size_per_head,
                                       size_t max_seq_len, size_t elem_bits, size_t max_entry_count, size_t chunk_size, int device)
{
    if (!out || !layer_num || !head_num || !size_per_head || !max_seq_len || !elem_bits || elem_bits % 8 || !max_entry_count
        || !chunk_size) {
        return TM_ERR_INVALID_ARG;
    }
    auto* m        = new tm_cache_manager;
    m->cache_bytes = layer_num * head_num * max_seq_len * size_per_head * elem_bits / 8;
    m->max_entries = max_entry_count, m->chunk_size = chunk_size, m->max_seq_len = max_seq_len, m->device = device;
    int prev = 0, rc = TM_OK;
    if (device >= 0) {
        cudaGetDevice(&prev);
        if (cudaSetDevice(device) != cudaSuccess) {
            delete m;
            return TM_ERR_CUDA;
        }
    }
    m->allocate(true, &rc);  // the first chunk up front, as the reference's constructor does (LlamaCacheManager.h:38)
    if (device >= 0) cudaSetDevice(prev);
    if (rc != TM_OK) {
        delete m;
        return rc;
    }
    *out = m;
    return TM_OK;
}

extern "C" int tm_cache_manager_destroy(tm_cache_manager* m)
{
    if (!m) return TM_OK;
    for (void* p : m->chunks) m->raw_free(p);
    delete m;
    return TM_OK;
}

// LlamaCacheManager.cc:59-83: an existing id is erased first; the new slab is zero-filled on `stream`
extern "C" int tm_cache_create(tm_cache_manager* m, uint64_t id, void* stream, tm_cache_sequence* out)
{
    if (!m || !out) return TM_ERR_INVALID_ARG;
    if (m->entries.count(id)) tm_cache_erase(m, id);
    int   rc = TM_OK;
    void* p  = m->allocate(false, &rc);
    if (!p) return rc;
    if ((rc = m->zero(p, (cudaStream_t)stream)) != TM_OK) {
        m->free_slabs.push_back(p);
        return rc;
    }
    tm_cache_manager::Entry e;
    e.id = id, e.k_cache = p, e.order = m->created++;
    m->fill(m->entries.emplace(id, std::move(e)).first->second, out);
    return TM_OK;
}

// LlamaCacheManager.cc:96-112: unknown id is an error; an evicted sequence gets a zeroed slab; the entry is pinned
extern "C" int tm_cache_fetch(tm_cache_manager* m, uint64_t id, void* stream, tm_cache_sequence* out)
{
    if (!m || !out) return TM_ERR_INVALID_ARG;
    auto it = m->entries.find(id);
    if (it == m->entries.end()) return TM_ERR_INVALID_ARG;
    tm_cache_manager::Entry& e = it->second;
    if (!e.k_cache) {
        int   rc = TM_OK;
        void* p  = m->allocate(false, &rc);
        if (!p) return rc;
        if ((rc = m->zero(p, (cudaStream_t)stream)) != TM_OK) {
            m->free_slabs.push_back(p);
            return rc;
        }
        e.k_cache = p;
    }
    e.timestamp = ~0ull;
    m->fill(e, out);
    return TM_OK;
}

// LlamaCacheManager.cc:114-126: stamps the entry (it becomes evictable) and stores its tokens and cached length
extern "C" int tm_cache_update(tm_cache_manager* m, const tm_cache_sequence* seq, const int* token_ids, size_t token_count)
{
    if (!m || !seq || (token_count && !token_ids)) return TM_ERR_INVALID_ARG;
    auto it = m->entries.find(seq->id);
    if (it == m->entries.end()) return TM_ERR_INVALID_ARG;
    tm_cache_manager::Entry& e = it->second;
    if (seq->k_cache != e.k_cache) return TM_ERR_INVALID_ARG;  // FT_CHECK(seq.k_cache == entry->k_cache ...)
    e.timestamp = ++m->clock;
    e.token_ids.assign(token_ids, token_ids + token_count);
    e.cache_len = seq->cache_len;
    return TM_OK;
}

extern "C" int tm_cache_tokens(const tm_cache_manager* m, uint64_t id, int* token_ids, size_t capacity, size_t* token_count)
{
    if (!m || !token_count) return TM_ERR_INVALID_ARG;
    auto it = m->entries.find(id);
    if (it == m->entries.end()) return TM_ERR_INVALID_ARG;
    *token_count = it->second.token_ids.size();
    if (token_ids) {
        if (capacity < *token_count) return TM_ERR_WORKSPACE;
        if (*token_count) std::memcpy(token_ids, it->second.token_ids.data(), *token_count * sizeof(int));  // an empty vector's data() may be null
    }
    return TM_OK;
}

// LlamaCacheManager.cc:128-143
extern "C" int tm_cache_erase(tm_cache_manager* m, uint64_t id)
{
    if (!m) return TM_ERR_INVALID_ARG;
    auto it = m->entries.find(id);
    if (it == m->entries.end()) return TM_ERR_INVALID_ARG;
    if (it->second.k_cache) m->free_slabs.push_back(it->second.k_cache);
    m->entries.erase(it);
    return TM_OK;
}

extern "C" int tm_cache_contains(const tm_cache_manager* m, uint64_t id)
{
    return m && m->entries.count(id) ? 1 : 0;
}
