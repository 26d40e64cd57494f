"""CPU restatement of the reference's KV slab manager policy (LlamaCacheManager, lmdeploy v0.0.9:
src/turbomind/models/llama/LlamaCacheManager.cc:16-183), with slabs as small integers instead of memory.

Test infrastructure only: nothing under lmdeploy_b200/ imports this module.  The reference has no test or golden vector
for this class; this file follows the source line by line (linear scans, vector order, FT_CHECK as exceptions) and is
pinned against the reference class itself: LlamaCacheManager.cc is compiled unmodified into oracle/_ref/libtm_ref.so (a
cudaMalloc allocator stub behind it), tests/golden/make_ref_cache_manager_trace.py recorded its answers to seeded
operation streams on a B200 (tests/golden/ref_cache_manager_trace.npz, replayed on the CPU by tests/test_cache_manager.py),
and tests/test_gpu_cache_manager.py runs reference and library side by side."""
from __future__ import annotations

NEVER = 2 ** 64 - 1   # static_cast<uint64_t>(-1): "in use"


class NoFreeSlab(RuntimeError):
    """FT_CHECK_WITH_INFO(mem_ptr, "No enough cache entries.") (LlamaCacheManager.cc:54)"""


class UnknownSequence(KeyError):
    """FT_CHECK(0) in getEntryOrThrow (LlamaCacheManager.cc:85-94)"""


class Sequence:
    def __init__(self, id, slab):
        self.id, self.token_ids, self.cache_len, self.slab, self.timestamp = id, [], 0, slab, NEVER


class CacheManager:
    def __init__(self, max_entry_count: int, chunk_size: int):
        self.max_entry_count, self.chunk_size = max_entry_count, chunk_size
        self.free, self.entry_count, self.clock = [], 0, 0
        self.cache = []                        # std::vector<Sequence> device_cache_, insertion order
        self.zeroed = []                       # slabs zero-filled, in order (cudaMemsetAsync calls)
        self._allocate(True)                   # LlamaCacheManager.h:38

    def _allocate(self, preallocate):          # .cc:16-57
        slab = None
        if self.free:
            slab = self.free.pop(0)
        elif self.entry_count < self.max_entry_count:
            n = min(self.chunk_size, self.max_entry_count - self.entry_count)
            self.free += list(range(self.entry_count, self.entry_count + n))
            self.entry_count += n
            if not preallocate:
                slab = self.free.pop(0)
        else:
            slab = self._evict()
            if slab is None:
                raise NoFreeSlab()
        return slab

    def _evict(self):                          # .cc:145-166
        it = min(self.cache, key=lambda s: s.timestamp) if self.cache else None   # first minimum in vector order
        if it is None or it.timestamp == NEVER:
            return None
        slab, it.slab, it.cache_len, it.timestamp = it.slab, None, 0, NEVER
        return slab

    def _entry(self, id):
        for s in self.cache:
            if s.id == id:
                return s
        raise UnknownSequence(id)

    def create(self, id):                      # .cc:59-83
        if any(s.id == id for s in self.cache):
            self.erase(id)
        slab = self._allocate(False)
        self.zeroed.append(slab)
        self.cache.append(Sequence(id, slab))
        return self.cache[-1]

    def fetch(self, id):                       # .cc:96-112
        e = self._entry(id)
        if e.slab is None:
            assert e.cache_len == 0
            e.slab = self._allocate(False)
            self.zeroed.append(e.slab)
        e.timestamp = NEVER
        return e

    def update(self, id, slab, token_ids, cache_len):   # .cc:114-126
        e = self._entry(id)
        self.clock += 1
        e.timestamp, e.token_ids, e.cache_len = self.clock, list(token_ids), cache_len
        assert slab == e.slab

    def erase(self, id):                       # .cc:128-143
        e = self._entry(id)
        if e.slab is not None:
            self.free.append(e.slab)
        self.cache.remove(e)

    def contains(self, id):                    # .cc:168-173
        return any(s.id == id for s in self.cache)
