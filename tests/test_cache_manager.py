"""CPU: the KV slab manager (tm_cache_*, host-memory mode) against the restated policy of the reference's
LlamaCacheManager (oracle/cache_manager.py): hand-written scenarios and a long random sequence of operations compared
step by step (which slab every sequence holds, cached lengths, stored tokens, error cases)."""
import ctypes as C

import numpy as np
import pytest

from lmdeploy_b200 import lib as l
from oracle import cache_manager as oc

SLAB = 2 * 2 * 2 * 16 * 8 * 2   # k + v: 2 layers x 2 heads x 16 positions x 8 dims x fp16


class Manager:
    def __init__(self, max_entries, chunk):
        self.m = C.c_void_p()
        l.check(l.lib.tm_cache_manager_create(C.byref(self.m), 2, 2, 8, 16, 16, max_entries, chunk, -1), "create")
        self.base = {}      # slab address -> small integer in order of first appearance per chunk

    def _seq(self):
        return l.TmCacheSequence()

    def create(self, id):
        s = self._seq()
        return l.lib.tm_cache_create(self.m, id, None, C.byref(s)), s

    def fetch(self, id):
        s = self._seq()
        return l.lib.tm_cache_fetch(self.m, id, None, C.byref(s)), s

    def update(self, s, tokens, cache_len):
        s.cache_len = cache_len
        arr = (C.c_int * len(tokens))(*tokens)
        return l.lib.tm_cache_update(self.m, C.byref(s), arr, len(tokens))

    def tokens(self, id):
        n = C.c_size_t(0)
        assert l.lib.tm_cache_tokens(self.m, id, None, 0, C.byref(n)) == l.TM_OK
        arr = (C.c_int * max(n.value, 1))()
        assert l.lib.tm_cache_tokens(self.m, id, arr, n.value, C.byref(n)) == l.TM_OK
        return list(arr[:n.value])

    def erase(self, id):
        return l.lib.tm_cache_erase(self.m, id)

    def contains(self, id):
        return bool(l.lib.tm_cache_contains(self.m, id))

    def close(self):
        l.lib.tm_cache_manager_destroy(self.m)


def test_slab_layout_zero_fill_and_reuse():
    m = Manager(3, 2)
    rc, a = m.create(10)
    assert rc == l.TM_OK and a.cache_len == 0 and a.max_seq_len == 16 and a.timestamp == oc.NEVER
    assert a.v_cache - a.k_cache == SLAB // 2
    buf = (C.c_ubyte * SLAB).from_address(a.k_cache)
    assert not any(buf)
    for i in range(SLAB):
        buf[i] = 0xAB
    rc, b = m.create(11)
    assert rc == l.TM_OK and b.k_cache - a.k_cache == SLAB           # second slab of the first chunk
    assert m.erase(10) == l.TM_OK and not m.contains(10) and m.contains(11)
    rc, c = m.create(12)                                             # the freed slab of 10 first, zero-filled again
    rc2, d = m.create(13)                                            # then a new chunk of one slab (3 - 2)
    assert rc == l.TM_OK and rc2 == l.TM_OK and c.k_cache == a.k_cache and d.k_cache not in (a.k_cache, b.k_cache)
    assert not any((C.c_ubyte * SLAB).from_address(c.k_cache))
    assert m.create(14)[0] == l.TM_ERR_WORKSPACE                     # three slabs, all in use
    m.close()


def test_lru_eviction_and_pinned_sequences():
    m = Manager(2, 2)
    _, a = m.create(1)
    _, b = m.create(2)
    rc, _ = m.create(3)
    assert rc == l.TM_ERR_WORKSPACE and not m.contains(3)            # both slabs in use: "No enough cache entries."
    assert m.update(a, [5, 6, 7], 3) == l.TM_OK                      # 1 becomes evictable (stamp 1)
    assert m.update(b, [8], 1) == l.TM_OK                            # stamp 2
    rc, c = m.create(3)
    assert rc == l.TM_OK and c.k_cache == a.k_cache                  # the least recently updated loses its slab
    assert m.contains(1) and m.tokens(1) == [5, 6, 7]                # ... but stays known, tokens kept
    rc, a2 = m.fetch(1)                                              # needs a slab again: evicts 2
    assert rc == l.TM_OK and a2.cache_len == 0 and a2.k_cache == b.k_cache and a2.token_count == 3
    rc, _ = m.fetch(2)
    assert rc == l.TM_ERR_WORKSPACE                                  # 1 and 3 are pinned
    assert m.fetch(99)[0] == l.TM_ERR_INVALID_ARG and m.erase(99) == l.TM_ERR_INVALID_ARG
    stale = l.TmCacheSequence()
    stale.id, stale.k_cache = 1, a.k_cache
    assert m.update(stale, [], 0) == l.TM_ERR_INVALID_ARG            # a slab pointer from before the eviction
    m.close()


@pytest.mark.parametrize("seed,max_entries,chunk", [(0, 4, 2), (1, 7, 3), (2, 1, 1), (3, 16, 16)])
def test_random_operations_follow_the_reference_policy(seed, max_entries, chunk):
    rng = np.random.default_rng(seed)
    m, o = Manager(max_entries, chunk), oc.CacheManager(max_entries, chunk)
    slab_of = {}            # address -> the oracle's slab number, learnt as slabs appear (addresses are per chunk)
    held = {}               # id -> last TmCacheSequence handed out

    def same_slab(addr, number):
        if addr is None or number is None:
            assert addr is None and number is None
            return
        assert slab_of.setdefault(addr, number) == number, "a sequence holds a different slab than the policy gives it"

    for step in range(3000):
        op = rng.choice(["create", "fetch", "update", "erase"], p=[0.3, 0.3, 0.3, 0.1])
        id = int(rng.integers(0, 2 * max_entries + 2))
        if op == "create":
            try:
                want = o.create(id)
            except oc.NoFreeSlab:
                want = None
            rc, s = m.create(id)
            if want is None:
                assert rc == l.TM_ERR_WORKSPACE
                held.pop(id, None)
            else:
                assert rc == l.TM_OK
                same_slab(s.k_cache, want.slab)
                held[id] = s
        elif op == "fetch":
            try:
                want = o.fetch(id)
            except oc.UnknownSequence:
                assert m.fetch(id)[0] == l.TM_ERR_INVALID_ARG
                continue
            except oc.NoFreeSlab:
                assert m.fetch(id)[0] == l.TM_ERR_WORKSPACE
                continue
            rc, s = m.fetch(id)
            assert rc == l.TM_OK and s.cache_len == want.cache_len and s.token_count == len(want.token_ids)
            same_slab(s.k_cache, want.slab)
            held[id] = s
        elif op == "update":
            if id not in held or not o.contains(id) or o._entry(id).slab is None or o._entry(id).timestamp != oc.NEVER:
                continue    # the engine only updates sequences it fetched and still holds
            toks = [int(t) for t in rng.integers(0, 1000, size=int(rng.integers(0, 6)))]
            o.update(id, o._entry(id).slab, toks, len(toks))
            assert m.update(held[id], toks, len(toks)) == l.TM_OK
        else:
            if o.contains(id):
                o.erase(id)
                assert m.erase(id) == l.TM_OK
                held.pop(id, None)
            else:
                assert m.erase(id) == l.TM_ERR_INVALID_ARG
        # the whole visible state after every operation
        for i in range(2 * max_entries + 2):
            assert m.contains(i) == o.contains(i)
            if o.contains(i):
                assert m.tokens(i) == o._entry(i).token_ids
    m.close()


@pytest.mark.parametrize("seed,max_entries,chunk", [(0, 4, 2), (1, 7, 3), (2, 1, 1), (3, 16, 16)])
def test_outcomes_recorded_from_the_reference_manager(seed, max_entries, chunk):
    """The golden file holds what the reference's own LlamaCacheManager (compiled unmodified, run on a B200 by
    tests/golden/make_ref_cache_manager_trace.py) answered to a seeded stream of 1500 operations: which slab every
    create / fetch handed out, cached lengths, token counts, pinned or not, which ids exist after every operation.
    Both the CPU restatement and the library (host slabs) must give the same answers."""
    import os
    from tests import cache_trace as ct
    assert os.path.exists(ct.GOLDEN), "tests/golden/ref_cache_manager_trace.npz is missing"
    want = np.load(ct.GOLDEN)[f"rows_{seed}"]
    ops = ct.gen_ops(seed, max_entries)
    for adapter in (ct.OracleAdapter(max_entries, chunk), ct.LibAdapter(max_entries, chunk, -1)):
        got = ct.run(adapter, ops, 2 * max_entries + 2)
        adapter.close()
        bad = np.nonzero((got != want).any(axis=1))[0]
        assert bad.size == 0, f"{type(adapter).__name__}: first difference at operation {bad[0]}: {ops[bad[0]]} got {got[bad[0]]} want {want[bad[0]]}"
