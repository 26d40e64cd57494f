"""Shared by the KV slab manager tests: one seeded stream of create / fetch / update / erase operations, and adapters
that apply it to (a) the reference's own LlamaCacheManager built into oracle/_ref/libtm_ref.so (GPU only: it zero-fills
slabs with cudaMemsetAsync), (b) this library's tm_cache_* (device or host slabs), (c) the CPU restatement in
oracle/cache_manager.py.  An outcome row is (rc, slab, cache_len, token_count, timestamp_is_never, contains bitmask):
rc 0 ok / 1 unknown id / 2 no free slab; slab = number of the slab in order of first appearance (-1: none)."""
import ctypes as C
import os

import numpy as np

NEVER = 2 ** 64 - 1
OK, UNKNOWN, NO_SLAB = 0, 1, 2
GEOMETRY = (2, 2, 8, 16, 16)     # layers, heads, size_per_head, max_seq_len, elem_bits


def gen_ops(seed, max_entries, n=1500):
    """-> list of (op, id, tokens): op 0 create, 1 fetch, 2 update (of the sequence last handed out for id), 3 erase."""
    rng = np.random.default_rng(seed)
    ops = []
    for _ in range(n):
        op = int(rng.choice(4, p=[0.3, 0.3, 0.3, 0.1]))
        id = int(rng.integers(0, 2 * max_entries + 2))
        toks = [int(t) for t in rng.integers(0, 1000, size=int(rng.integers(0, 6)))] if op == 2 else []
        ops.append((op, id, toks))
    return ops


class _Slabs:
    """pointer -> small number in order of first appearance"""

    def __init__(self):
        self.n = {}

    def __call__(self, ptr):
        if not ptr:
            return -1
        return self.n.setdefault(int(ptr), len(self.n))


def run(adapter, ops, n_ids):
    """Applies `ops`; an update is issued only for a sequence the caller still holds pinned with a slab (what the
    engine does; the reference aborts otherwise).  Returns the outcome rows [n, 6] (int64)."""
    held = {}
    rows = []
    for op, id, toks in ops:
        row = [OK, -1, 0, 0, 0]
        if op in (0, 1):
            rc, seq = adapter.get(op, id)
            row[0] = rc
            if rc == OK:
                row[1:5] = [seq["slab"], seq["cache_len"], seq["token_count"], int(seq["timestamp"] == NEVER)]
                held[id] = seq
            elif op == 0:
                held.pop(id, None)
        elif op == 2:
            seq = held.get(id)
            if seq is None or not adapter.contains(id) or not adapter.updatable(id, seq):
                row[0] = -1          # skipped
            else:
                row[0] = adapter.update(seq, toks)
                seq["timestamp"] = 0     # no longer pinned: not updatable again until fetched
        else:
            row[0] = adapter.erase(id)
            if row[0] == OK:
                held.pop(id, None)
        mask = 0
        for i in range(n_ids):
            mask |= int(adapter.contains(i)) << i
        rows.append(row + [mask])
    return np.asarray(rows, np.int64)


class RefAdapter:
    """the reference's LlamaCacheManager through oracle/_ref/libtm_ref.so (needs a GPU)"""

    def __init__(self, lib, max_entries, chunk):
        u64, sz, vp = C.c_ulonglong, C.c_size_t, C.c_void_p
        lib.ref_cache_manager_create.restype = vp
        lib.ref_cache_manager_create.argtypes = [sz] * 7
        lib.ref_cache_manager_destroy.argtypes = [vp]
        lib.ref_cache_get.argtypes = [vp, C.c_int, u64, C.POINTER(u64), C.POINTER(C.c_int), sz]
        lib.ref_cache_update.argtypes = [vp, C.POINTER(u64), C.POINTER(C.c_int), sz]
        lib.ref_cache_erase.argtypes = [vp, u64]
        lib.ref_cache_contains.argtypes = [vp, u64]
        self.lib, self.slabs = lib, _Slabs()
        self.m = lib.ref_cache_manager_create(*GEOMETRY, max_entries, chunk)
        assert self.m

    def get(self, op, id):
        out, toks = (C.c_ulonglong * 7)(), (C.c_int * 64)()
        rc = self.lib.ref_cache_get(self.m, op, id, out, toks, 64)
        if rc != 0:
            # the reference throws for both causes; which one follows from whether the id is known
            return (NO_SLAB if (op == 0 or self.contains(id)) else UNKNOWN), None
        return OK, dict(raw=out, slab=self.slabs(out[4]), cache_len=int(out[2]), token_count=int(out[3]), timestamp=int(out[6]))

    def updatable(self, id, seq):
        return seq["timestamp"] == NEVER and seq["slab"] >= 0

    def update(self, seq, toks):
        seq["raw"][2] = len(toks)
        arr = (C.c_int * max(len(toks), 1))(*toks)
        return OK if self.lib.ref_cache_update(self.m, seq["raw"], arr, len(toks)) == 0 else UNKNOWN

    def erase(self, id):
        if not self.contains(id):
            return UNKNOWN           # the reference aborts on an unknown id: not exercised
        return OK if self.lib.ref_cache_erase(self.m, id) == 0 else UNKNOWN

    def contains(self, id):
        return bool(self.lib.ref_cache_contains(self.m, id))

    def close(self):
        self.lib.ref_cache_manager_destroy(self.m)


class LibAdapter:
    """tm_cache_* of this library; device = -1 keeps the slabs in host memory"""

    def __init__(self, max_entries, chunk, device=-1):
        from lmdeploy_b200 import lib as l
        self.l, self.slabs = l, _Slabs()
        self.m = C.c_void_p()
        l.check(l.lib.tm_cache_manager_create(C.byref(self.m), *GEOMETRY, max_entries, chunk, device), "tm_cache_manager_create")

    def _rc(self, rc):
        return {self.l.TM_OK: OK, self.l.TM_ERR_INVALID_ARG: UNKNOWN, self.l.TM_ERR_WORKSPACE: NO_SLAB}[rc]

    def get(self, op, id):
        s = self.l.TmCacheSequence()
        rc = (self.l.lib.tm_cache_create if op == 0 else self.l.lib.tm_cache_fetch)(self.m, id, None, C.byref(s))
        if rc != self.l.TM_OK:
            return self._rc(rc), None
        return OK, dict(raw=s, slab=self.slabs(s.k_cache), cache_len=int(s.cache_len), token_count=int(s.token_count),
                        timestamp=int(s.timestamp))

    def updatable(self, id, seq):
        return seq["timestamp"] == NEVER and seq["slab"] >= 0

    def update(self, seq, toks):
        seq["raw"].cache_len = len(toks)
        arr = (C.c_int * max(len(toks), 1))(*toks)
        return self._rc(self.l.lib.tm_cache_update(self.m, C.byref(seq["raw"]), arr, len(toks)))

    def erase(self, id):
        return self._rc(self.l.lib.tm_cache_erase(self.m, id))

    def contains(self, id):
        return bool(self.l.lib.tm_cache_contains(self.m, id))

    def close(self):
        self.l.lib.tm_cache_manager_destroy(self.m)


class OracleAdapter:
    """oracle/cache_manager.py"""

    def __init__(self, max_entries, chunk):
        from oracle import cache_manager as oc
        self.oc, self.o = oc, oc.CacheManager(max_entries, chunk)

    def get(self, op, id):
        try:
            e = self.o.create(id) if op == 0 else self.o.fetch(id)
        except self.oc.NoFreeSlab:
            return NO_SLAB, None
        except self.oc.UnknownSequence:
            return UNKNOWN, None
        return OK, dict(slab=e.slab, cache_len=e.cache_len, token_count=len(e.token_ids), timestamp=e.timestamp)

    def updatable(self, id, seq):
        return seq["timestamp"] == NEVER and seq["slab"] is not None and seq["slab"] >= 0

    def update(self, seq, toks):
        e = next(s for s in self.o.cache if s.slab == seq["slab"])
        self.o.update(e.id, seq["slab"], toks, len(toks))
        return OK

    def erase(self, id):
        if not self.o.contains(id):
            return UNKNOWN
        self.o.erase(id)
        return OK

    def contains(self, id):
        return self.o.contains(id)

    def close(self):
        pass


CASES = [(0, 4, 2), (1, 7, 3), (2, 1, 1), (3, 16, 16)]      # (seed, max_entry_count, chunk_size)
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_cache_manager_trace.npz")
