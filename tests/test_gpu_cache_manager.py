"""GPU: slabs handed out by the KV slab manager (tm_cache_*, device mode) are zero-filled device memory with keys then
values, usable as the per-sequence cache pointers of the prefill writers."""
import ctypes as C

import numpy as np
import pytest
import torch

from lmdeploy_b200 import lib as l

pytestmark = pytest.mark.gpu


def test_slabs_serve_as_kv_cache_of_the_writers():
    from lmdeploy_b200 import turbomind as tm
    layers, H, D, S_max, B = 2, 4, 128, 32, 3
    m = C.c_void_p()
    l.check(l.lib.tm_cache_manager_create(C.byref(m), layers, H, D, S_max, 16, 4, 2, 0), "tm_cache_manager_create")
    seqs = []
    for i in range(B):
        s = l.TmCacheSequence()
        assert l.lib.tm_cache_create(m, 100 + i, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(s)) == l.TM_OK
        assert s.v_cache - s.k_cache == layers * H * S_max * D * 2
        seqs.append(s)
    kp = torch.tensor([s.k_cache for s in seqs], dtype=torch.int64, device="cuda")
    vp = torch.tensor([s.v_cache for s in seqs], dtype=torch.int64, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(1)
    k_src = torch.randn((B, H, 8, D), device="cuda", dtype=torch.float16, generator=g)
    v_src = torch.randn((B, H, 8, D), device="cuda", dtype=torch.float16, generator=g)
    lens = torch.tensor([8, 3, 0], dtype=torch.int32, device="cuda")
    hist = torch.tensor([0, 5, 0], dtype=torch.int32, device="cuda")
    off = 1 * H * S_max * D                                   # layer 1
    tm.invokeExtendKVCache(kp, vp, off, k_src, v_src, B, lens, 8, hist, S_max, D, H)
    kt = torch.full((B, H, S_max, D), 7.0, dtype=torch.float16, device="cuda")
    vt = torch.full_like(kt, 7.0)
    full = torch.full((B,), S_max, dtype=torch.int32, device="cuda")
    tm.invokeTransposeKVCache(kt, vt, kp, vp, off, B, full, S_max, S_max, D, H, 1)
    torch.cuda.synchronize()
    assert torch.equal(kt[0, :, :8], k_src[0]) and torch.equal(vt[1, :, 5:8], v_src[1, :, :3])
    assert float(kt[0, :, 8:].abs().max()) == 0 and float(vt[2].abs().max()) == 0 and float(kt[1, :, :5].abs().max()) == 0
    # an erased slab comes back zero-filled for the next sequence
    assert l.lib.tm_cache_erase(m, 100) == l.TM_OK
    s = l.TmCacheSequence()
    assert l.lib.tm_cache_create(m, 200, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(s)) == l.TM_OK
    assert s.k_cache not in [q.k_cache for q in seqs]          # the fourth slab (second chunk), never used before
    assert l.lib.tm_cache_create(m, 201, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(s)) == l.TM_OK
    assert s.k_cache == seqs[0].k_cache                        # then the slab that 100 gave back
    kp2 = torch.tensor([s.k_cache], dtype=torch.int64, device="cuda")
    vp2 = torch.tensor([s.v_cache], dtype=torch.int64, device="cuda")
    tm.invokeTransposeKVCache(kt[:1], vt[:1], kp2, vp2, off, 1, full[:1], S_max, S_max, D, H, 1)
    torch.cuda.synchronize()
    assert float(kt[0].abs().max()) == 0 and float(vt[0].abs().max()) == 0
    l.lib.tm_cache_manager_destroy(m)


@pytest.mark.parametrize("seed,max_entries,chunk", [(0, 4, 2), (1, 7, 3), (2, 1, 1), (3, 16, 16)])
def test_same_answers_as_the_reference_manager_side_by_side(seed, max_entries, chunk):
    """The reference's own LlamaCacheManager (LlamaCacheManager.cc compiled unmodified into oracle/_ref, a cudaMalloc
    allocator stub behind it) and tm_cache_* with device slabs, driven by the same 1500 seeded operations: same slab
    for every sequence at every step, same lengths, same pinned state, same set of known ids."""
    import ctypes as C
    import os
    from tests import cache_trace as ct
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libtm_ref.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libtm_ref.so not built (python oracle/build_ref.py needs the reference tree)")
    ref = C.CDLL(path)
    if not hasattr(ref, "ref_cache_manager_create"):
        pytest.skip("oracle/_ref/libtm_ref.so predates the cache manager entry layer")
    ops = ct.gen_ops(seed, max_entries)
    a, b = ct.RefAdapter(ref, max_entries, chunk), ct.LibAdapter(max_entries, chunk, torch.cuda.current_device())
    want, got = ct.run(a, ops, 2 * max_entries + 2), ct.run(b, ops, 2 * max_entries + 2)
    a.close()
    b.close()
    bad = np.nonzero((got != want).any(axis=1))[0]
    assert bad.size == 0, f"first difference at operation {bad[0]}: {ops[bad[0]]} got {got[bad[0]]} want {want[bad[0]]}"
    if os.path.exists(ct.GOLDEN):
        assert np.array_equal(np.load(ct.GOLDEN)[f"rows_{seed}"], want), "the committed golden trace is stale"
