"""GPU: slabs handed out by the KV slab manager (tm_cache_*, device mode) are zero-filled device memory with keys then
values, usable as the per-sequence cache pointers of the prefill writers."""
import ctypes as C

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
