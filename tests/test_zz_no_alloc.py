"""GPU: the allocation-free GEMM entry point (``tm_gemm_s4_f16_noalloc``).

It exists for hosts that may not call the CUDA allocator (memory owned by an embedding server,
everything already given to a KV-cache pool, loops that cannot afford cudaMalloc's device-wide
sync): its split-K scratch is a fixed 8 MB array inside the library.  The test calls it through the
C ABI twice in a row — the shared array keeps the first call's contents, so the second call proves
that nothing stale leaks — and compares with the handle-based entry point on the same inputs.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import gemm as ogemm
from tests.helpers import assert_close, dev, make_linear

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,k,t,fused", [(4096, 4096, 4, False), (22016, 4096, 16, True), (160, 384, 1, False)])
def test_noalloc_matches_handle_entry_point_twice(n, k, t, fused):
    from lmdeploy_b200 import lib as l
    lin = make_linear(n, k, 3)
    A, Q = dev(lin["A"], torch.int32), dev(lin["Q"])
    g = torch.Generator().manual_seed(t)
    xs = [torch.randn(t, k, generator=g).half() for _ in range(2)]
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    n_out = n // 2 if fused else n
    h = l.default_handle(torch.cuda.current_device())
    for x in xs:                                   # two calls in a row, different activations
        xd = x.cuda()
        ref = torch.empty(t, n_out, dtype=torch.float16, device="cuda")
        out = torch.full((t, n_out), 123.0, dtype=torch.float16, device="cuda")
        assert l.lib.tm_gemm_s4_f16(h.ptr, ref.data_ptr(), A.data_ptr(), xd.data_ptr(), Q.data_ptr(), n, t, k, 128,
                                    int(fused), None, 0, st) == l.TM_OK
        assert l.lib.tm_gemm_s4_f16_noalloc(out.data_ptr(), A.data_ptr(), xd.data_ptr(), Q.data_ptr(), n, t, k, 128,
                                            int(fused), st) == l.TM_OK
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), ref.cpu().numpy(), "noalloc vs handle entry", rel_slack=2.0 ** -9 if fused else 0.0)
        assert_close(out.cpu().numpy(), ogemm.gemm_s4_f16(x.numpy(), lin["w_kn"], fused_silu=fused), "noalloc vs oracle",
                     rel_slack=2.0 ** -9 if fused else 0.0)


def test_noalloc_largest_llama_shape_fits_up_to_eight_tokens():
    """The un-sharded Llama-2-70B gate_up projection (m = 57344, k = 8192) is the largest shape of the two models:
    its partial tiles fit the built-in 8 MB up to 8 tokens; at 9..16 tokens the plan needs 8.5 MB and the entry
    point says so instead of overrunning the array."""
    from lmdeploy_b200 import lib as l
    n, k = 57344, 8192
    g = torch.Generator(device="cuda").manual_seed(5)
    A = torch.randint(-2 ** 31, 2 ** 31 - 1, (k, n // 8), dtype=torch.int32, device="cuda", generator=g)   # any nibbles are a weight
    z = torch.randint(64, 80, (k // 128, n, 1), device="cuda", generator=g).half()
    s = (torch.rand(k // 128, n, 1, device="cuda", generator=g) * 0.01 + 0.002).half()
    Q = torch.cat([z, s], dim=-1).contiguous()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    h = l.default_handle(torch.cuda.current_device())
    for t in (1, 8):
        x = torch.randn(t, k, device="cuda", generator=g).half()
        ref = torch.empty(t, n // 2, dtype=torch.float16, device="cuda")
        cols = torch.empty(t, n // 2, dtype=torch.float16, device="cuda")
        out = torch.full((t, n // 2), 123.0, dtype=torch.float16, device="cuda")
        # the handle entry picks the column-owner kernel for this shape; the allocation-free entry always runs the
        # split-K kernel: bit-identical with the handle entry told to do the same, within the tolerance otherwise
        assert l.lib.tm_gemm_s4_f16(h.ptr, cols.data_ptr(), A.data_ptr(), x.data_ptr(), Q.data_ptr(), n, t, k, 128, 1, None, 0, st) == l.TM_OK
        h.set_option("gemv_cols", 0)
        try:
            assert l.lib.tm_gemm_s4_f16(h.ptr, ref.data_ptr(), A.data_ptr(), x.data_ptr(), Q.data_ptr(), n, t, k, 128, 1, None, 0, st) == l.TM_OK
        finally:
            h.set_option("gemv_cols", 1)
        assert l.lib.tm_gemm_s4_f16_noalloc(out.data_ptr(), A.data_ptr(), x.data_ptr(), Q.data_ptr(), n, t, k, 128, 1, st) == l.TM_OK
        torch.cuda.synchronize()
        assert torch.equal(out, ref), "same kernel, same plan: bit-identical"
        assert_close(cols.cpu().numpy(), ref.cpu().numpy(), f"column-owner kernel vs split-K kernel, {t} tokens", rel_slack=2.0 ** -9)
    x = torch.randn(16, k, device="cuda", generator=g).half()
    out = torch.empty(16, n // 2, dtype=torch.float16, device="cuda")
    assert l.lib.tm_gemm_s4_f16_noalloc(out.data_ptr(), A.data_ptr(), x.data_ptr(), Q.data_ptr(), n, 16, k, 128, 1, st) == l.TM_ERR_WORKSPACE


def test_noalloc_rejects_what_does_not_fit():
    from lmdeploy_b200 import lib as l
    buf = torch.zeros(1 << 20, dtype=torch.float16, device="cuda")
    p = buf.data_ptr()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert l.lib.tm_gemm_s4_f16_noalloc(p, p, p, p, 4096, 17, 4096, 128, 0, st) == l.TM_ERR_WORKSPACE     # > 16 tokens
    assert l.lib.tm_gemm_s4_f16_noalloc(p, p, p, p, 1 << 22, 16, 128, 128, 0, st) == l.TM_ERR_WORKSPACE   # partials > 8 MB
    assert l.lib.tm_gemm_s4_f16_noalloc(p, p, p, p, 4096, 1, 4096, 64, 0, st) == l.TM_ERR_UNSUPPORTED
    assert l.lib.tm_gemm_s4_f16_noalloc(None, p, p, p, 4096, 1, 4096, 128, 0, st) == l.TM_ERR_INVALID_ARG
