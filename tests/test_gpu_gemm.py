"""GPU: W4A16 GEMM through the C ABI against the CPU oracle (fp32-accumulated torch linear on
the reference's pseudo-quant weight).  Tolerance: max-abs 2e-2, mean-rel 1e-3 on fp16 outputs."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import gemm as ogemm
from tests.helpers import assert_close, dev, make_linear

pytestmark = pytest.mark.gpu

_cache = {}


def _linear(n, k, seed):
    key = (n, k, seed)
    if key not in _cache:
        lin = make_linear(n, k, seed)
        lin["A_dev"] = dev(lin["A"], torch.int32)
        lin["Q_dev"] = dev(lin["Q"])
        _cache[key] = lin
    return _cache[key]


def _run(lin, x, n, k, fused=False, guard=True):
    from lmdeploy_b200 import turbomind as tm
    t = x.shape[0]
    n_out = n // 2 if fused else n
    buf = torch.full((t + 2, n_out), 777.0, dtype=torch.float16, device="cuda")   # guard rows around the output
    out = buf[1:t + 1]
    w = tm.LlamaDenseWeight(k, n, lin["A_dev"], tm.WeightType.kINT4, None, lin["Q_dev"], 128)
    op = tm.LlamaLinear()
    op.forward(out, dev(x), t, w, op.kFusedSiluFfn if fused else op.kGemm)
    op.gemm_s4_f16_.handle.check_device_status(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert (buf[0] == 777.0).all() and (buf[t + 1] == 777.0).all(), "wrote outside the output rows"
    return out.cpu().numpy()


def _x(t, k, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(t, k, generator=g).half().numpy()


SMALL = [(32, 128), (96, 256), (160, 384), (128, 1024), (544, 2048)]


@pytest.mark.parametrize("n,k", SMALL)
@pytest.mark.parametrize("t", [1, 2, 3, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64, 70])
def test_small_shapes_all_token_counts(n, k, t):
    lin = _linear(n, k, n + k)
    x = _x(t, k, t)
    y = _run(lin, x, n, k)
    assert_close(y, ogemm.gemm_s4_f16(x, lin["w_kn"]), f"gemm n={n} k={k} t={t}")


@pytest.mark.parametrize("n,k", [(64, 128), (192, 512), (22016, 4096), (7168, 2048)])   # the last: one strip per CTA slot, fused, at every token count
@pytest.mark.parametrize("t", [1, 2, 8, 16, 40])
def test_fused_silu(n, k, t):
    lin = _linear(n, k, 11)
    x = _x(t, k, 100 + t)
    y = _run(lin, x, n, k, fused=True)
    # silu(gate) * up reaches |y| > 16 on these inputs, where one fp16 ulp is 1.6e-2: allow 2 ulp
    # (2^-9 relative) on top of the absolute tolerance
    assert_close(y, ogemm.gemm_s4_f16(x, lin["w_kn"], fused_silu=True), f"silu n={n} k={k} t={t}", rel_slack=2.0 ** -9)
    # the epilogue alone, pinned on the kernel's own un-fused output: at most one fp16 ulp apart
    plain = _run(lin, x, n, k)
    want = ogemm.silu_mul_interleaved(torch.from_numpy(plain)).numpy().astype(np.float32)
    assert (np.abs(y.astype(np.float32) - want) <= 2.0 ** -10 * np.abs(want) + 1e-7).all()


LLAMA7B = [("qkv", 12288, 4096), ("o", 4096, 4096), ("gate_up", 22016, 4096), ("down", 4096, 11008)]


@pytest.mark.parametrize("name,n,k", LLAMA7B)
@pytest.mark.parametrize("t", [1, 2, 8, 16, 17, 64, 128])
def test_llama7b_projections(name, n, k, t):
    lin = _linear(n, k, 0)
    x = _x(t, k, t)
    y = _run(lin, x, n, k)
    assert_close(y, ogemm.gemm_s4_f16(x, lin["w_kn"]), f"{name} t={t}")


@pytest.mark.parametrize("name,n,k", LLAMA7B)
@pytest.mark.parametrize("t", [32, 512, 2048])
def test_llama7b_projections_benchmark_grid(name, n, k, t):
    """The remaining token counts of the benchmark's shape sweep ({1, 8, 32, 128, 512, 2048} x the four
    Llama-2-7B projections; 1, 8 and 128 are in test_llama7b_projections).  gate_up also runs with the
    fused SiLU epilogue (output [t, 11008]); 512 and 2048 tokens take several passes of 128 tokens."""
    lin = _linear(n, k, 0)
    x = _x(t, k, 1000 + t)
    w = torch.from_numpy(lin["w_kn"])
    want = (torch.from_numpy(x).float() @ w.float()).half()
    assert_close(_run(lin, x, n, k), want.numpy(), f"{name} t={t}")
    if name == "gate_up":
        y = _run(lin, x, n, k, fused=True)
        assert_close(y, ogemm.silu_mul_interleaved(want).numpy(), f"{name} silu t={t}", rel_slack=2.0 ** -9)


def test_baseline_config0_exact_case():
    """BASELINE config 0 as written: torch.manual_seed(0); X = randn(16, 4096).half(); W = (randn(11008, 4096)
    * 0.02).half(); group-128 asymmetric int4 (q and z clamped to 0..15); Y = X . dequant(W)^T, fp32
    accumulate, fp16 out.  Weight packing and layout conversion by the oracle, GEMM through tm_gemm_s4_f16."""
    from oracle import awq, s4_format as f
    torch.manual_seed(0)
    x = torch.randn(16, 4096).half()
    w = (torch.randn(11008, 4096) * 0.02).half()
    qr = awq.quantize(w, 128)
    t = awq.to_awq_tensors(qr)
    a, q = f.convert_s4_k_m8(t.qweight, t.scales, t.qzeros, 11008, 4096, 128)
    w_nk = awq.pseudo_quant_weight(qr, 128)
    lin = dict(A_dev=dev(a, torch.int32), Q_dev=dev(q))
    want = (x.float() @ w_nk.float().t()).half().numpy()
    assert_close(_run(lin, x.numpy(), 11008, 4096), want, "config 0")


@pytest.mark.parametrize("t", [5, 128])
@pytest.mark.parametrize("n,k", [(1280, 8192), (8192, 1024), (8192, 3584), (2560, 8192), (8192, 2048)])
def test_llama70b_tp8_and_tp4_shapes(n, k, t):
    """per-rank projection shapes of Llama-2-70B at tp=8 (qkv, o, w2) and tp=4 (qkv, o), both GEMM kernels"""
    lin = _linear(n, k, 1)
    x = _x(t, k, 5)
    y = _run(lin, x, n, k)
    assert_close(y, ogemm.gemm_s4_f16(x, lin["w_kn"]), f"70b/tp n={n} k={k} t={t}")


@pytest.mark.parametrize("t", [129, 200, 512])
def test_more_tokens_than_one_tile(t):
    n, k = 4096, 4096
    lin = _linear(n, k, 0)
    x = _x(t, k, t)
    assert_close(_run(lin, x, n, k), ogemm.gemm_s4_f16(x, lin["w_kn"]), f"o t={t}")


def test_deterministic_and_repeatable_tensor_core_path():
    n, k = 4096, 11008
    lin = _linear(n, k, 0)
    x = _x(64, k, 9)
    a = _run(lin, x, n, k)
    for _ in range(3):
        assert np.array_equal(a.view(np.uint16), _run(lin, x, n, k).view(np.uint16))


def test_deterministic_and_repeatable():
    n, k = 4096, 4096
    lin = _linear(n, k, 0)
    x = _x(4, k, 9)
    a = _run(lin, x, n, k)
    for _ in range(5):
        assert np.array_equal(a.view(np.uint16), _run(lin, x, n, k).view(np.uint16))


def test_linearity_and_zero_input():
    n, k = 4096, 11008
    lin = _linear(n, k, 0)
    x = _x(8, k, 3)
    y1 = _run(lin, x, n, k).astype(np.float32)
    y2 = _run(lin, (x.astype(np.float32) * 0.5).astype(np.float16), n, k).astype(np.float32)
    assert np.abs(y2 - 0.5 * y1).max() <= 2e-3          # exact scaling by 2 up to fp16 output rounding
    z = _run(lin, np.zeros_like(x), n, k)
    assert not z.any()


def test_caller_workspace_and_error_codes():
    from lmdeploy_b200 import lib as l
    n, k, t = 4096, 4096, 4
    lin = _linear(n, k, 0)
    x = _x(t, k, 4)
    h = l.default_handle(torch.cuda.current_device())
    need = l.lib.tm_gemm_s4_f16_workspace_bytes(n, t, k)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    out = torch.empty(t, n, dtype=torch.float16, device="cuda")
    xd = dev(x)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = (h.ptr, out.data_ptr(), lin["A_dev"].data_ptr(), xd.data_ptr(), lin["Q_dev"].data_ptr())
    for _ in range(2):       # twice: the tickets must have reset themselves
        assert l.lib.tm_gemm_s4_f16(*args, n, t, k, 128, 0, ws.data_ptr(), need, st) == l.TM_OK
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), ogemm.gemm_s4_f16(x, lin["w_kn"]), "caller workspace")
    assert l.lib.tm_gemm_s4_f16(*args, n, t, k, 128, 0, ws.data_ptr(), 16, st) == l.TM_ERR_WORKSPACE
    assert l.lib.tm_gemm_s4_f16(*args, n, t, k, 64, 0, None, 0, st) == l.TM_ERR_UNSUPPORTED
    assert l.lib.tm_gemm_s4_f16(*args, n, t, k + 1, 128, 0, None, 0, st) == l.TM_ERR_UNSUPPORTED
    assert l.lib.tm_gemm_s4_f16(*args, n + 8, t, k, 128, 0, None, 0, st) == l.TM_ERR_UNSUPPORTED
    assert l.lib.tm_gemm_s4_f16(*args, n, 0, k, 128, 0, None, 0, st) == l.TM_ERR_INVALID_ARG
    assert l.lib.tm_gemm_s4_f16(h.ptr, None, None, None, None, n, t, k, 128, 0, None, 0, st) == l.TM_ERR_INVALID_ARG
    assert l.lib.tm_gemm_s4_f16(*args, n, t, k, 128, 7, None, 0, st) == l.TM_ERR_UNSUPPORTED
