"""GPU: int4 layout converters through the C ABI, bit exact against the numpy oracle."""
import numpy as np
import pytest
import torch

from oracle import awq, s4_format as f
from tests.helpers import dev

pytestmark = pytest.mark.gpu


def _rand_words(shape, seed):
    return np.random.default_rng(seed).integers(0, 2 ** 32, size=shape, dtype=np.uint64).astype(np.uint32)


@pytest.mark.parametrize("n,k", [(32, 32), (64, 128), (96, 256), (160, 384), (4096, 512)])
def test_convert_s4_k_m8_bit_exact(n, k):
    from lmdeploy_b200 import turbomind as tm
    a_src = _rand_words((k, n // 8), 1)
    qz = _rand_words((k // 128 if k >= 128 else 1, n // 8), 2)
    g = 128 if k >= 128 else k
    scales = np.random.default_rng(3).standard_normal((k // g, n)).astype(np.float16)
    A_dst = torch.full((k, n // 8), -1, dtype=torch.int32, device="cuda")     # poison: every word must be overwritten
    Q_dst = torch.full((k // g, n, 2), float("nan"), dtype=torch.float16, device="cuda")
    ws = torch.empty(k // g * n, dtype=torch.float16, device="cuda")
    tm.convert_s4_k_m8(A_dst, Q_dst, ws, dev(a_src, torch.int32), dev(scales), dev(qz, torch.int32), n, k, g)
    a_want, q_want = f.convert_s4_k_m8(a_src, scales, qz, n, k, g)
    assert np.array_equal(A_dst.cpu().numpy().view(np.uint32), a_want)
    assert np.array_equal(Q_dst.cpu().numpy().view(np.uint16), q_want.view(np.uint16))
    assert np.array_equal(ws.cpu().numpy().view(np.uint16), f.dequantize_s4_offset_64(qz).view(np.uint16))


@pytest.mark.parametrize("heads,k", [(1, 8), (3, 40), (32, 64)])
def test_transpose_qk(heads, k):
    from lmdeploy_b200 import turbomind as tm
    m = heads * 128
    src = _rand_words((k, m // 8), 4)
    dst = torch.full((k, m // 8), -1, dtype=torch.int32, device="cuda")
    tm.transpose_qk_s4_k_m8(dev(src, torch.int32), dst, m, k, 128)
    assert np.array_equal(dst.cpu().numpy().view(np.uint32), f.transpose_qk_s4_k_m8_hf(src, m, k, 128))


@pytest.mark.parametrize("m,k", [(64, 8), (352, 24), (11008, 16)])
def test_fuse_w1_w3(m, k):
    from lmdeploy_b200 import turbomind as tm
    src = _rand_words((2, k, m // 8), 5)
    dst = torch.full((k, m // 4), -1, dtype=torch.int32, device="cuda")
    tm.fuse_w1_w3_s4_k_m8(dev(src, torch.int32), dst, m, k)
    assert np.array_equal(dst.cpu().numpy().view(np.uint32), f.fuse_w1_w3_s4_k_m8(src, m, k))


def test_dequantize_s4_and_empty():
    from lmdeploy_b200 import turbomind as tm
    src = _rand_words((1000,), 6)
    dst = torch.empty(8000, dtype=torch.float16, device="cuda")
    tm.dequantize_s4(dev(src, torch.int32), dst)
    assert np.array_equal(dst.cpu().numpy().view(np.uint16), f.dequantize_s4(src).view(np.uint16))
    with pytest.raises(ValueError):
        tm.dequantize_s4(dev(src, torch.int32), torch.empty(8, dtype=torch.float16, device="cuda"))
    tm.dequantize_s4(torch.empty(0, dtype=torch.int32, device="cuda"), torch.empty(0, dtype=torch.float16, device="cuda"))


def test_format_error_codes():
    from lmdeploy_b200 import lib as l
    a = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = a.data_ptr()
    assert l.lib.tm_reformat_s4_k_m8(p, p, 32, 32, None) == l.TM_ERR_INVALID_ARG      # aliasing
    assert l.lib.tm_reformat_s4_k_m8(p, None, 32, 32, None) == l.TM_ERR_INVALID_ARG
    assert l.lib.tm_reformat_s4_k_m8(p + 4 * 32, p, 33, 32, None) == l.TM_ERR_UNSUPPORTED
