"""Self-consistency of the int4 layout oracle: the permute_u4 emulation, the closed form
of the runtime layout and the column permutations must agree with their logical meaning."""
import numpy as np
import pytest
import torch

from oracle import awq, s4_format as f


def _rand_q(k, n, seed):
    return np.random.default_rng(seed).integers(0, 16, size=(k, n), dtype=np.uint8)


@pytest.mark.parametrize("k,n", [(32, 32), (128, 64), (256, 96), (384, 160)])
def test_reformat_matches_closed_form(k, n):
    q = _rand_q(k, n, k + n)
    a = awq.pack_awq(q)                       # layout A [k, n/8]
    b = f.reformat_s4_k_m8(a, n, k)
    assert np.array_equal(f.unpack_runtime_layout(b, n, k), q)
    # the permutation is a bijection on nibbles
    kk, nn = np.meshgrid(np.arange(k), np.arange(n), indexing="ij")
    idx = f.runtime_layout_index(kk, nn, n).reshape(-1)
    assert np.array_equal(np.sort(idx), np.arange(k * n))


def test_dequantize_orders():
    w = np.array([0x76543210, 0xFEDCBA98], dtype=np.uint32)
    assert f.dequantize_s4(w).tolist() == [0, 4, 1, 5, 2, 6, 3, 7, 8, 12, 9, 13, 10, 14, 11, 15]
    assert f.dequantize_s4_offset_64(w).tolist() == [64 + v for v in f.dequantize_s4(w).tolist()]
    # AWQ packing followed by the dequant order gives back logical column order
    q = _rand_q(4, 16, 0)
    assert np.array_equal(f.dequantize_s4(awq.pack_awq(q)).reshape(4, 16), q.astype(np.float16))


@pytest.mark.parametrize("heads", [1, 3])
def test_transpose_qk(heads):
    k, d = 8, 128
    q = _rand_q(k, heads * d, 7)
    out = awq.unpack_awq(f.transpose_qk_s4_k_m8_hf(awq.pack_awq(q), heads * d, k, d))
    qh = q.reshape(k, heads, 2, d // 2)            # [k, head, half, j]
    want = qh.transpose(0, 1, 3, 2).reshape(k, heads * d)   # new[2j+h] = old[64h+j]
    assert np.array_equal(out, want)


def test_fuse_w1_w3():
    k, m = 8, 64
    w1, w3 = _rand_q(k, m, 1), _rand_q(k, m, 2)
    src = np.stack([awq.pack_awq(w1), awq.pack_awq(w3)])
    out = awq.unpack_awq(f.fuse_w1_w3_s4_k_m8(src, m, k))
    assert np.array_equal(out[:, 0::2], w1) and np.array_equal(out[:, 1::2], w3)


@pytest.mark.parametrize("n,k,seed", [(64, 256, 0), (96, 384, 1)])
def test_convert_and_dequant_equal_pseudo_quant_weight(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).half()
    qr = awq.quantize(w, 128)
    t = awq.to_awq_tensors(qr)
    a, q = f.convert_s4_k_m8(t.qweight, t.scales, t.qzeros, n, k, 128)
    assert np.array_equal(q[..., 0], (64 + qr.zeros.t().numpy()).astype(np.float16))
    assert np.array_equal(q[..., 1].view(np.uint16), t.scales.view(np.uint16))
    wd = f.dequantize_runtime_weight(a, q, n, k, 128)          # [k, n]
    want = awq.pseudo_quant_weight(qr, 128).t().numpy()
    assert np.array_equal(wd.view(np.uint16), want.view(np.uint16))
