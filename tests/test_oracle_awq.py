"""The quantiser / packing oracle against vectors produced by the reference's own torch
code (tests/golden/make_awq_reference_vectors.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import awq

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "awq_reference_vectors.npz"))
CASES = ["a", "b", "c", "d"]


@pytest.mark.parametrize("c", CASES)
def test_qparams_and_unclamped_quant_match_reference(c):
    w = torch.from_numpy(G[f"{c}_w"])
    qr = awq.quantize(w, 128, clamp=False)
    assert np.array_equal(qr.scales.numpy().view(np.uint16), G[f"{c}_scales"].view(np.uint16))
    assert np.array_equal(qr.zeros.numpy(), G[f"{c}_zeros"].astype(np.int32))
    assert np.array_equal(qr.q.numpy(), G[f"{c}_real"])
    fake = awq.pseudo_quant_weight(qr, 128)
    assert np.array_equal(fake.numpy().view(np.uint16), G[f"{c}_fake"].view(np.uint16))
    assert qr.n_clamped == int(G[f"{c}_overflow"])


@pytest.mark.parametrize("c", [c for c in CASES if f"{c}_qweight" in G.files])
def test_packing_matches_from_linear(c):
    w = torch.from_numpy(G[f"{c}_w"])
    qr = awq.quantize(w, 128)
    assert qr.n_clamped == 0
    t = awq.to_awq_tensors(qr)
    assert np.array_equal(t.qweight, G[f"{c}_qweight"].view(np.uint32))
    assert np.array_equal(t.qzeros, G[f"{c}_qzeros"].view(np.uint32))
    assert np.array_equal(t.scales.view(np.uint16), G[f"{c}_qscales"].view(np.uint16))
    assert np.array_equal(awq.unpack_awq(t.qweight), qr.q.t().numpy().astype(np.uint8))


@pytest.mark.parametrize("c", CASES)
def test_clamp_only_touches_overflowing_elements(c):
    w = torch.from_numpy(G[f"{c}_w"])
    a, b = awq.quantize(w, 128, clamp=False), awq.quantize(w, 128, clamp=True)
    diff = (a.q != b.q)
    assert int(diff.sum()) <= a.n_clamped
    assert b.q.min() >= 0 and b.q.max() <= 15 and b.zeros.min() >= 0 and b.zeros.max() <= 15


@pytest.mark.parametrize("c", CASES)
def test_linear_matches_reference_torch_path(c):
    from oracle import gemm
    w = torch.from_numpy(G[f"{c}_w"])
    qr = awq.quantize(w, 128, clamp=False)
    fake = awq.pseudo_quant_weight(qr, 128)
    y = gemm.linear_f32acc(torch.from_numpy(G[f"{c}_x"]), fake.t().contiguous())
    assert np.array_equal(y.numpy().view(np.uint16), G[f"{c}_y"].view(np.uint16))
