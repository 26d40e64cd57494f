"""Shared test helpers: seeded AWQ linears, tolerance checks (oracle side = CPU)."""
import numpy as np
import torch

from oracle import awq, s4_format as f

MAX_ABS = 2e-2     # tolerance of the hot path against the fp32-accumulated torch oracle (fp16 outputs)
MEAN_REL = 1e-3


def make_linear(n, k, seed, std=0.02):
    """-> dict with AWQ tensors (numpy), runtime-layout tensors (numpy) and the fp16 weight [K, N]."""
    t, w_nk, n_clamped = awq.make_awq_linear(n, k, seed, 128, std)
    a, q = f.convert_s4_k_m8(t.qweight, t.scales, t.qzeros, n, k, 128)
    return dict(awq=t, A=a, Q=q, w_kn=w_nk.t().contiguous().numpy(), n_clamped=n_clamped)


def assert_close(got: np.ndarray, want: np.ndarray, what: str, max_abs=MAX_ABS, mean_rel=MEAN_REL, rel_slack=0.0):
    """max |got - want| <= max_abs (+ rel_slack * |want| elementwise) and
    mean|got - want| / mean|want| <= mean_rel.  ``rel_slack`` is only for outputs whose
    magnitude makes one fp16 ulp comparable to max_abs (|y| >= 16 -> ulp 1.6e-2)."""
    g = np.asarray(got, np.float32)
    w = np.asarray(want, np.float32)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    err = np.abs(g - w)
    ma = float(err.max(initial=0.0))
    mr = float(err.mean() / max(float(np.abs(w).mean()), 1e-12))
    worst = float((err - rel_slack * np.abs(w)).max(initial=0.0))
    assert worst <= max_abs and mr <= mean_rel, \
        f"{what}: max-abs {ma:.3e} (<= {max_abs} + {rel_slack}|y|), mean-rel {mr:.3e} (<= {mean_rel})"
    return ma, mr


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.view(dtype) if t.element_size() == torch.empty(0, dtype=dtype).element_size() else t.to(dtype)
    return t.cuda()
