"""Oracle: AWQ group-wise asymmetric int4 quantiser and the AWQ ("layout A") packing.

TEST INFRASTRUCTURE.  Restates, with the same torch operator sequence:

* ``cal_qparams_per_group_minmax``   lmdeploy/lite/utils/cal_qparams.py:75-99
* ``WeightQuantizer.quant``          lmdeploy/lite/quantization/weight/quantizer.py:105-156
* ``WeightOnlyQLinear.from_linear``  lmdeploy/pytorch/modules/linear.py:64-126
  (vectorised instead of the per-column Python loop)

One deliberate difference: the reference quantiser does not clamp, so
``round(w/s) + round(-min/s)`` can reach 16 and its ``|=`` packing then corrupts the
neighbouring nibble.  ``quantize`` clamps q and z to [0, 15] (what the benchmark
configuration prescribes) and returns how many elements were clamped;
``quantize(..., clamp=False)`` reproduces the reference bit for bit.
"""
from __future__ import annotations

from typing import NamedTuple

import numpy as np
import torch

AWQ_PACK_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)  # linear.py:87


class QuantResult(NamedTuple):
    q: torch.Tensor        # int32 [N, K]   quantised weight, values 0..15
    zeros: torch.Tensor    # int32 [N, K/g]
    scales: torch.Tensor   # same dtype as w, [N, K/g]
    n_clamped: int         # elements of q (and z) that fell outside 0..15


@torch.no_grad()
def cal_qparams_per_group_minmax(w: torch.Tensor, n_bits: int, group_size: int):
    """cal_qparams.py:75-99 — scales/zero points per (row, group); dtype of ``w``."""
    outc, inc = w.shape
    assert inc >= group_size and inc % group_size == 0
    wg = w.reshape(outc, -1, group_size)
    w_min = wg.min(dim=-1, keepdim=True)[0]
    w_max = wg.max(dim=-1, keepdim=True)[0]
    q_max = 2 ** n_bits - 1
    scales = (w_max - w_min)
    scales = scales.clamp_(min=1e-5).div_(q_max)
    zero_points = (-w_min / scales).round()
    return scales, zero_points


@torch.no_grad()
def quantize(w: torch.Tensor, group_size: int = 128, n_bits: int = 4, clamp: bool = True) -> QuantResult:
    """quantizer.py:128-156 with ``real=True``; q = round(w/s) + z, all in w's dtype."""
    n, k = w.shape
    scales, zp = cal_qparams_per_group_minmax(w, n_bits, group_size)
    wg = w.reshape(n, scales.shape[1], -1)
    q = (wg / scales).round() + zp
    q = q.reshape(n, k).to(torch.int32)
    z = zp.squeeze(-1).to(torch.int32)
    q_max = 2 ** n_bits - 1
    n_clamped = int(((q < 0) | (q > q_max)).sum()) + int(((z < 0) | (z > q_max)).sum())
    if clamp:
        q = q.clamp(0, q_max)
        z = z.clamp(0, q_max)
    return QuantResult(q, z, scales.squeeze(-1), n_clamped)


@torch.no_grad()
def pseudo_quant_weight(qr: QuantResult, group_size: int = 128) -> torch.Tensor:
    """quantizer.py:147 — ``(q - z) * s`` in the scale dtype; the weight the GEMM must see."""
    n, k = qr.q.shape
    dt = qr.scales.dtype
    qg = qr.q.reshape(n, -1, group_size).to(dt)
    w = (qg - qr.zeros.unsqueeze(-1).to(dt)) * qr.scales.unsqueeze(-1)
    return w.reshape(n, k)


def pack_awq(v: np.ndarray) -> np.ndarray:
    """linear.py:100-108 — int values [R, C] (C % 8 == 0) -> uint32 [R, C/8];
    nibble i of word c holds v[:, 8c + AWQ_PACK_ORDER[i]].  Values must be 0..15."""
    v = np.asarray(v)
    assert v.ndim == 2 and v.shape[1] % 8 == 0
    assert v.min(initial=0) >= 0 and v.max(initial=0) <= 15, "value outside 0..15 would corrupt a neighbour nibble"
    v = v.astype(np.uint32).reshape(v.shape[0], -1, 8)
    out = np.zeros(v.shape[:2], dtype=np.uint32)
    for i, src in enumerate(AWQ_PACK_ORDER):
        out |= v[:, :, src] << np.uint32(4 * i)
    return out


def unpack_awq(words: np.ndarray) -> np.ndarray:
    """Inverse of :func:`pack_awq`: uint32 [R, C/8] -> uint8 [R, C]."""
    words = np.asarray(words).astype(np.uint32)
    out = np.zeros(words.shape + (8,), dtype=np.uint8)
    for i, dst in enumerate(AWQ_PACK_ORDER):
        out[:, :, dst] = (words >> np.uint32(4 * i)) & 0xF
    return out.reshape(words.shape[0], -1)


class AwqTensors(NamedTuple):
    qweight: np.ndarray  # uint32 [K, N/8]   layout A
    qzeros: np.ndarray   # uint32 [K/g, N/8] layout A
    scales: np.ndarray   # float16 [K/g, N]


def to_awq_tensors(qr: QuantResult) -> AwqTensors:
    """linear.py:96-122 — the three tensors of an AWQ checkpoint linear."""
    qweight = pack_awq(qr.q.t().contiguous().numpy())
    qzeros = pack_awq(qr.zeros.t().contiguous().numpy())
    scales = qr.scales.t().contiguous().to(torch.float16).numpy()
    return AwqTensors(qweight, qzeros, scales)


def make_awq_linear(n: int, k: int, seed: int, group_size: int = 128, std: float = 0.02):
    """Seeded synthetic linear of the benchmark configurations: W ~ N(0, std) fp16 [N, K],
    quantised.  Returns (AwqTensors, fp16 pseudo-quant weight [N, K], n_clamped)."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * std).half()
    qr = quantize(w, group_size)
    return to_awq_tensors(qr), pseudo_quant_weight(qr, group_size), qr.n_clamped
