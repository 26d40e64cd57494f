"""Weight preparation on the GPU: AWQ group-wise asymmetric int4 quantisation with torch ops and
conversion to the runtime layout with the library's format kernels.

The arithmetic is lmdeploy.lite's (``cal_qparams_per_group_minmax``,
lmdeploy/lite/utils/cal_qparams.py:75-99; ``WeightQuantizer.quant``,
lmdeploy/lite/quantization/weight/quantizer.py:128-156; nibble order of
``WeightOnlyQLinear.from_linear``, lmdeploy/pytorch/modules/linear.py:87-108), with the integer
weight and zero point clamped to 0..15 before packing; the layout conversion is what
lmdeploy/serve/turbomind/deploy.py:656-666 does through ``_turbomind.convert_s4_k_m8``.
"""
from __future__ import annotations

import torch

from . import turbomind as tm

AWQ_PACK_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


@torch.no_grad()
def quantize_awq(w: torch.Tensor, group_size: int = 128):
    """w half [N, K] (CUDA) -> (qweight int32 [K, N/8], qzeros int32 [K/g, N/8], scales half [K/g, N])."""
    n, k = w.shape
    wg = w.reshape(n, k // group_size, group_size)
    w_min = wg.min(dim=-1, keepdim=True)[0]
    w_max = wg.max(dim=-1, keepdim=True)[0]
    scales = (w_max - w_min).clamp_(min=1e-5).div_(15)
    zeros = (-w_min / scales).round()
    q = ((wg / scales).round() + zeros).clamp_(0, 15).reshape(n, k).to(torch.int32)
    z = zeros.squeeze(-1).clamp_(0, 15).to(torch.int32)
    return pack_awq(q.t().contiguous()), pack_awq(z.t().contiguous()), scales.squeeze(-1).t().contiguous().half()


@torch.no_grad()
def pack_awq(v: torch.Tensor) -> torch.Tensor:
    """int32 [R, C] values 0..15 -> int32 [R, C/8]; nibble i of a word holds column 8c + order[i]."""
    r, c = v.shape
    v = v.reshape(r, c // 8, 8).to(torch.int64)
    out = torch.zeros(r, c // 8, dtype=torch.int64, device=v.device)
    for i, src in enumerate(AWQ_PACK_ORDER):
        out |= v[:, :, src] << (4 * i)
    return torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)


@torch.no_grad()
def to_runtime_layout(qweight, qzeros, scales, n, k, group_size=128):
    """AWQ tensors -> (kernel int32 [K, N/8] runtime layout, scales_and_zeros half [K/g, N, 2])."""
    kernel = torch.empty_like(qweight)
    sz = torch.empty(k // group_size, n, 2, dtype=torch.float16, device=qweight.device)
    ws = torch.empty(k // group_size * n, dtype=torch.float16, device=qweight.device)
    tm.convert_s4_k_m8(kernel, sz, ws, qweight, scales, qzeros, n, k, group_size)
    return kernel, sz


@torch.no_grad()
def random_linear(n, k, gen, std=0.02, group_size=128):
    """Seeded synthetic W ~ N(0, std) half [N, K], quantised and converted -> LlamaDenseWeight."""
    w = (torch.randn(n, k, device=gen.device, generator=gen) * std).half()
    qw, qz, s = quantize_awq(w, group_size)
    del w
    kernel, sz = to_runtime_layout(qw, qz, s, n, k, group_size)
    return tm.LlamaDenseWeight(k, n, kernel, tm.WeightType.kINT4, None, sz, group_size)
