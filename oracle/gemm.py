"""Oracle: W4A16 linear — ``Y = X . dequant(W)^T`` with fp32 accumulate, fp16 output.

TEST INFRASTRUCTURE.  This is the reference's torch path for the linear
(pseudo-quant weight of lmdeploy/lite/quantization/weight/quantizer.py:147, then an
fp32 matmul) plus the two epilogues of the CUDA GEMM:

* identity        src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.cu:22-29
  (``__float22half2_rn`` of the fp32 accumulators, gemm_template.h:278)
* fused SiLU      gemm_s4_f16.cu:31-43 — works on the fp16-rounded pair
  ``(gate, up) = (Y[:, 2j], Y[:, 2j+1])``: ``fp16(silu(gate) * up)`` in fp32.

Pinned against GemmS4F16::Run of the reference on a B200 (tests/golden/ref_kernel_vectors.npz,
tests/test_gpu_reference_kernels.py).

Argument names: T tokens, N output features, K input features.
"""
from __future__ import annotations

import numpy as np
import torch


def linear_f32acc(x: np.ndarray | torch.Tensor, w_kn: np.ndarray | torch.Tensor) -> torch.Tensor:
    """x fp16 [T, K], w_kn fp16 [K, N]  ->  fp16 [T, N] (fp32 accumulate)."""
    x = torch.as_tensor(np.asarray(x)) if not isinstance(x, torch.Tensor) else x
    w = torch.as_tensor(np.asarray(w_kn)) if not isinstance(w_kn, torch.Tensor) else w_kn
    return (x.float() @ w.float()).half()


def silu_mul_interleaved(y: torch.Tensor) -> torch.Tensor:
    """gemm_s4_f16.cu:31-43 on fp16 ``y [T, 2I]`` with interleaved (gate, up) columns."""
    u = y.float()
    gate, up = u[:, 0::2], u[:, 1::2]
    silu = gate / (1.0 + torch.exp(-gate))
    return (silu * up).half()


def gemm_s4_f16(x: np.ndarray, w_kn_f16: np.ndarray, fused_silu: bool = False) -> np.ndarray:
    """The operator ``GemmS4F16::Run`` (gemm_s4_f16.h:41-51) on an already dequantised
    fp16 weight ``[K, N]`` (see ``oracle.s4_format.dequantize_runtime_weight``)."""
    y = linear_f32acc(x, w_kn_f16)
    if fused_silu:
        y = silu_mul_interleaved(y)
    return y.numpy()
