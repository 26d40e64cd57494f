"""Oracle: RMSNorm and the fused residual-add + RMSNorm of the decoder loop.

TEST INFRASTRUCTURE.  Follows

* ``rootMeanSquareNorm``          src/turbomind/models/llama/llama_kernels.cu:14-44
* ``fusedAddBiasResidualNorm``    src/turbomind/models/llama/llama_decoder_kernels.cu:104-145
  (sum of squares taken from the un-rounded fp32 sum, the residual stored as fp16, the
  normalisation applied to the stored fp16 residual; ops at :41-63)

The fused residual-add form is pinned against the reference kernel's outputs on a B200
(tests/golden/ref_kernel_vectors.npz, tests/test_gpu_reference_kernels.py); the plain form is pinned
against the reference kernel run beside it (tests/test_gpu_reference_kernels.py,
test_rmsnorm_matches_reference_kernel).
"""
from __future__ import annotations

import numpy as np


def rmsnorm(x: np.ndarray, scale: np.ndarray, eps: float) -> np.ndarray:
    xf = np.asarray(x, np.float16).astype(np.float32)
    inv = 1.0 / np.sqrt((xf * xf).mean(axis=-1, keepdims=True, dtype=np.float32) + np.float32(eps))
    return (xf * inv.astype(np.float32) * np.asarray(scale, np.float16).astype(np.float32)).astype(np.float16)


def add_residual_rmsnorm(residual: np.ndarray, x: np.ndarray, bias, scale: np.ndarray, eps: float):
    """returns (new residual fp16, normed output fp16)."""
    r = np.asarray(residual, np.float16).astype(np.float32) + np.asarray(x, np.float16).astype(np.float32)
    if bias is not None:
        r = r + np.asarray(bias, np.float16).astype(np.float32)
    ss = (r * r).mean(axis=-1, keepdims=True, dtype=np.float32)
    r16 = r.astype(np.float16)
    inv = (1.0 / np.sqrt(ss + np.float32(eps))).astype(np.float32)
    out = (r16.astype(np.float32) * np.asarray(scale, np.float16).astype(np.float32) * inv).astype(np.float16)
    return r16, out
