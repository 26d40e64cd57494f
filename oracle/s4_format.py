"""Oracle: int4 layout conversions of TurboMind's ``format.cu`` (numpy, bit exact).

TEST INFRASTRUCTURE.  The reference has only CUDA code for these; this file restates

* ``permute_u4``                    src/turbomind/kernels/gemm_s_f16/format.cu:24-59
* ``reformat_s4_k_m8``              format.cu:69-75
* ``dequantize_s4_offset_64`` / ``dequantize_s4_to_fp16x2_v2``
                                    format.cu:77-82, common.h:115-156
* ``merge_Q``                       format.cu:84-95
* ``convert_s4_k_m8``               format.cu:97-113
* ``transpose_qk_s4_k_m8_hf``       format.cu:115-121
* ``fuse_w1_w3_s4_k_m8``            format.cu:123-130
* ``dequantize_s4`` / ``dequantize_s4_to_fp16x2``  format.cu:132-142, common.h:47-113
* ``apply_Q``                       common.h:218-235

A "flat nibble array" is the word array read nibble by nibble, least significant
nibble of word 0 first (``read_u4`` format.cu:19-22).

Naming follows the reference: ``m`` = output features (N of the linear), ``k`` = input
features.  Pinned bit for bit against the reference's CUDA kernels run on a B200
(tests/golden/ref_kernel_vectors.npz, tests/test_gpu_reference_kernels.py).
"""
from __future__ import annotations

import numpy as np

# order in which dequantize_s4_to_fp16x2(_v2) emits the 8 nibbles of a word (common.h:70-84)
DEQUANT_NIBBLE_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)


def to_nibbles(words: np.ndarray) -> np.ndarray:
    """uint32 words (any shape) -> flat uint8 nibble array."""
    w = np.ascontiguousarray(words).astype(np.uint32).reshape(-1, 1)
    sh = (np.arange(8, dtype=np.uint32) * 4).reshape(1, 8)
    return ((w >> sh) & 0xF).astype(np.uint8).reshape(-1)


def from_nibbles(nib: np.ndarray) -> np.ndarray:
    """flat nibble array (len % 8 == 0) -> uint32 words."""
    n = np.asarray(nib).astype(np.uint32).reshape(-1, 8)
    sh = (np.arange(8, dtype=np.uint32) * 4).reshape(1, 8)
    return (n << sh).sum(axis=1, dtype=np.uint64).astype(np.uint32)


def permute_u4(src_words: np.ndarray, dims, order) -> np.ndarray:
    """format.cu:24-59 — view the flat nibble array with shape ``dims`` (row major) and
    write element ``indices`` to the position whose (row-major) index is taken over the
    axes listed in ``order``: a plain ``transpose(order)``."""
    nib = to_nibbles(src_words)
    assert nib.size == int(np.prod(dims)), (nib.size, dims)
    out = nib.reshape(dims).transpose(order)
    return from_nibbles(np.ascontiguousarray(out).reshape(-1))


def reformat_s4_k_m8(src_words: np.ndarray, m: int, k: int) -> np.ndarray:
    """format.cu:69-75 — AWQ layout ``[k, m/8]`` -> runtime layout ``[k/32][m/32][32 lanes] uint4``."""
    dims = (k // 32, 2, 2, 4, 2, m // 32, 2, 2, 2, 4)
    return permute_u4(src_words, dims, (0, 5, 9, 8, 3, 1, 6, 4, 2, 7)).reshape(k, m // 8)


def runtime_layout_index(kk: np.ndarray, nn: np.ndarray, m: int) -> np.ndarray:
    """Closed form of the permutation above: flat nibble index, inside the runtime layout,
    of logical element ``q[kk][nn]`` (nn = output feature).  Derived independently of
    :func:`reformat_s4_k_m8`; the tests require both to agree."""
    lane = (nn % 8) * 4 + (kk % 8) // 2
    w = ((kk // 16) % 2) * 2 + (nn // 16) % 2
    nib = (kk % 2) * 4 + ((kk // 8) % 2) * 2 + (nn // 8) % 2
    return ((((kk // 32) * (m // 32) + nn // 32) * 32 + lane) * 4 + w) * 8 + nib


def unpack_runtime_layout(a_words: np.ndarray, m: int, k: int) -> np.ndarray:
    """runtime layout words -> logical uint8 ``q[k][m]``."""
    nib = to_nibbles(a_words)
    kk, nn = np.meshgrid(np.arange(k), np.arange(m), indexing="ij")
    return nib[runtime_layout_index(kk, nn, m)]


def _u16_as_f16(bits: np.ndarray) -> np.ndarray:
    return bits.astype(np.uint16).view(np.float16)


def dequantize_s4_offset_64(words: np.ndarray) -> np.ndarray:
    """common.h:115-156 (the live ``else`` branch) — each word -> 8 halves, nibble order
    [0,4,1,5,2,6,3,7], value fp16 bit pattern ``0x5400 | nib << 4`` == 64 + nib."""
    w = np.asarray(words).astype(np.uint32).reshape(-1, 1)
    sh = (np.array(DEQUANT_NIBBLE_ORDER, dtype=np.uint32) * 4).reshape(1, 8)
    nib = (w >> sh) & 0xF
    return _u16_as_f16(0x5400 | (nib << 4)).reshape(-1)


def dequantize_s4(words: np.ndarray) -> np.ndarray:
    """format.cu:132-142 / common.h:47-113 — each word -> 8 halves holding the plain
    integer 0..15, nibble order [0,4,1,5,2,6,3,7]."""
    w = np.asarray(words).astype(np.uint32).reshape(-1, 1)
    sh = (np.array(DEQUANT_NIBBLE_ORDER, dtype=np.uint32) * 4).reshape(1, 8)
    return ((w >> sh) & 0xF).astype(np.float16).reshape(-1)


def merge_q(scales: np.ndarray, zeros_f16: np.ndarray) -> np.ndarray:
    """format.cu:84-95 — ``Q[i] = half2{zeros[i], scales[i]}`` -> float16 [..., 2]."""
    return np.stack([np.asarray(zeros_f16, np.float16), np.asarray(scales, np.float16)], axis=-1)


def convert_s4_k_m8(a_src: np.ndarray, scales: np.ndarray, qzeros: np.ndarray, m: int, k: int, group_size: int):
    """format.cu:97-113 — returns (A_dst uint32 [k, m/8] runtime layout,
    Q_dst float16 [k/g, m, 2] = {64 + z, s})."""
    zeros = dequantize_s4_offset_64(qzeros)[: k // group_size * m]
    q = merge_q(np.asarray(scales, np.float16).reshape(-1), zeros).reshape(k // group_size, m, 2)
    return reformat_s4_k_m8(a_src, m, k), q


def transpose_qk_s4_k_m8_hf(src_words: np.ndarray, m: int, k: int, size_per_head: int) -> np.ndarray:
    """format.cu:115-121 — per head, output feature ``2j+h`` takes HF feature ``64h + j``
    (half-rotation -> interleaved RoPE pairs), done on AWQ-packed words ``[k, m/8]``."""
    dims = (k, m // size_per_head, 2, size_per_head // 2 // 8, 2, 2, 2)
    return permute_u4(src_words, dims, (0, 1, 3, 5, 2, 6, 4)).reshape(k, m // 8)


def fuse_w1_w3_s4_k_m8(src_words: np.ndarray, m: int, k: int) -> np.ndarray:
    """format.cu:123-130 — ``[2, k, m/8]`` (w1 then w3) -> ``[k, 2m/8]`` with output
    features interleaved ``[w1_0, w3_0, w1_1, w3_1, ...]``."""
    dims = (2, k, m // 8, 2, 2, 2)
    return permute_u4(src_words, dims, (1, 2, 4, 0, 5, 3)).reshape(k, 2 * m // 8)


def _ftz16(x: np.ndarray) -> np.ndarray:
    """flush fp16 subnormals to (signed) zero, as ``.ftz`` does."""
    x = np.asarray(x, np.float16).copy()
    b = x.view(np.uint16)
    sub = (b & 0x7C00) == 0
    b[sub] &= 0x8000
    return x


def apply_q(x64: np.ndarray, q: np.ndarray) -> np.ndarray:
    """common.h:218-235 — ``(x - Q.x) * Q.y`` with ``sub.ftz.f16x2`` / ``mul.ftz.f16x2``."""
    x = _ftz16(x64).astype(np.float32)
    z = _ftz16(q[..., 0]).astype(np.float32)
    s = _ftz16(q[..., 1]).astype(np.float32)
    d = _ftz16((x - z).astype(np.float16)).astype(np.float32)
    return _ftz16((d * s).astype(np.float16))


def dequantize_runtime_weight(a_words: np.ndarray, q: np.ndarray, m: int, k: int, group_size: int) -> np.ndarray:
    """The fp16 weight ``[k, m]`` that ``gemm_s4_f16`` multiplies with: unpack the runtime
    layout, add the +64 carried by ``dequantize_s4_to_fp16x2_v2`` and apply ``apply_Q``
    (warp_iterator.h:56-83)."""
    nib = unpack_runtime_layout(a_words, m, k)
    x64 = _u16_as_f16(0x5400 | (nib.astype(np.uint16) << 4))
    qq = np.repeat(np.asarray(q, np.float16).reshape(k // group_size, m, 2), group_size, axis=0)
    return apply_q(x64, qq)
