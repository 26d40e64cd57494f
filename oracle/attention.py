"""Oracle: one decode step of masked multi-head attention over a per-sequence KV cache.

TEST INFRASTRUCTURE.  numpy restatement of
``mmha::masked_multihead_attention_kernel``
(src/turbomind/kernels/decoder_masked_multihead_attention/
decoder_masked_multihead_attention_template.cuh:1218-1913) as LLaMA drives it
(parameter packing: src/turbomind/models/llama/LlamaDecoderSelfAttentionLayer.cc:87-161):

* finished sequences are skipped, neither ``out`` nor the cache is touched (:1298-1300)
* q/k (+bias) get the interleaved-pair rotary embedding at position
  ``timestep - total_padding_tokens[b]`` (:1391-1395; coefficients
  decoder_masked_multihead_attention_utils.h:885-904: ``pos / base^(2i/dim)``, fp32)
* the new K (after RoPE) and V go to cache slot ``tlength % memory_max_len`` of KV head
  ``h / (H / Hkv)`` (:1421-1440, :1811-1838); int8 cache: ``round(clamp((x - zp) / scale,
  -128, 127))`` with round-half-away (:976-981)
* scores over cached steps ``[first_step, tlength)`` use the cache content (int8:
  ``q8 * scale + zp`` in fp32, rounded to fp16, :1057-1107, :1558-1568); the new token's
  own score and value use the un-quantised fp16 k / v (:1447, :1798-1861)
* softmax: ``exp(s - max)``, ``1 / (sum + 1e-6)``, probabilities rounded to fp16
  (:1627-1666); PV accumulates in fp32 (MMHA_USE_FP32_ACUM_FOR_OUT, :34), fp16 output.

The reference multiplies q.k in fp16 FMA chains; this oracle uses fp32 dot products
(the reference's "own fp32-accumulated torch implementation" the tolerance is stated
against).  Pinned against the reference kernel's outputs on a B200
(tests/golden/ref_kernel_vectors.npz, tests/test_gpu_reference_kernels.py).

Cache layout per sequence (one layer): ``[Hkv, S_max, D]`` for K and for V, element
fp16 or int8 (LlamaCacheManager.h:32, template.cuh:1425-1426).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np


@dataclass
class KvQuant:
    """past_kv_scale: 4 floats (LlamaDecoderLayerWeight.cc:296-306)."""
    k_scale: float
    k_zp: float
    v_scale: float
    v_zp: float


def rope_coefficients(pos: float, rot_dim: int, base: float):
    """utils.h:885-889 — returns (cos, sin) fp32 arrays of rot_dim/2 pair angles."""
    zid = np.arange(0, rot_dim, 2, dtype=np.float32)
    denom = np.power(np.float32(base), zid / np.float32(rot_dim), dtype=np.float32)
    ang = (np.float32(pos) / denom).astype(np.float32)
    return np.cos(ang.astype(np.float64)).astype(np.float32), np.sin(ang.astype(np.float64)).astype(np.float32)


def apply_rope(x: np.ndarray, pos: float, rot_dim: int, base: float) -> np.ndarray:
    """utils.h:891-904 — x fp16 [..., D]; pairs (x[2i], x[2i+1]) rotated in fp32 -> fp16."""
    c, s = rope_coefficients(pos, rot_dim, base)
    xf = np.asarray(x, np.float16).astype(np.float32)
    out = xf.copy()
    a, b = xf[..., 0:rot_dim:2], xf[..., 1:rot_dim:2]
    out[..., 0:rot_dim:2] = c * a - s * b
    out[..., 1:rot_dim:2] = c * b + s * a
    return out.astype(np.float16)


def quant_int8(x_f16: np.ndarray, scale: float, zp: float) -> np.ndarray:
    """template.cuh:976-981 — fp32 divide, clamp, round half away from zero."""
    v = (np.asarray(x_f16, np.float16).astype(np.float32) - np.float32(zp)) / np.float32(scale)
    v = np.clip(v, np.float32(-128.0), np.float32(127.0))
    return (np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))).astype(np.int8)


def dequant_int8(q8: np.ndarray, scale: float, zp: float) -> np.ndarray:
    """template.cuh:1057-1061 then conversion to the fp16 compute type."""
    return (np.asarray(q8, np.int8).astype(np.float32) * np.float32(scale) + np.float32(zp)).astype(np.float16)


def mmha_decode(qkv: np.ndarray,
                k_cache: list,
                v_cache: list,
                lengths: np.ndarray,
                num_heads: int,
                num_kv_heads: int,
                head_dim: int,
                memory_max_len: int,
                rope_base: float = 10000.0,
                rot_dim: Optional[int] = None,
                finished: Optional[np.ndarray] = None,
                positions: Optional[np.ndarray] = None,
                qkv_bias: Optional[np.ndarray] = None,
                kv_quant: Optional[KvQuant] = None,
                inv_sqrt_dh: Optional[float] = None,
                out: Optional[np.ndarray] = None) -> np.ndarray:
    """One decode step.  ``k_cache[b]`` / ``v_cache[b]`` are numpy arrays
    ``[Hkv, memory_max_len, D]`` (float16, or int8 when ``kv_quant`` is given) and are
    UPDATED IN PLACE with the new token.  ``lengths[b]`` = tokens already cached.
    ``positions[b]`` = RoPE position (defaults to ``lengths[b]``, which is what the engine
    feeds: step - 1 - padding == cached length).  Returns ``out`` fp16 ``[B, H*D]``."""
    B = qkv.shape[0]
    H, Hkv, D = num_heads, num_kv_heads, head_dim
    rot_dim = D if rot_dim is None else rot_dim
    rep = H // Hkv
    isd = np.float32(1.0 / np.sqrt(D)) if inv_sqrt_dh is None else np.float32(inv_sqrt_dh)
    if out is None:
        out = np.zeros((B, H * D), np.float16)
    qkv = np.asarray(qkv, np.float16)
    if qkv_bias is not None:
        qkv = (qkv + np.asarray(qkv_bias, np.float16)[None, :]).astype(np.float16)  # fp16 add, :1381-1382
    for b in range(B):
        if finished is not None and finished[b]:
            continue
        t = int(lengths[b])
        pos = float(t if positions is None else positions[b])
        first = max(0, t + 1 - memory_max_len)
        slot = t % memory_max_len
        q = qkv[b, : H * D].reshape(H, D)
        k = qkv[b, H * D: (H + Hkv) * D].reshape(Hkv, D)
        v = qkv[b, (H + Hkv) * D:].reshape(Hkv, D)
        if rot_dim > 0:
            q = apply_rope(q, pos, rot_dim, rope_base)
            k = apply_rope(k, pos, rot_dim, rope_base)
        steps = np.arange(first, t) % memory_max_len
        if kv_quant is None:
            kc = k_cache[b][:, steps, :]
            vc = v_cache[b][:, steps, :]
            k_cache[b][:, slot, :] = k
            v_cache[b][:, slot, :] = v
        else:
            kc = dequant_int8(k_cache[b][:, steps, :], kv_quant.k_scale, kv_quant.k_zp)
            vc = dequant_int8(v_cache[b][:, steps, :], kv_quant.v_scale, kv_quant.v_zp)
            k_cache[b][:, slot, :] = quant_int8(k, kv_quant.k_scale, kv_quant.k_zp)
            v_cache[b][:, slot, :] = quant_int8(v, kv_quant.v_scale, kv_quant.v_zp)
        kc = kc.astype(np.float32)
        vc = vc.astype(np.float32)
        qf = q.astype(np.float32).reshape(Hkv, rep, D)
        s_past = np.einsum("grd,gsd->grs", qf, kc).astype(np.float32) * isd          # [Hkv, rep, L]
        s_new = (qf * k.astype(np.float32)[:, None, :]).sum(-1, dtype=np.float32)[..., None] * isd
        s = np.concatenate([s_past, s_new], axis=-1)
        e = np.exp(s - s.max(axis=-1, keepdims=True)).astype(np.float32)
        inv = np.float32(1.0) / (e.sum(axis=-1, keepdims=True, dtype=np.float32) + np.float32(1e-6))
        p = (e * inv).astype(np.float16).astype(np.float32)
        o = np.einsum("grs,gsd->grd", p[..., :-1], vc) + p[..., -1:] * v.astype(np.float32)[:, None, :]
        out[b] = o.reshape(H * D).astype(np.float16)
    return out
