"""CPU restatement (numpy) of the reference's prefill-side writers around the KV cache and of its context attention,
lmdeploy v0.0.9.

Test infrastructure only: nothing under lmdeploy_b200/ imports this module.  Pinned against the
reference kernels themselves (oracle/_ref, built from the reference sources where they lie) by
tests/test_gpu_prefill.py, and against vectors those kernels produced (tests/golden/ref_prefill_vectors.npz,
tests/test_oracle_prefill_vectors.py).  Context attention is pinned against the reference's unfused route (its cache
transpose, mask and softmax kernels, GEMMs by cuBLAS); its flash-attention kernel needs CUTLASS and is not built.

  add_fused_qkv_bias_transpose  src/turbomind/kernels/unfused_attention_kernels.cu:852-976
  extend_kv_cache               src/turbomind/models/llama/llama_kernels.cu:245-464
  transpose_kv_cache            src/turbomind/models/llama/llama_kernels.cu:497-660
  context_attention             src/turbomind/models/llama/LlamaContextAttentionLayer.cc:257-420
"""
from __future__ import annotations

import numpy as np

from .attention import apply_rope

D = 128


def ntk_base(context_len: int, max_pos: int, rot_dim: int, base: float) -> np.float32:
    """decoder_masked_multihead_attention_utils.h:862-871"""
    f = np.float32
    if f(context_len) < f(max_pos):
        return f(base)
    alpha = max(f(np.exp2(np.ceil(np.log2(f(context_len) / f(max_pos)) + f(1)))) - f(1), f(1))
    return f(f(base) * np.power(f(alpha), f(rot_dim) / (f(rot_dim) - f(2)), dtype=np.float32))


def logn_scaling(seq_len: int, max_pos: int) -> np.float32:
    """decoder_masked_multihead_attention_utils.h:854-860"""
    if seq_len <= max_pos:
        return np.float32(1)
    return np.float32(np.log2(np.float32(seq_len)) / np.log2(np.float32(max_pos)))


def add_fused_qkv_bias_transpose(qkv, bias, padding_offset, history_length, input_length, batch_size, seq_len, head_num,
                                 kv_head_num, rot_dim=D, base=10000.0, max_pos=2048, use_dynamic_ntk=False,
                                 use_logn_attn=False):
    """qkv fp16 [token_num, (H + 2 Hkv) * D] -> q [B, H, seq_len, D], k, v [B, Hkv, seq_len, D]; rows that no token
    maps to stay zero (the reference leaves them unwritten)."""
    qkv = np.asarray(qkv, np.float16)
    token_num = qkv.shape[0]
    H, Hkv = head_num, kv_head_num
    x = qkv.reshape(token_num, H + 2 * Hkv, D)
    if bias is not None:
        x = x + np.asarray(bias, np.float16).reshape(1, H + 2 * Hkv, D)  # fp16 add, :903-904,913-916
    q = np.zeros((batch_size, H, seq_len, D), np.float16)
    k = np.zeros((batch_size, Hkv, seq_len, D), np.float16)
    v = np.zeros((batch_size, Hkv, seq_len, D), np.float16)
    for t in range(token_num):
        tgt = t + (0 if padding_offset is None else int(padding_offset[t]))  # :877-878
        b, s = divmod(tgt, seq_len)
        hist = int(history_length[b])
        step = hist + s  # :929
        rb = base
        if use_dynamic_ntk:
            rb = ntk_base(hist + int(input_length[b]), max_pos, rot_dim, base)  # :928,931-934
        qt = apply_rope(x[t, :H], float(step), rot_dim, float(rb))
        kt = apply_rope(x[t, H:H + Hkv], float(step), rot_dim, float(rb))
        if use_logn_attn:
            qt = (np.float16(logn_scaling(step + 1, max_pos)) * qt).astype(np.float16)  # :940-950, fp16 multiply
        q[b, :, s] = qt
        k[b, :, s] = kt
        v[b, :, s] = x[t, H + Hkv:]
    return q, k, v


def quant_int8_rne(x_f16, scale: float, zp: float) -> np.ndarray:
    """llama_kernels.cu:318-341,382-388: (x - zp) / scale in fp32, round to nearest even, saturate."""
    v = (np.asarray(x_f16, np.float16).astype(np.float32) - np.float32(zp)) / np.float32(scale)
    return np.clip(np.rint(v), -128, 127).astype(np.int8)


def dequant_int8(q8, scale: float, zp: float) -> np.ndarray:
    """llama_kernels.cu:309-316: q * scale + zp as one fp32 fused multiply-add, then fp16."""
    v = np.asarray(q8, np.int8).astype(np.float64) * np.float64(np.float32(scale)) + np.float64(np.float32(zp))
    return v.astype(np.float32).astype(np.float16)


def extend_kv_cache(k_cache, v_cache, layer_offset_rows_head, k_src, v_src, query_length, history_length, kv_scale=None):
    """k_cache / v_cache: one array per sequence, viewed as [heads_total, max_seq_len, D] (fp16 or int8), modified in
    place; layer_offset_rows_head = first head row of this layer in that view.  k_src / v_src [B, Hkv, max_q_len, D]."""
    B, Hkv = k_src.shape[0], k_src.shape[1]
    for b in range(B):
        n, t0 = int(query_length[b]), int(history_length[b])
        for cache, src, sc in ((k_cache[b], k_src[b], kv_scale[0:2] if kv_scale is not None else None),
                               (v_cache[b], v_src[b], kv_scale[2:4] if kv_scale is not None else None)):
            rows = src[:, :n]
            if cache.dtype == np.int8:
                rows = quant_int8_rne(rows, sc[0], sc[1])
            cache[layer_offset_rows_head:layer_offset_rows_head + Hkv, t0:t0 + n] = rows


def transpose_kv_cache(k_cache, v_cache, layer_offset_rows_head, key_length, max_kv_len, head_num, head_n_rep, kv_scale=None):
    """-> (k, v) fp16 [B, head_num, max_kv_len, D]; rows beyond key_length[b] stay zero."""
    B = len(k_cache)
    Hkv = head_num // head_n_rep
    outs = []
    for caches, sc in ((k_cache, kv_scale[0:2] if kv_scale is not None else None),
                       (v_cache, kv_scale[2:4] if kv_scale is not None else None)):
        out = np.zeros((B, head_num, max_kv_len, D), np.float16)
        for b in range(B):
            n = int(key_length[b])
            rows = caches[b][layer_offset_rows_head:layer_offset_rows_head + Hkv, :n]
            if rows.dtype == np.int8:
                rows = dequant_int8(rows, sc[0], sc[1])
            out[b, :, :n] = np.repeat(rows, head_n_rep, axis=0)  # query head h reads cached head h / n_rep (:526)
        outs.append(out)
    return outs[0], outs[1]


def context_attention(q, k_cache, v_cache, layer_offset_rows_head, cu_seqlens, context_lengths, head_num, kv_head_num,
                      kv_scale=None):
    """Causal attention of the new tokens over the cache, as the reference's unfused route defines it
    (src/turbomind/models/llama/LlamaContextAttentionLayer.cc:316-420: transposed cache -> q k^T (fp32 accumulate) ->
    invokeMaskedSoftmax with scale 1/sqrt(d), probabilities stored as fp16 -> p v (fp32 accumulate) -> fp16) and as its
    flash-attention route computes up to rounding (:257-313).  The mask is invokeCreateCausalMasks
    (src/turbomind/models/llama/llama_kernels.cu:179-201): query i sees key j iff j <= i + (k_len - q_len).

    q fp16 [B, H, max_q_len, D]; caches as in extend_kv_cache; -> fp16 [token_num, H * D] (packed by cu_seqlens)."""
    B = len(k_cache)
    n_rep = head_num // kv_head_num
    out = np.zeros((int(cu_seqlens[B]), head_num * D), np.float16)
    scale = np.float32(1.0 / np.sqrt(np.float32(D)))
    for b in range(B):
        tok0, q_len, ctx = int(cu_seqlens[b]), int(cu_seqlens[b + 1] - cu_seqlens[b]), int(context_lengths[b])
        hist = ctx - q_len
        for h in range(head_num):
            row = layer_offset_rows_head + h // n_rep
            k, v = k_cache[b][row, :ctx], v_cache[b][row, :ctx]
            if k.dtype == np.int8:
                k, v = dequant_int8(k, kv_scale[0], kv_scale[1]), dequant_int8(v, kv_scale[2], kv_scale[3])
            s = (q[b, h, :q_len].astype(np.float32) @ k.astype(np.float32).T) * scale
            s[np.arange(ctx)[None, :] > (hist + np.arange(q_len))[:, None]] = -np.inf
            p = np.exp(s - s.max(axis=1, keepdims=True))
            p = (p / p.sum(axis=1, keepdims=True)).astype(np.float16)
            out[tok0:tok0 + q_len, h * D:(h + 1) * D] = (p.astype(np.float32) @ v.astype(np.float32)).astype(np.float16)
    return out
