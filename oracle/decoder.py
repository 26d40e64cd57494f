"""Oracle: one LLaMA decode step for a batch (embedding -> layers -> lm-head -> greedy pick).

TEST INFRASTRUCTURE and the timed CPU baseline.  Order of operations and precisions follow
LlamaDecoder::forward (src/turbomind/models/llama/LlamaDecoder.cc:198-237): the residual stream is
kept in fp16, norms in fp32, every linear is the fp32-accumulated pseudo-quant linear of
``oracle.gemm`` with fp16 output, attention is ``oracle.attention.mmha_decode``; the lm-head uses
fp16 weights and fp32 logits (LlamaV2.cc:319-336); greedy = argmax, lowest id on ties (the
reference has no dedicated greedy path: top_k = 1 sampling, tie-breaking unpinned).

Weights of a layer (numpy): ``attn_norm``, ``ffn_norm`` fp16 [hidden]; ``w_qkv`` fp16
[hidden, (H + 2 Hkv) * 128] (dequantised, q/k columns already in interleaved-RoPE order),
``w_o`` [H * 128, hidden], ``w13`` [hidden, 2 * inter] with (gate, up) interleaved, ``w2``
[inter, hidden]; ``kv_quant``: ``oracle.attention.KvQuant`` or None.
"""
from __future__ import annotations

import numpy as np
import torch

from . import attention, gemm, norm


def decode_step(ids, lengths, layers, globals_, k_caches, v_caches, cfg, active=None):
    """ids int [B]; lengths int [B] (tokens cached); k_caches[l][b] / v_caches[l][b] numpy
    [Hkv, S, 128] updated in place.  Returns (normed hidden fp16 [B, hidden], logits f32 [B, V],
    picked int [B])."""
    H, Hkv, S = cfg["head_num"], cfg["kv_head_num"], cfg["session_len"]
    eps = cfg["norm_eps"]
    B = len(ids)
    finished = None if active is None else ~np.asarray(active, bool)
    x = globals_["tok_embeddings"][np.asarray(ids)].astype(np.float16)
    h = norm.rmsnorm(x, layers[0]["attn_norm"], eps)
    for l, w in enumerate(layers):
        qkv = gemm.gemm_s4_f16(h, w["w_qkv"])
        ctx = np.zeros((B, H * 128), np.float16)
        attention.mmha_decode(qkv, k_caches[l], v_caches[l], lengths, H, Hkv, 128, S, rope_base=cfg["rope_theta"],
                              finished=finished, kv_quant=w.get("kv_quant"), out=ctx)
        a = gemm.gemm_s4_f16(ctx, w["w_o"])
        x, h = norm.add_residual_rmsnorm(x, a, None, w["ffn_norm"], eps)
        f = gemm.gemm_s4_f16(h, w["w13"], fused_silu=True)
        f = gemm.gemm_s4_f16(f, w["w2"])
        nxt = layers[l + 1]["attn_norm"] if l + 1 < len(layers) else globals_["output_norm"]
        x, h = norm.add_residual_rmsnorm(x, f, None, nxt, eps)
    logits = (torch.from_numpy(h).float() @ torch.from_numpy(globals_["output_weight"]).float().t()).numpy()
    return h, logits, logits.argmax(axis=-1).astype(np.int32)
