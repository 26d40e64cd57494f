"""AWQ checkpoint -> TurboMind W4A16 workspace, the converter side of the on-disk format.

What ``deploy_awq`` + ``export`` of lmdeploy v0.0.9 do (lmdeploy/serve/turbomind/deploy.py:554-783, 111-248), for a
checkpoint already in memory: HF-named AWQ tensors (``model.layers.N.self_attn.q_proj.qweight`` ...; qweight / qzeros
int32 with 8 nibbles per word, scales fp16) go through the int4 format kernels of ``libtm_b200.so`` (``_tm_b200``) and
come out as the per-rank files that ``tm_llama_load_workspace`` / LlamaDecoderLayerWeight::loadModel read, plus
``config.ini``.  Needs a GPU (the format helpers are CUDA kernels, as in the reference).

    q, k   rotary pairs from the HF half-rotation layout to interleaved (deploy.py:631-637, 371-382)
    qkv    per tensor-parallel rank  [q_r | k_r | v_r]                     (deploy.py:251-260)
    w1|w3  interleaved gate / up columns                                    (deploy.py:638-654)
    all    AWQ nibble order -> runtime layout, {64 + zero, scale} pairs     (deploy.py:656-666)
    qkv, w13  runtime layout regrouped so that each rank's columns are one contiguous slice (deploy.py:668-670)
    export    column-split w_qkv / w13, row-split wo / w2, one file per rank (deploy.py:142-198), config.ini (:209-248)
"""
from __future__ import annotations

import configparser
import os
from typing import Dict

import torch

from . import _tm_b200 as _tm

HEAD = 128      # size_per_head, the only one the kernels serve


def rotary_interleave(x: torch.Tensor) -> torch.Tensor:
    """fp16 tensor whose LAST axis runs over q or k output features: within every head, feature 64 h + j moves to
    2 j + h (deploy.py:371-382 for matrices; scales of shape [groups, features] are matrices here too)."""
    heads = x.shape[-1] // HEAD
    return x.reshape(*x.shape[:-1], heads, 2, HEAD // 2).transpose(-1, -2).reshape(x.shape)


def _qk_s4(x: torch.Tensor, group_size: int) -> torch.Tensor:
    out = torch.empty_like(x)
    _tm.transpose_qk_s4_k_m8(x, out, x.shape[-1] * 8, x.shape[0], group_size)    # size_per_head = group_size, as deploy.py:634
    return out


def _per_rank_concat(parts, tp: int) -> torch.Tensor:
    """[rows, cols_i] tensors -> [rows, sum cols]: rank r's slice of every part, side by side, rank after rank"""
    rows = parts[0].shape[0]
    return torch.cat([p.reshape(rows, tp, -1) for p in parts], dim=-1).reshape(rows, -1).contiguous()


def _interleave_s4(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    both = torch.cat((a, b)).contiguous()
    out = torch.empty_like(both)
    _tm.fuse_w1_w3_s4_k_m8(both, out, a.shape[-1] * 8, a.shape[0])
    return out.view(a.shape[0], -1)


def _to_runtime(qw: torch.Tensor, qz: torch.Tensor, s: torch.Tensor, group_size: int):
    a = torch.empty_like(qw)
    q = torch.empty(s.shape, dtype=torch.int32, device=s.device)       # half2 {64 + zero, scale} per weight column
    ws = torch.empty_like(s)
    _tm.convert_s4_k_m8(a, q, ws, qw.contiguous(), s.contiguous(), qz.contiguous(), qw.shape[-1] * 8, qw.shape[0], group_size)
    return a, q


def _rank_major(a: torch.Tensor, tp: int) -> torch.Tensor:
    """runtime layout [K/32 slabs][tiles of 32 columns][128 words]: tiles regrouped so that splitting the flat row of a
    slab into tp equal parts hands every rank its own tiles (deploy.py:668-670)"""
    return a.view(a.shape[0] // 32, tp, -1, 128).permute(0, 2, 3, 1).contiguous()


def convert_awq_checkpoint(params: Dict[str, torch.Tensor], num_layer: int, tp: int, group_size: int = 128) -> Dict[str, torch.Tensor]:
    """HF-named AWQ tensors -> TurboMind-named tensors, still whole (export() splits them per rank)."""
    out = {}

    def get(name):
        return params[name].cuda().contiguous()

    for i in range(num_layer):
        att, mlp = f"model.layers.{i}.self_attn.", f"model.layers.{i}.mlp."
        qw, qz, sc = {}, {}, {}
        for p in ("q", "k", "v", "o"):
            qw[p], qz[p], sc[p] = get(att + p + "_proj.qweight"), get(att + p + "_proj.qzeros"), get(att + p + "_proj.scales")
        for p in ("q", "k"):
            qw[p], qz[p], sc[p] = _qk_s4(qw[p], group_size), _qk_s4(qz[p], group_size), rotary_interleave(sc[p])
        qkv = [_per_rank_concat([t["q"], t["k"], t["v"]], tp) for t in (qw, qz, sc)]
        a, q = _to_runtime(*qkv, group_size)
        out[f"layers.{i}.attention.w_qkv.qweight"], out[f"layers.{i}.attention.w_qkv.scales_zeros"] = _rank_major(a, tp), q
        out[f"layers.{i}.attention.wo.qweight"], out[f"layers.{i}.attention.wo.scales_zeros"] = _to_runtime(qw["o"], qz["o"], sc["o"], group_size)
        if att + "q_proj.bias" in params:
            b = [rotary_interleave(get(att + "q_proj.bias")[None])[0], rotary_interleave(get(att + "k_proj.bias")[None])[0],
                 get(att + "v_proj.bias")]
            out[f"layers.{i}.attention.w_qkv.bias"] = torch.cat([x.reshape(tp, -1) for x in b], dim=-1).reshape(-1)
            out[f"layers.{i}.attention.wo.bias"] = get(att + "o_proj.bias")

        g = {n: (get(mlp + n + "_proj.qweight"), get(mlp + n + "_proj.qzeros"), get(mlp + n + "_proj.scales")) for n in ("gate", "down", "up")}
        w13_s = torch.stack((g["gate"][2], g["up"][2]), dim=-1).reshape(g["gate"][2].shape[0], -1).contiguous()
        a, q = _to_runtime(_interleave_s4(g["gate"][0], g["up"][0]), _interleave_s4(g["gate"][1], g["up"][1]), w13_s, group_size)
        out[f"layers.{i}.feed_forward.w13.qweight"], out[f"layers.{i}.feed_forward.w13.scales_zeros"] = _rank_major(a, tp), q
        out[f"layers.{i}.feed_forward.w2.qweight"], out[f"layers.{i}.feed_forward.w2.scales_zeros"] = _to_runtime(*g["down"], group_size)
        out[f"layers.{i}.attention_norm.weight"] = get(f"model.layers.{i}.input_layernorm.weight")
        out[f"layers.{i}.ffn_norm.weight"] = get(f"model.layers.{i}.post_attention_layernorm.weight")
    out["tok_embeddings.weight"] = get("model.embed_tokens.weight")
    out["norm.weight"] = get("model.norm.weight")
    out["output.weight"] = get("lm_head.weight")
    return out


def export_workspace(tensors: Dict[str, torch.Tensor], weights_dir: str, tp: int, *, model_name: str, num_layer: int, norm_eps: float,
                     kv_head_num: int, group_size: int, rope_theta: float = 10000.0, session_len: int = 2056, start_id: int = 1,
                     end_id: int = 2, size_per_head: int = HEAD) -> None:
    """One raw little-endian file per tensor and rank, and config.ini (deploy.py:111-248)."""
    os.makedirs(weights_dir, exist_ok=True)

    def dump(t: torch.Tensor, name: str):
        if t.dtype in (torch.float32, torch.bfloat16):
            t = t.half()
        t.contiguous().cpu().numpy().tofile(os.path.join(weights_dir, name))

    vocab, dim = tensors["tok_embeddings.weight"].shape
    if vocab % tp:                                   # rows of zeros up to a multiple of tp (deploy.py:150-160)
        pad = (vocab + tp - 1) // tp * tp - vocab
        for n in ("tok_embeddings.weight", "output.weight"):
            tensors[n] = torch.nn.functional.pad(tensors[n], (0, 0, 0, pad))
        vocab += pad
    inter, attn_bias = 0, 0
    for name, t in tensors.items():
        key, ext = name.split(".")[-2:]
        stem = name[: -len(ext) - 1]
        if key == "w_qkv" and ext == "bias":
            attn_bias = 1
        if key == "w13":
            inter = max(inter, t.shape[-1] // 2)
        if key in ("w_qkv", "w13"):                  # output features split: last axis
            for r, part in enumerate(torch.chunk(t, tp, dim=-1)):
                dump(part, f"{stem}.{r}.{ext}")
        elif key in ("wo", "w2") and ext != "bias":  # input features split: first axis
            for r, part in enumerate(torch.chunk(t, tp, dim=0)):
                dump(part, f"{stem}.{r}.{ext}")
        elif key in ("wo", "w2"):                    # bias of a row-split linear: every rank gets the whole
            for r in range(tp):
                dump(t, f"{stem}.{r}.{ext}")
        else:
            dump(t, name)
    assert inter > 0
    cfg = configparser.ConfigParser()
    cfg["llama"] = dict(model_name=model_name, head_num=dim // size_per_head, kv_head_num=kv_head_num, size_per_head=size_per_head,
                        vocab_size=vocab, num_layer=num_layer, rotary_embedding=size_per_head, rope_theta=rope_theta,
                        inter_size=inter, norm_eps=norm_eps, attn_bias=attn_bias, start_id=start_id, end_id=end_id,
                        weight_type="int4", group_size=group_size, max_batch_size=32, max_context_token_num=4,
                        session_len=session_len, step_length=1, cache_max_entry_count=48, cache_chunk_size=1,
                        use_context_fmha=1, quant_policy=0, tensor_para_size=tp, max_position_embeddings=0, use_dynamic_ntk=0,
                        use_logn_attn=0)
    with open(os.path.join(weights_dir, "config.ini"), "w") as f:
        cfg.write(f)


def deploy_awq(params: Dict[str, torch.Tensor], hf_config: dict, out_dir: str, tp: int = 1, group_size: int = 128,
               model_name: str = "llama2", session_len: int = 2056) -> str:
    """-> ``out_dir``/weights, loadable by ``LlamaModel.load_workspace`` (tm_llama_load_workspace)."""
    n = hf_config["num_hidden_layers"]
    tensors = convert_awq_checkpoint(params, n, tp, group_size)
    weights = os.path.join(out_dir, "weights")
    export_workspace(tensors, weights, tp, model_name=model_name, num_layer=n, norm_eps=hf_config["rms_norm_eps"],
                     kv_head_num=hf_config.get("num_key_value_heads", hf_config["num_attention_heads"]), group_size=group_size,
                     rope_theta=float(hf_config.get("rope_theta", 10000.0)), session_len=session_len)
    return weights
