"""Helpers around tests/golden/ref_workspace.npz (a tiny AWQ checkpoint and the TurboMind workspaces that the reference's
own deploy.py wrote for it, tp = 1 and 2; see tests/golden/make_ref_workspace_fixture.py): unpacking the files, and an
independent restatement of what every per-rank file must hold, computed from the checkpoint with the CPU oracle."""
import json
import os

import numpy as np

from oracle import awq as oawq
from oracle import s4_format as f

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_workspace.npz")
G = 128


def load():
    z = np.load(GOLDEN)
    cfg = json.loads(bytes(z["hf_config"]).decode())
    hf = {k[3:]: z[k] for k in z.files if k.startswith("hf/")}
    files = {tp: {k.split("/", 1)[1]: z[k] for k in z.files if k.startswith(f"tp{tp}/")} for tp in (1, 2)}
    return cfg, hf, files


def unpack_to(dir_, files):
    os.makedirs(dir_, exist_ok=True)
    for name, data in files.items():
        data.tofile(os.path.join(dir_, name))
    return dir_


def rotary_cols(n_heads):
    """column permutation HF half-rotation -> interleaved pairs: new column 128 h + 2 j + p takes old column 128 h + 64 p + j"""
    new = np.arange(n_heads * 128)
    h, r = new // 128, new % 128
    return h * 128 + (r % 2) * 64 + r // 2


class Linear:
    """one linear of the checkpoint as plain integer / fp16 matrices [K, N] (q), [K / 128, N] (z, s)"""

    def __init__(self, hf, name):
        self.q = oawq.unpack_awq(hf[name + ".qweight"].view(np.uint32))
        self.z = oawq.unpack_awq(hf[name + ".qzeros"].view(np.uint32))
        self.s = hf[name + ".scales"].view(np.float16)

    def cols(self, idx):
        out = Linear.__new__(Linear)
        out.q, out.z, out.s = self.q[:, idx], self.z[:, idx], self.s[:, idx]
        return out

    def rows(self, lo, hi):
        out = Linear.__new__(Linear)
        out.q, out.z, out.s = self.q[lo:hi], self.z[lo // G:hi // G], self.s[lo // G:hi // G]
        return out

    @staticmethod
    def hcat(parts):
        out = Linear.__new__(Linear)
        out.q, out.z, out.s = (np.concatenate([getattr(p, a) for p in parts], axis=1) for a in ("q", "z", "s"))
        return out

    def runtime(self):
        """-> (qweight words, scales_zeros half2) exactly as a .qweight / .scales_zeros file holds them"""
        k, n = self.q.shape
        a, q = f.convert_s4_k_m8(oawq.pack_awq(self.q), np.ascontiguousarray(self.s), oawq.pack_awq(self.z), n, k, G)
        return a, q

    def weight(self):
        """fp16 [K, N] = fp16((q - z) * s), the weight the GEMM must see"""
        z = np.repeat(self.z.astype(np.float16), G, axis=0)
        s = np.repeat(self.s, G, axis=0)
        return ((self.q.astype(np.float16) - z) * s).astype(np.float16)


def rank_linears(cfg, hf, layer, tp, rank):
    """the four linears of `layer` as tensor-parallel rank `rank` must hold them (LlamaDecoderLayerWeight.cc:49-77)"""
    H, Hkv, inter = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"]
    p = f"model.layers.{layer}."
    q = Linear(hf, p + "self_attn.q_proj").cols(rotary_cols(H))
    k = Linear(hf, p + "self_attn.k_proj").cols(rotary_cols(Hkv))
    v = Linear(hf, p + "self_attn.v_proj")
    hq, hkv = H // tp * 128, Hkv // tp * 128
    sl = lambda n: np.arange(rank * n, (rank + 1) * n)
    qkv = Linear.hcat([q.cols(sl(hq)), k.cols(sl(hkv)), v.cols(sl(hkv))])
    o = Linear(hf, p + "self_attn.o_proj").rows(rank * hq, (rank + 1) * hq)
    gate, up = Linear(hf, p + "mlp.gate_proj").cols(sl(inter // tp)), Linear(hf, p + "mlp.up_proj").cols(sl(inter // tp))
    inter_cols = np.arange(2 * (inter // tp))
    w13 = Linear.hcat([gate, up]).cols((inter_cols % 2) * (inter // tp) + inter_cols // 2)      # gate_j, up_j, gate_j+1, ...
    w2 = Linear(hf, p + "mlp.down_proj").rows(rank * (inter // tp), (rank + 1) * (inter // tp))
    return {"attention.w_qkv": qkv, "attention.wo": o, "feed_forward.w13": w13, "feed_forward.w2": w2}
