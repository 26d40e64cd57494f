"""Writes tests/golden/ref_workspace.npz: a tiny AWQ checkpoint and the TurboMind workspaces (tp = 1 and tp = 2) that the
REFERENCE's own converter makes of it.

lmdeploy/serve/turbomind/deploy.py is loaded by file path from the reference tree and its ``deploy_awq`` runs unmodified:
``permute`` (:371-382), ``merge_qkv`` (:251-260), ``fuse_w1_w3_s4`` (:638-654), ``convert_s4`` (:656-666), ``tp_m_s4``
(:668-670), ``export`` / ``save_bin`` / config.ini (:111-248).  What it cannot have here is stubbed, nothing else:
  * ``fire``, ``lmdeploy`` (package import), ``lmdeploy.model.MODELS`` (needs mmengine): inert stand-ins;
  * ``SentencePieceProcessor``: a stand-in that reports the vocabulary size (no tokenizer model in the fixture);
  * ``_turbomind`` (the compiled extension): the int4 format helpers restated in oracle/s4_format.py, which are pinned bit
    for bit against the reference's own format.cu kernels (tests/golden/ref_kernel_vectors.npz);
  * ``Tensor.cuda()``: identity (the restated helpers run on the CPU).
The checkpoint is seeded random: W ~ N(0, 0.05) quantised by oracle/awq.py (pinned against the reference quantiser).

    python tests/golden/make_ref_workspace_fixture.py [/path/to/lmdeploy]
"""
import importlib.util
import json
import os
import sys
import tempfile
import types

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import awq as oawq  # noqa: E402
from oracle import s4_format as f  # noqa: E402

REFERENCE = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TM_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))
HF_CONFIG = dict(num_hidden_layers=2, rms_norm_eps=1e-6, num_attention_heads=2, num_key_value_heads=2, rope_theta=10000.0,
                 hidden_size=256, intermediate_size=256, vocab_size=96)


def make_checkpoint(seed=0):
    """HF / AWQ naming: qweight int32 [in, out / 8], qzeros int32 [in / 128, out / 8], scales fp16 [in / 128, out]"""
    cfg, p = HF_CONFIG, {}
    hid, inter = cfg["hidden_size"], cfg["intermediate_size"]
    kv = cfg["num_key_value_heads"] * 128
    g = torch.Generator().manual_seed(seed)
    for i in range(cfg["num_hidden_layers"]):
        shapes = {"self_attn.q_proj": (hid, hid), "self_attn.k_proj": (kv, hid), "self_attn.v_proj": (kv, hid), "self_attn.o_proj": (hid, hid),
                  "mlp.gate_proj": (inter, hid), "mlp.up_proj": (inter, hid), "mlp.down_proj": (hid, inter)}
        for j, (name, (n, k)) in enumerate(shapes.items()):
            t, _, _ = oawq.make_awq_linear(n, k, 1000 * seed + 10 * i + j, 128, 0.05)
            p[f"model.layers.{i}.{name}.qweight"] = torch.from_numpy(t.qweight.view(np.int32).copy())
            p[f"model.layers.{i}.{name}.qzeros"] = torch.from_numpy(t.qzeros.view(np.int32).copy())
            p[f"model.layers.{i}.{name}.scales"] = torch.from_numpy(t.scales.copy())
        p[f"model.layers.{i}.input_layernorm.weight"] = (1 + 0.1 * torch.randn(hid, generator=g)).half()
        p[f"model.layers.{i}.post_attention_layernorm.weight"] = (1 + 0.1 * torch.randn(hid, generator=g)).half()
    p["model.embed_tokens.weight"] = (torch.randn(cfg["vocab_size"], hid, generator=g) * 0.5).half()
    p["model.norm.weight"] = (1 + 0.1 * torch.randn(hid, generator=g)).half()
    p["lm_head.weight"] = (torch.randn(cfg["vocab_size"], hid, generator=g) * 0.05).half()
    return p


def _words(t):
    return t.contiguous().numpy().view(np.uint32)


def turbomind_standin():
    m = types.ModuleType("_turbomind")

    def transpose_qk_s4_k_m8(src, dst, mm, k, size_per_head):
        dst.copy_(torch.from_numpy(f.transpose_qk_s4_k_m8_hf(_words(src), mm, k, size_per_head).view(np.int32)).view_as(dst))

    def fuse_w1_w3_s4_k_m8(src, dst, mm, k):
        dst.copy_(torch.from_numpy(f.fuse_w1_w3_s4_k_m8(_words(src), mm, k).view(np.int32)).view_as(dst))

    def convert_s4_k_m8(A_dst, Q_dst, ws, A_src, scales, qzeros, mm, k, group_size):
        a, q = f.convert_s4_k_m8(_words(A_src), scales.contiguous().numpy(), _words(qzeros), mm, k, group_size)
        A_dst.copy_(torch.from_numpy(a.view(np.int32)).view_as(A_dst))
        Q_dst.copy_(torch.from_numpy(np.ascontiguousarray(q).view(np.int32)).view_as(Q_dst))

    m.transpose_qk_s4_k_m8, m.fuse_w1_w3_s4_k_m8, m.convert_s4_k_m8 = transpose_qk_s4_k_m8, fuse_w1_w3_s4_k_m8, convert_s4_k_m8
    return m


def load_reference_deploy():
    class _Model:
        session_len = 2048

    class _Registry:
        def get(self, name):
            return _Model

    lm = types.ModuleType("lmdeploy")
    lm.__file__ = os.path.join(REFERENCE, "lmdeploy", "__init__.py")
    lm_model = types.ModuleType("lmdeploy.model")
    lm_model.MODELS = _Registry()
    for name, mod in (("fire", types.ModuleType("fire")), ("lmdeploy", lm), ("lmdeploy.model", lm_model), ("_turbomind", turbomind_standin())):
        sys.modules[name] = mod
    spec = importlib.util.spec_from_file_location("ref_deploy", os.path.join(REFERENCE, "lmdeploy", "serve", "turbomind", "deploy.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    class _Sp:
        def __init__(self, model_file):
            pass

        def vocab_size(self):
            return HF_CONFIG["vocab_size"]

        def bos_id(self):
            return 1

        def eos_id(self):
            return 2

    mod.SentencePieceProcessor = _Sp
    return mod


def main():
    deploy = load_reference_deploy()
    torch.Tensor.cuda = lambda self, *a, **k: self           # the stand-in helpers run on the CPU
    ckpt = make_checkpoint()
    out = {"hf/" + k: v.numpy() for k, v in ckpt.items()}
    out["hf_config"] = np.frombuffer(json.dumps(HF_CONFIG).encode(), np.uint8)
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "hf")
        os.makedirs(src)
        torch.save(ckpt, os.path.join(src, "pytorch_model.bin"))
        json.dump(HF_CONFIG, open(os.path.join(src, "config.json"), "w"))
        open(os.path.join(src, "tokenizer.model"), "wb").write(b"fixture without a tokenizer")
        for tp in (1, 2):
            dst = os.path.join(tmp, f"ws{tp}")
            os.makedirs(os.path.join(dst, "tokenizer"))
            assert deploy.deploy_awq("llama2", src, None, dst, tp, None, 128)
            wdir = os.path.join(dst, "weights")
            for name in sorted(os.listdir(wdir)):
                out[f"tp{tp}/{name}"] = np.fromfile(os.path.join(wdir, name), np.uint8)
    path = os.path.join(ROOT, "tests", "golden", "ref_workspace.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "entries")


if __name__ == "__main__":
    main()
