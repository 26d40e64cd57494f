"""GPU: the workspace written by the reference's own deploy.py (tests/golden/ref_workspace.npz) is loaded by
tm_llama_load_workspace and decodes like the CPU oracle fed with weights derived independently from the checkpoint;
this library's converter (lmdeploy_b200/deploy.py over the CUDA format kernels) writes the same files byte for byte."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import decoder as odec
from tests import ref_workspace as rw

pytestmark = pytest.mark.gpu


def _oracle_model(cfg, hf):
    layers = []
    for i in range(cfg["num_hidden_layers"]):
        lin = rw.rank_linears(cfg, hf, i, 1, 0)
        layers.append(dict(attn_norm=hf[f"model.layers.{i}.input_layernorm.weight"].view(np.float16),
                           ffn_norm=hf[f"model.layers.{i}.post_attention_layernorm.weight"].view(np.float16),
                           w_qkv=lin["attention.w_qkv"].weight(), w_o=lin["attention.wo"].weight(),
                           w13=lin["feed_forward.w13"].weight(), w2=lin["feed_forward.w2"].weight(), kv_quant=None))
    g = dict(tok_embeddings=hf["model.embed_tokens.weight"].view(np.float16), output_norm=hf["model.norm.weight"].view(np.float16),
             output_weight=hf["lm_head.weight"].view(np.float16))
    return layers, g


def test_reference_written_workspace_loads_and_decodes_like_the_oracle(tmp_path):
    from lmdeploy_b200 import lib as l, llama
    cfg, hf, files = rw.load()
    d = rw.unpack_to(str(tmp_path / "ws"), files[1])
    c = l.TmLlamaConfig()
    assert l.lib.tm_llama_read_config(d.encode(), C.byref(c), None) == l.TM_OK
    S = 32
    mcfg = llama.LlamaConfig(c.head_num, c.kv_head_num, c.inter_size, c.num_layer, c.vocab_size, norm_eps=c.norm_eps,
                             rope_theta=c.rope_theta, quant_policy=c.quant_policy)
    model = llama.LlamaModel(mcfg, max_batch_size=2, session_len=S, device=0)
    model.load_workspace(d)
    layers, g = _oracle_model(cfg, hf)
    ocfg = dict(head_num=c.head_num, kv_head_num=c.kv_head_num, session_len=S, norm_eps=c.norm_eps, rope_theta=c.rope_theta)
    B, steps = 2, 6
    tokens = np.random.default_rng(0).integers(0, c.vocab_size, size=(steps, B)).astype(np.int32)
    kc = [[np.zeros((c.kv_head_num, S, 128), np.float16) for _ in range(B)] for _ in range(c.num_layer)]
    vc = [[np.zeros((c.kv_head_num, S, 128), np.float16) for _ in range(B)] for _ in range(c.num_layer)]
    lengths = np.zeros(B, np.int32)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        st = model.new_state(B, steps, None, tokens, keep_hidden=True, keep_logits=True)
        for s in range(steps):
            want_h, want_l, _ = odec.decode_step(tokens[s], lengths, layers, g, kc, vc, ocfg)
            model.decode(st, 1, use_graph=False)
            model.check_status(stream.cuda_stream)
            eh = np.abs(st.hidden.cpu().numpy().astype(np.float32) - want_h.astype(np.float32))
            el = np.abs(st.logits.cpu().numpy() - want_l)
            assert eh.max() <= 3e-2 and eh.mean() / np.abs(want_h.astype(np.float32)).mean() <= 5e-3, (s, eh.max())
            assert el.max() <= 3e-2 and el.mean() / np.abs(want_l).mean() <= 5e-3, (s, el.max())
            gk, gv = st.k_cache.cpu().numpy(), st.v_cache.cpu().numpy()
            for li in range(c.num_layer):          # the oracle continues from the GPU's cache: identical history every step
                for b in range(B):
                    d_k = np.abs(gk[b, li][:, lengths[b]].astype(np.float32) - kc[li][b][:, lengths[b]].astype(np.float32))
                    assert d_k.max() <= 2e-2, (s, li, b, d_k.max())
                    kc[li][b][...] = gk[b, li]
                    vc[li][b][...] = gv[b, li]
            lengths = lengths + 1
    model.close()


@pytest.mark.parametrize("tp", [1, 2])
def test_own_converter_writes_the_same_files_as_the_reference(tp, tmp_path):
    from lmdeploy_b200 import deploy, lib as l
    cfg, hf, files = rw.load()
    params = {k: torch.from_numpy(v.copy()) for k, v in hf.items()}
    wdir = deploy.deploy_awq(params, cfg, str(tmp_path / "out"), tp=tp, group_size=128, model_name="llama2")
    want = files[tp]
    got = set(os.listdir(wdir))
    assert got == set(want), (sorted(got - set(want)), sorted(set(want) - got))
    for name, data in want.items():
        if name == "config.ini":
            continue
        assert np.array_equal(np.fromfile(os.path.join(wdir, name), np.uint8), data), name
    # config.ini: same values through the reader (key order and float formatting are configparser's business)
    ref_dir = rw.unpack_to(str(tmp_path / "ref"), {"config.ini": want["config.ini"]})
    a, b, ia, ib = l.TmLlamaConfig(), l.TmLlamaConfig(), l.TmLlamaWorkspaceInfo(), l.TmLlamaWorkspaceInfo()
    assert l.lib.tm_llama_read_config(wdir.encode(), C.byref(a), C.byref(ia)) == l.TM_OK
    assert l.lib.tm_llama_read_config(ref_dir.encode(), C.byref(b), C.byref(ib)) == l.TM_OK
    assert bytes(a) == bytes(b) and bytes(ia) == bytes(ib)
