"""CPU: a workspace written by the REFERENCE's own converter (lmdeploy/serve/turbomind/deploy.py run unmodified on a tiny
AWQ checkpoint, tests/golden/ref_workspace.npz).  Its config.ini goes through tm_llama_read_config; every per-rank file
is compared, byte for byte, with what the CPU oracle derives independently from the checkpoint tensors (rotary interleave
of q / k, [q_r | k_r | v_r] per rank, interleaved gate / up, runtime int4 layout, row slices of o / w2) at tp = 1 and 2."""
import ctypes as C

import numpy as np
import pytest

from lmdeploy_b200 import lib as l
from tests import ref_workspace as rw


def test_config_ini_written_by_the_reference_reads_back(tmp_path):
    cfg, _, files = rw.load()
    for tp in (1, 2):
        d = rw.unpack_to(str(tmp_path / f"ws{tp}"), {"config.ini": files[tp]["config.ini"]})
        c, info = l.TmLlamaConfig(), l.TmLlamaWorkspaceInfo()
        assert l.lib.tm_llama_read_config(d.encode(), C.byref(c), C.byref(info)) == l.TM_OK
        assert (c.head_num, c.kv_head_num, c.size_per_head, c.inter_size, c.num_layer, c.vocab_size) == (2, 2, 128, 256, 2, 96)
        assert abs(c.norm_eps - 1e-6) < 1e-12 and c.rope_theta == 10000.0 and c.group_size == 128 and c.quant_policy == 0
        assert (c.tensor_para_size, c.tensor_para_rank, c.max_batch_size, c.session_len) == (tp, 0, 32, 2056)
        assert info.model_name == b"llama2" and info.weight_type == b"int4" and (info.start_id, info.end_id) == (1, 2)
        assert (info.rotary_embedding_dim, info.step_length, info.cache_max_entry_count, info.cache_chunk_size) == (128, 1, 48, 1)
        assert info.max_context_token_num == 4 * 2056 and info.use_context_fmha == 1 and info.attn_bias == 0


def test_config_ini_defaults_and_errors(tmp_path):
    d = tmp_path / "ws"
    d.mkdir()
    c = l.TmLlamaConfig()
    assert l.lib.tm_llama_read_config(str(d).encode(), C.byref(c), None) == l.TM_ERR_IO
    (d / "config.ini").write_text("[llama]\nhead_num = 4\nsize_per_head = 128\ninter_size = 512\nnum_layer = 3\nvocab_size = 100\n"
                                  "norm_eps = 1e-5\nstart_id = 1\nend_id = 2\nrotary_embedding = 128\n")
    info = l.TmLlamaWorkspaceInfo()
    assert l.lib.tm_llama_read_config(str(d).encode(), C.byref(c), C.byref(info)) == l.TM_OK
    # handleMissingParams (LlamaTritonModel.cc:59-98)
    assert (c.kv_head_num, c.max_batch_size, c.session_len, c.tensor_para_size) == (4, 32, 2160, 1) and c.rope_theta == 10000.0
    assert (info.step_length, info.cache_max_entry_count, info.cache_chunk_size, info.max_context_token_num) == (1, 32, 32, 5 * 2160)
    (d / "config.ini").write_text("[llama]\nhead_num = 4\n")
    assert l.lib.tm_llama_read_config(str(d).encode(), C.byref(c), None) == l.TM_ERR_INVALID_ARG
    (d / "config.ini").write_text("[other]\nhead_num = 4\n")
    assert l.lib.tm_llama_read_config(str(d).encode(), C.byref(c), None) == l.TM_ERR_IO


@pytest.mark.parametrize("tp", [1, 2])
def test_every_per_rank_file_matches_the_oracle_derivation(tp):
    cfg, hf, files = rw.load()
    ws = files[tp]
    for layer in range(cfg["num_hidden_layers"]):
        for rank in range(tp):
            for name, lin in rw.rank_linears(cfg, hf, layer, tp, rank).items():
                a, q = lin.runtime()
                stem = f"layers.{layer}.{name}.{rank}"
                assert np.array_equal(ws[stem + ".qweight"], a.view(np.uint8).reshape(-1)), stem + ".qweight"
                assert np.array_equal(ws[stem + ".scales_zeros"], np.ascontiguousarray(q).view(np.uint8).reshape(-1)), stem + ".scales_zeros"
        for norm, hf_name in (("attention_norm", "input_layernorm"), ("ffn_norm", "post_attention_layernorm")):
            assert np.array_equal(ws[f"layers.{layer}.{norm}.weight"], hf[f"model.layers.{layer}.{hf_name}.weight"].view(np.uint8).reshape(-1))
    for ours, theirs in (("tok_embeddings.weight", "model.embed_tokens.weight"), ("norm.weight", "model.norm.weight"), ("output.weight", "lm_head.weight")):
        assert np.array_equal(ws[ours], hf[theirs].view(np.uint8).reshape(-1))
    n_files = cfg["num_hidden_layers"] * (8 * tp + 2) + 3 + 1
    assert len(ws) == n_files, sorted(ws)
