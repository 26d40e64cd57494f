"""CPU: the prefill oracle against golden vectors produced by the REFERENCE's own CUDA kernels
(tests/golden/ref_prefill_vectors.npz, written by tests/golden/make_ref_prefill_vectors.py on a B200 from the reference
sources compiled as they are).  Copies and int8 rounding bit for bit; rotated values within one fp16 step; attention
within the fp16 tolerances of the GPU parity tests."""
import os

import numpy as np
import pytest

from oracle import prefill as op
from tests.helpers import assert_close

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_prefill_vectors.npz")
if not os.path.exists(_PATH):
    pytest.skip("tests/golden/ref_prefill_vectors.npz not generated yet", allow_module_level=True)
G = np.load(_PATH)


def test_qkv_bias_rope_transpose():
    q, k, v = op.add_fused_qkv_bias_transpose(G["qkv_in"], G["qkv_bias"], G["qkv_pad"], G["qkv_history"], G["qkv_input"], 3, 12, 4, 2)
    assert np.array_equal(v.view(np.uint16), G["qkv_v"].view(np.uint16))
    for got, want in ((q, G["qkv_q"]), (k, G["qkv_k"])):
        g, w = got.astype(np.float32), want.astype(np.float32)
        assert (np.abs(g - w) <= np.maximum(np.abs(w) * 2.0 ** -10 * 1.01, 1e-3)).all()   # position 300: see the GPU test
        assert (g != w).mean() < 0.05


def test_extend_and_transpose_kv_cache():
    sc = G["kv_scale"]
    for tag, scale in (("f16", None), ("s8", sc)):
        kc, vc = [a.copy() for a in G[f"ext_{tag}_k_in"]], [a.copy() for a in G[f"ext_{tag}_v_in"]]
        op.extend_kv_cache(kc, vc, 2, G[f"ext_{tag}_k_src"], G[f"ext_{tag}_v_src"], [10, 3], [0, 21], scale)
        assert np.array_equal(np.stack(kc), G[f"ext_{tag}_k_out"]) and np.array_equal(np.stack(vc), G[f"ext_{tag}_v_out"])
        kt, vt = op.transpose_kv_cache(list(G[f"ext_{tag}_k_in"]), list(G[f"ext_{tag}_v_in"]), 2, [24, 6], 24, 4, 2, scale)
        assert np.array_equal(kt.view(np.uint16), G[f"tr_{tag}_k"].view(np.uint16))
        assert np.array_equal(vt.view(np.uint16), G[f"tr_{tag}_v"].view(np.uint16))


def test_causal_mask_and_context_attention():
    for tag, scale in (("f16", None), ("s8", G["attn_kv_scale"])):
        cu, ctx = G[f"attn_{tag}_cu"], G[f"attn_{tag}_ctx"]
        mask = G[f"attn_{tag}_mask"]
        for b in range(len(ctx)):
            q_len, k_len = int(cu[b + 1] - cu[b]), int(ctx[b])
            i, j = np.arange(mask.shape[1])[:, None], np.arange(mask.shape[2])[None, :]
            want = (i < q_len) & (j < k_len) & (j <= i + (k_len - q_len))
            assert np.array_equal(mask[b] != 0, want)
        out = op.context_attention(G[f"attn_{tag}_q"], list(G[f"attn_{tag}_k"]), list(G[f"attn_{tag}_v"]), 0, cu, ctx, 4, 2, scale)
        assert_close(out, G[f"attn_{tag}_out"], f"oracle vs reference unfused route ({tag})")
