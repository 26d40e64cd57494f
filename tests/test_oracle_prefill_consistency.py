"""CPU: the two attention oracles agree where they overlap.  One new token per sequence pushed through the prefill
chain (QKV bias + RoPE + transpose -> cache extend -> context attention, oracle/prefill.py) must give what the decode
oracle gives for the same token (oracle/attention.py, pinned against the reference's decode kernel): same cache rows,
same output within the fp16 tolerance of the path.  Also the degenerate inputs of the writers."""
import numpy as np

from oracle import attention as oa, prefill as op
from tests.helpers import assert_close

D = 128


def test_one_token_prefill_equals_a_decode_step():
    rng = np.random.default_rng(41)
    B, H, Hkv, S_max = 3, 4, 2, 40
    lengths = np.asarray([0, 7, 31], np.int32)
    qkv = rng.standard_normal((B, (H + 2 * Hkv) * D)).astype(np.float16)
    bias = (rng.standard_normal((H + 2 * Hkv) * D) * 0.1).astype(np.float16)
    kc = [rng.standard_normal((Hkv, S_max, D)).astype(np.float16) for _ in range(B)]
    vc = [rng.standard_normal((Hkv, S_max, D)).astype(np.float16) for _ in range(B)]
    kd, vd = [a.copy() for a in kc], [a.copy() for a in vc]
    want = oa.mmha_decode(qkv, kd, vd, lengths, H, Hkv, D, S_max, qkv_bias=bias)
    # the same token as a prefill of length 1 on top of `lengths` cached tokens
    ones = np.ones(B, np.int32)
    q, k, v = op.add_fused_qkv_bias_transpose(qkv, bias, None, lengths, ones, B, 1, H, Hkv)
    op.extend_kv_cache(kc, vc, 0, k, v, ones, lengths)
    got = op.context_attention(q, kc, vc, 0, np.arange(B + 1, dtype=np.int32), lengths + 1, H, Hkv)
    for a, b in zip(kc + vc, kd + vd):
        assert np.array_equal(a.view(np.uint16), b.view(np.uint16)), "appended cache rows differ between the two oracles"
    assert_close(got, want, "prefill oracle vs decode oracle, one new token")


def test_degenerate_inputs():
    q, k, v = op.add_fused_qkv_bias_transpose(np.zeros((0, 4 * D), np.float16), None, None, np.zeros(2, np.int32),
                                              np.zeros(2, np.int32), 2, 3, 2, 1)
    assert q.shape == (2, 2, 3, D) and not q.any() and not k.any() and not v.any()
    kc, vc = [np.ones((2, 8, D), np.float16)], [np.ones((2, 8, D), np.float16)]
    op.extend_kv_cache(kc, vc, 0, np.zeros((1, 2, 4, D), np.float16), np.zeros((1, 2, 4, D), np.float16), [0], [3])
    assert kc[0].all() and vc[0].all()                                   # nothing to append: untouched
    kt, vt = op.transpose_kv_cache(kc, vc, 0, [0], 8, 2, 1)
    assert not kt.any() and not vt.any()
    x = np.asarray([-1000.0, -0.5, 0.5, 1.5, 2.5, 1000.0], np.float16)
    assert op.quant_int8_rne(x, 1.0, 0.0).tolist() == [-128, 0, 0, 2, 2, 127]    # ties to even, saturation
