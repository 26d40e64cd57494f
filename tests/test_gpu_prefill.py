"""GPU: the prefill-side writers around the KV cache (QKV bias + RoPE + transpose, cache extend, cache
transpose) through the C ABI, three ways: this library, the reference's own kernels (oracle/_ref, when
built) and the CPU oracle.  Integer / copy results must agree bit for bit; rotated values within one
fp16 rounding of the oracle and bit for bit with the reference kernel."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import prefill as op
from tests.helpers import dev

pytestmark = pytest.mark.gpu

D = 128
_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libtm_ref.so")


def load_ref():
    if not os.path.exists(_REF):
        return None
    lib = C.CDLL(_REF)
    vp, i, f32, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
    lib.ref_add_fused_qkv_bias_transpose.argtypes = [vp] * 8 + [i] * 7 + [f32, i, i, i, vp]
    lib.ref_extend_kv_cache.argtypes = [vp, vp, sz, vp, vp, i, vp, i, vp, i, i, i, vp, i, C.POINTER(f32)]
    lib.ref_transpose_kv_cache.argtypes = [vp, vp, vp, vp, sz, i, vp, i, i, i, i, i, vp, i, C.POINTER(f32)]
    lib.ref_create_causal_masks.argtypes = [vp, vp, vp, i, i, i, vp]
    lib.ref_masked_softmax.argtypes = [vp, vp, vp, i, i, i, i, f32, vp]
    for n in ("ref_add_fused_qkv_bias_transpose", "ref_extend_kv_cache", "ref_transpose_kv_cache", "ref_create_causal_masks",
              "ref_masked_softmax"):
        getattr(lib, n).restype = i
    return lib


@pytest.fixture(scope="module")
def ref():
    return load_ref()


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p()


def qkv_case(lengths, history, seq_len, H, Hkv, seed, bias=True, padded=True):
    """packed tokens of a ragged batch -> inputs of invokeAddFusedQKVBiasTranspose"""
    rng = np.random.default_rng(seed)
    B = len(lengths)
    token_num = int(sum(lengths)) if padded else B * seq_len
    qkv = rng.standard_normal((token_num, (H + 2 * Hkv) * D)).astype(np.float16)
    b = (rng.standard_normal((H + 2 * Hkv) * D) * 0.1).astype(np.float16) if bias else None
    pad = None
    if padded:
        tgt = np.concatenate([bi * seq_len + np.arange(n) for bi, n in enumerate(lengths)])
        pad = (tgt - np.arange(token_num)).astype(np.int32)
    else:
        lengths = [seq_len] * B
    return dict(qkv=qkv, bias=b, pad=pad, history=np.asarray(history, np.int32), input=np.asarray(lengths, np.int32), B=B,
                seq_len=seq_len, token_num=token_num, H=H, Hkv=Hkv)


def run_qkv(case, which, ref, rot_dim=D, base=10000.0, max_pos=2048, ntk=False, logn=False):
    from lmdeploy_b200 import turbomind as tm
    c = case
    q = torch.zeros((c["B"], c["H"], c["seq_len"], D), dtype=torch.float16, device="cuda")
    k = torch.zeros((c["B"], c["Hkv"], c["seq_len"], D), dtype=torch.float16, device="cuda")
    v = torch.zeros_like(k)
    qkv = dev(c["qkv"])
    b = None if c["bias"] is None else dev(c["bias"])
    pad = None if c["pad"] is None else dev(c["pad"])
    hist, inp = dev(c["history"]), dev(c["input"])
    args = (c["B"], c["seq_len"], c["token_num"], c["H"], c["Hkv"], D, rot_dim, base, max_pos, int(ntk), int(logn))
    if which == "reference":
        assert ref.ref_add_fused_qkv_bias_transpose(_p(q), _p(k), _p(v), _p(qkv), _p(b), _p(pad), _p(hist), _p(inp), *args,
                                                    None) == 0
    else:
        tm.invokeAddFusedQKVBiasTranspose(q, k, v, qkv, b, pad, hist, inp, *args)
        torch.cuda.synchronize()
        assert np.array_equal(qkv.cpu().numpy(), c["qkv"]), "the fused QKV buffer must not be modified"
    return q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy()


def _near_fp16(got, want, what, abs_tol=1e-6):
    """rotated values: fp32 math rounded once to fp16; libm and fused-multiply-add differences (1e-6 absolute where
    the two products cancel) may move a value by one fp16 step"""
    g, w = got.astype(np.float32), want.astype(np.float32)
    tol = np.maximum(np.abs(w) * 2.0 ** -10 * 1.01, abs_tol)
    bad = np.abs(g - w) > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} values differ by more than one fp16 step (+ {abs_tol})"
    assert (g != w).mean() < (0.02 if abs_tol <= 1e-6 else 0.2), f"{what}: {(g != w).mean():.4f} of the values differ"


QKV_CASES = [
    dict(lengths=[24, 7, 15], history=[0, 5, 100], seq_len=24, H=4, Hkv=2, kw={}),
    dict(lengths=[3, 1], history=[0, 9], seq_len=3, H=40, Hkv=40, kw={}, bias=False),                 # 120 heads: two passes of 64 per CTA
    # dynamic NTK + log-n at positions ~2000: the angle is position / powf(base', .), so one fp32 rounding of the
    # rescaled base moves it by ~2e-4 rad; against the CPU oracle (numpy's pow / log2) that is an absolute 4e-3
    dict(lengths=[16, 9], history=[60, 2000], seq_len=16, H=8, Hkv=1, kw=dict(max_pos=64, ntk=True, logn=True), abs_tol=4e-3),
    dict(lengths=[5, 5], history=[0, 3], seq_len=5, H=2, Hkv=2, kw=dict(rot_dim=64, base=1e6), padded=False),
    dict(lengths=[512, 300, 77, 512], history=[0, 5, 1000, 3000], seq_len=512, H=8, Hkv=8, kw={}, abs_tol=2e-3),      # 4 M values each
]


@pytest.mark.parametrize("idx", range(len(QKV_CASES)))
def test_qkv_bias_rope_transpose(ref, idx):
    cs = QKV_CASES[idx]
    case = qkv_case(cs["lengths"], cs["history"], cs["seq_len"], cs["H"], cs["Hkv"], 100 + idx, cs.get("bias", True),
                    cs.get("padded", True))
    ours = run_qkv(case, "ours", ref, **cs["kw"])
    kw = dict(cs["kw"])
    want = op.add_fused_qkv_bias_transpose(case["qkv"], case["bias"], case["pad"], case["history"], case["input"], case["B"],
                                           case["seq_len"], case["H"], case["Hkv"], kw.get("rot_dim", D), kw.get("base", 10000.0),
                                           kw.get("max_pos", 2048), kw.get("ntk", False), kw.get("logn", False))
    for name, g, w in zip("qkv", ours, want):
        _near_fp16(g, w, f"library vs oracle ({name})", cs.get("abs_tol", 1e-6))
    assert np.array_equal(ours[2].view(np.uint16), want[2].view(np.uint16)), "v is a copy (+ fp16 bias add): bit exact"
    if ref is not None:
        theirs = run_qkv(case, "reference", ref, **cs["kw"])
        for name, g, w in zip("qkv", ours, theirs):
            assert np.array_equal(g.view(np.uint16), w.view(np.uint16)), f"library != reference kernel ({name})"


def cache_case(B, Hkv, layers, layer, S_max, max_q, q_len, hist, seed, int8):
    rng = np.random.default_rng(seed)
    k_src = rng.standard_normal((B, Hkv, max_q, D)).astype(np.float16)
    v_src = (rng.standard_normal((B, Hkv, max_q, D)) * 2 + 0.5).astype(np.float16)
    dt = np.int8 if int8 else np.float16
    fill = (lambda: rng.integers(-128, 128, size=(layers * Hkv, S_max, D)).astype(np.int8)) if int8 else \
        (lambda: rng.standard_normal((layers * Hkv, S_max, D)).astype(np.float16))
    kc, vc = [fill() for _ in range(B)], [fill() for _ in range(B)]
    scale = np.asarray([0.031, 0.11, 0.067, -0.4], np.float32) if int8 else None
    return dict(B=B, Hkv=Hkv, layer=layer, S_max=S_max, max_q=max_q, q_len=np.asarray(q_len, np.int32),
                hist=np.asarray(hist, np.int32), k_src=k_src, v_src=v_src, kc=kc, vc=vc, scale=scale, dtype=dt)


def _cache_tensors(c):
    kd = [torch.from_numpy(a.copy()).reshape(-1).cuda() for a in c["kc"]]
    vd = [torch.from_numpy(a.copy()).reshape(-1).cuda() for a in c["vc"]]
    kp = torch.tensor([t.data_ptr() for t in kd], dtype=torch.int64, device="cuda")
    vp = torch.tensor([t.data_ptr() for t in vd], dtype=torch.int64, device="cuda")
    return kd, vd, kp, vp


def run_extend(c, which, ref):
    from lmdeploy_b200 import turbomind as tm
    kd, vd, kp, vp = _cache_tensors(c)
    ks, vs, ql, hl = dev(c["k_src"]), dev(c["v_src"]), dev(c["q_len"]), dev(c["hist"])
    off = c["layer"] * c["Hkv"] * c["S_max"] * D
    quant = 4 if c["scale"] is not None else 0
    if which == "reference":
        sc = None if c["scale"] is None else (C.c_float * 4)(*[float(x) for x in c["scale"]])
        assert ref.ref_extend_kv_cache(_p(kp), _p(vp), off, _p(ks), _p(vs), c["B"], _p(ql), c["max_q"], _p(hl), c["S_max"], D,
                                       c["Hkv"], None, quant, sc) == 0
    else:
        tm.invokeExtendKVCache(kp, vp, off, ks, vs, c["B"], ql, c["max_q"], hl, c["S_max"], D, c["Hkv"], None, quant, c["scale"])
        torch.cuda.synchronize()
    shape = c["kc"][0].shape
    return [t.cpu().numpy().reshape(shape) for t in kd], [t.cpu().numpy().reshape(shape) for t in vd]


@pytest.mark.parametrize("int8", [False, True])
def test_extend_kv_cache(ref, int8):
    c = cache_case(B=3, Hkv=2, layers=3, layer=1, S_max=48, max_q=20, q_len=[20, 1, 0], hist=[0, 47, 13], seed=7, int8=int8)
    ours_k, ours_v = run_extend(c, "ours", ref)
    want_k, want_v = [a.copy() for a in c["kc"]], [a.copy() for a in c["vc"]]
    op.extend_kv_cache(want_k, want_v, c["layer"] * c["Hkv"], c["k_src"], c["v_src"], c["q_len"], c["hist"], c["scale"])
    for g, w in zip(ours_k + ours_v, want_k + want_v):
        assert np.array_equal(g, w), "library != oracle (rows outside the appended range must stay untouched)"
    if ref is not None:
        ref_k, ref_v = run_extend(c, "reference", ref)
        for g, w in zip(ours_k + ours_v, ref_k + ref_v):
            assert np.array_equal(g, w), "library != reference kernel"


def run_transpose(c, key_len, max_kv, n_rep, which, ref):
    from lmdeploy_b200 import turbomind as tm
    kd, vd, kp, vp = _cache_tensors(c)
    H = c["Hkv"] * n_rep
    kt = torch.zeros((c["B"], H, max_kv, D), dtype=torch.float16, device="cuda")
    vt = torch.zeros_like(kt)
    kl = dev(np.asarray(key_len, np.int32))
    off = c["layer"] * c["Hkv"] * c["S_max"] * D
    quant = 4 if c["scale"] is not None else 0
    if which == "reference":
        sc = None if c["scale"] is None else (C.c_float * 4)(*[float(x) for x in c["scale"]])
        assert ref.ref_transpose_kv_cache(_p(kt), _p(vt), _p(kp), _p(vp), off, c["B"], _p(kl), max_kv, c["S_max"], D, H, n_rep,
                                          None, quant, sc) == 0
    else:
        tm.invokeTransposeKVCache(kt, vt, kp, vp, off, c["B"], kl, max_kv, c["S_max"], D, H, n_rep, None, quant, c["scale"])
        torch.cuda.synchronize()
    return kt.cpu().numpy(), vt.cpu().numpy()


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("n_rep", [1, 4])
def test_transpose_kv_cache(ref, int8, n_rep):
    c = cache_case(B=3, Hkv=2, layers=2, layer=1, S_max=48, max_q=1, q_len=[0] * 3, hist=[0] * 3, seed=11, int8=int8)
    key_len, max_kv = [48, 5, 0], 48
    ours = run_transpose(c, key_len, max_kv, n_rep, "ours", ref)
    want = op.transpose_kv_cache(c["kc"], c["vc"], c["layer"] * c["Hkv"], key_len, max_kv, c["Hkv"] * n_rep, n_rep, c["scale"])
    for g, w in zip(ours, want):
        assert np.array_equal(g.view(np.uint16), w.view(np.uint16)), "library != oracle"
    if ref is not None:
        theirs = run_transpose(c, key_len, max_kv, n_rep, "reference", ref)
        for g, w in zip(ours, theirs):
            assert np.array_equal(g.view(np.uint16), w.view(np.uint16)), "library != reference kernel"


@pytest.mark.parametrize("int8", [False, True])
def test_extend_then_transpose_round_trip_at_full_size(int8):
    """Llama-2-7B prefill shape (8 x 2048 tokens, 32 heads): what extend writes, transpose reads back — exactly for an
    fp16 cache, within half a quantisation step for an int8 cache."""
    from lmdeploy_b200 import turbomind as tm
    B, H, S, S_max = 8, 32, 2048, 2048 + 64
    g = torch.Generator(device="cuda").manual_seed(5)
    k_src = torch.randn((B, H, S, D), device="cuda", dtype=torch.float16, generator=g)
    v_src = torch.randn((B, H, S, D), device="cuda", dtype=torch.float16, generator=g)
    lens = torch.tensor([2048, 1, 777, 2048, 1024, 5, 2000, 64], dtype=torch.int32, device="cuda")
    hist = torch.tensor([0, 64, 3, 64, 0, 1, 7, 0], dtype=torch.int32, device="cuda")
    esz = 1 if int8 else 2
    caches = [torch.zeros(H * S_max * D * esz, dtype=torch.uint8, device="cuda") for _ in range(2 * B)]
    kp = torch.tensor([t.data_ptr() for t in caches[:B]], dtype=torch.int64, device="cuda")
    vp = torch.tensor([t.data_ptr() for t in caches[B:]], dtype=torch.int64, device="cuda")
    scale = [6.5 / 127, 0.0, 6.5 / 127, 0.0] if int8 else None
    quant = 4 if int8 else 0
    tm.invokeExtendKVCache(kp, vp, 0, k_src, v_src, B, lens, S, hist, S_max, D, H, None, quant, scale)
    total = lens + hist
    max_kv = int(total.max())
    kt = torch.zeros((B, H, max_kv, D), dtype=torch.float16, device="cuda")
    vt = torch.zeros_like(kt)
    tm.invokeTransposeKVCache(kt, vt, kp, vp, 0, B, total, max_kv, S_max, D, H, 1, None, quant, scale)
    torch.cuda.synchronize()
    for b in range(B):
        n, h0 = int(lens[b]), int(hist[b])
        for src, got in ((k_src, kt), (v_src, vt)):
            a, o = src[b, :, :n], got[b, :, h0:h0 + n]
            if int8:
                assert float((a.float() - o.float()).abs().max()) <= 0.5 * scale[0] + 2e-3
            else:
                assert torch.equal(a, o)
            assert float(got[b, :, :h0].abs().max()) == 0 if h0 else True   # never-written cache rows read back as zeros


def test_argument_checks():
    from lmdeploy_b200 import lib as l
    x = torch.zeros(4096, dtype=torch.float16, device="cuda")
    i32 = torch.zeros(4, dtype=torch.int32, device="cuda")
    p, ip = C.c_void_p(x.data_ptr()), C.c_void_p(i32.data_ptr())
    f = l.lib.tm_add_fused_qkv_bias_transpose
    assert f(None, p, p, p, None, None, ip, ip, 1, 1, 1, 1, 1, D, D, 1e4, 2048, 0, 0, None) == l.TM_ERR_INVALID_ARG
    assert f(p, p, p, p, None, None, ip, ip, 1, 1, 1, 1, 1, 64, 64, 1e4, 2048, 0, 0, None) == l.TM_ERR_UNSUPPORTED
    assert f(p, p, p, p, None, None, ip, ip, 1, 1, 1, 1, 1, D, 0, 1e4, 2048, 0, 0, None) == l.TM_ERR_INVALID_ARG
    assert f(p, p, p, p, None, None, ip, ip, 1, 1, 0, 1, 1, D, D, 1e4, 2048, 0, 0, None) == l.TM_OK          # no tokens
    e = l.lib.tm_extend_kv_cache
    assert e(ip, ip, 0, p, p, 1, ip, 1, ip, 16, D, 1, None, 4, None) == l.TM_ERR_INVALID_ARG                     # int8 needs scales
    assert e(ip, ip, 8, p, p, 1, ip, 1, ip, 16, D, 1, None, 0, None) == l.TM_ERR_INVALID_ARG                     # offset % 16
    assert e(ip, ip, 0, p, p, 0, ip, 1, ip, 16, D, 1, None, 0, None) == l.TM_OK
    t = l.lib.tm_transpose_kv_cache
    assert t(p, p, ip, ip, 0, 1, ip, 1, 16, D, 3, 2, None, 0, None) == l.TM_ERR_INVALID_ARG                      # 3 heads, groups of 2


# ------------------------------------------------------------------------------- context attention

def attention_case(q_lens, hist, H, Hkv, S_max, layers, layer, seed, int8):
    rng = np.random.default_rng(seed)
    B = len(q_lens)
    max_q = max(q_lens)
    q = rng.standard_normal((B, H, max_q, D)).astype(np.float16)
    if int8:
        kc = [rng.integers(-128, 128, size=(layers * Hkv, S_max, D)).astype(np.int8) for _ in range(B)]
        vc = [rng.integers(-128, 128, size=(layers * Hkv, S_max, D)).astype(np.int8) for _ in range(B)]
        scale = np.asarray([0.011, 0.05, 0.013, -0.1], np.float32)
    else:
        kc = [rng.standard_normal((layers * Hkv, S_max, D)).astype(np.float16) for _ in range(B)]
        vc = [rng.standard_normal((layers * Hkv, S_max, D)).astype(np.float16) for _ in range(B)]
        scale = None
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    ctx = (np.asarray(q_lens) + np.asarray(hist)).astype(np.int32)
    return dict(q=q, kc=kc, vc=vc, scale=scale, cu=cu, ctx=ctx, B=B, H=H, Hkv=Hkv, S_max=S_max, layer=layer, max_q=max_q)


def run_attention(c):
    from lmdeploy_b200 import turbomind as tm
    kd, vd, kp, vp = _cache_tensors(c)
    out = torch.zeros((int(c["cu"][-1]), c["H"] * D), dtype=torch.float16, device="cuda")
    tm.fusedMultiHeadAttention(out, dev(c["q"]), kp, vp, c["layer"] * c["Hkv"] * c["S_max"] * D, dev(c["cu"]), dev(c["ctx"]),
                               c["B"], c["max_q"], c["S_max"], c["H"], c["Hkv"], D, 4 if c["scale"] is not None else 0, c["scale"])
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("q_lens,hist,H,Hkv", [
    ([1, 64, 65], [0, 0, 0], 2, 2),             # single token, exactly one tile, one row into the second tile
    ([130, 17, 200], [0, 100, 37], 4, 1),       # history, ragged lengths, grouped-query heads
    ([300], [211], 8, 2),                       # many key tiles, the diagonal in the middle of a tile
])
def test_context_attention_matches_oracle(int8, q_lens, hist, H, Hkv):
    from tests.helpers import assert_close
    S_max = max(a + b for a, b in zip(q_lens, hist)) + 3
    c = attention_case(q_lens, hist, H, Hkv, S_max, layers=2, layer=1, seed=23, int8=int8)
    got = run_attention(c)
    want = op.context_attention(c["q"], c["kc"], c["vc"], c["layer"] * c["Hkv"], c["cu"], c["ctx"], H, Hkv, c["scale"])
    assert_close(got, want, f"context attention (int8={int8})")   # max-abs 2e-2, mean-rel 1e-3: the fp16 bar of the path


@pytest.mark.parametrize("int8", [False, True])
def test_context_attention_against_the_reference_unfused_route(ref, int8):
    """The reference's own kernels for everything but the two batched GEMMs (which it hands to cuBLAS, as torch.matmul does
    here): invokeTransposeKVCache -> q k^T (fp16 out) -> invokeCreateCausalMasks + invokeMaskedSoftmax -> p v
    (src/turbomind/models/llama/LlamaContextAttentionLayer.cc:316-420).  Pins the CPU oracle and the kernel to it."""
    from tests.helpers import assert_close
    if ref is None:
        pytest.skip("oracle/_ref/libtm_ref.so not built")
    q_lens, hist, H, Hkv = [130, 17, 200], [0, 100, 37], 4, 2
    S_max = 240
    c = attention_case(q_lens, hist, H, Hkv, S_max, layers=2, layer=1, seed=29, int8=int8)
    B, max_q, max_k = c["B"], c["max_q"], int(c["ctx"].max())
    # --- the reference route
    kd, vd, kp, vp = _cache_tensors(c)
    kt = torch.zeros((B, H, max_k, D), dtype=torch.float16, device="cuda")
    vt = torch.zeros_like(kt)
    ctx_d, ql_d = dev(c["ctx"]), dev(np.asarray(q_lens, np.int32))
    sc = None if c["scale"] is None else (C.c_float * 4)(*[float(x) for x in c["scale"]])
    assert ref.ref_transpose_kv_cache(_p(kt), _p(vt), _p(kp), _p(vp), c["layer"] * Hkv * S_max * D, B, _p(ctx_d), max_k, S_max, D,
                                      H, H // Hkv, None, 4 if int8 else 0, sc) == 0
    qd = dev(c["q"])
    qk = torch.matmul(qd, kt.transpose(2, 3)).contiguous()                      # half [B, H, max_q, max_k]
    mask = torch.zeros((B, max_q, max_k), dtype=torch.float16, device="cuda")
    assert ref.ref_create_causal_masks(_p(mask), _p(ql_d), _p(ctx_d), max_q, max_k, B, None) == 0
    assert ref.ref_masked_softmax(_p(qk), _p(qk), _p(mask), B, max_q, max_k, H, 1.0 / np.sqrt(D), None) == 0
    o = torch.matmul(qk, vt)                                                    # [B, H, max_q, D]
    theirs = np.concatenate([o[b, :, :n].transpose(0, 1).reshape(n, H * D).cpu().numpy() for b, n in enumerate(q_lens)])
    # --- the oracle and the kernel
    want = op.context_attention(c["q"], c["kc"], c["vc"], c["layer"] * Hkv, c["cu"], c["ctx"], H, Hkv, c["scale"])
    got = run_attention(c)
    assert_close(want, theirs, f"CPU oracle vs reference unfused route (int8={int8})")
    assert_close(got, theirs, f"kernel vs reference unfused route (int8={int8})")


def test_context_attention_properties_at_full_size():
    """Llama-2-7B prefill shape (4 x 2048 tokens, 32 heads).  (1) With every value row equal to one vector the output is
    that vector whatever the scores are.  (2) Causality: changing the keys / values of the LAST position changes no
    output row except the last one of each sequence."""
    from lmdeploy_b200 import turbomind as tm
    B, H, S = 4, 32, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn((B, H, S, D), device="cuda", dtype=torch.float16, generator=g)
    kc = [torch.randn((H, S, D), device="cuda", dtype=torch.float16, generator=g) for _ in range(B)]
    vrow = torch.randn((H, 1, D), device="cuda", dtype=torch.float16, generator=g)
    vc = [vrow.expand(H, S, D).contiguous() for _ in range(B)]
    kp = torch.tensor([t.data_ptr() for t in kc], dtype=torch.int64, device="cuda")
    vp = torch.tensor([t.data_ptr() for t in vc], dtype=torch.int64, device="cuda")
    lens = [2048, 1000, 1, 2047]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    ctx = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = torch.zeros((sum(lens), H * D), dtype=torch.float16, device="cuda")
    tm.fusedMultiHeadAttention(out, q, kp, vp, 0, cu, ctx, B, S, S, H, H, D)
    torch.cuda.synchronize()
    want = vrow.reshape(1, H * D).float()
    assert float((out.float() - want).abs().max()) <= 2e-3 * float(want.abs().max()) + 1e-3
    # causality
    vc2 = [torch.randn((H, S, D), device="cuda", dtype=torch.float16, generator=g) for _ in range(B)]
    vp2 = torch.tensor([t.data_ptr() for t in vc2], dtype=torch.int64, device="cuda")
    a = torch.zeros_like(out)
    tm.fusedMultiHeadAttention(a, q, kp, vp2, 0, cu, ctx, B, S, S, H, H, D)
    for b, n in enumerate(lens):
        kc[b][:, n - 1] += 1.0
        vc2[b][:, n - 1] -= 3.0
    b2 = torch.zeros_like(out)
    tm.fusedMultiHeadAttention(b2, q, kp, vp2, 0, cu, ctx, B, S, S, H, H, D)
    torch.cuda.synchronize()
    last = torch.zeros(sum(lens), dtype=torch.bool, device="cuda")
    last[(cu[1:] - 1).long()] = True
    assert torch.equal(a[~last], b2[~last])
    assert not torch.equal(a[last], b2[last])


def test_writers_never_leave_their_buffers():
    """More new tokens than a cache head has rows left: the surplus rows are dropped, the next head's rows stay as they
    were; a padding offset that points past the batch writes nothing."""
    from lmdeploy_b200 import turbomind as tm
    c = cache_case(B=1, Hkv=2, layers=1, layer=0, S_max=16, max_q=8, q_len=[8], hist=[12], seed=31, int8=False)
    kd, vd, kp, vp = _cache_tensors(c)
    tm.invokeExtendKVCache(kp, vp, 0, dev(c["k_src"]), dev(c["v_src"]), 1, dev(c["q_len"]), 8, dev(c["hist"]), 16, D, 2)
    torch.cuda.synchronize()
    got = kd[0].cpu().numpy().reshape(2, 16, D)
    assert np.array_equal(got[:, 12:], c["k_src"][0, :, :4]) and np.array_equal(got[:, :12], c["kc"][0][:, :12])
    case = qkv_case([4], [0], 4, 2, 1, 33)
    case["pad"] = np.asarray([0, 0, 100, -50], np.int32)          # tokens 2 and 3 point outside [1, 4]
    q, k, v = run_qkv(case, "ours", None)
    assert q[0, :, :2].any() and not q[0, :, 2:].any() and not k[0, :, 2:].any() and not v[0, :, 2:].any()
