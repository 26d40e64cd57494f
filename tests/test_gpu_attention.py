"""GPU: decode attention (fused RoPE + KV append + split-KV softmax) and RMSNorm through the C ABI
against the numpy oracle.  Tolerance for attention outputs: max-abs 2e-2, mean-rel 1e-3."""
import math

import numpy as np
import pytest
import torch

from oracle import attention as oa
from oracle import norm as onorm
from tests.helpers import assert_close, dev

pytestmark = pytest.mark.gpu


def make_case(B, H, Hkv, S_max, lengths, seed, int8, bias=False, std=1.0):
    rng = np.random.default_rng(seed)
    D = 128
    qkv = (rng.standard_normal((B, (H + 2 * Hkv) * D)) * std).astype(np.float16)
    kq = None
    kc, vc = [], []
    kf = [(rng.standard_normal((Hkv, S_max, D))).astype(np.float16) for _ in range(B)]
    vf = [(rng.standard_normal((Hkv, S_max, D))).astype(np.float16) for _ in range(B)]
    if int8:
        ks = float(max(np.abs(k).max() for k in kf)) / 127.0
        vs = float(max(np.abs(v).max() for v in vf)) / 127.0
        kq = oa.KvQuant(ks, 0.0, vs, 0.0)
        kc = [oa.quant_int8(k, ks, 0.0) for k in kf]
        vc = [oa.quant_int8(v, vs, 0.0) for v in vf]
    else:
        kc, vc = kf, vf
    b = (rng.standard_normal(((H + 2 * Hkv) * D)) * 0.1).astype(np.float16) if bias else None
    return dict(B=B, H=H, Hkv=Hkv, S_max=S_max, lengths=np.asarray(lengths, np.int32), qkv=qkv, kc=kc, vc=vc, kq=kq,
                bias=b)


def run_gpu(case, finished=None, positions=None, chunk_env=None, layer_offset_tokens=0):
    from lmdeploy_b200 import turbomind as tm
    B, H, Hkv, S_max = case["B"], case["H"], case["Hkv"], case["S_max"]
    D = 128
    int8 = case["kq"] is not None
    # per-sequence slabs with room for a leading "other layer" so that the element offset is exercised
    pad = layer_offset_tokens * Hkv * D
    kd = [torch.cat([torch.zeros(pad, dtype=torch.from_numpy(k).dtype), torch.from_numpy(k).reshape(-1)]).cuda()
          for k in case["kc"]]
    vd = [torch.cat([torch.zeros(pad, dtype=torch.from_numpy(v).dtype), torch.from_numpy(v).reshape(-1)]).cuda()
          for v in case["vc"]]
    kp = torch.tensor([t.data_ptr() for t in kd], dtype=torch.int64, device="cuda")
    vp = torch.tensor([t.data_ptr() for t in vd], dtype=torch.int64, device="cuda")
    qkv = dev(case["qkv"])
    out = torch.full((B, H * D), 555.0, dtype=torch.float16, device="cuda")
    lengths = dev(case["lengths"])
    timestep = int(case["lengths"].max())
    pos = case["lengths"] if positions is None else np.asarray(positions, np.int32)
    timestep = max(timestep, int(pos.max()))
    padding = dev((timestep - pos).astype(np.int32))
    p = tm.Masked_multihead_attention_params(
        out=out, q=qkv, k=qkv[:, H * D:], v=qkv[:, (H + Hkv) * D:], stride=(H + 2 * Hkv) * D, batch_size=B,
        memory_max_len=S_max, num_heads=H, num_kv_heads=Hkv, timestep=timestep, inv_sqrt_dh=1.0 / math.sqrt(D),
        total_padding_tokens=padding, length_per_sample=lengths, k_cache_per_sample=kp, v_cache_per_sample=vp,
        kv_cache_per_sample_offset=pad, finished=None if finished is None else dev(np.asarray(finished, np.bool_)))
    if case["bias"] is not None:
        bias = dev(case["bias"])
        p.q_bias, p.k_bias, p.v_bias = bias, bias[H * D:], bias[(H + Hkv) * D:]
    if int8:
        p.int8_mode = tm.QUANT_POLICY_CACHE_KV_INT8
        q = case["kq"]
        p.attention_k_scale, p.attention_k_zp, p.attention_v_scale, p.attention_v_zp = q.k_scale, q.k_zp, q.v_scale, q.v_zp
    from lmdeploy_b200 import lib as l
    tm.masked_multihead_attention(p)
    l.default_handle(torch.cuda.current_device()).check_device_status(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    kout = [t[pad:].cpu().numpy().reshape(Hkv, S_max, D) for t in kd]
    vout = [t[pad:].cpu().numpy().reshape(Hkv, S_max, D) for t in vd]
    return out.cpu().numpy(), kout, vout


def run_oracle(case, finished=None, positions=None):
    kc = [k.copy() for k in case["kc"]]
    vc = [v.copy() for v in case["vc"]]
    out = np.full((case["B"], case["H"] * 128), 555.0, np.float16)
    oa.mmha_decode(case["qkv"], kc, vc, case["lengths"], case["H"], case["Hkv"], 128, case["S_max"], finished=finished,
                   positions=positions, qkv_bias=case["bias"], kv_quant=case["kq"], out=out)
    return out, kc, vc


def check_cache(got, want, int8, lengths, S_max, finished=None):
    for b, (g, w) in enumerate(zip(got, want)):
        slot = int(lengths[b]) % S_max
        mask = np.ones(S_max, bool)
        mask[slot] = False
        assert np.array_equal(g[:, mask], w[:, mask]), "touched cache rows other than the new token's"
        if finished is not None and finished[b]:
            assert np.array_equal(g[:, slot], w[:, slot])
            continue
        if int8:
            d = np.abs(g[:, slot].astype(np.int32) - w[:, slot].astype(np.int32))
            assert d.max() <= 1 and (d != 0).mean() < 0.02, "int8 row differs by more than 1 LSB / too often"
        else:
            d = np.abs(g[:, slot].astype(np.float32) - w[:, slot].astype(np.float32))
            # RoPE mixes the two elements of a pair, so the error scale is the pair's magnitude (|x| ~ 1
            # here, angle error ~ position * 1e-7), not the magnitude of the single rotated element
            assert (d <= 2.0 ** -9 * np.abs(w[:, slot].astype(np.float32)) + 2e-3).all(), "appended fp16 row is off"


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("H,Hkv", [(4, 4), (8, 1), (16, 2), (3, 1)])
def test_mha_and_gqa_small(int8, H, Hkv):
    lengths = [0, 1, 15, 16, 17, 63, 64, 65, 200, 257, 511]
    case = make_case(len(lengths), H, Hkv, 640, lengths, 1, int8)
    out, kc, vc = run_gpu(case)
    want, kw, vw = run_oracle(case)
    assert_close(out, want, f"mmha H={H} Hkv={Hkv} int8={int8}")
    check_cache(kc, kw, int8, case["lengths"], 640)
    check_cache(vc, vw, int8, case["lengths"], 640)


@pytest.mark.parametrize("int8", [False, True])
def test_bias_finished_positions_and_offset(int8):
    lengths = [5, 130, 64, 300]
    case = make_case(4, 8, 2, 512, lengths, 2, int8, bias=True)
    finished = [False, True, False, False]
    positions = [5, 130, 70, 300]          # one sequence whose RoPE position differs from its cached length
    out, kc, vc = run_gpu(case, finished, positions, layer_offset_tokens=3)
    want, kw, vw = run_oracle(case, finished, positions)
    assert (out[1] == 555.0).all(), "a finished sequence must not be written"
    assert_close(out, want, f"mmha bias/finished int8={int8}")
    check_cache(kc, kw, int8, case["lengths"], 512, finished)
    check_cache(vc, vw, int8, case["lengths"], 512, finished)


@pytest.mark.parametrize("int8", [False, True])
def test_ring_buffer_wraparound(int8):
    S_max = 128
    lengths = [127, 128, 129, 300, 1000]
    case = make_case(5, 4, 2, S_max, lengths, 3, int8)
    out, kc, vc = run_gpu(case)
    want, kw, vw = run_oracle(case)
    assert_close(out, want, f"mmha ring int8={int8}")
    check_cache(kc, kw, int8, case["lengths"], S_max)


@pytest.mark.parametrize("int8", [False, True])
def test_benchmark_shape_long_sequences(int8):
    """32 heads of 128, lengths up to 4096 (a slice of the batch-64 configuration)."""
    rng = np.random.default_rng(7)
    lengths = [4096, 128] + list(rng.integers(128, 4097, size=4))
    case = make_case(len(lengths), 32, 32, 4224, lengths, 4, int8)
    out, kc, vc = run_gpu(case)
    want, kw, vw = run_oracle(case)
    assert_close(out, want, f"mmha config-2 slice int8={int8}")
    check_cache(kc, kw, int8, case["lengths"], 4224)


@pytest.mark.parametrize("int8", [False, True])
@pytest.mark.parametrize("warps", [1, 2, 4])
@pytest.mark.parametrize("chunk", [0, 64, 192])
def test_every_cta_shape_and_split_size(int8, warps, chunk):
    """The kernel exists with 1, 2 and 4 warps per CTA and splits a sequence into chunks; which one
    runs is a tuning decision, so every combination is forced here (MHA, GQA, bias, ragged lengths)."""
    from lmdeploy_b200 import lib as l
    h = l.default_handle(torch.cuda.current_device())
    lengths = [0, 1, 17, 64, 65, 200, 511, 600]
    case = make_case(len(lengths), 16, 2, 640, lengths, 11, int8, bias=True)
    try:
        h.set_option("mmha_warps", warps)
        h.set_option("mmha_chunk", chunk)
        out, kc, vc = run_gpu(case)
    finally:
        h.set_option("mmha_warps", 0)
        h.set_option("mmha_chunk", 0)
    want, kw, vw = run_oracle(case)
    assert_close(out, want, f"mmha warps={warps} chunk={chunk} int8={int8}")
    check_cache(kc, kw, int8, case["lengths"], 640)
    check_cache(vc, vw, int8, case["lengths"], 640)


def test_split_merge_is_deterministic_and_tickets_reset():
    case = make_case(3, 8, 8, 2048, [2000, 700, 64], 5, True)
    a, _, _ = run_gpu(case)
    for _ in range(3):
        b, _, _ = run_gpu(case)
        assert np.array_equal(a.view(np.uint16), b.view(np.uint16))


def test_mmha_error_codes():
    from lmdeploy_b200 import lib as l
    h = l.default_handle(torch.cuda.current_device())
    c = l.TmMmhaParams()
    assert l.lib.tm_mmha_decode(h.ptr, c, None) == l.TM_ERR_INVALID_ARG
    assert l.lib.tm_mmha_decode(None, c, None) == l.TM_ERR_INVALID_ARG
    buf = torch.zeros(4096, dtype=torch.float16, device="cuda")
    ptrs = torch.zeros(1, dtype=torch.int64, device="cuda")
    ln = torch.zeros(1, dtype=torch.int32, device="cuda")
    c.out = c.q = buf.data_ptr()
    c.k, c.v = buf.data_ptr() + 256, buf.data_ptr() + 512
    c.length_per_sample, c.k_cache_per_sample, c.v_cache_per_sample = ln.data_ptr(), ptrs.data_ptr(), ptrs.data_ptr()
    c.batch_size, c.num_heads, c.num_kv_heads, c.memory_max_len, c.stride = 1, 1, 1, 16, 384
    c.hidden_size_per_head = 64
    assert l.lib.tm_mmha_decode(h.ptr, c, None) == l.TM_ERR_UNSUPPORTED      # only head dim 128 is built
    c.hidden_size_per_head, c.num_heads, c.num_kv_heads = 128, 3, 2
    assert l.lib.tm_mmha_decode(h.ptr, c, None) == l.TM_ERR_UNSUPPORTED


@pytest.mark.parametrize("m,n", [(1, 4096), (64, 4096), (5, 8192), (3, 128), (2, 11008)])
def test_rmsnorm_and_fused_residual(m, n):
    from lmdeploy_b200 import turbomind as tm
    rng = np.random.default_rng(m + n)
    x = rng.standard_normal((m, n)).astype(np.float16)
    r = rng.standard_normal((m, n)).astype(np.float16)
    w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float16)
    b = (0.1 * rng.standard_normal(n)).astype(np.float16)
    out = torch.empty(m, n, dtype=torch.float16, device="cuda")
    tm.invokeRootMeanSquareNorm(out, dev(x), dev(w), 1e-6, m, n)
    assert_close(out.cpu().numpy(), onorm.rmsnorm(x, w, 1e-6), "rmsnorm", max_abs=4e-3)
    for bias in (None, b):
        rd, xd = dev(r), dev(x)
        tm.invokeFusedAddBiasResidualRMSNorm(rd, xd, None if bias is None else dev(bias), dev(w), 1e-6, m, n)
        r_want, o_want = onorm.add_residual_rmsnorm(r, x, bias, w, 1e-6)
        assert np.array_equal(rd.cpu().numpy().view(np.uint16), r_want.view(np.uint16)), "residual must be bit exact"
        assert_close(xd.cpu().numpy(), o_want, "fused add + rmsnorm", max_abs=4e-3)
