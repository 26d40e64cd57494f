"""GPU: token sampling (tm_sample_topk, tm_sample_topp) and the lm-head kernel (tm_lm_head_f16).

Sampling is checked two ways: against oracle/sampling.py with caller-supplied uniform numbers (draws that sit on an
interval boundary are left out), and step by step against the reference's own penalty and top-k sampling kernels
compiled unmodified into oracle/_ref, both sides drawing from curand states seeded alike: ids identical and the
rewritten logits bit-identical over several steps with the history growing.
The lm-head is compared with an fp32 matmul of the same fp16 operands (tolerance: fp32 accumulation order only).
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import sampling as osamp

pytestmark = pytest.mark.gpu

_REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libtm_ref.so")


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _params(l, logits, ids, **kw):
    p = l.TmSamplingParams()
    p.logits, p.ld, p.vocab_size, p.batch_size = logits.data_ptr(), logits.stride(0), kw.pop("vocab", logits.shape[1]), logits.shape[0]
    p.ids = ids.data_ptr()
    p.max_top_k, p.top_p = 1, 1.0
    for k, v in kw.items():
        setattr(p, k, v.data_ptr() if isinstance(v, torch.Tensor) else v)
    return p


@pytest.mark.parametrize("B,V,ld", [(7, 32000, 32000), (3, 1000, 1024), (64, 32000, 32000), (2, 50001, 50008)])
def test_sampling_matches_oracle(B, V, ld):
    from lmdeploy_b200 import lib as l
    rng = np.random.default_rng(B * 1000 + V)
    h = l.default_handle(torch.cuda.current_device())
    x = (rng.standard_normal((B, ld)) * 3).astype(np.float32)
    step, max_in = 12, 6
    out_ids = rng.integers(0, V, size=(step, B)).astype(np.int32)
    out_ids[3] = out_ids[2]                                   # repeated tokens are penalised once
    in_len = rng.integers(1, max_in + 1, size=B).astype(np.int32)
    temps = rng.uniform(0.3, 1.5, B).astype(np.float32)
    reps = rng.uniform(1.0, 1.3, B).astype(np.float32)
    min_len = rng.integers(0, 12, B).astype(np.int32)
    seq_len = np.full(B, step - 1, np.int32)
    end_ids = rng.integers(0, V, B).astype(np.int32)
    top_ks = rng.integers(1, 65, B).astype(np.int32)
    top_ks[0] = 1
    top_ps = rng.uniform(0.3, 1.0, B).astype(np.float32)
    us = rng.uniform(1e-3, 1.0, B).astype(np.float32)
    finished = np.zeros(B, np.uint8)
    finished[B // 2] = 1
    d = {k: torch.from_numpy(v).cuda() for k, v in dict(x=x, out_ids=out_ids, in_len=in_len, temps=temps, reps=reps, min_len=min_len,
                                                         seq_len=seq_len, end_ids=end_ids, top_ks=top_ks, top_ps=top_ps, us=us,
                                                         finished=finished).items()}
    ids = torch.full((B,), -7, dtype=torch.int32, device="cuda")
    p = _params(l, d["x"], ids, vocab=V, output_ids=d["out_ids"], step=step, input_lengths=d["in_len"], max_input_length=max_in,
                temperatures=d["temps"], repetition_penalties=d["reps"], min_lengths=d["min_len"], sequence_lengths=d["seq_len"],
                end_ids=d["end_ids"], top_ks=d["top_ks"], top_ps=d["top_ps"], uniforms=d["us"], finished=d["finished"])
    assert l.lib.tm_sample_topk(h.ptr, C.byref(p), _stream()) == l.TM_OK
    torch.cuda.synchronize()
    want_x = osamp.apply_penalties(x[:, :V], temps, reps, out_ids, in_len, max_in, min_len, end_ids, seq_len)
    want_ids, margins = osamp.sample(want_x, top_ks, top_ps, us, finished, end_ids)
    got_x = d["x"].cpu().numpy()
    live = finished == 0
    np.testing.assert_allclose(got_x[live][:, :V], want_x[live], rtol=2e-6, atol=0)
    np.testing.assert_array_equal(got_x[~live], x[~live])            # finished rows are left alone
    if ld > V:
        np.testing.assert_array_equal(got_x[:, V:], x[:, V:])
    got = ids.cpu().numpy()
    sure = (margins > 1e-5) | (finished == 1)
    assert sure.sum() >= B - 1
    np.testing.assert_array_equal(got[sure], want_ids[sure])
    assert got[0] == int(np.argmax(want_x[0])) or finished[0]         # top_k = 1 is greedy


def test_sampling_matches_reference_kernels_over_steps():
    from lmdeploy_b200 import lib as l
    if not os.path.exists(_REF):
        pytest.skip("oracle/_ref/libtm_ref.so not built")
    ref = C.CDLL(_REF)
    if not hasattr(ref, "ref_batch_topk_sampling"):
        pytest.skip("oracle/_ref/libtm_ref.so predates the sampling entry layer")
    ref.ref_curand_state_bytes.restype = C.c_size_t
    assert ref.ref_curand_state_bytes() == l.lib.tm_sampling_rng_state_bytes()
    B, V, steps, max_in = 16, 32000, 6, 4
    h = l.default_handle(torch.cuda.current_device())
    g = torch.Generator(device="cuda").manual_seed(17)
    seeds = torch.arange(100, 100 + B, dtype=torch.int64, device="cuda")
    nbytes = int(l.lib.tm_sampling_rng_state_bytes())
    st_a = torch.zeros(B * nbytes, dtype=torch.uint8, device="cuda")
    st_b = torch.zeros_like(st_a)
    assert l.lib.tm_sampling_rng_init(st_a.data_ptr(), B, seeds.data_ptr(), 0, _stream()) == l.TM_OK
    vp = C.c_void_p
    assert ref.ref_curand_batch_init(vp(st_b.data_ptr()), B, vp(seeds.data_ptr()), _stream()) == 0
    temps = (torch.rand(B, device="cuda", generator=g) + 0.4).float()
    reps = (torch.rand(B, device="cuda", generator=g) * 0.3 + 1.0).float()
    top_ks = torch.randint(1, 65, (B,), device="cuda", generator=g, dtype=torch.int32)
    top_ps = (torch.rand(B, device="cuda", generator=g) * 0.6 + 0.4).float()
    end_ids = torch.full((B,), 2, dtype=torch.int32, device="cuda")
    min_len = torch.full((B,), 3, dtype=torch.int32, device="cuda")
    in_len = torch.randint(1, max_in + 1, (B,), device="cuda", generator=g, dtype=torch.int32)
    hist = torch.randint(0, V, (max_in + steps, B), device="cuda", generator=g, dtype=torch.int32)
    hist_b = hist.clone()
    fin_a = torch.zeros(B, dtype=torch.uint8, device="cuda")
    fin_b = torch.zeros(B, dtype=torch.bool, device="cuda")
    len_a = torch.full((B,), max_in - 1, dtype=torch.int32, device="cuda")
    len_b = len_a.clone()
    ws_bytes = C.c_size_t(0)
    ref.ref_batch_topk_sampling(None, C.byref(ws_bytes), None, None, None, None, None, 64, None, None, V, None, B, None, _stream())
    ws = torch.zeros(ws_bytes.value + 256, dtype=torch.uint8, device="cuda")
    was_finished = torch.zeros(B, dtype=torch.bool, device="cuda")
    for s in range(steps):
        step = max_in + s
        logits = torch.randn(B, V, device="cuda", generator=g) * 4
        if s == 2:
            logits[3, 2] = 100.0       # sequence 3 draws its end id once the minimum length allows it
        if s == 4:
            logits[3, 2] = 100.0
        xa, xb = logits.clone(), logits.clone()
        p = _params(l, xa, hist[step], output_ids=hist, step=step, input_lengths=in_len, max_input_length=max_in, temperatures=temps,
                    repetition_penalties=reps, min_lengths=min_len, sequence_lengths=len_a, end_ids=end_ids, top_ks=top_ks,
                    top_ps=top_ps, rng_states=st_a, finished=fin_a, sequence_lengths_out=len_a)
        assert l.lib.tm_sample_topk(h.ptr, C.byref(p), _stream()) == l.TM_OK
        assert ref.ref_sampling_penalties(vp(xb.data_ptr()), B, V, vp(temps.data_ptr()), vp(reps.data_ptr()), vp(hist_b.data_ptr()),
                                          vp(in_len.data_ptr()), max_in, step, vp(min_len.data_ptr()), vp(end_ids.data_ptr()),
                                          vp(len_b.data_ptr()), _stream()) == 0
        assert ref.ref_batch_topk_sampling(vp(ws.data_ptr()), C.byref(ws_bytes), vp(xb.data_ptr()), vp(hist_b[step].data_ptr()),
                                           vp(len_b.data_ptr()), vp(fin_b.data_ptr()), vp(st_b.data_ptr()), 64, vp(top_ks.data_ptr()),
                                           vp(top_ps.data_ptr()), V, vp(end_ids.data_ptr()), B, None, _stream()) == 0
        torch.cuda.synchronize()
        live = ~was_finished          # the library leaves the logits of finished sequences alone
        assert torch.equal(xa[live], xb[live]), f"step {s}: penalised logits differ"
        assert torch.equal(hist[step], hist_b[step]), f"step {s}: {hist[step].tolist()} vs {hist_b[step].tolist()}"
        assert torch.equal(fin_a.bool(), fin_b) and torch.equal(len_a, len_b)
        was_finished = fin_b.clone()
    assert bool(fin_b[3])     # the forced end id was taken


@pytest.mark.parametrize("B,V,ld", [(9, 32000, 32000), (4, 1000, 1024), (64, 32000, 32000), (2, 50001, 50008)])
def test_topp_sampling_matches_oracle(B, V, ld):
    """tm_sample_topp against oracle/sampling.py with caller-supplied uniform numbers: rows that stop at the most probable
    token, rows that walk, a row of few distinct values (equal probabilities are passed in token order), a finished row,
    a skipped row."""
    from lmdeploy_b200 import lib as l
    rng = np.random.default_rng(B * 77 + V)
    h = l.default_handle(torch.cuda.current_device())
    x = (rng.standard_normal((B, ld)) * 3).astype(np.float32)
    x[1, :V] = rng.integers(0, 4, V).astype(np.float32)          # four distinct probabilities, thousands of equals
    step, max_in = 10, 5
    out_ids = rng.integers(0, V, size=(step, B)).astype(np.int32)
    in_len = rng.integers(1, max_in + 1, size=B).astype(np.int32)
    temps = rng.uniform(0.5, 1.5, B).astype(np.float32)
    reps = rng.uniform(1.0, 1.2, B).astype(np.float32)
    temps[1], reps[1] = 1.0, 1.0
    end_ids = rng.integers(0, V, B).astype(np.int32)
    top_ps = rng.uniform(0.02, 1.0, B).astype(np.float32)
    top_ps[0], top_ps[1] = 1e-3, 0.9                             # row 0 certainly stops at its most probable token
    us = rng.uniform(1e-3, 1.0, B).astype(np.float32)
    finished = np.zeros(B, np.uint8)
    skip = np.zeros(B, np.uint8)
    if B > 2:
        finished[B // 2] = 1
        skip[B - 1] = 1
    d = {k: torch.from_numpy(v).cuda() for k, v in dict(x=x, out_ids=out_ids, in_len=in_len, temps=temps, reps=reps, end_ids=end_ids,
                                                         top_ps=top_ps, us=us, finished=finished, skip=skip).items()}
    ids = torch.full((B,), -7, dtype=torch.int32, device="cuda")
    p = _params(l, d["x"], ids, vocab=V, output_ids=d["out_ids"], step=step, input_lengths=d["in_len"], max_input_length=max_in,
                temperatures=d["temps"], repetition_penalties=d["reps"], end_ids=d["end_ids"], top_ps=d["top_ps"], uniforms=d["us"],
                finished=d["finished"], skip_decode=d["skip"])
    assert l.lib.tm_sample_topp(h.ptr, C.byref(p), _stream()) == l.TM_OK
    torch.cuda.synchronize()
    want_x = osamp.apply_penalties(x[:, :V], temps, reps, out_ids, in_len, max_in)
    got_x, got = d["x"].cpu().numpy(), ids.cpu().numpy()
    live = (finished == 0) & (skip == 0)
    np.testing.assert_allclose(got_x[live][:, :V], want_x[live], rtol=2e-6, atol=0)
    np.testing.assert_array_equal(got_x[~live], x[~live])
    assert (got[skip == 1] == -7).all() and (got[finished == 1] == end_ids[finished == 1]).all()
    n_sure, n_top, n_walk = 0, 0, 0
    for b in np.nonzero(live)[0]:
        want, margin = osamp.topp_sample(got_x[b, :V], top_ps[b], us[b])      # from the logits the kernel left behind
        top = float(osamp.softmax_topp(got_x[b, :V]).max())
        n_top += top >= top_ps[b]
        n_walk += top < top_ps[b]
        if margin > 2e-6:
            n_sure += 1
            assert got[b] == want, f"row {b}: {got[b]} vs {want} (margin {margin:.2e}, top_p {top_ps[b]:.3f}, u {us[b]:.3f})"
    assert n_sure >= live.sum() - 1 and n_top >= 1 and n_walk >= 1


def test_topp_sampling_matches_reference_kernels_over_steps():
    """tm_sample_topp step by step against the reference's penalty kernels, softmax, segmented sort and topp_sampling
    (compiled unmodified into oracle/_ref), both sides drawing from curand states seeded alike; odd rows belong to the
    top-k layer and are skipped by both.  Then the top_p decay."""
    from lmdeploy_b200 import lib as l
    if not os.path.exists(_REF):
        pytest.skip("oracle/_ref/libtm_ref.so not built")
    ref = C.CDLL(_REF)
    if not hasattr(ref, "ref_batch_topp_sampling"):
        pytest.skip("oracle/_ref/libtm_ref.so predates the top-p entry layer")
    B, V, steps, max_in = 16, 32000, 6, 4
    h = l.default_handle(torch.cuda.current_device())
    g = torch.Generator(device="cuda").manual_seed(23)
    seeds = torch.arange(500, 500 + B, dtype=torch.int64, device="cuda")
    nbytes = int(l.lib.tm_sampling_rng_state_bytes())
    st_a = torch.zeros(B * nbytes, dtype=torch.uint8, device="cuda")
    st_b = torch.zeros_like(st_a)
    vp = C.c_void_p
    assert l.lib.tm_sampling_rng_init(st_a.data_ptr(), B, seeds.data_ptr(), 0, _stream()) == l.TM_OK
    assert ref.ref_curand_batch_init(vp(st_b.data_ptr()), B, vp(seeds.data_ptr()), _stream()) == 0
    temps = (torch.rand(B, device="cuda", generator=g) + 0.5).float()
    reps = (torch.rand(B, device="cuda", generator=g) * 0.2 + 1.0).float()
    top_ps = (torch.rand(B, device="cuda", generator=g) * 0.9 + 0.1).float()
    top_ps[0] = 0.01                                   # stops at the most probable token every step
    top_ps_b = top_ps.clone()
    initial = top_ps.clone()
    decay = torch.full((B,), 0.9, device="cuda")
    p_min = torch.full((B,), 0.2, device="cuda")
    reset = torch.full((B,), -1, dtype=torch.int32, device="cuda")
    skip = torch.zeros(B, dtype=torch.uint8, device="cuda")
    skip[1::2] = 1
    end_ids = torch.full((B,), 2, dtype=torch.int32, device="cuda")
    min_len = torch.full((B,), 3, dtype=torch.int32, device="cuda")
    in_len = torch.randint(1, max_in + 1, (B,), device="cuda", generator=g, dtype=torch.int32)
    hist = torch.randint(3, V, (max_in + steps, B), device="cuda", generator=g, dtype=torch.int32)
    hist_b = hist.clone()
    fin_a = torch.zeros(B, dtype=torch.uint8, device="cuda")
    fin_b = torch.zeros(B, dtype=torch.bool, device="cuda")
    len_a = torch.full((B,), max_in - 1, dtype=torch.int32, device="cuda")
    len_b = len_a.clone()
    ref.ref_batch_topp_sampling.argtypes = [vp, vp, vp, vp, vp, C.c_float, vp, C.c_int, vp, C.c_int, vp, vp]
    ref.ref_compute_topp_decay.argtypes = [vp, vp, vp, vp, vp, vp, C.c_int, vp]
    for s in range(steps):
        step = max_in + s
        logits = torch.randn(B, V, device="cuda", generator=g) * 4
        if s in (3, 4):
            logits[4, 2] = 100.0                       # sequence 4 draws its end id once the minimum length allows it
        if s == 1:
            reset[6] = -1
        xa, xb = logits.clone(), logits.clone()
        p = _params(l, xa, hist[step], output_ids=hist, step=step, input_lengths=in_len, max_input_length=max_in, temperatures=temps,
                    repetition_penalties=reps, min_lengths=min_len, sequence_lengths=len_a, end_ids=end_ids, top_ps=top_ps,
                    rng_states=st_a, finished=fin_a, sequence_lengths_out=len_a, skip_decode=skip)
        assert l.lib.tm_sample_topp(h.ptr, C.byref(p), _stream()) == l.TM_OK
        assert ref.ref_sampling_penalties(vp(xb.data_ptr()), B, V, vp(temps.data_ptr()), vp(reps.data_ptr()), vp(hist_b.data_ptr()),
                                          vp(in_len.data_ptr()), max_in, step, vp(min_len.data_ptr()), vp(end_ids.data_ptr()),
                                          vp(len_b.data_ptr()), _stream()) == 0
        assert ref.ref_batch_topp_sampling(xb.data_ptr(), hist_b[step].data_ptr(), len_b.data_ptr(), fin_b.data_ptr(), st_b.data_ptr(),
                                           float(top_ps_b.max()), top_ps_b.data_ptr(), V, end_ids.data_ptr(), B,
                                           skip.view(torch.bool).data_ptr(), _stream().value) == 0
        torch.cuda.synchronize()
        mine = skip == 0
        assert torch.equal(hist[step][mine], hist_b[step][mine]), f"step {s}: {hist[step].tolist()} vs {hist_b[step].tolist()}"
        assert torch.equal(fin_a.bool()[mine], fin_b[mine]) and torch.equal(len_a[mine], len_b[mine])
        # the layer's decay after the draw (reset id of sequence 6 = what it just drew, once)
        if s == 2:
            reset[6] = hist[step][6]
        assert l.lib.tm_top_p_decay(top_ps.data_ptr(), initial.data_ptr(), hist[step].data_ptr(), decay.data_ptr(), p_min.data_ptr(),
                                    reset.data_ptr(), B, _stream()) == l.TM_OK
        assert ref.ref_compute_topp_decay(top_ps_b.data_ptr(), initial.data_ptr(), hist_b[step].data_ptr(), decay.data_ptr(),
                                          p_min.data_ptr(), reset.data_ptr(), B, _stream().value) == 0
        torch.cuda.synchronize()
        assert torch.equal(top_ps[mine], top_ps_b[mine])
        if s == 2:
            assert float(top_ps[6]) == float(initial[6])
    assert bool(fin_b[4]) and float(top_ps[0]) == float(np.float32(0.2))


@pytest.mark.parametrize("T,V,H,ld", [(1, 32000, 4096, 32000), (64, 32000, 4096, 32000), (5, 1000, 128, 1008), (128, 4000, 8192, 4000),
                                      (200, 512, 256, 512), (300, 256, 128, 256)])
def test_lm_head_matches_fp32_matmul(T, V, H, ld):
    from lmdeploy_b200 import lib as l
    h = l.default_handle(torch.cuda.current_device())
    g = torch.Generator(device="cuda").manual_seed(T + V)
    x = torch.randn(T, H, device="cuda", generator=g).half()
    w = (torch.randn(V, H, device="cuda", generator=g) * 0.05).half()
    out = torch.full((T, ld), 123.0, dtype=torch.float32, device="cuda")
    for _ in range(2):   # twice: the second launch meets used barriers / TMEM of the first
        assert l.lib.tm_lm_head_f16(h.ptr, out.data_ptr(), ld, x.data_ptr(), w.data_ptr(), T, V, H, _stream()) == l.TM_OK
    torch.cuda.synchronize()
    h.check_device_status(torch.cuda.current_stream().cuda_stream)     # raises if a bounded wait gave up
    want = x.float() @ w.float().t()
    err = (out[:, :V] - want).abs().max().item()
    assert err <= 2e-3 * max(1.0, want.abs().max().item()), err
    if ld > V:
        assert bool((out[:, V:] == 123.0).all())


def _word_lists(rng, B, V, length):
    """per sequence a [2, length] list: a few items of 1..3 tokens, offsets padded with -1"""
    out = np.zeros((B, 2, length), np.int32)
    out[:, 1, :] = -1
    for b in range(B):
        pos, i = 0, 0
        while True:
            n = int(rng.integers(1, 4))
            if pos + n > length or i >= length:
                break
            out[b, 0, pos:pos + n] = rng.integers(1, V, n)
            pos += n
            out[b, 1, i] = pos
            i += 1
    return out


@pytest.mark.parametrize("share", [False, True])
def test_word_lists_match_the_reference_kernels_and_the_oracle(share):
    from lmdeploy_b200 import lib as l
    rng = np.random.default_rng(21 + int(share))
    B, V, steps, L = 9, 500, 7, 12
    words = _word_lists(rng, 1 if share else B, V, L)
    ids = rng.integers(1, V, (steps, B)).astype(np.int32)
    # plant matches: the history of sequence b ends with the head of one of its items at some steps
    for b in range(B):
        w = words[0 if share else b]
        ends = [e for e in w[1] if e >= 0]
        if len(ends) >= 2:
            s0, e0 = int(ends[0]), int(ends[1])
            item = w[0, s0:e0]
            ids[steps - 1 - len(item) + 1: steps, b] = item          # whole item ends at the last step
            if len(item) > 1:
                ids[2: 2 + len(item) - 1, b] = item[:-1]               # head of the item ends at step 2 + len - 2
    d_ids, d_words = torch.from_numpy(ids).cuda(), torch.from_numpy(words if not share else words[0]).cuda().contiguous()
    ref = C.CDLL(_REF) if os.path.exists(_REF) else None
    if ref is not None and not hasattr(ref, "ref_ban_bad_words"):
        ref = None
    vp = C.c_void_p
    for step in range(steps):
        x = (rng.standard_normal((B, V))).astype(np.float32)
        xa = torch.from_numpy(x).cuda()
        assert l.lib.tm_ban_bad_words(xa.data_ptr(), V, V, B, d_ids.data_ptr(), 0, d_words.data_ptr(), L, int(share), step, _stream()) == l.TM_OK
        torch.cuda.synchronize()
        want = osamp.ban_bad_words(x, ids, words[0] if share else words, share, step)
        np.testing.assert_array_equal(xa.cpu().numpy(), want)
        if ref is not None:
            xb = torch.from_numpy(x).cuda()
            assert ref.ref_ban_bad_words(vp(xb.data_ptr()), vp(d_ids.data_ptr()), B, vp(d_words.data_ptr()), int(share), L, V, step, _stream()) == 0
            assert torch.equal(xa, xb), f"step {step}"
    if not share:
        for step in range(steps):
            fa = torch.zeros(B, dtype=torch.uint8, device="cuda")
            assert l.lib.tm_stop_words_criterion(d_ids.data_ptr(), 0, d_words.data_ptr(), L, fa.data_ptr(), B, step, _stream()) == l.TM_OK
            torch.cuda.synchronize()
            want = osamp.stop_words_criterion(ids, words, np.zeros(B, bool), step)
            np.testing.assert_array_equal(fa.cpu().numpy().astype(bool), want)
            if ref is not None:
                fb = torch.zeros(B, dtype=torch.bool, device="cuda")
                assert ref.ref_stop_words_criterion(vp(d_ids.data_ptr()), vp(d_words.data_ptr()), vp(fb.data_ptr()), L, B, step, _stream()) == 0
                assert torch.equal(fa.bool(), fb), f"step {step}"
        assert want.any()                                  # the planted endings were found at the last step
        limits = torch.tensor(rng.integers(0, 10, B), dtype=torch.int32, device="cuda")
        fin = torch.from_numpy(want.astype(np.uint8)).cuda()
        count = torch.zeros(1, dtype=torch.int32, device="cuda")
        assert l.lib.tm_length_criterion(fin.data_ptr(), limits.data_ptr(), B, 5, count.data_ptr(), _stream()) == l.TM_OK
        torch.cuda.synchronize()
        f2, n2 = osamp.length_criterion(want, limits.cpu().numpy(), 5)
        np.testing.assert_array_equal(fin.cpu().numpy().astype(bool), f2)
        assert int(count.item()) == n2
