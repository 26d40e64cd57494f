"""GPU: the persistent-batch scheduler (tm_batch_*).

The same requests are run one at a time (a scheduler with a single slot) and with continuous batching (four slots, six
requests of different lengths, so that sequences join and leave while others are mid-generation): every request must
get the same tokens either way - a sequence's result may not depend on who shares the batch with it.  Context decode is
issued one prompt per call in both runs (max_context_token_num = 1), so both feed identical inputs to identical
kernels.  Also: stopping at the end id, zero-length requests, a session continued from its cached tokens, and sampling
that depends on the seed and on nothing else.
"""
import numpy as np
import pytest
import torch

from tests.test_gpu_llama import CFG, build

pytestmark = pytest.mark.gpu


def _requests():
    rng = np.random.default_rng(11)
    lens = [(9, 12), (1, 20), (17, 5), (4, 9), (30, 14), (2, 3)]
    return [(100 + i, list(rng.integers(3, CFG["vocab_size"], size=p)), o) for i, (p, o) in enumerate(lens)]


def _run(model, slots, reqs, llama, **kw):
    b = llama.Batch(model, slots, start_id=1, end_id=kw.pop("end_id", 2), max_context_token_num=1)
    for sid, prompt, out_len in reqs:
        assert b.submit(sid, prompt, out_len, ignore_eos=kw.get("ignore_eos", True), **{k: v for k, v in kw.items() if k != "ignore_eos"}) == 0
    b.run(max_rounds=2000)
    res = {sid: b.output(sid) for sid, _, _ in reqs}
    c = b.counts()
    b.close()
    return res, c


def test_continuous_batching_gives_every_request_the_tokens_it_gets_alone():
    from lmdeploy_b200 import llama
    model, _, _ = build(False)
    reqs = _requests()
    alone, c1 = _run(model, 1, reqs, llama)
    together, c4 = _run(model, 4, reqs, llama)
    for sid, prompt, out_len in reqs:
        toks, state = together[sid]
        assert state == llama.Batch.FINISHED and len(toks) == out_len
        assert toks == alone[sid][0], f"request {sid}: {toks} vs {alone[sid][0]}"
    assert c1["steps"] == sum(o for _, _, o in reqs)                 # one sequence per step when alone
    assert max(o for _, _, o in reqs) <= c4["steps"] < c1["steps"] // 2  # shared steps when batched
    assert c1["prefill_tokens"] == c4["prefill_tokens"] == sum(len(p) - 1 for _, p, _ in reqs)
    model.close()


def test_end_id_zero_length_and_failures():
    from lmdeploy_b200 import llama
    model, _, _ = build(False)
    sid, prompt, _ = _requests()[0]
    free, _ = _run(model, 2, [(sid, prompt, 8)], llama)
    toks = free[sid][0]
    stop = toks[2]
    first = toks.index(stop)
    res, _ = _run(model, 2, [(sid, prompt, 8), (sid + 1, prompt, 0)], llama, end_id=stop, ignore_eos=False)
    assert res[sid][0] == toks[:first + 1] and res[sid][1] == llama.Batch.FINISHED       # the end id is the last token out
    assert res[sid + 1] == ([], llama.Batch.FINISHED)
    # a stop token of the request's own ends it the same way, with the end id left alone
    b = llama.Batch(model, 2)
    assert b.submit(sid, prompt, 8, ignore_eos=True, stop_ids=[toks[4], 999999]) == 0
    b.run(max_rounds=50)
    assert b.output(sid) == (toks[:toks.index(toks[4]) + 1], llama.Batch.FINISHED)
    b.close()
    b = llama.Batch(model, 2)
    assert b.submit(7, [1, 2, 3], 4, start=False) != 0                                   # continuing a session nobody started
    assert b.submit(8, [CFG["vocab_size"]], 4) != 0                                      # token outside the vocabulary
    assert b.submit(9, list(range(3, 3 + CFG["session_len"])), 4) == 0                   # accepted, then refused at intake: no room
    b.run(max_rounds=10)
    assert b.output(9) == ([], llama.Batch.FAILED) and not b.has_session(9)
    b.close()
    model.close()


def test_session_continues_from_its_cached_tokens():
    from lmdeploy_b200 import llama
    model, _, _ = build(False)
    rng = np.random.default_rng(3)
    p1, p2 = list(rng.integers(3, CFG["vocab_size"], size=6)), list(rng.integers(3, CFG["vocab_size"], size=4))
    b = llama.Batch(model, 2)
    assert b.submit(1, p1, 5, end=False, ignore_eos=True) == 0
    b.run(max_rounds=50)
    g1, state = b.output(1)
    assert state == llama.Batch.FINISHED and len(g1) == 5 and b.has_session(1)
    before = b.counts()["prefill_tokens"]
    assert b.submit(1, p2, 4, start=False, end=True, ignore_eos=True) == 0
    b.run(max_rounds=50)
    g2, state = b.output(1)
    assert state == llama.Batch.FINISHED and len(g2) == 4 and not b.has_session(1)
    assert b.forget(1) == 0 and b.forget(1) != 0          # the record goes once
    # only what had no keys / values was context-decoded: the last token of round one and the new prompt but its last token
    assert b.counts()["prefill_tokens"] - before == 1 + len(p2) - 1
    b.close()
    # the same conversation as one fresh prompt
    res, _ = _run(model, 1, [(2, p1 + g1 + p2, 4)], llama)
    assert res[2][0] == g2, (res[2][0], g2)
    model.close()


def test_session_rewound_to_a_step_equals_the_truncated_conversation():
    """The `step` input of a continued request: the session keeps its first `step` tokens only."""
    from lmdeploy_b200 import llama
    model, _, _ = build(False)
    rng = np.random.default_rng(4)
    p1, p2 = [int(t) for t in rng.integers(3, CFG["vocab_size"], size=6)], [int(t) for t in rng.integers(3, CFG["vocab_size"], size=3)]
    b = llama.Batch(model, 2)
    assert b.submit(1, p1, 5, end=False, ignore_eos=True) == 0
    b.run(max_rounds=50)
    g1 = b.output(1)[0]
    assert b.submit(1, p2, 4, start=False, end=True, ignore_eos=True, step=8) == 0      # 6 prompt tokens + the first 2 generated
    b.run(max_rounds=50)
    g2 = b.output(1)[0]
    b.close()
    res, _ = _run(model, 1, [(2, (p1 + g1)[:8] + p2, 4)], llama)
    assert res[2][0] == g2, (res[2][0], g2)
    model.close()


def test_sampling_depends_on_the_seed_only():
    from lmdeploy_b200 import llama
    model, _, _ = build(False)
    _, prompt, _ = _requests()[2]
    b = llama.Batch(model, 4)
    for sid, seed in ((1, 5), (2, 5), (3, 6)):
        assert b.submit(sid, prompt, 12, top_k=40, top_p=0.9, temperature=1.5, repetition_penalty=1.1, random_seed=seed, ignore_eos=True) == 0
    assert b.submit(4, prompt, 12, ignore_eos=True) == 0      # greedy neighbour
    b.run(max_rounds=100)
    out = {sid: b.output(sid)[0] for sid in (1, 2, 3, 4)}
    b.close()
    assert out[1] == out[2] and out[1] != out[3]
    alone, _ = _run(model, 1, [(9, prompt, 12)], llama)
    assert alone[9][0] == out[4]
    model.close()


def test_requests_with_only_a_top_p_are_drawn_over_the_whole_vocabulary():
    """A batch that mixes the reference's two sampling layers: top-k requests, top-p-only requests, a greedy one.  Every
    kind depends on its own seed only, the greedy neighbour is untouched, and a tiny top_p is greedy."""
    from lmdeploy_b200 import llama
    model, _, _ = build(False)
    _, prompt, _ = _requests()[2]
    b = llama.Batch(model, 4)          # six requests for four slots: two wait for a free slot
    assert b.submit(1, prompt, 10, top_p=0.95, temperature=2.0, random_seed=5, ignore_eos=True) == 0
    assert b.submit(2, prompt, 10, top_p=0.95, temperature=2.0, random_seed=5, ignore_eos=True) == 0
    assert b.submit(3, prompt, 10, top_p=0.95, temperature=2.0, random_seed=6, ignore_eos=True) == 0
    assert b.submit(4, prompt, 10, top_k=30, temperature=2.0, random_seed=5, ignore_eos=True) == 0
    assert b.submit(5, prompt, 10, top_p=1e-4, random_seed=9, ignore_eos=True) == 0      # the top token alone reaches it
    assert b.submit(6, prompt, 10, ignore_eos=True) == 0
    b.run(max_rounds=100)
    out = {sid: b.output(sid)[0] for sid in range(1, 7)}
    b.close()
    assert out[1] == out[2] and out[1] != out[3]
    assert out[5] == out[6]
    alone, _ = _run(model, 1, [(9, prompt, 10)], llama)
    assert alone[9][0] == out[6]
    model.close()


def test_banned_tokens_are_never_drawn():
    """bad_words_list of a request (single tokens, as the reference's scheduler takes them): the greedy answer changes at
    the first banned token and holds none of them; the neighbour without a list is untouched."""
    from lmdeploy_b200 import llama
    model, _, _ = build(False)
    sid, prompt, _ = _requests()[1]
    free, _ = _run(model, 2, [(sid, prompt, 8)], llama)
    toks = free[sid][0]
    banned = [toks[0], toks[3]]
    b = llama.Batch(model, 3)
    assert b.submit(1, prompt, 8, ignore_eos=True, bad_ids=banned) == 0
    assert b.submit(2, prompt, 8, ignore_eos=True) == 0
    assert b.submit(3, prompt, 8, ignore_eos=True, bad_ids=list(range(1, 40))) != 0      # more than 32 tokens
    b.run(max_rounds=50)
    got, other = b.output(1)[0], b.output(2)[0]
    b.close()
    assert other == toks
    assert len(got) == 8 and got[0] != toks[0] and not set(got) & set(banned)
    model.close()
