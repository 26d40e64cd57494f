"""CPU: known answers for the sampling oracle (oracle/sampling.py)."""
import numpy as np

from oracle import sampling as osamp


def test_topk_sample_known_answers():
    x = np.array([0.0, 2.0, 1.0, -1.0, 2.0], np.float32)
    # candidates in descending order, ties by id: 1, 4, 2 ; e = 1, 1, e^-1
    tot = 2 + np.exp(-1.0)
    assert osamp.topk_sample(x, 3, 1.0, 0.2)[0] == 1            # target 0.2 * tot < 1
    assert osamp.topk_sample(x, 3, 1.0, 1.5 / tot)[0] == 4      # 1 < target < 2
    assert osamp.topk_sample(x, 3, 1.0, 1.0)[0] == 2            # target = whole sum: last candidate
    assert osamp.topk_sample(x, 3, 0.4, 1.0)[0] == 1            # top_p shrinks the target: 0.4 * tot < 1
    assert osamp.topk_sample(x, 1, 1.0, 0.99)[0] == 1           # k = 1 is greedy
    assert osamp.topk_sample(x, 99, 1.0, 1e-9)[0] == 1          # k larger than the vocabulary


def test_penalties_known_answers():
    x = np.array([[1.0, -2.0, 4.0, 8.0]], np.float32)
    y = osamp.apply_penalties(x, temperatures=[0.5])
    np.testing.assert_allclose(y, x / np.float32(0.5 + 1e-6), rtol=1e-6)
    # token 2 twice and token 1 once in the history; row 1 is prompt padding (input length 1 of 2)
    ids = np.array([[2], [3], [1], [2]])
    y = osamp.apply_penalties(x, repetition_penalties=[2.0], output_ids=ids, input_lengths=[1], max_input_length=2)
    np.testing.assert_array_equal(y, np.array([[1.0, -4.0, 2.0, 8.0]], np.float32))
    # generated so far = sequence_length + 1 - max_input_length = 1 < 3: the end id is masked
    y = osamp.apply_penalties(x, min_lengths=[3], end_ids=[3], sequence_lengths=[2], max_input_length=2)
    assert y[0, 3] == -osamp.FLT_MAX and (y[0, :3] == x[0, :3]).all()
    y = osamp.apply_penalties(x, min_lengths=[1], end_ids=[3], sequence_lengths=[2], max_input_length=2)
    assert (y == x).all()


def test_finished_rows_emit_the_end_id():
    x = np.random.default_rng(0).standard_normal((3, 50)).astype(np.float32)
    ids, _ = osamp.sample(x, [5, 5, 5], [1.0, 1.0, 1.0], [0.5, 0.5, 0.5], finished=[0, 1, 0], end_ids=[2, 2, 2])
    assert ids[1] == 2


def test_word_lists_known_answers():
    # two items for sequence 0: [5] and [7, 8]; one for sequence 1: [9, 9, 4]; padded with -1 offsets
    words = np.array([[[5, 7, 8, 0], [1, 3, -1, -1]], [[9, 9, 4, 0], [3, -1, -1, -1]]])
    ids = np.array([[1, 9], [7, 9], [3, 2]])                 # steps 0..2
    x = np.zeros((2, 12), np.float32)
    y = osamp.ban_bad_words(x, ids, words, False, 2)         # about to draw step 2: history = steps 0, 1
    assert y[0, 5] == -np.inf and y[0, 8] == -np.inf        # single token always; [7, 8] because 7 was drawn last
    assert y[1, 4] == -np.inf and np.isinf(y).sum() == 3    # [9, 9, 4]: the last two were 9, 9
    y = osamp.ban_bad_words(x, ids, words, False, 1)         # one step earlier: 7 not drawn yet, only one 9
    assert y[0, 5] == -np.inf and np.isinf(y).sum() == 1
    ids2 = np.array([[7, 9], [8, 9], [5, 4]])
    f = osamp.stop_words_criterion(ids2, words, [False, False], 1)
    assert list(f) == [True, False]                          # sequence 0 ends with 7, 8
    f = osamp.stop_words_criterion(ids2, words, [False, False], 2)
    assert list(f) == [True, True]                           # 5 ; 9, 9, 4
    f, n = osamp.length_criterion([False, True, False], [5, 9, 3], 4)
    assert list(f) == [False, True, True] and n == 2


def test_topp_sample_known_answers():
    # probabilities 0.5, 0.25, 0.125, 0.125 (up to the 1e-6 in the denominator): logits = log2 scaled
    x = (np.log(np.array([0.125, 0.5, 0.125, 0.25])) + 3.0).astype(np.float32)
    assert osamp.topp_sample(x, 0.4, 0.9)[0] == 1               # the top token alone reaches top_p: no walk
    assert osamp.topp_sample(x, 0.5 - 1e-3, 0.01)[0] == 1
    # walk: target = u * top_p against the running sums 0.5, 0.75, 0.875, 1.0 in the order 1, 3, 0, 2
    assert osamp.topp_sample(x, 0.8, 0.5)[0] == 1               # 0.40
    assert osamp.topp_sample(x, 0.8, 0.8)[0] == 3               # 0.64
    assert osamp.topp_sample(x, 1.0, 0.8)[0] == 0               # 0.80: equal probabilities in token order
    assert osamp.topp_sample(x, 1.0, 0.9)[0] == 2               # 0.90
    assert osamp.topp_sample(x, 1.0, 1.0)[0] == 1               # the row sums to just under 1: falls back to the top token
    tok, margin = osamp.topp_sample(x, 0.8, 0.8)
    assert abs(margin - 0.11) < 1e-3                            # 0.64 is 0.14 above 0.5 and 0.11 below 0.75
    p = osamp.softmax_topp(x)
    assert abs(float(p.sum()) - 1.0) < 1e-5 and p.dtype == np.float32


def test_top_p_decay_known_answers():
    out = osamp.top_p_decay([0.8, 0.8, 0.05], [0.9, 0.9, 0.9], [7, 3, 1], [0.5, 0.5, 0.5], [0.1, 0.1, 0.1], [3, 3, -1])
    np.testing.assert_allclose(out, [0.4, 0.9, 0.1], rtol=1e-6)
