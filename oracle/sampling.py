"""CPU restatement of the reference's token sampling for fp32 logits.  Test infrastructure only: nothing under
``lmdeploy_b200/`` may import this.

Follows, in the order of ``BaseSamplingLayer<T>::forward``
(src/turbomind/layers/sampling_layers/BaseSamplingLayer.cc:300-353):

* ``batchApplyTemperaturePenalty``  (src/turbomind/kernels/sampling_penalty_kernels.cu:118-146)
* ``batchApplyRepetitionPenalty``   (sampling_penalty_kernels.cu:386-430, multiplicative; a token that occurs several
  times is penalised once, because every occurrence writes the value computed from the unpenalised logit)
* ``batchApplyMinLengthPenalty``    (sampling_penalty_kernels.cu:486-500)
* ``topk_stage1`` + ``topk_stage2_sampling`` (src/turbomind/kernels/sampling_topk_kernels.cu:125-312): the k largest
  logits in descending order, ``e_i = exp(l_i - l_max)``, target ``u * top_p * sum(e)``, first i whose running sum
  reaches the target (the last one otherwise).
* ``addBiasSoftMax`` + ``topp_beam_topk_kernel`` + segmented sort + ``topp_sampling``
  (src/turbomind/kernels/sampling_topp_kernels.cu:802-1004, 1295-1346) for the sequences without a top-k:
  probabilities ``exp(l - max) / (sum + 1e-6)``; the most probable token at once when it alone reaches ``top_p``;
  otherwise the first token, by descending probability, at which the running sum reaches ``u * top_p``.

Pinned on a GPU against those kernels compiled unmodified into ``oracle/_ref`` (tests/test_gpu_sampling.py), where the
uniform numbers come from the same curand states.  Here the uniform number is an input.
"""
import numpy as np

FLT_MAX = np.float32(3.4028234663852886e38)


def apply_penalties(logits, temperatures=None, repetition_penalties=None, output_ids=None, input_lengths=None,
                    max_input_length=0, min_lengths=None, end_ids=None, sequence_lengths=None):
    """logits [batch, vocab] float32 -> penalised copy.  output_ids [step, batch]."""
    x = np.array(logits, dtype=np.float32, copy=True)
    B = x.shape[0]
    if temperatures is not None:
        inv = (np.float32(1.0) / (np.asarray(temperatures, np.float32) + np.float32(1e-6))).astype(np.float32)
        x = (x * inv[:, None]).astype(np.float32)
    if repetition_penalties is not None and output_ids is not None and len(output_ids) > 0:
        ids = np.asarray(output_ids)
        for b in range(B):
            in_len = max_input_length if input_lengths is None else int(input_lengths[b])
            keep = [s for s in range(ids.shape[0]) if not (in_len <= s < max_input_length)]
            toks = np.unique(ids[keep, b])
            pen = np.float32(repetition_penalties[b])
            old = x[b, toks]
            x[b, toks] = np.where(old < 0, old * pen, old / pen).astype(np.float32)
    if min_lengths is not None:
        for b in range(B):
            if int(sequence_lengths[b]) + 1 - max_input_length < int(min_lengths[b]):
                x[b, int(end_ids[b])] = -FLT_MAX
    return x


def topk_sample(logits, top_k, top_p, u):
    """One row.  Returns (token id, margin): margin is the distance of the target from the nearest boundary of the
    chosen candidate's interval, relative to the sum - a test can skip draws that sit on a boundary."""
    x = np.asarray(logits, dtype=np.float32)
    k = max(1, min(int(top_k), x.shape[0]))
    order = np.lexsort((np.arange(x.shape[0]), -x.astype(np.float64)))[:k]      # descending value, then ascending id
    e = np.exp((x[order] - x[order[0]]).astype(np.float32)).astype(np.float32)
    total = np.float32(0)
    for v in e:
        total = np.float32(total + v)
    r = np.float32(np.float32(np.float32(u) * np.float32(top_p)) * total)
    target = float(r)
    run = 0.0
    for i in range(k):
        r = np.float32(r - e[i])
        lo, run = run, run + float(e[i])
        if r <= 0 or i == k - 1:
            margin = min(abs(target - lo), abs(run - target)) / float(total)
            return int(order[i]), margin
    raise AssertionError("unreachable")


def sample(logits, top_ks, top_ps, uniforms, finished=None, end_ids=None):
    """Batch version: ids [batch], margins [batch]."""
    B = len(logits)
    ids, margins = np.zeros(B, np.int32), np.ones(B)
    for b in range(B):
        if finished is not None and finished[b]:
            ids[b] = end_ids[b]
            continue
        ids[b], margins[b] = topk_sample(logits[b], top_ks[b], top_ps[b], uniforms[b])
    return ids, margins


def softmax_topp(logits):
    """addBiasSoftMax for a sequence that is not finished (src/turbomind/kernels/sampling_topp_kernels.cu:1295-1346):
    exp(l - max) / (sum + 1e-6), float32."""
    x = np.asarray(logits, dtype=np.float32)
    e = np.exp((x - x.max()).astype(np.float32)).astype(np.float32)
    # The kernels add per-thread partial sums and then a tree (blockReduceSum), which stays within an ulp or two of the
    # exact sum; a sequential float32 loop over 32 000 terms does not (1e-4 off on rows of equal values).  The exact sum
    # rounded to float stands for the kernels' order; the tests allow a margin for the last ulp.
    total = np.float32(e.astype(np.float64).sum())
    return (e / np.float32(total + np.float32(1e-6))).astype(np.float32)


def topp_sample(logits, top_p, u):
    """One row of invokeBatchTopPSampling (sampling_topp_kernels.cu:802-858, 878-1004).  Returns (token id, margin):
    margin is how far the decision was from flipping (distance of u * top_p from the chosen interval's ends, or of the
    largest probability from top_p), so that a test can leave out draws that float rounding decides."""
    p = softmax_topp(logits)
    order = np.lexsort((np.arange(p.shape[0]), -p.astype(np.float64)))      # descending, equal values in token order
    top = float(p[order[0]])
    if top >= np.float32(top_p):                                            # topp_beam_topk_kernel: no sort, no walk
        return int(order[0]), abs(top - float(np.float32(top_p)))
    gate = abs(top - float(np.float32(top_p)))
    r = float(np.float32(np.float32(u) * np.float32(top_p)))
    # The running sum is kept in double here.  The reference's block scan rounds it in float, in an order no loop
    # reproduces (an error of a few 1e-6 after thousands of terms): the margin is what a test must leave for that.
    run = 0.0
    for i in order:
        lo, run = run, run + float(p[i])
        if r <= run:
            return int(i), min(gate, abs(r - lo), abs(run - r))
    return int(order[0]), min(gate, abs(r - run))                           # the row sums to less than the target


def top_p_decay(top_p, initial, ids, decay, top_p_min, reset_ids):
    """invokeComputeToppDecay (sampling_topp_kernels.cu:1381-1426)."""
    top_p, initial = np.asarray(top_p, np.float32), np.asarray(initial, np.float32)
    stepped = np.maximum((top_p * np.asarray(decay, np.float32)).astype(np.float32), np.asarray(top_p_min, np.float32))
    return np.where(np.asarray(ids) == np.asarray(reset_ids), initial, stepped).astype(np.float32)


def _items(words):
    """words: int array [2, len] (tokens back to back | exclusive end offsets, -1 padded) -> list of token lists."""
    toks, offs = np.asarray(words[0]), np.asarray(words[1])
    out, start = [], 0
    for i, end in enumerate(offs):
        if end < 0:
            out.append(None)        # padding entry: the kernels skip it but keep using its offset as the next start
            continue
        out.append(list(toks[start:end]))
        start = int(end)
    # the reference takes the start of item i from offs[i - 1] whatever its sign; with -1 padding only at the tail that is
    # the running `start` above
    return [o for o in out if o is not None]


def ban_bad_words(logits, output_ids, bad_words, share_words, step):
    """src/turbomind/kernels/ban_bad_words.cu:22-84, beam width 1.  logits [batch, vocab] float32 -> copy with the banned
    tokens at -inf; output_ids [steps, batch]; bad_words [batch, 2, len] or [2, len] when shared."""
    x = np.array(logits, dtype=np.float32, copy=True)
    B, V = x.shape
    for b in range(B):
        for item in _items(bad_words if share_words else bad_words[b]):
            n = len(item)
            ban = n == 1
            if n > 1 and step >= n - 1:
                ban = all(int(output_ids[step - (n - 1) + k, b]) == int(item[k]) for k in range(n - 1))
            if ban and 0 < int(item[-1]) < V:
                x[b, int(item[-1])] = -np.inf
    return x


def stop_words_criterion(output_ids, stop_words, finished, step):
    """src/turbomind/kernels/stop_criteria_kernels.cu:25-84, beam width 1: finished[b] set when the tokens up to and
    including `step` end with one of the sequence's items."""
    f = np.array(finished, dtype=bool, copy=True)
    for b in range(len(f)):
        for item in _items(stop_words[b]):
            n = len(item)
            if step + 1 >= n and all(int(output_ids[step - (n - 1) + k, b]) == int(item[k]) for k in range(n)):
                f[b] = True
    return f


def length_criterion(finished, limits, step):
    """stop_criteria_kernels.cu:107-132: finished |= step >= limit; also how many are finished."""
    f = np.array(finished, dtype=bool, copy=True) | (step >= np.asarray(limits))
    return f, int(f.sum())
