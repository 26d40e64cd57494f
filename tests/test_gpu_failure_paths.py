"""GPU: the paths that report trouble instead of faulting.  Nothing here faults, traps or hangs the GPU: a bounded
wait is made to run out by giving it a budget of one clock cycle, a prefill is given more tokens than the cache
holds (the writers drop the surplus rows), a decode step runs with every sequence inactive."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import gemm as ogemm
from tests.helpers import assert_close, dev, make_linear
from tests.test_gpu_llama import CFG, build

pytestmark = pytest.mark.gpu


def test_split_tile_wait_that_runs_out_is_reported_and_the_next_call_is_clean():
    """tcgen05 GEMM, a shape whose column tiles are shared by several CTAs: with a wait budget of one cycle the
    first CTA to finish a tile gives up on its partners at once, sets the status bit and leaves its share of the
    tile unreduced; tm_check_device_status turns the word into TM_ERR_DEVICE_TIMEOUT.  The arrival counts
    still reset themselves, so the next call (default budget) is correct."""
    from lmdeploy_b200 import lib as l
    n, k, t = 4096, 4096, 64
    lin = make_linear(n, k, 0)
    A, Q = dev(lin["A"], torch.int32), dev(lin["Q"])
    x = torch.randn(t, k, generator=torch.Generator().manual_seed(1)).half()
    xd = x.cuda()
    out = torch.zeros(t, n, dtype=torch.float16, device="cuda")
    h = l.Handle(torch.cuda.current_device())          # a handle of its own: the option must not leak into other tests
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = (h.ptr, out.data_ptr(), A.data_ptr(), xd.data_ptr(), Q.data_ptr(), n, t, k, 128, 0, None, 0, st)
    try:
        h.set_option("gemm_wait_cycles", 1)
        w = C.c_uint(0)
        for attempt in range(5):
            # whether some CTA polls before its last partner has arrived is a matter of timing: practically always,
            # but a launch in which every CTA happens to find its tile complete at the first look is legal
            assert l.lib.tm_gemm_s4_f16(*args) == l.TM_OK   # the launch itself succeeds
            rc = l.lib.tm_check_device_status(h.ptr, st, C.byref(w))
            if rc == l.TM_ERR_DEVICE_TIMEOUT:
                break
            assert rc == l.TM_OK
        assert rc == l.TM_ERR_DEVICE_TIMEOUT, "no wait ran out in five launches"
        assert w.value & (1 << 3), hex(w.value)
        assert l.lib.tm_check_device_status(h.ptr, st, C.byref(w)) == l.TM_OK   # read and cleared
        h.set_option("gemm_wait_cycles", 0)
        for _ in range(2):
            out.zero_()
            assert l.lib.tm_gemm_s4_f16(*args) == l.TM_OK
            h.check_device_status(torch.cuda.current_stream().cuda_stream)
            assert_close(out.cpu().numpy(), ogemm.gemm_s4_f16(x.numpy(), lin["w_kn"]), "after a time-out")
    finally:
        h.close()


def test_prefill_past_the_cache_is_reported_and_writes_nothing_outside():
    """history + new tokens > session_len: the surplus rows are dropped by the writers (no write outside a cache
    head), and tm_llama_check_status reports the caller's mistake."""
    from lmdeploy_b200 import lib as l
    model, _, _ = build(True)
    S = CFG["session_len"]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        st = model.new_state(2, 8, None, None)
        guard_k, guard_v = st.k_cache.clone(), st.v_cache.clone()
        model.prefill(st, [list(range(1, S - 3)), [5, 6, 7]])          # fits: S - 4 and 3 tokens
        model.check_status(stream.cuda_stream)
        k_ok = st.k_cache.clone()
        assert not torch.equal(k_ok, guard_k)
        model.prefill(st, [list(range(1, 11)), [9]])                   # sequence 0: S - 4 + 10 > S
        with pytest.raises(l.TmError) as e:
            model.check_status(stream.cuda_stream)
        assert e.value.status == l.TM_ERR_DEVICE_TIMEOUT and "0x20" in str(e.value)
        # rows [0, S - 4) of sequence 0 are as the first call left them: nothing wrapped around or spilled over
        assert torch.equal(st.k_cache[0, :, :, : S - 4], k_ok[0, :, :, : S - 4])
        model.check_status(stream.cuda_stream)                          # cleared by the read
    model.close()


def test_steps_with_every_sequence_inactive_keep_the_launch_chain_intact():
    """Decode steps in which no sequence is active (all start later) make every attention CTA exit early.  They
    must still wait for the kernel before them: otherwise the GEMM after the attention could overlap the GEMM
    before it, and both use the same split-K scratch and arrival counts.  Same tokens with and without
    programmatic dependent launch, bit for bit, through idle steps followed by active ones."""
    outs = []
    for pdl in (1, 0):
        model, _, _ = build(True)
        model.handle.set_option("pdl", pdl)
        B, idle, active = 3, 5, 6
        steps = idle + active
        start = np.full(B, idle, np.int32)
        forced = np.full((steps, B), -1, np.int32)
        forced[idle] = [11, 22, 33]
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            st = model.new_state(B, steps, start, forced, keep_logits=True)
            model.decode(st, steps, use_graph=True)
            model.check_status(stream.cuda_stream)
            ids = st.output_ids.cpu().numpy()
            assert (ids[:idle] == -1).all() and (ids[idle:] >= 0).all()
            outs.append((ids, st.logits.cpu().numpy(), st.k_cache.cpu().numpy()))
        model.handle.set_option("pdl", 1)
        model.close()
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a, b)
