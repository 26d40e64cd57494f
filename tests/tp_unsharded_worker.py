"""Worker of tests/test_gpu_tp_vs_single.py: one tensor-parallel rank per GPU (torchrun, NCCL, world = 2).

ONE set of weights, sharded per rank the way the reference shards it (LlamaDecoderLayerWeight.cc:49-77: q | k | v heads
and gate / up pairs by column, o / w2 by row, lm-head by vocabulary rows), is run at tp = world and compared with the
un-sharded run of the same weights on one GPU and with the CPU oracle:
  (a) the workspace the reference's own deploy.py wrote at tp = 2 (tests/golden/ref_workspace.npz) against its tp = 1
      workspace;
  (b) a larger seeded checkpoint (GQA: 8 query / 4 KV heads) converted by lmdeploy_b200/deploy.py at tp = world and tp = 1.
Teacher-forced tokens, logits of every step and the cached K rows (rank r holds KV heads [r Hkv / tp, (r + 1) Hkv / tp)),
decode steps and a prefill, fp16 cache.  Tolerance: max-abs 3e-2, mean-rel 5e-3 (fp16 all-reduce included)."""
import ctypes as C
import os
import sys
import tempfile

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def read_cfg(d, l, llama):
    c = l.TmLlamaConfig()
    assert l.lib.tm_llama_read_config(d.encode(), C.byref(c), None) == l.TM_OK
    return llama.LlamaConfig(c.head_num, c.kv_head_num, c.inter_size, c.num_layer, c.vocab_size, norm_eps=c.norm_eps,
                             rope_theta=c.rope_theta, quant_policy=0)


def run_model(llama, mcfg, wdir, comm, local, tokens, prompts, S):
    """-> (logits of every decode step [steps, B, V], K cache after the steps, logits after a prefill + one step)"""
    B, steps = tokens.shape[1], tokens.shape[0]
    model = llama.LlamaModel(mcfg, B, S, local, comm)
    model.load_workspace(wdir)
    out = []
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        st = model.new_state(B, steps, None, tokens, keep_logits=True)
        for _ in range(steps):
            model.decode(st, 1, use_graph=True)
            out.append(st.logits.cpu().numpy().copy())
        model.check_status(stream.cuda_stream)
        k = st.k_cache.float().cpu().numpy()
        st2 = model.new_state(B, 1, None, np.asarray([[p[-1] for p in prompts]], np.int32), keep_logits=True)
        model.prefill(st2, [p[:-1] for p in prompts])
        model.decode(st2, 1, use_graph=False)
        model.check_status(stream.cuda_stream)
        pre = st2.logits.cpu().numpy().copy()
    model.close()
    return np.stack(out), k, pre


class _DevMem:
    """a zero-copy torch view of device memory that the library owns"""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = dict(shape=shape, typestr="<f2", data=(int(ptr), False), version=2, strides=None)


def slot_view(ptr, rows, cols):
    return torch.as_tensor(_DevMem(ptr, (rows, cols)), device="cuda")


def close(a, b):
    err = np.abs(a - b)
    return float(err.max()), float(err.mean() / max(np.abs(b).mean(), 1e-9))


def main():
    from lmdeploy_b200 import deploy, lib as l, llama
    from tests import ref_workspace as rw
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = llama.Comm(world, rank, local)
    ok, report = True, []
    tmp = tempfile.mkdtemp(prefix=f"tm_tp_{rank}_")
    S = 48
    rng = np.random.default_rng(11)

    cases = []
    # (a) reference-written workspaces (every rank unpacks its own copy)
    cfg_a, hf_a, files = rw.load()
    if world == 2:
        cases.append(("reference-written", rw.unpack_to(os.path.join(tmp, "a_tp"), files[2]), rw.unpack_to(os.path.join(tmp, "a_1"), files[1])))
    # (b) a GQA checkpoint through this library's converter
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import make_ref_workspace_fixture as fx
    fx.HF_CONFIG.update(num_attention_heads=8, num_key_value_heads=4, hidden_size=1024, intermediate_size=512, vocab_size=256)
    ckpt = fx.make_checkpoint(seed=7)
    b_tp = deploy.deploy_awq(ckpt, fx.HF_CONFIG, os.path.join(tmp, "b_tp"), tp=world)
    b_1 = deploy.deploy_awq(ckpt, fx.HF_CONFIG, os.path.join(tmp, "b_1"), tp=1)
    cases.append(("own converter, GQA", b_tp, b_1))

    for name, d_tp, d_1 in cases:
        mcfg = read_cfg(d_1, l, llama)
        B, steps = 3, 5
        tokens = rng.integers(0, mcfg.vocab_size, size=(steps, B)).astype(np.int32)
        prompts = [list(rng.integers(0, mcfg.vocab_size, size=n)) for n in (9, 17, 3)]
        lg_tp, k_tp, pre_tp = run_model(llama, mcfg, d_tp, comm, local, tokens, prompts, S)
        lg_1, k_1, pre_1 = run_model(llama, mcfg, d_1, None, local, tokens, prompts, S)      # every rank: the un-sharded run
        hkv = mcfg.kv_head_num // world
        a = close(lg_tp, lg_1)
        b = close(pre_tp, pre_1)
        kerr = float(np.abs(k_tp[:, :, :, :steps] - k_1[:, :, rank * hkv:(rank + 1) * hkv, :steps]).max())
        good = a[0] <= 3e-2 and a[1] <= 5e-3 and b[0] <= 3e-2 and b[1] <= 5e-3 and kerr <= 2e-2 and np.isfinite(lg_tp).all()
        ok = ok and good
        report.append(f"{name}: decode max_abs={a[0]:.2e} mean_rel={a[1]:.2e}; prefill max_abs={b[0]:.2e} mean_rel={b[1]:.2e}; "
                      f"k rows max_abs={kerr:.2e} {'ok' if good else 'FAIL'}")
    # (c) the peer-memory all-reduce + residual add + RMSNorm by itself, against the same arithmetic in torch on the
    #     gathered partial sums (rank order, fp16 rounding of the sum, fp32 add, fp16 residual, norm)
    if comm.p2p:
        h = l.default_handle(local)
        status = torch.zeros(64, dtype=torch.int32, device="cuda")
        # both hand-over schemes: 1 = every rank reads every slot, 2 = token rows dealt to owner ranks (the default
        # beyond two ranks), where a rank updates the residual of its own rows only
        # ... and both ways of fetching a peer's rows: bulk copies into shared memory (the default) or 16-byte loads
        cases = [(mode, 1, shape) for mode in (1, 2) for shape in [(5, 1024), (64, 4096), (128, 8192), (3, 16384), (1, 256), (130, 4096)]]
        cases += [(mode, 0, shape) for mode in (1, 2) for shape in [(64, 4096), (3, 16384)]]
        for it, (mode, bulk, (m_rows, n)) in enumerate(cases):
            slot = it % 2
            assert l.lib.tm_comm_set_option(comm.ptr, b"p2p_mode", mode) == l.TM_OK
            assert l.lib.tm_comm_set_option(comm.ptr, b"p2p_bulk", bulk) == l.TM_OK
            g = torch.Generator(device="cuda").manual_seed(100 + 7 * it + rank)
            part = torch.randn(m_rows, n, device="cuda", generator=g).half()
            g0 = torch.Generator(device="cuda").manual_seed(55 + it)
            resid = torch.randn(m_rows, n, device="cuda", generator=g0).half()
            scale = (1 + 0.1 * torch.randn(n, device="cuda", generator=g0)).half()
            ptr = l.lib.tm_comm_p2p_slot(comm.ptr, slot)
            # the partial goes into the slot (in the model the GEMM writes there directly)
            slot_view(ptr, m_rows, n).copy_(part)
            torch.cuda.synchronize()
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            out = torch.empty_like(resid)
            r_in = resid.clone()
            st = torch.cuda.current_stream().cuda_stream
            assert l.lib.tm_allreduce_add_residual_rmsnorm(comm.ptr, slot, r_in.data_ptr(), out.data_ptr(), scale.data_ptr(), 1e-6,
                                                           m_rows, n, status.data_ptr(), st) == l.TM_OK
            torch.cuda.synchronize()
            total = torch.zeros(m_rows, n, device="cuda")
            for pj in parts:
                total += pj.float()
            want_r = (resid.float() + total.half().float()).half()
            inv = torch.rsqrt((resid.float() + total.half().float()).pow(2).mean(dim=-1, keepdim=True) + 1e-6)
            want_o = (want_r.float() * scale.float() * inv).half()
            if mode == 2:   # rows of other owners keep the residual they had
                per = (m_rows + world - 1) // world
                mine = torch.zeros(m_rows, 1, dtype=torch.bool, device="cuda")
                mine[rank * per:(rank + 1) * per] = True
                want_r = torch.where(mine, want_r, resid)
            good = torch.equal(r_in, want_r) and (out.float() - want_o.float()).abs().max().item() <= 2e-3 * max(1.0, want_o.float().abs().max().item())
            good = good and int(status[0].item()) == 0
            ok = ok and good
            report.append(f"all-reduce + add + norm [{m_rows}, {n}] slot {slot} scheme {mode} bulk {bulk}: residual bit-exact {torch.equal(r_in, want_r)}, "
                          f"out max_abs {(out.float() - want_o.float()).abs().max().item():.2e} {'ok' if good else 'FAIL'}")
        assert l.lib.tm_comm_set_option(comm.ptr, b"p2p_bulk", -1) == l.TM_OK
        # (d) the decode step with NCCL instead of the peer-memory path gives the same logits within tolerance
        h.set_option("p2p_allreduce", 0)
        mcfg = read_cfg(b_1, l, llama)
        tokens = rng.integers(0, mcfg.vocab_size, size=(4, 3)).astype(np.int32)
        prompts = [list(rng.integers(0, mcfg.vocab_size, size=n)) for n in (4, 6, 2)]
        lg_nccl, _, _ = run_model(llama, mcfg, b_tp, comm, local, tokens, prompts, S)
        h.set_option("p2p_allreduce", 1)
        for mode in (1, 2):
            assert l.lib.tm_comm_set_option(comm.ptr, b"p2p_mode", mode) == l.TM_OK
            lg_p2p, _, _ = run_model(llama, mcfg, b_tp, comm, local, tokens, prompts, S)
            a = close(lg_p2p, lg_nccl)
            good = a[0] <= 3e-2 and a[1] <= 5e-3
            ok = ok and good
            report.append(f"decode, peer-memory all-reduce (scheme {mode}) vs NCCL: max_abs={a[0]:.2e} mean_rel={a[1]:.2e} {'ok' if good else 'FAIL'}")
        assert l.lib.tm_comm_set_option(comm.ptr, b"p2p_mode", 0) == l.TM_OK
        # (e) last: a peer that does not show up.  Rank 0 alone calls, with a wait bound of a few microseconds: the kernel
        #     gives up, sets the status bit and returns; nothing hangs.  No all-reduce follows (the call counts now differ).
        dist.barrier()
        if rank == 0:
            assert l.lib.tm_comm_set_option(comm.ptr, b"p2p_wait_cycles", 20000) == l.TM_OK
            x = torch.zeros(2, 256, dtype=torch.float16, device="cuda")
            y = torch.ones(256, dtype=torch.float16, device="cuda")
            status.zero_()
            assert l.lib.tm_allreduce_add_residual_rmsnorm(comm.ptr, 0, x.data_ptr(), x.clone().data_ptr(), y.data_ptr(), 1e-6, 2, 256,
                                                           status.data_ptr(), torch.cuda.current_stream().cuda_stream) == l.TM_OK
            torch.cuda.synchronize()
            good = int(status[0].item()) == (1 << 6)
            assert l.lib.tm_comm_set_option(comm.ptr, b"p2p_mode", 2) == l.TM_OK     # same with rows dealt to owners
            status.zero_()
            assert l.lib.tm_allreduce_add_residual_rmsnorm(comm.ptr, 1, x.data_ptr(), x.clone().data_ptr(), y.data_ptr(), 1e-6, 2, 256,
                                                           status.data_ptr(), torch.cuda.current_stream().cuda_stream) == l.TM_OK
            torch.cuda.synchronize()
            good = good and int(status[0].item()) == (1 << 6)
            ok = ok and good
            report.append(f"absent peer: status word 0x{int(status[0].item()):x} {'ok' if good else 'FAIL'}")
        dist.barrier()
    else:
        report.append("peer-memory all-reduce not set up on this machine: NCCL path only")
    flag = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("\n".join(report))
        print(f"TP_VS_SINGLE world={world} {'OK' if int(flag.item()) else 'FAIL'}", flush=True)
    comm.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) else 1)


if __name__ == "__main__":
    main()
