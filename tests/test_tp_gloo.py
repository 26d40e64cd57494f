"""CPU, world_size 2 over gloo: the tensor-parallel sharding the decode driver assumes
(LlamaDecoderLayerWeight.cc:49-77) — column-split qkv / w13, row-split o / w2, one sum-allreduce
after o_proj and after down_proj — reproduces the un-sharded oracle layer."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention as oa
from oracle import gemm, norm

H, HKV, INTER, S = 4, 2, 512, 32
HID = H * 128


def _weights():
    rng = np.random.default_rng(0)
    f = lambda *s: (rng.standard_normal(s) * 0.05).astype(np.float16)
    return dict(w_qkv=f(HID, (H + 2 * HKV) * 128), w_o=f(HID, HID), w13=f(HID, 2 * INTER), w2=f(INTER, HID),
                ffn_norm=np.ones(HID, np.float16), x=f(3, HID) * 10, h=f(3, HID) * 10)


def _layer(w, cols, heads, kv_heads, reduce):
    """attention + ffn of one decode step on (a shard of) the weights; `reduce` sums partial outputs."""
    lengths = np.array([0, 1, 2], np.int32)
    rng = np.random.default_rng(1)
    kc_full = [rng.standard_normal((HKV, S, 128)).astype(np.float16) for _ in range(3)]
    vc_full = [rng.standard_normal((HKV, S, 128)).astype(np.float16) for _ in range(3)]
    kvh0 = cols["kv_head0"]
    kc = [k[kvh0:kvh0 + kv_heads].copy() for k in kc_full]
    vc = [v[kvh0:kvh0 + kv_heads].copy() for v in vc_full]
    qkv = gemm.gemm_s4_f16(w["h"], w["w_qkv"][:, cols["qkv_cols"]])
    ctx = np.zeros((3, heads * 128), np.float16)
    oa.mmha_decode(qkv, kc, vc, lengths, heads, kv_heads, 128, S, out=ctx)
    a = reduce(gemm.gemm_s4_f16(ctx, w["w_o"][cols["o_rows"]]))
    x, h = norm.add_residual_rmsnorm(w["x"], a, None, w["ffn_norm"], 1e-6)
    f = gemm.gemm_s4_f16(h, w["w13"][:, cols["w13_cols"]], fused_silu=True)
    f = reduce(gemm.gemm_s4_f16(f, w["w2"][cols["w2_rows"]]))
    return x, f


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from lmdeploy_b200.llama import LlamaConfig, tp_column_index
    cfg = LlamaConfig(H, HKV, INTER, 1, vocab_size=1000)
    cols = tp_column_index(cfg, world, rank)
    cols["kv_head0"] = rank * (HKV // world)

    def reduce(partial):
        t = torch.from_numpy(partial.astype(np.float32))      # fp16 sum like ncclHalf, emulated in fp32 then rounded
        dist.all_reduce(t)
        return t.numpy().astype(np.float16)

    x, f = _layer(_weights(), cols, H // world, HKV // world, reduce)
    if rank == 0:
        q.put((x, f))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded_layer():
    from lmdeploy_b200.llama import LlamaConfig, tp_column_index
    cfg = LlamaConfig(H, HKV, INTER, 1, vocab_size=1000)
    full = tp_column_index(cfg, 1, 0)
    full["kv_head0"] = 0
    x_want, f_want = _layer(_weights(), full, H, HKV, lambda p: p)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    x_got, f_got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert np.abs(x_got.astype(np.float32) - x_want.astype(np.float32)).max() <= 2e-2
    assert np.abs(f_got.astype(np.float32) - f_want.astype(np.float32)).max() <= 2e-2


def test_column_index_covers_everything_once():
    from lmdeploy_b200.llama import LLAMA2_70B, tp_column_index
    for tp in (1, 2, 4, 8):
        parts = [tp_column_index(LLAMA2_70B, tp, r) for r in range(tp)]
        for key, total in (("qkv_cols", (64 + 16) * 128), ("o_rows", 8192), ("w13_cols", 2 * 28672), ("w2_rows", 28672)):
            allidx = np.concatenate([p[key] for p in parts])
            assert len(allidx) == total and len(np.unique(allidx)) == total
        assert all(len(p["qkv_cols"]) % 128 == 0 and len(p["w2_rows"]) % 128 == 0 for p in parts)
