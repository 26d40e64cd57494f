"""Worker of tests/test_gpu_tp_prefill.py: one tensor-parallel rank per GPU (torchrun, NCCL).  A small random-init model
is run two ways on every rank — prompts through tm_llama_prefill then one decode step, and the same prompts token by
token through the decode driver — and the logits after the last prompt token and the cached keys must agree.  Both
routes end in the same all-reduce / all-gather sequence, so agreement also means the ranks stayed in step."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from lmdeploy_b200 import llama
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = llama.Comm(world, rank, local)
    cfg = llama.LlamaConfig(head_num=8, kv_head_num=4, inter_size=2048, num_layer=2, vocab_size=1024, quant_policy=0, name="tiny")
    model = llama.LlamaModel(cfg, 4, 64, local, comm)
    model.random_init(seed=3)
    rng = np.random.default_rng(5)
    prompts = [list(rng.integers(0, cfg.vocab_size, size=n)) for n in (20, 33, 7, 2)]
    B, pmax = len(prompts), max(len(p) for p in prompts)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        # token by token
        start = np.array([pmax - len(p) for p in prompts], np.int32)
        forced = np.full((pmax, B), -1, np.int32)
        for b, p in enumerate(prompts):
            forced[start[b]:pmax, b] = p
        st = model.new_state(B, pmax, start, forced, keep_logits=True)
        model.decode(st, pmax, use_graph=True)
        model.handle.check_device_status(stream.cuda_stream)
        logits_a, k_a = st.logits.cpu().numpy(), st.k_cache.float().cpu().numpy()
        # prefill + one step
        st2 = model.new_state(B, 1, np.zeros(B, np.int32), np.asarray([[p[-1] for p in prompts]], np.int32), keep_logits=True)
        model.prefill(st2, [p[:-1] for p in prompts])
        model.decode(st2, 1, use_graph=False)
        model.handle.check_device_status(stream.cuda_stream)
        logits_b, k_b = st2.logits.cpu().numpy(), st2.k_cache.float().cpu().numpy()
    err = np.abs(logits_a - logits_b)
    rel = err.mean() / np.abs(logits_a).mean()
    kerr = max(np.abs(k_a[b, :, :, :len(p)] - k_b[b, :, :, :len(p)]).max() for b, p in enumerate(prompts))
    ok = err.max() <= 3e-2 and rel <= 5e-3 and kerr <= 3e-2 and np.isfinite(logits_b).all()
    flag = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"TP_PREFILL world={world} max_abs={err.max():.3e} mean_rel={rel:.3e} k_max_abs={kerr:.3e} "
              f"{'OK' if int(flag.item()) else 'FAIL'}", flush=True)
    model.close()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) else 1)


if __name__ == "__main__":
    main()
