"""Benchmark of the B200 W4A16 decode hot path.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (``config.workload``):
  gemm      W4A16 GEMM over the four Llama-2-7B projections at ``--tokens`` tokens; a step is one
            pass over the four linears of a layer.  Inputs larger than L2: the weights of every
            projection are replicated until they exceed twice the L2 size and each launch takes
            the next replica.

The timed region is bracketed by a barrier + ``torch.cuda.synchronize()``; device time comes from
CUDA events on the launching stream; SM clocks and throttle reasons are sampled with nvidia-smi
during the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LLAMA7B_PROJ = [("qkv", 12288, 4096, False), ("o", 4096, 4096, False), ("gate_up", 22016, 4096, True),
                ("down", 4096, 11008, False)]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def gemm_bytes(n, k, t, fused):
    """algorithmic bytes of one W4A16 GEMM: int4 weight + {zero, scale} + activations in + out."""
    n_out = n // 2 if fused else n
    return k * n // 2 + (k // 128) * n * 4 + t * k * 2 + t * n_out * 2


def build_gemm_case(name, n, k, fused, tokens, l2_bytes, device, seed):
    """Random packed weights (any nibble pattern is a valid int4 weight) replicated beyond 2x L2."""
    g = torch.Generator(device=device).manual_seed(seed)
    per = k * n // 2 + (k // 128) * n * 4
    reps = max(2, int(2 * l2_bytes // per) + 1)
    A = torch.randint(-2 ** 31, 2 ** 31 - 1, (reps, k, n // 8), dtype=torch.int32, device=device, generator=g)
    z = torch.randint(64, 80, (reps, k // 128, n, 1), device=device, generator=g).half()
    s = (torch.rand(reps, k // 128, n, 1, device=device, generator=g) * 0.01 + 0.002).half()
    Q = torch.cat([z, s], dim=-1).contiguous()
    X = torch.randn(reps, tokens, k, device=device, generator=g).half()
    Y = torch.empty(reps, tokens, n // 2 if fused else n, dtype=torch.float16, device=device)
    return dict(name=name, n=n, k=k, fused=fused, A=A, Q=Q, X=X, Y=Y, reps=reps)


def run_gemm_workload(args, rank, world, device):
    from lmdeploy_b200 import turbomind as tm
    from lmdeploy_b200 import lib as l
    torch.cuda.set_device(device)
    h = l.default_handle(device)
    l2 = torch.cuda.get_device_properties(device).L2_cache_size
    T = args.tokens
    cases = [build_gemm_case(nm, n, k, fz, T, l2, device, 1000 + i) for i, (nm, n, k, fz) in enumerate(LLAMA7B_PROJ)]
    op = tm.LlamaLinear(device)
    weights = [[tm.LlamaDenseWeight(c["k"], c["n"], c["A"][r], tm.WeightType.kINT4, None, c["Q"][r], 128)
                for r in range(c["reps"])] for c in cases]

    def step(i):
        for c, ws in zip(cases, weights):
            r = i % c["reps"]
            op.forward(c["Y"][r], c["X"][r], T, ws[r], op.kFusedSiluFfn if c["fused"] else op.kGemm)

    def one(c, ws, i):
        r = i % c["reps"]
        op.forward(c["Y"][r], c["X"][r], T, ws[r], op.kFusedSiluFfn if c["fused"] else op.kGemm)

    # The launches are replayed from CUDA graphs so that the device, not the Python caller,
    # sets the pace.  One graph = `ring` consecutive steps (every step takes the next replica).
    ring = max(c["reps"] for c in cases)
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step(i)
        h.check_device_status(stream.cuda_stream)
        g_step = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_step, stream=stream):
            for i in range(ring):
                step(i)
        g_one = {}
        for c, ws in zip(cases, weights):
            g_one[c["name"]] = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_one[c["name"]], stream=stream):
                for i in range(c["reps"]):
                    one(c, ws, i)
        n_replay = max(1, (args.steps + ring - 1) // ring)
        steps_done = n_replay * ring
        g_step.replay()
        barrier(world)
        torch.cuda.synchronize()
        sampler = ClockSampler(device)
        sampler.start()
        launches0 = h.launch_count()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record(stream)
        for _ in range(n_replay):
            g_step.replay()
        ev[1].record(stream)
        torch.cuda.synchronize()
        barrier(world)
        ms = ev[0].elapsed_time(ev[1])
        launches = n_replay * ring * len(cases)
        h.check_device_status(stream.cuda_stream)

        # per-kernel device time: a graph of `reps` launches of one projection, replayed
        per = {}
        for c in cases:
            g = g_one[c["name"]]
            n_rep = max(3, 200 // c["reps"])
            g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(n_rep):
                g.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (n_rep * c["reps"])
            b = gemm_bytes(c["n"], c["k"], T, c["fused"])
            per[c["name"]] = dict(us=round(us, 3), gbs=round(b / us * 1e-3, 1), bytes=b)
        clocks = sampler.stop()
    args.steps = steps_done

    bytes_step = sum(gemm_bytes(c["n"], c["k"], T, c["fused"]) for c in cases)
    ms_step = max_over_ranks(ms / args.steps, world)
    peaks = measured_peaks()
    gbs = bytes_step / (ms_step * 1e-3) * 1e-9 * world
    dom = per["gate_up"]
    out = {
        "metric": "W4 GEMM HBM GB/s vs peak (Llama-2-7B projections)", "value": round(gbs, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 x int4 -> f32 accumulate",
        "data": "synthetic",
        "config": {"workload": "gemm", "tokens": T, "shapes": [c["name"] for c in cases],
                   "l2": "inputs larger than L2: weights replicated beyond 2x L2, next replica each launch",
                   "parallelism": "replicas only" if world > 1 else "single GPU"},
        "roofline": {"bound": "hbm", "kernel": "gemm_s4_f16_small_kernel (gate_up)", "achieved": dom["gbs"],
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(dom["gbs"] / peaks["hbm_gbs"], 4),
                     "peak_source": peaks["source"], "traffic": None},
        "per_kernel": per, "clocks": clocks, "gpu_launches": int(launches),
    }
    return out


def mmha_bytes(lengths, H, Hkv, e):
    """algorithmic bytes of one decode-attention call (KV counted once per KV head)."""
    B = len(lengths)
    return int(sum(2 * Hkv * int(L) * 128 * e for L in lengths) + B * (H + 2 * Hkv) * 128 * 2 + B * H * 128 * 2
               + B * 2 * Hkv * 128 * e)


def run_mmha_workload(args, rank, world, device):
    """Decode attention, batch 64, 32 heads of 128, KV length ~ U[128, 4096], int8 or fp16 cache.
    Inputs larger than L2: one call reads ~1.1 GB (int8) / ~2.2 GB (fp16) of cache."""
    import math
    from lmdeploy_b200 import turbomind as tm
    from lmdeploy_b200 import lib as l
    torch.cuda.set_device(device)
    h = l.default_handle(device)
    B, H, Hkv, D, S_max = args.batch, args.heads, args.kv_heads, 128, 4224
    int8 = args.kv == "int8"
    rng = np.random.default_rng(1234 + rank)
    lengths = rng.integers(128, 4097, size=B).astype(np.int32)
    g = torch.Generator(device=device).manual_seed(7 + rank)
    if int8:
        kc = torch.randint(-127, 128, (B, Hkv, S_max, D), dtype=torch.int8, device=device, generator=g)
        vc = torch.randint(-127, 128, (B, Hkv, S_max, D), dtype=torch.int8, device=device, generator=g)
    else:
        kc = torch.randn(B, Hkv, S_max, D, device=device, generator=g).half()
        vc = torch.randn(B, Hkv, S_max, D, device=device, generator=g).half()
    kp = torch.tensor([kc[b].data_ptr() for b in range(B)], dtype=torch.int64, device=device)
    vp = torch.tensor([vc[b].data_ptr() for b in range(B)], dtype=torch.int64, device=device)
    qkv = torch.randn(B, (H + 2 * Hkv) * D, device=device, generator=g).half()
    out = torch.empty(B, H * D, dtype=torch.float16, device=device)
    ld = torch.from_numpy(lengths).to(device)
    ts = int(lengths.max())
    pad = torch.from_numpy((ts - lengths).astype(np.int32)).to(device)
    p = tm.Masked_multihead_attention_params(
        out=out, q=qkv, k=qkv[:, H * D:], v=qkv[:, (H + Hkv) * D:], stride=(H + 2 * Hkv) * D, batch_size=B,
        memory_max_len=S_max, num_heads=H, num_kv_heads=Hkv, timestep=ts, inv_sqrt_dh=1.0 / math.sqrt(D),
        total_padding_tokens=pad, length_per_sample=ld, k_cache_per_sample=kp, v_cache_per_sample=vp)
    if int8:
        p.int8_mode = tm.QUANT_POLICY_CACHE_KV_INT8
        p.attention_k_scale = p.attention_v_scale = 4.0 / 127.0
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            tm.masked_multihead_attention(p)
        h.check_device_status(stream.cuda_stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            tm.masked_multihead_attention(p)
        graph.replay()
        barrier(world)
        torch.cuda.synchronize()
        sampler = ClockSampler(device)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        barrier(world)
        ms = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop()
        h.check_device_status(stream.cuda_stream)
    ms = max_over_ranks(ms, world)
    nbytes = mmha_bytes(lengths, H, Hkv, 1 if int8 else 2)
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) * 1e-9
    return {
        "metric": "decode MMHA HBM GB/s vs peak", "value": round(gbs * world, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": f"f16 q, {args.kv} KV, f32 softmax/accumulate",
        "data": "synthetic",
        "config": {"workload": "mmha", "batch": B, "heads": H, "kv_heads": Hkv, "kv": args.kv,
                   "kv_len": "uniform 128..4096", "l2": "inputs larger than L2 (one call reads > 1 GB of KV cache)",
                   "parallelism": "replicas only" if world > 1 else "single GPU"},
        "roofline": {"bound": "hbm", "kernel": "mmha_decode_kernel", "achieved": round(gbs, 1),
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                     "peak_source": peaks["source"], "traffic": None},
        "clocks": clocks, "gpu_launches": args.steps,
    }


def barrier(world):
    if world > 1:
        torch.distributed.barrier()


def max_over_ranks(v, world):
    if world == 1:
        return v
    t = torch.tensor([v], dtype=torch.float64, device="cuda")
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="gemm")
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=32)
    ap.add_argument("--kv", default="int8", choices=["int8", "fp16"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))

    if args.workload == "gemm":
        out = run_gemm_workload(args, rank, world, local)
    elif args.workload == "mmha":
        out = run_mmha_workload(args, rank, world, local)
    else:
        raise SystemExit(f"unknown workload {args.workload}")
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
