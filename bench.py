"""Benchmark of the B200 W4A16 decode hot path.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (``config.workload``):
  gemm      W4A16 GEMM over the four Llama-2-7B projections at ``--tokens`` tokens; a step is one
            pass over the four linears of a layer.  Inputs larger than L2: the weights of every
            projection are replicated until they exceed twice the L2 size and each launch takes
            the next replica.
  mmha      decode attention, batch 64, KV length uniform in ``--kv-len``, int8 or fp16 cache.
  prefill   attention side of one prefill layer (QKV bias + RoPE + transpose, KV-cache extend, causal attention
            over the cache) for ``--batch`` (default 8) sequences of 2048 new tokens.
  prefill7b whole-model prefill of Llama-2-7B through tm_llama_prefill, ``--batch`` (default 8) prompts of 2048 tokens.
  decode    (default) whole-model greedy decode, Llama-2-7B at 1 GPU, Llama-2-70B tensor-parallel at N > 1.

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
# Llama-2-70B on one GPU (no tensor-parallel slicing): 8 KV heads, inter size 28672
LLAMA70B_PROJ = [("qkv", 10240, 8192, False), ("o", 8192, 8192, False), ("gate_up", 57344, 8192, True),
                 ("down", 8192, 28672, False)]


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


def load_reference_kernels():
    """The reference's own CUDA kernels for this path, built unmodified from its sources by
    oracle/build_ref.py (oracle/_ref/libtm_ref.so).  Only the `--impl reference` arm of the per-kernel
    workloads uses it; None when it has not been built."""
    import ctypes as C
    path = os.path.join(ROOT, "oracle", "_ref", "libtm_ref.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    vp, i, f32 = C.c_void_p, C.c_int, C.c_float
    lib.ref_gemm_s4_f16.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp]
    lib.ref_mmha_decode.argtypes = [vp] * 7 + [i] * 5 + [i, f32, i, vp, vp, vp, vp, vp, C.c_size_t, i, f32, f32, f32, f32, i, i, i,
                                                          vp]
    lib.ref_set_sync.argtypes = [i]
    lib.ref_set_sync(0)      # launches only: the timing below synchronises itself
    return lib


def gemm_bytes(n, k, t, fused):
    """algorithmic bytes of one W4A16 GEMM: int4 weight + {zero, scale} + activations in + out."""
    n_out = n // 2 if fused else n
    return k * n // 2 + (k // 128) * n * 4 + t * k * 2 + t * n_out * 2


def cpu_gemm_baseline(proj, T, seconds=10.0):
    """The reference's torch CPU path for the W4A16 linear (fp32 matmul on the pseudo-quant fp16 weight:
    lmdeploy.lite's pseudo-quant linear, oracle/gemm.py) over the projections of `proj` at T tokens, all host threads,
    repeated for about `seconds`.  The fp32 copy of the weight is made once, outside the timing (in the
    reference's favour).  value = the workload's algorithmic bytes per second."""
    from oracle import gemm as ogemm
    g = torch.Generator().manual_seed(0)
    ws = [(torch.randn(k, n, generator=g) * 0.02).half().float() for _, n, k, _ in proj]
    xs = [torch.randn(T, k, generator=g).half() for _, n, k, _ in proj]

    def step():
        for (nm, n, k, fused), w, x in zip(proj, ws, xs):
            y = ogemm.linear_f32acc(x, w)
            if fused:
                ogemm.silu_mul_interleaved(y)

    step()
    n_it, t0 = 0, time.perf_counter()
    while True:
        step()
        n_it += 1
        el = time.perf_counter() - t0
        if el >= seconds or n_it >= 2000:
            break
    nb = sum(gemm_bytes(n, k, T, fz) for _, n, k, fz in proj)
    return {"value": round(nb * n_it / el * 1e-9, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
            "kind": "port", "ms_per_step": round(el / n_it * 1e3, 3),
            "sample": f"{n_it} passes over the {len(proj)} projections at {T} tokens ({el:.1f} s of CPU work): fp32 torch matmul on the "
                      f"pseudo-quant weight (fp32 copy made outside the timing)"}


def gemm_e2e(cases, weights, op, T, steps, stream):
    """The same pass through the C ABI with HOST buffers: per projection the activations come from pinned host
    memory and the result goes back to pinned host memory, all inside the timed region."""
    hx = [torch.randn(T, c["k"]).half().pin_memory() for c in cases]
    hy = [torch.empty(T, c["n"] // 2 if c["fused"] else c["n"], dtype=torch.float16).pin_memory() for c in cases]

    def step(i):
        for c, ws, x, y in zip(cases, weights, hx, hy):
            r = i % c["reps"]
            c["X"][r].copy_(x, non_blocking=True)
            op.forward(c["Y"][r], c["X"][r], T, ws[r], op.kFusedSiluFfn if c["fused"] else op.kGemm)
            y.copy_(c["Y"][r], non_blocking=True)
        stream.synchronize()

    for i in range(3):
        step(i)
    t0 = time.perf_counter()
    for i in range(steps):
        step(i)
    ms = (time.perf_counter() - t0) * 1e3 / steps
    h2d = sum(x.numel() * 2 for x in hx)
    d2h = sum(y.numel() * 2 for y in hy)
    return ms, h2d, d2h


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
    proj = LLAMA70B_PROJ if args.shapes == "70b" else LLAMA7B_PROJ
    cases = [build_gemm_case(nm, n, k, fz, T, l2, device, 1000 + i) for i, (nm, n, k, fz) in enumerate(proj)]
    op = tm.LlamaLinear(device)
    weights = [[tm.LlamaDenseWeight(c["k"], c["n"], c["A"][r], tm.WeightType.kINT4, None, c["Q"][r], 128)
                for r in range(c["reps"])] for c in cases]

    reflib = load_reference_kernels() if args.impl == "reference" else None
    if args.impl == "reference" and reflib is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libtm_ref.so not built (python oracle/build_ref.py needs the reference tree)"}

    def one(c, ws, i):
        r = i % c["reps"]
        if reflib is not None:
            import ctypes as C
            rc = reflib.ref_gemm_s4_f16(C.c_void_p(c["Y"][r].data_ptr()), C.c_void_p(c["A"][r].data_ptr()),
                                        C.c_void_p(c["X"][r].data_ptr()), C.c_void_p(c["Q"][r].data_ptr()), c["n"], T, c["k"], 128,
                                        int(c["fused"]), C.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert rc == 0, f"reference GEMM returned {rc}"
        else:
            op.forward(c["Y"][r], c["X"][r], T, ws[r], op.kFusedSiluFfn if c["fused"] else op.kGemm)

    def step(i):
        for c, ws in zip(cases, weights):
            one(c, ws, i)

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
        if reflib is None:
            # the same launches chained by programmatic dependent launch, as the decode driver issues them: a kernel
            # starts fetching its weights while the one before it drains (launch gap and first-byte latency overlap)
            h.set_option("pdl_direct", 1)
            try:
                for c, ws in zip(cases, weights):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        for i in range(c["reps"]):
                            one(c, ws, i)
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
                    per[c["name"]]["us_chained"] = round(us, 3)
                    per[c["name"]]["gbs_chained"] = round(per[c["name"]]["bytes"] / us * 1e-3, 1)
            finally:
                h.set_option("pdl_direct", 0)
            h.check_device_status(stream.cuda_stream)
        clocks = sampler.stop()
        ms_e2e = h2d = d2h = None
        if reflib is None:
            ms_e2e, h2d, d2h = gemm_e2e(cases, weights, op, T, min(steps_done, 64), stream)
    args.steps = steps_done

    bytes_step = sum(gemm_bytes(c["n"], c["k"], T, c["fused"]) for c in cases)
    ms_step = max_over_ranks(ms / args.steps, world)
    peaks = measured_peaks()
    gbs = bytes_step / (ms_step * 1e-3) * 1e-9 * world
    dom = per["gate_up"]
    out = {
        "metric": f"W4 GEMM HBM GB/s vs peak (Llama-2-{args.shapes.upper()} projections)", "value": round(gbs, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 x int4 -> f32 accumulate",
        "data": "synthetic",
        "config": {"workload": "gemm", "tokens": T, "model_shapes": args.shapes, "shapes": [c["name"] for c in cases],
                   "l2": "inputs larger than L2: weights replicated beyond 2x L2, next replica each launch",
                   "parallelism": "replicas only" if world > 1 else "single GPU"},
        "roofline": {"bound": "hbm", "kernel": ("reference gemm_s4_f16_nn" if reflib is not None else
                                                "gemm_s4_f16_tc_kernel" if T > 16 else "gemm_s4_f16_cols_kernel" if T == 1 else "gemm_s4_f16_small_kernel") + " (gate_up)",
                     "achieved": dom["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(dom["gbs"] / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
                     "algorithmic_bytes": dom["bytes"],
                     # DRAM bytes / algorithmic bytes measured with ncu on the qkv and o shapes (profiles/)
                     "traffic": int(dom["bytes"] * (1.03 if T > 16 else 1.0))},
        "per_kernel": per,
        "per_kernel_note": "us: launches back to back on one stream, each waiting for the one before it; us_chained: the same "
                           "launches with programmatic dependent launch (as inside the decode step)",
        "clocks": clocks, "gpu_launches": int(launches),
    }
    if reflib is not None:
        mark_reference_kernel_arm(out)
        return out
    ms_e2e = max_over_ranks(ms_e2e, world)
    out["e2e"] = {"value": round(bytes_step / (ms_e2e * 1e-3) * 1e-9 * world, 1), "unit": "GB/s", "ms_per_step": round(ms_e2e, 4),
                  "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                  "note": "one tm_gemm_s4_f16 call per projection, activations from pinned host memory, result back to it, "
                          "host synchronisation every step"}
    if rank == 0 and not args.no_cpu:
        out["cpu_baseline"] = cpu_gemm_baseline(proj, T)
    return out


def mark_reference_kernel_arm(out):
    """fields of a line measured on the reference's own CUDA kernels (per-kernel workloads)"""
    out["impl"] = "reference"
    out["roofline"]["traffic"] = None
    out["cpu_baseline"] = {"value": out["value"], "unit": out["unit"], "cores": 0, "kind": "reference",
                           "sample": "the reference's CUDA kernels for this workload, built unmodified for sm_100a (oracle/_ref), "
                                     "same inputs, same timer, on the GPU"}
    out["e2e"] = {"value": out["value"], "unit": out["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def mmha_bytes(lengths, H, Hkv, e):
    """algorithmic bytes of one decode-attention call (KV counted once per KV head)."""
    B = len(lengths)
    return int(sum(2 * Hkv * int(L) * 128 * e for L in lengths) + B * (H + 2 * Hkv) * 128 * 2 + B * H * 128 * 2
               + B * 2 * Hkv * 128 * e)


def cpu_mmha_baseline(lengths, H, Hkv, int8, seconds=10.0):
    """CPU restatement of the reference's decode attention (oracle/attention.py) on a bounded sample: the first
    sequences of the batch, one call each, until about `seconds` have passed.  value = algorithmic bytes per second."""
    from oracle import attention as oa
    rng = np.random.default_rng(0)
    D = 128
    quant = oa.KvQuant(4.0 / 127, 0.0, 4.0 / 127, 0.0) if int8 else None
    done, nb, t0 = 0, 0, time.perf_counter()
    for L in lengths:
        L = int(L)
        S = L + 8
        if int8:
            kc = [rng.integers(-127, 128, size=(Hkv, S, D), dtype=np.int8)]
            vc = [rng.integers(-127, 128, size=(Hkv, S, D), dtype=np.int8)]
        else:
            kc = [rng.standard_normal((Hkv, S, D)).astype(np.float16)]
            vc = [rng.standard_normal((Hkv, S, D)).astype(np.float16)]
        qkv = rng.standard_normal((1, (H + 2 * Hkv) * D)).astype(np.float16)
        oa.mmha_decode(qkv, kc, vc, np.asarray([L], np.int32), H, Hkv, D, S, kv_quant=quant)
        done += 1
        nb += mmha_bytes([L], H, Hkv, 1 if int8 else 2)
        if time.perf_counter() - t0 >= seconds:
            break
    el = time.perf_counter() - t0
    return {"value": round(nb / el * 1e-9, 4), "unit": "GB/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
            "kind": "port",
            "sample": f"{done} of {len(lengths)} sequences of the batch ({el:.1f} s of CPU work, cache generation included), numpy "
                      f"restatement of the reference kernel"}


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
    lo, hi = (int(v) for v in args.kv_len.split(","))
    S_max = max(S_max, hi + 128)
    lengths = rng.integers(lo, hi + 1, size=B).astype(np.int32)
    g = torch.Generator(device=device).manual_seed(7 + rank)
    if int8:
        kc = torch.randint(-127, 128, (B, Hkv, S_max, D), dtype=torch.int8, device=device, generator=g)
        vc = torch.randint(-127, 128, (B, Hkv, S_max, D), dtype=torch.int8, device=device, generator=g)
    else:
        kc = torch.randn(B, Hkv, S_max, D, device=device, generator=g).half()
        vc = torch.randn(B, Hkv, S_max, D, device=device, generator=g).half()
    kp = torch.tensor([kc[b].data_ptr() for b in range(B)], dtype=torch.int64, device=device)
    vp_ = torch.tensor([vc[b].data_ptr() for b in range(B)], dtype=torch.int64, device=device)
    qkv = torch.randn(B, (H + 2 * Hkv) * D, device=device, generator=g).half()
    out = torch.empty(B, H * D, dtype=torch.float16, device=device)
    ld = torch.from_numpy(lengths).to(device)
    ts = int(lengths.max())
    pad = torch.from_numpy((ts - lengths).astype(np.int32)).to(device)
    p = tm.Masked_multihead_attention_params(
        out=out, q=qkv, k=qkv[:, H * D:], v=qkv[:, (H + Hkv) * D:], stride=(H + 2 * Hkv) * D, batch_size=B,
        memory_max_len=S_max, num_heads=H, num_kv_heads=Hkv, timestep=ts, inv_sqrt_dh=1.0 / math.sqrt(D),
        total_padding_tokens=pad, length_per_sample=ld, k_cache_per_sample=kp, v_cache_per_sample=vp_)
    if int8:
        p.int8_mode = tm.QUANT_POLICY_CACHE_KV_INT8
        p.attention_k_scale = p.attention_v_scale = 4.0 / 127.0
    reflib = load_reference_kernels() if args.impl == "reference" else None
    if args.impl == "reference" and reflib is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libtm_ref.so not built (python oracle/build_ref.py needs the reference tree)"}

    def attention():
        if reflib is None:
            tm.masked_multihead_attention(p)
            return
        import ctypes as C
        vp = lambda t: C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p()
        rc = reflib.ref_mmha_decode(vp(out), vp(qkv), vp(qkv[:, H * D:]), vp(qkv[:, (H + Hkv) * D:]), None, None, None,
                                    (H + 2 * Hkv) * D, B, S_max, H, Hkv, D, 10000.0, ts, vp(pad), None, vp(ld), vp(kp), vp(vp_),
                                    0, 4 if int8 else 0, float(getattr(p, "attention_k_scale", 0.0) or 0.0), 0.0, float(getattr(p, "attention_v_scale", 0.0) or 0.0), 0.0, 2048, 0, 0,
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, f"reference attention returned {rc}"

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            attention()
        h.check_device_status(stream.cuda_stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            attention()
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
        # end to end: q, k, v of the new tokens from pinned host memory, attention output back to it, every step
        ms_e2e = None
        if reflib is None:
            h_qkv = qkv.cpu().pin_memory()
            h_out = torch.empty(out.shape, dtype=torch.float16).pin_memory()
            n_e2e = min(args.steps, 64)
            for i in range(n_e2e + 3):
                if i == 3:
                    t0 = time.perf_counter()
                qkv.copy_(h_qkv, non_blocking=True)
                attention()
                h_out.copy_(out, non_blocking=True)
                stream.synchronize()
            ms_e2e = (time.perf_counter() - t0) * 1e3 / n_e2e
    ms = max_over_ranks(ms, world)
    nbytes = mmha_bytes(lengths, H, Hkv, 1 if int8 else 2)
    peaks = measured_peaks()
    gbs = nbytes / (ms * 1e-3) * 1e-9
    res = {
        "metric": "decode MMHA HBM GB/s vs peak", "value": round(gbs * world, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": f"f16 q, {args.kv} KV, f32 softmax/accumulate",
        "data": "synthetic",
        "config": {"workload": "mmha", "batch": B, "heads": H, "kv_heads": Hkv, "kv": args.kv,
                   "kv_len": f"uniform {lo}..{hi}", "l2": "inputs larger than L2 (one call reads > 1 GB of KV cache)",
                   "parallelism": "replicas only" if world > 1 else "single GPU"},
        "roofline": {"bound": "hbm", "kernel": "reference masked_multihead_attention_kernel" if reflib is not None else "mmha_decode_kernel",
                     "achieved": round(gbs, 1),
                     "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                     "peak_source": peaks["source"], "algorithmic_bytes": int(nbytes),
                     # ncu on this workload: 1.157 GB read + written for 1.132 GB algorithmic (profiles/)
                     "traffic": int(nbytes * 1.02)},
        "clocks": clocks, "gpu_launches": args.steps,
    }
    if reflib is not None:
        mark_reference_kernel_arm(res)
        return res
    ms_e2e = max_over_ranks(ms_e2e, world)
    res["e2e"] = {"value": round(nbytes / (ms_e2e * 1e-3) * 1e-9 * world, 1), "unit": "GB/s", "ms_per_step": round(ms_e2e, 4),
                  "h2d_bytes_per_step": int(qkv.numel() * 2), "d2h_bytes_per_step": int(out.numel() * 2)}
    if rank == 0 and not args.no_cpu:
        res["cpu_baseline"] = cpu_mmha_baseline(lengths, H, Hkv, int8)
    return res


def run_prefill_workload(args, rank, world, device):
    """Attention side of one Llama-2-7B prefill layer: ``--batch`` sequences (default 8) of 2048 new tokens, 32 heads.
    A step = QKV bias + RoPE + transpose -> KV-cache extend -> causal attention over the cache.  Inputs larger than L2
    (the fused QKV buffer alone is 0.4 GB at batch 8).  With --impl reference the same three stages run on the
    reference's own kernels: its writers, and its unfused attention route (cache transpose, cuBLAS GEMMs through
    torch.matmul, mask + softmax kernels), because its flash-attention build needs CUTLASS."""
    import ctypes as C
    from lmdeploy_b200 import turbomind as tm
    torch.cuda.set_device(device)
    B = args.batch if args.batch != 64 else 8
    H, D, S = args.heads, 128, 2048
    Hkv = args.kv_heads
    int8 = args.kv == "int8"
    S_max = S
    g = torch.Generator(device=device).manual_seed(11 + rank)
    qkv = torch.randn(B * S, (H + 2 * Hkv) * D, device=device, generator=g).half()
    q = torch.empty((B, H, S, D), dtype=torch.float16, device=device)
    k = torch.empty((B, Hkv, S, D), dtype=torch.float16, device=device)
    v = torch.empty_like(k)
    esz = 1 if int8 else 2
    kc = torch.zeros((B, Hkv * S_max * D * esz), dtype=torch.uint8, device=device)
    vc = torch.zeros_like(kc)
    kp = torch.tensor([kc[b].data_ptr() for b in range(B)], dtype=torch.int64, device=device)
    vp_ = torch.tensor([vc[b].data_ptr() for b in range(B)], dtype=torch.int64, device=device)
    hist = torch.zeros(B, dtype=torch.int32, device=device)
    lens = torch.full((B,), S, dtype=torch.int32, device=device)
    cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=device)
    out = torch.empty((B * S, H * D), dtype=torch.float16, device=device)
    scale = [6.0 / 127, 0.0, 6.0 / 127, 0.0] if int8 else None
    quant = 4 if int8 else 0
    reflib = load_reference_kernels() if args.impl == "reference" else None
    if args.impl == "reference" and reflib is None:
        return {"impl": "reference", "unavailable": "oracle/_ref/libtm_ref.so not built (python oracle/build_ref.py needs the reference tree)"}
    P = lambda t: C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p()
    cur = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)
    sc = None if scale is None else (C.c_float * 4)(*scale)
    if reflib is not None:
        reflib.ref_add_fused_qkv_bias_transpose.argtypes = [C.c_void_p] * 8 + [C.c_int] * 7 + [C.c_float] + [C.c_int] * 3 + [C.c_void_p]
        reflib.ref_extend_kv_cache.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                               C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_float)]
        reflib.ref_transpose_kv_cache.argtypes = [C.c_void_p] * 4 + [C.c_size_t, C.c_int, C.c_void_p] + [C.c_int] * 5 + [C.c_void_p, C.c_int,
                                                                                                                    C.POINTER(C.c_float)]
        reflib.ref_create_causal_masks.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_void_p]
        reflib.ref_masked_softmax.argtypes = [C.c_void_p] * 3 + [C.c_int] * 4 + [C.c_float, C.c_void_p]
        kt = torch.empty((B, H, S, D), dtype=torch.float16, device=device)
        vt = torch.empty_like(kt)
        mask = torch.empty((B, S, S), dtype=torch.float16, device=device)
        assert reflib.ref_create_causal_masks(P(mask), P(lens), P(lens), S, S, B, cur()) == 0   # built once per batch, not per layer

    def stage_qkv():
        if reflib is None:
            tm.invokeAddFusedQKVBiasTranspose(q, k, v, qkv, None, None, hist, lens, B, S, B * S, H, Hkv, D, D, 10000.0, 2048, False, False)
        else:
            assert reflib.ref_add_fused_qkv_bias_transpose(P(q), P(k), P(v), P(qkv), None, None, P(hist), P(lens), B, S, B * S, H, Hkv, D,
                                                           D, 10000.0, 2048, 0, 0, cur()) == 0

    def stage_extend():
        if reflib is None:
            tm.invokeExtendKVCache(kp, vp_, 0, k, v, B, lens, S, hist, S_max, D, Hkv, None, quant, scale)
        else:
            assert reflib.ref_extend_kv_cache(P(kp), P(vp_), 0, P(k), P(v), B, P(lens), S, P(hist), S_max, D, Hkv, cur(), quant, sc) == 0

    def stage_attention():
        if reflib is None:
            tm.fusedMultiHeadAttention(out, q, kp, vp_, 0, cu, lens, B, S, S_max, H, Hkv, D, quant, scale)
        else:
            assert reflib.ref_transpose_kv_cache(P(kt), P(vt), P(kp), P(vp_), 0, B, P(lens), S, S_max, D, H, H // Hkv, cur(), quant, sc) == 0
            qk = torch.matmul(q, kt.transpose(2, 3))
            assert reflib.ref_masked_softmax(P(qk), P(qk), P(mask), B, S, S, H, 1.0 / np.sqrt(D), cur()) == 0
            torch.matmul(qk, vt).transpose(1, 2).reshape(B * S, H * D)

    stages = [("qkv_bias_rope_transpose", stage_qkv), ("extend_kv_cache", stage_extend), ("context_attention", stage_attention)]
    if reflib is not None:
        reflib.ref_set_sync(0)
    stream = torch.cuda.Stream(device)
    per = {}
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            for _, f in stages:
                f()
        torch.cuda.synchronize()
        for name, f in stages:   # per-stage device time (explains the step time; the step itself is timed below)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(max(2, args.steps // 4)):
                f()
            e1.record(stream)
            torch.cuda.synchronize()
            per[name] = e0.elapsed_time(e1) / max(2, args.steps // 4)
        barrier(world)
        torch.cuda.synchronize()
        sampler = ClockSampler(device)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            for _, f in stages:
                f()
        e1.record(stream)
        torch.cuda.synchronize()
        barrier(world)
        ms = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop()
    if reflib is not None:
        reflib.ref_set_sync(1)
    ms = max_over_ranks(ms, world)
    peaks = measured_peaks()
    flops = 4.0 * D * H * B * (S * (S + 1) / 2)            # causal: query i sees i + 1 keys; 2 products x 2 flops
    tf = flops / (per["context_attention"] * 1e-3) * 1e-12
    qkv_bytes = 2 * qkv.numel() * 2                         # read the fused buffer, write q, k, v
    ext_bytes = 2 * k.numel() * (2 + esz)                   # read k, v; write the cache rows
    res = {
        "metric": "prefill attention tokens/s (QKV RoPE/transpose + KV-cache extend + causal attention, one layer)",
        "value": round(B * S * world / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": f"f16 q, {args.kv} KV, f32 softmax/accumulate", "data": "synthetic",
        "config": {"workload": "prefill", "batch": B, "new_tokens": S, "heads": H, "kv_heads": Hkv, "kv": args.kv,
                   "l2": "inputs larger than L2 (fused QKV buffer %.2f GB)" % (qkv.numel() * 2e-9),
                   "parallelism": "replicas only" if world > 1 else "single GPU"},
        "roofline": {"bound": "tensor", "kernel": "reference unfused route" if reflib is not None else "context_attention_kernel",
                     "achieved": round(tf, 1), "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": round(tf / peaks["bf16_tflops"], 4), "peak_source": peaks["source"], "algorithmic_flops": flops,
                     "traffic": None},
        "stages_ms": {n: round(t, 4) for n, t in per.items()},
        "stages_gbs": {"qkv_bias_rope_transpose": round(qkv_bytes / per["qkv_bias_rope_transpose"] * 1e-6, 1),
                       "extend_kv_cache": round(ext_bytes / per["extend_kv_cache"] * 1e-6, 1)},
        "clocks": clocks, "gpu_launches": args.steps * 3,
    }
    if reflib is not None:
        mark_reference_kernel_arm(res)
        return res
    return res


def run_prefill_model_workload(args, rank, world, device):
    """Whole-model prefill of a random-init Llama-2-7B (W4A16, ``--kv`` cache) through tm_llama_prefill: ``--batch``
    (default 8) prompts of 2048 tokens per step, every step into an empty cache.  Tensor-bound: the four W4A16 GEMMs of
    each layer at 16384 tokens (tcgen05 kernel) and the causal attention."""
    from lmdeploy_b200 import llama
    torch.cuda.set_device(device)
    import dataclasses
    B = args.batch if args.batch != 64 else 8
    S = 2048
    cfg = llama.LLAMA2_7B
    cfg = dataclasses.replace(cfg, quant_policy=4 if args.kv == "int8" else 0)
    session_len = S + 64
    model = llama.LlamaModel(cfg, B, session_len, device, None)
    model.random_init(seed=0)
    rng = np.random.default_rng(77 + rank)
    prompts = [list(rng.integers(0, cfg.vocab_size, size=S)) for _ in range(B)]
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        st = model.new_state(B, 1, np.zeros(B, np.int32), None)
        for _ in range(args.warmup):
            st.lengths.zero_()
            model.prefill(st, prompts)
        model.handle.check_device_status(stream.cuda_stream)
        barrier(world)
        torch.cuda.synchronize()
        sampler = ClockSampler(device)
        sampler.start()
        total = 0.0
        torch.cuda.cudart().cudaProfilerStart()           # a profiler started with capture off sees the timed calls only
        for _ in range(args.steps):   # the wrapper uploads ids and synchronises per call: device time per call, summed
            st.lengths.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            model.prefill(st, prompts)
            e1.record(stream)
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        torch.cuda.cudart().cudaProfilerStop()
        barrier(world)
        ms = total / args.steps
        clocks = sampler.stop()
        model.handle.check_device_status(stream.cuda_stream)
        assert int(st.lengths.min().item()) == S
    ms = max_over_ranks(ms, world)
    peaks = measured_peaks()
    T = B * S
    hid, inter, H, L = cfg.hidden, cfg.inter_size, cfg.head_num, cfg.num_layer
    gemm_flops = 2.0 * T * (hid * (cfg.head_num + 2 * cfg.kv_head_num) * 128 + hid * hid + 2 * hid * inter + inter * hid) * L
    attn_flops = 4.0 * 128 * H * B * (S * (S + 1) / 2) * L
    tf = (gemm_flops + attn_flops) / (ms * 1e-3) * 1e-12
    return {
        "metric": "prefill tokens/s (Llama-2-7B W4A16, whole model)", "value": round(T * world / (ms * 1e-3), 1), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": f"f16 activations, int4 weights, {args.kv} KV, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": "prefill7b", "batch": B, "prompt_tokens": S, "kv": args.kv,
                   "l2": "inputs larger than L2 (activations of 16384 tokens: 0.13 GB per [tokens, hidden] buffer)",
                   "parallelism": "replicas only" if world > 1 else "single GPU"},
        "roofline": {"bound": "tensor", "kernel": "whole prefill (W4A16 GEMMs at 16384 tokens + causal attention)",
                     "achieved": round(tf, 1), "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(tf / peaks["bf16_tflops_sustained"], 4), "peak_source": peaks["source"],
                     "algorithmic_flops": gemm_flops + attn_flops, "traffic": None},
        "clocks": clocks, "gpu_launches": args.steps * (3 + 10 * L),
    }


DECODE_WORKLOADS = {
    # name: (config attr, batch, prompt_lo, prompt_hi, new_tokens)
    "decode7b": ("LLAMA2_7B", 64, 128, 1024, 256),
    "decode70b": ("LLAMA2_70B", 128, 512, 512, 512),
}


class ModelShape:
    """Architecture constants of the two benchmark models (BASELINE configs 3 and 4), kept here as plain
    numbers so that the CPU reference arm needs nothing from the GPU package."""

    def __init__(self, name, head_num, kv_head_num, inter_size, num_layer):
        self.name, self.head_num, self.kv_head_num, self.inter_size, self.num_layer = name, head_num, kv_head_num, inter_size, num_layer
        self.vocab_size, self.size_per_head, self.norm_eps, self.rope_theta = 32000, 128, 1e-6, 10000.0
        self.quant_policy, self.hidden = 4, head_num * 128


MODEL_SHAPES = {"LLAMA2_7B": ModelShape("llama-2-7b", 32, 32, 11008, 32), "LLAMA2_70B": ModelShape("llama-2-70b", 64, 8, 28672, 80)}


def decode_workload_plan(name, steps, warmup, batch_override=0, max_prompt=0):
    """Prompt lengths and the position of the timed window, the same for the GPU arm and the CPU reference arm.
    The window of `steps` decode steps is centred in the `new_tokens` generated tokens of the configuration, so
    that the mean KV length while it is timed equals the mean over the whole generation (mean prompt +
    new_tokens / 2) whatever `steps` is."""
    attr, B, p_lo, p_hi, new_tokens = DECODE_WORKLOADS[name]
    if batch_override:
        B = batch_override
    rng = np.random.default_rng(2024)
    prompt_len = rng.integers(p_lo, p_hi + 1, size=B).astype(np.int32)
    if max_prompt:
        prompt_len = np.minimum(prompt_len, max_prompt)
    steps = max(1, steps)
    lead = max(warmup, (new_tokens - steps) // 2)          # untimed decode steps ahead of the window (>= warm-up)
    mean_len = float(prompt_len.mean()) + lead + (steps - 1) / 2.0   # cached tokens + the new one, averaged over the window
    return dict(attr=attr, B=B, p_lo=p_lo, p_hi=p_hi, new_tokens=new_tokens, prompt_len=prompt_len, lead=lead, rng=rng,
                mean_len=mean_len)


def decode_step_bytes(cfg, tp, batch, mean_len, kv_bytes):
    """algorithmic HBM bytes of one decode step on ONE rank: int4 weights + {zero, scale} of the four
    projections of every layer, the lm-head slice, the KV cache at the current lengths."""
    hid = cfg.hidden
    shapes = [((cfg.head_num + 2 * cfg.kv_head_num) * 128 // tp, hid), (hid, hid // tp),
              (2 * cfg.inter_size // tp, hid), (hid, cfg.inter_size // tp)]
    w = sum(k * n // 2 + (k // 128) * n * 4 for n, k in shapes) * cfg.num_layer
    head = cfg.vocab_size // tp * hid * 2
    kv = batch * mean_len * 2 * cfg.num_layer * (cfg.kv_head_num // tp) * 128 * kv_bytes
    return w + head + kv, w, head, kv


def run_decode_workload(args, rank, world, device, name):
    """Greedy decode of a random-init Llama-2 (W4A16, int8 KV): the prompts go through the prefill path
    (tm_llama_prefill, not timed), then untimed decode steps up to a window of `steps` timed steps centred
    in the generation (decode_workload_plan); the timed region is `steps` steps = steps * batch generated
    tokens."""
    from lmdeploy_b200 import llama
    from lmdeploy_b200 import lib as l
    from lmdeploy_b200 import turbomind as tm
    torch.cuda.set_device(device)
    K, W = args.steps, args.warmup
    plan = decode_workload_plan(name, K, W, args.batch_override, args.max_prompt)
    attr, B, p_lo, p_hi, new_tokens = plan["attr"], plan["B"], plan["p_lo"], plan["p_hi"], plan["new_tokens"]
    cfg = getattr(llama, attr)
    prompt_len, rng, lead = plan["prompt_len"], plan["rng"], plan["lead"]
    pmax = int(prompt_len.max())
    max_steps = lead + 2 * K + 8
    session_len = ((pmax + max_steps + 8 + 63) // 64) * 64
    comm = llama.Comm(world, rank, device) if world > 1 else None
    t0 = time.time()
    model = llama.LlamaModel(cfg, B, session_len, device, comm)
    model.random_init(seed=0)
    torch.cuda.synchronize()
    t_init = time.time() - t0
    prompts = [rng.integers(0, cfg.vocab_size, size=int(n)).astype(np.int32) for n in prompt_len]
    # step 0 of the decode loop takes the last prompt token; everything before it goes through the prefill path
    forced = np.full((max_steps, B), -1, np.int32)
    forced[0] = [int(t[-1]) for t in prompts]
    h = model.handle
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        st = model.new_state(B, max_steps, None, forced)
        t0 = time.time()
        # prompts (not timed): tm_llama_prefill, a few sequences per call to bound the activation buffers
        group = max(1, min(B, 16384 // max(pmax, 1)))
        for b0 in range(0, B, group):
            part = [prompts[b][:-1].tolist() if b0 <= b < b0 + group else [] for b in range(B)]
            if any(part):                                     # one-token prompts have nothing to prefill
                model.prefill(st, part)
        assert bool((st.lengths.cpu().numpy() == prompt_len - 1).all())
        model.decode(st, lead, use_graph=True)            # untimed decode steps up to the window (>= warm-up)
        h.check_device_status(stream.cuda_stream)
        t_prefill = time.time() - t0
        barrier(world)
        torch.cuda.synchronize()
        sampler = ClockSampler(device)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        lengths_at_window, step_at_window = st.lengths.clone(), st.step.clone()   # the end-to-end leg re-runs the same window
        torch.cuda.cudart().cudaProfilerStart()           # a profiler started with capture off sees the timed steps only
        e0.record(stream)
        model.decode(st, K, use_graph=True)
        e1.record(stream)
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
        barrier(world)
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        launches = model.last_launches()
        h.check_device_status(stream.cuda_stream)
        # KV length seen by the attention of a timed step, averaged over the window (cached tokens + the new one)
        mean_len = float(st.lengths.float().mean().item()) - K / 2.0 + 0.5
        assert abs(mean_len - plan["mean_len"]) < 1.0, (mean_len, plan["mean_len"])
        assert int(st.step.item()) == lead + K
        assert bool((st.output_ids[lead: lead + K] >= 0).all()), "a sequence produced no token in the timed region"
        pmax_w = lead   # first step index of the timed window

        # ---- end to end: one C-ABI call per step, host buffers in and out, over the SAME window (the sequences are
        # ---- set back to where the window began, so both numbers see the same KV lengths; the cache rows of the
        # ---- window are simply written again)
        ids_host = torch.empty(B, dtype=torch.int32).pin_memory()
        out_host = torch.empty(B, dtype=torch.int32).pin_memory()
        ids_host.copy_(st.output_ids[pmax_w - 1].cpu())
        st.lengths.copy_(lengths_at_window)
        st.step.copy_(step_at_window)
        torch.cuda.synchronize()
        barrier(world)
        w0 = time.perf_counter()
        e0.record(stream)
        for i in range(K):
            s_idx = pmax_w + i
            st.forced_ids[s_idx].copy_(ids_host, non_blocking=True)       # H2D: this step's input tokens
            model.decode(st, 1, use_graph=True)
            out_host.copy_(st.output_ids[s_idx], non_blocking=True)       # D2H: the picked tokens
            stream.synchronize()
            ids_host.copy_(out_host)
        e1.record(stream)
        torch.cuda.synchronize()
        barrier(world)
        ms_e2e = max((time.perf_counter() - w0) * 1e3, e0.elapsed_time(e1))

        # ---- per-kernel device time on the same tensors (events around runs of launches) ------
        per = time_decode_kernels(model, st, cfg, B, world, stream, tm, session_len)
        # the metric's second half, "W4 GEMM HBM GB/s vs peak": the GEMV at one token on the same weights
        m1 = time_layer_gemms(model, cfg, 1, stream, tm, st.lengths.device, chained=False)
        m1c = time_layer_gemms(model, cfg, 1, stream, tm, st.lengths.device, chained=True)
        m1_large = time_large_gemv(stream, tm, st.lengths.device) if world == 1 else None
        h.check_device_status(stream.cuda_stream)

    ms_step = max_over_ranks(ms / K, world)
    ms_e2e_step = max_over_ranks(ms_e2e / K, world)
    peaks = measured_peaks()
    kv_b = 1 if cfg.quant_policy & 4 else 2
    total_b, w_b, head_b, kvb = decode_step_bytes(cfg, world, B, mean_len, kv_b)
    dom = max(((k, v) for k, v in per.items() if not k.startswith("gemm ")), key=lambda kv: kv[1]["us_per_step"])
    # DRAM bytes per launch of the dominant kernel: ratio measured once with ncu on the same shapes
    # (dram__bytes_read.sum + dram__bytes_write.sum over algorithmic bytes; profiles/), applied to this launch
    traffic_ratio = {"gemm_s4_f16_tc_kernel": 1.03, "gemm_s4_f16_small_kernel": 1.0, "gemm_s4_f16_cols_kernel": 1.0, "mmha_decode_kernel": 1.02}
    ratio = next((r for k, r in traffic_ratio.items() if dom[0].startswith(k)), None)
    out = {
        "metric": "decode tokens/s Llama-2 W4A16", "value": round(B * 1e3 / ms_step, 1), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "int4 weights x f16 activations, f32 accumulate, int8 KV", "data": "synthetic",
        "config": {"workload": f"{cfg.name} W4A16 g128, int8 KV, greedy decode", "global_batch": B,
                   "prompt_len": f"uniform {p_lo}..{p_hi}" if p_lo != p_hi else p_lo, "new_tokens": new_tokens,
                   "mean_kv_len_timed": round(plan["mean_len"], 1), "untimed_decode_steps_before_window": lead,
                   "prompts": "tm_llama_prefill (untimed)",
                   "parallelism": f"tp{world}", "weights": "random init N(0,0.02), AWQ int4",
                   "l2": "inputs larger than L2: every step streams all layer weights and the KV cache (GBs)"},
        "e2e": {"value": round(B * 1e3 / ms_e2e_step, 1), "unit": "tokens/s", "h2d_bytes_per_step": B * 4,
                "d2h_bytes_per_step": B * 4,
                "note": "one tm_llama_decode call per step over the same steps as the device-timed window (sequences set back to "
                        "its start): input ids from pinned host memory, picked ids read back, host synchronisation every step"},
        "roofline": {"bound": "hbm", "kernel": dom[0], "achieved": dom[1]["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(dom[1]["gbs"] / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
                     "algorithmic_bytes": dom[1]["bytes"], "traffic": int(dom[1]["bytes"] * ratio) if ratio else None},
        "step_roofline": {"bytes_per_step_per_gpu": int(total_b), "weights": int(w_b), "lm_head": int(head_b), "kv": int(kvb),
                          "achieved_gbs_per_gpu": round(total_b / (ms_step * 1e-3) * 1e-9, 1),
                          "frac_of_hbm_peak": round(total_b / (ms_step * 1e-3) * 1e-9 / peaks["hbm_gbs"], 4)},
        "per_kernel_m1": {k: dict(v, frac=round(v["gbs"] / peaks["hbm_gbs"], 4), us_chained=m1c[k]["us"], gbs_chained=m1c[k]["gbs"],
                                  frac_chained=round(m1c[k]["gbs"] / peaks["hbm_gbs"], 4)) for k, v in m1.items()},
        "per_kernel_m1_note": "the 1-token GEMM on this model's weights (per-rank shapes; gemm_s4_f16_cols_kernel where the weight has a "
                              "64-column strip per SM: qkv and gate_up, gemm_s4_f16_small_kernel otherwise); us / gbs / frac: launches "
                              "back to back, each waiting for the one before it; *_chained: with programmatic dependent launch, as "
                              "inside the decode step",
        "per_kernel_m1_large": None if m1_large is None else {
            k: dict(v, frac=round(v["gbs"] / peaks["hbm_gbs"], 4)) for k, v in m1_large.items()},
        "per_kernel_m1_large_note": "same kernel at 1 token on the un-sharded Llama-2-70B projection shapes (seeded random nibbles and "
                                    "scales; copies of each weight alternate so that every launch reads HBM): the launch's fixed cost "
                                    "weighs less there",
        "per_kernel": per,
        "per_kernel_note": "each kernel timed alone (no overlap with its neighbours), a different layer's weights / cache every "
                           "launch (L2-cold): the sum exceeds ms_per_step, where programmatic dependent launch overlaps them",
        "clocks": clocks, "gpu_launches": int(launches),
        "setup_s": {"weights": round(t_init, 1), "prompts_and_warmup": round(t_prefill, 1)},
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_decode_baseline(MODEL_SHAPES[attr], B, int(round(plan["mean_len"])), seconds=15.0)
    model.close()
    return out


def time_layer_gemms(model, cfg, tokens, stream, tm, dev, chained):
    """Device time of the four W4A16 projections of a layer at `tokens` tokens, each timed alone over the model's own
    layers (a different layer's weights every launch: 3.4 GB in all, far beyond L2).  chained: launches carry the
    programmatic-serialization attribute, as in the decode step."""
    layers = [model._keep[i:i + 6] for i in range(0, 6 * cfg.num_layer, 6)]   # norm, norm, qkv, o, w13, w2
    op = tm.LlamaLinear(dev.index)
    h = model.handle
    out = {}
    h.set_option("pdl_direct", int(chained))
    try:
        for nm, idx, fused in (("qkv", 2, False), ("o", 3, False), ("w13+silu", 4, True), ("w2", 5, False)):
            w0 = layers[0][idx]
            x = torch.randn(tokens, w0.input_dims, device=dev).half()
            y = torch.empty(tokens, w0.output_dims // (2 if fused else 1), dtype=torch.float16, device=dev)
            launch = lambda i: op.forward(y, x, tokens, layers[i % cfg.num_layer][idx], op.kFusedSiluFfn if fused else op.kGemm)
            n_it = max(cfg.num_layer, 32)
            for i in range(3):
                launch(i)
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                for i in range(n_it):
                    launch(i)
            gr.replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            gr.replay()
            b.record(stream)
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / n_it
            nb = gemm_bytes(w0.output_dims, w0.input_dims, tokens, fused)
            out[nm] = dict(us=round(us, 2), gbs=round(nb / us * 1e-3, 1), bytes=int(nb))
    finally:
        h.set_option("pdl_direct", 0)
    return out


def time_large_gemv(stream, tm, dev):
    """The 1-token GEMM on the four projection shapes of the un-sharded Llama-2-70B (k, n as LlamaDecoderLayerWeight.cc:49-77
    gives them at tp 1): the weights of one launch are 34..235 MB, so the launch's fixed cost weighs less than on the 7B
    shapes.  Any nibbles are a weight; launches wait for one another (no programmatic dependent launch)."""
    g = torch.Generator(device=dev).manual_seed(70)
    op = tm.LlamaLinear(dev.index)
    out = {}
    for nm, n, k, fused in (("qkv 10240x8192", 10240, 8192, False), ("o 8192x8192", 8192, 8192, False),
                            ("w13+silu 57344x8192", 57344, 8192, True), ("w2 8192x28672", 8192, 28672, False)):
        nbytes = n * k // 2
        copies = max(2, -(-400_000_000 // nbytes))        # at least 400 MB in rotation: three times L2
        ws = []
        for _ in range(copies):
            A = torch.randint(-2 ** 31, 2 ** 31 - 1, (k, n // 8), dtype=torch.int32, device=dev, generator=g)
            z = torch.randint(64, 80, (k // 128, n, 1), device=dev, generator=g).half()
            sc = (torch.rand(k // 128, n, 1, device=dev, generator=g) * 0.01 + 0.002).half()
            ws.append(tm.LlamaDenseWeight(k, n, A, tm.WeightType.kINT4, None, torch.cat([z, sc], dim=-1).contiguous(), 128))
        x = torch.randn(1, k, device=dev, generator=g).half()
        y = torch.empty(1, n // (2 if fused else 1), dtype=torch.float16, device=dev)
        launch = lambda i: op.forward(y, x, 1, ws[i % copies], op.kFusedSiluFfn if fused else op.kGemm)
        n_it = 4 * copies
        for i in range(3):
            launch(i)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=stream):
            for i in range(n_it):
                launch(i)
        gr.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        gr.replay()
        b.record(stream)
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / n_it
        nb = gemm_bytes(n, k, 1, fused)
        out[nm] = dict(us=round(us, 2), gbs=round(nb / us * 1e-3, 1), bytes=int(nb))
        del ws
    return out


def time_decode_kernels(model, st, cfg, B, tp, stream, tm, session_len):
    """Device time of the kernels of one decode step, each timed alone with CUDA events around a run
    of launches on the model's own tensors (weights of a different layer every launch: larger than
    L2 in total)."""
    import math
    dev = st.lengths.device
    per = {}
    ev = lambda: torch.cuda.Event(enable_timing=True)
    layers = [model._keep[i:i + 6] for i in range(0, 6 * cfg.num_layer, 6)]   # norm, norm, qkv, o, w13, w2
    op = tm.LlamaLinear(dev.index)
    hid = cfg.hidden
    names = [("gemm qkv", 2, False), ("gemm o", 3, False), ("gemm w13+silu", 4, True), ("gemm w2", 5, False)]
    def graph_time(launch, n_it):
        """device time per launch: `n_it` launches captured into one CUDA graph, replayed once warm and once timed"""
        for i in range(3):
            launch(i)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=stream):
            for i in range(n_it):
                launch(i)
        gr.replay()
        a, b = ev(), ev()
        a.record(stream)
        gr.replay()
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / n_it

    gemm_us = gemm_b = 0.0
    for nm, idx, fused in names:
        w0 = layers[0][idx]
        x = torch.randn(B, w0.input_dims, device=dev).half()
        y = torch.empty(B, w0.output_dims // (2 if fused else 1), dtype=torch.float16, device=dev)
        n_it = max(cfg.num_layer, 32)
        us = graph_time(lambda i: op.forward(y, x, B, layers[i % cfg.num_layer][idx], op.kFusedSiluFfn if fused else op.kGemm), n_it)
        nb = gemm_bytes(w0.output_dims, w0.input_dims, B, fused)
        gemm_us += us
        gemm_b += nb
        per[nm] = dict(us=round(us, 2), gbs=round(nb / us * 1e-3, 1), us_per_step=round(us * cfg.num_layer, 1), bytes=int(nb))
    kname = "gemm_s4_f16_tc_kernel" if B > 16 else "gemm_s4_f16_small_kernel" if B > 8 else "gemm_s4_f16_cols_kernel + gemm_s4_f16_small_kernel"
    per[f"{kname} (4 projections of a layer)"] = dict(us=round(gemm_us / 4, 2), gbs=round(gemm_b / gemm_us * 1e-3, 1),
                                                      us_per_step=round(gemm_us * cfg.num_layer, 1), bytes=int(gemm_b / 4))
    # attention over the caches as they stand (layer l of every sequence)
    Hl, Hkvl = cfg.head_num // tp, cfg.kv_head_num // tp
    qkv = torch.randn(B, (Hl + 2 * Hkvl) * 128, device=dev).half()
    out = torch.empty(B, Hl * 128, dtype=torch.float16, device=dev)
    lengths = st.lengths.clone()
    p = tm.Masked_multihead_attention_params(
        out=out, q=qkv, k=qkv[:, Hl * 128:], v=qkv[:, (Hl + Hkvl) * 128:], stride=(Hl + 2 * Hkvl) * 128, batch_size=B,
        memory_max_len=session_len, num_heads=Hl, num_kv_heads=Hkvl, timestep=session_len - 1,
        inv_sqrt_dh=1.0 / math.sqrt(128), length_per_sample=lengths, k_cache_per_sample=st.k_ptrs,
        v_cache_per_sample=st.v_ptrs)
    p.total_padding_tokens = (session_len - 1 - lengths).to(torch.int32)
    if cfg.quant_policy & 4:
        p.int8_mode, p.attention_k_scale, p.attention_v_scale = 4, 4.0 / 127, 4.0 / 127
    def attn(i):
        p.kv_cache_per_sample_offset = (i % cfg.num_layer) * Hkvl * session_len * 128
        tm.masked_multihead_attention(p)

    us = graph_time(attn, max(cfg.num_layer, 32))
    nb = mmha_bytes(lengths.cpu().numpy(), Hl, Hkvl, 1 if cfg.quant_policy & 4 else 2)
    per["mmha_decode_kernel"] = dict(us=round(us, 2), gbs=round(nb / us * 1e-3, 1), us_per_step=round(us * cfg.num_layer, 1), bytes=int(nb))
    return per


def cpu_decode_baseline(cfg, B, mean_len, seconds=15.0, layers_sample=1, threads=None):
    """The reference's torch CPU path (pseudo-quant fp16 weights, fp32-accumulated linears, numpy
    attention: the oracle) on a bounded sample: `layers_sample` decoder layers + the lm-head for one
    batch step at KV length `mean_len`, repeated for about `seconds`; per-token time extrapolated
    to the full depth."""
    from oracle import attention as oa, awq as oawq, decoder as odec
    if threads:
        torch.set_num_threads(threads)
    hid = cfg.hidden
    g = torch.Generator().manual_seed(0)
    small = dict(head_num=cfg.head_num, kv_head_num=cfg.kv_head_num, session_len=mean_len + 8, norm_eps=cfg.norm_eps,
                 rope_theta=cfg.rope_theta)

    def lin(n, k):
        w = (torch.randn(n, k, generator=g) * 0.02).half()
        return oawq.pseudo_quant_weight(oawq.quantize(w, 128), 128).t().contiguous().numpy()

    layers = []
    for _ in range(layers_sample):
        layers.append(dict(attn_norm=np.ones(hid, np.float16), ffn_norm=np.ones(hid, np.float16),
                           w_qkv=lin((cfg.head_num + 2 * cfg.kv_head_num) * 128, hid), w_o=lin(hid, hid),
                           w13=lin(2 * cfg.inter_size, hid), w2=lin(hid, cfg.inter_size),
                           kv_quant=oa.KvQuant(4.0 / 127, 0.0, 4.0 / 127, 0.0)))
    rng = np.random.default_rng(0)
    glob = dict(tok_embeddings=(rng.standard_normal((cfg.vocab_size, hid)) * 0.02).astype(np.float16),
                output_norm=np.ones(hid, np.float16),
                output_weight=(rng.standard_normal((cfg.vocab_size, hid)) * 0.02).astype(np.float16))
    S = mean_len + 8
    kc = [[rng.integers(-127, 128, size=(cfg.kv_head_num, S, 128), dtype=np.int8) for _ in range(B)] for _ in layers]
    vc = [[rng.integers(-127, 128, size=(cfg.kv_head_num, S, 128), dtype=np.int8) for _ in range(B)] for _ in layers]
    ids = rng.integers(0, cfg.vocab_size, size=B)
    lengths = np.full(B, mean_len, np.int32)
    odec.decode_step(ids, lengths, layers, glob, kc, vc, small)       # warm-up
    t_head0 = time.perf_counter()
    hfake = np.zeros((B, hid), np.float16)
    _ = (torch.from_numpy(hfake).float() @ torch.from_numpy(glob["output_weight"]).float().t())
    t_head = time.perf_counter() - t_head0
    n, t0 = 0, time.perf_counter()
    while True:
        odec.decode_step(ids, lengths, layers, glob, kc, vc, small)
        n += 1
        el = time.perf_counter() - t0
        if el >= seconds or n >= 50:
            break
    t_step = el / n
    t_layers = max(t_step - t_head, 1e-9) / layers_sample
    t_full = t_layers * cfg.num_layer + t_head
    return {"value": round(B / t_full, 3), "unit": "tokens/s", "cores": torch.get_num_threads(), "host_cpus": os.cpu_count(),
            "kind": "port",
            "sample": f"{n} x one batch-{B} decode step of {layers_sample} of {cfg.num_layer} layers + lm-head at KV length "
                      f"{mean_len} ({el:.1f} s of CPU work), per-token time extrapolated to {cfg.num_layer} layers"}


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's CPU implementation of the path (torch pseudo-quant linears
    + the attention restatement: the oracle port), all host threads, same config/metric/unit."""
    if rank != 0:
        return None
    name = "decode7b" if world == 1 and args.workload in ("decode", "decode7b") else "decode70b"
    if args.workload in DECODE_WORKLOADS:
        name = args.workload
    plan = decode_workload_plan(name, args.steps, args.warmup, args.batch_override, args.max_prompt)
    cfg, B = MODEL_SHAPES[plan["attr"]], plan["B"]
    mean_len = int(round(plan["mean_len"]))
    torch.set_num_threads(os.cpu_count() or 1)
    budget = min(120.0, max(10.0, 4.0 * (args.steps + args.warmup)))
    t0 = time.perf_counter()
    cb = cpu_decode_baseline(cfg, B, mean_len, seconds=budget)
    ms_step = B / cb["value"] * 1e3
    p_lo, p_hi = plan["p_lo"], plan["p_hi"]
    return {"impl": "reference", "metric": "decode tokens/s Llama-2 W4A16", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 2),
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "f16 pseudo-quant weights, f32 accumulate (torch CPU)", "data": "synthetic",
            "config": {"workload": f"{cfg.name} W4A16 g128, int8 KV, greedy decode", "global_batch": B,
                       "prompt_len": f"uniform {p_lo}..{p_hi}" if p_lo != p_hi else p_lo, "new_tokens": plan["new_tokens"],
                       "mean_kv_len_timed": round(plan["mean_len"], 1), "parallelism": "host cores"},
            # ms_per_step is NOT the duration of a measured step: the CPU cannot run `steps` full steps in minutes, so a
            # bounded sample (cpu_baseline.sample) is timed and the per-step time extrapolated to the model's depth
            "extrapolated": True, "measured_seconds": round(time.perf_counter() - t0, 1),
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}


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
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="decode",
                    help="decode (7B at 1 GPU, 70B tensor-parallel at N > 1) | decode7b | decode70b | gemm | mmha | prefill | prefill7b")
    ap.add_argument("--batch-override", type=int, default=0, help="smaller batch for smoke runs")
    ap.add_argument("--max-prompt", type=int, default=0, help="cap on the prompt length for smoke runs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--shapes", choices=["7b", "70b"], default="7b", help="projection shapes of the gemm workload")
    ap.add_argument("--kv-len", default="128,4096", help="lo,hi of the uniform KV lengths of the mmha workload")
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
    if args.impl == "reference" and args.workload == "prefill7b":
        if rank == 0:   # the reference's prefill needs its engine and its flash-attention build (CUTLASS): neither is built
            print(json.dumps({"impl": "reference", "unavailable": "whole-model prefill of the reference needs its engine and "
                              "CUTLASS flash attention; use --workload prefill for its kernels"}), flush=True)
        return
    if args.impl == "reference" and args.workload not in ("gemm", "mmha", "prefill"):
        # whole-model workloads: the reference's CPU path (the engine around its kernels is out of scope)
        out = run_reference_arm(args, rank, world)
        if rank == 0:
            print(json.dumps(out), flush=True)
        return
    if args.impl == "reference" and rank != 0:
        return   # per-kernel workloads: rank 0 alone times the reference's CUDA kernels
    if args.impl == "reference":
        world = 1
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))

    if args.workload in ("decode", "decode7b", "decode70b"):
        name = args.workload if args.workload != "decode" else ("decode7b" if world == 1 else "decode70b")
        out = run_decode_workload(args, rank, world, local, name)
    elif args.workload == "gemm":
        out = run_gemm_workload(args, rank, world, local)
    elif args.workload == "mmha":
        out = run_mmha_workload(args, rank, world, local)
    elif args.workload == "prefill":
        out = run_prefill_workload(args, rank, world, local)
    elif args.workload == "prefill7b":
        out = run_prefill_model_workload(args, rank, world, local)
    else:
        raise SystemExit(f"unknown workload {args.workload}")
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
