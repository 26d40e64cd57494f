"""Python face of the C++ decode driver (``tm_llama_*``): model set-up, tensor-parallel
communicator, KV-cache slabs and the decode loop.  torch provides device memory, streams and the
process group used to hand the NCCL id around; everything that computes is in ``libtm_b200.so``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import awq
from . import lib as _l
from . import turbomind as tm


@dataclass
class LlamaConfig:
    head_num: int
    kv_head_num: int
    inter_size: int
    num_layer: int
    vocab_size: int = 32000
    size_per_head: int = 128
    norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    quant_policy: int = 4          # int8 KV cache
    group_size: int = 128
    name: str = "llama"

    @property
    def hidden(self):
        return self.head_num * self.size_per_head


LLAMA2_7B = LlamaConfig(32, 32, 11008, 32, name="llama-2-7b")
LLAMA2_70B = LlamaConfig(64, 8, 28672, 80, name="llama-2-70b")


class Comm:
    """tm_comm: one rank of the tensor-parallel group (NCCL)."""

    def __init__(self, world: int, rank: int, device: int, p2p_slot_bytes: int = 4 << 20):
        import torch.distributed as dist
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_ubyte * 128)()
            _l.check(_l.lib.tm_comm_unique_id(buf), "tm_comm_unique_id")
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        if world > 1:
            t = ident.cuda(device) if dist.get_backend() == "nccl" else ident
            dist.broadcast(t, 0)
            ident = t.cpu()
        raw = (C.c_ubyte * 128)(*ident.tolist())
        self._c = C.c_void_p()
        _l.check(_l.lib.tm_comm_create(C.byref(self._c), world, rank, raw, device), "tm_comm_create")
        self.world, self.rank = world, rank
        self.p2p = False
        if 1 < world <= 8 and p2p_slot_bytes > 0:
            # peer-memory all-reduce of the decode step: every rank exports a region, all ranks map all of them
            mine = (C.c_ubyte * 64)()
            ok = _l.lib.tm_comm_p2p_export(self._c, p2p_slot_bytes, mine) == _l.TM_OK
            t = torch.tensor(list(mine) + [int(ok)], dtype=torch.uint8)
            t = t.cuda(device) if dist.get_backend() == "nccl" else t
            every = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(every, t)
            every = torch.stack(every).cpu()
            if bool(every[:, 64].all()):
                raw_all = (C.c_ubyte * (64 * world))(*every[:, :64].reshape(-1).tolist())
                ok = _l.lib.tm_comm_p2p_import(self._c, raw_all) == _l.TM_OK
                flag = torch.tensor([int(ok)], dtype=torch.uint8)
                flag = flag.cuda(device) if dist.get_backend() == "nccl" else flag
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                self.p2p = bool(flag.item())

    @property
    def ptr(self):
        return self._c

    def allreduce_sum_f16(self, t: torch.Tensor):
        _l.check(_l.lib.tm_allreduce_sum_f16(self._c, t.data_ptr(), t.numel(), torch.cuda.current_stream().cuda_stream),
                 "tm_allreduce_sum_f16")

    def close(self):
        if self._c:
            _l.lib.tm_comm_destroy(self._c)
            self._c = C.c_void_p()


class LlamaModel:
    """tm_llama + the tensors it points to."""

    def __init__(self, cfg: LlamaConfig, max_batch_size: int, session_len: int, device: int = 0,
                 comm: Optional[Comm] = None):
        self.cfg, self.device, self.comm = cfg, device, comm
        self.tp = comm.world if comm else 1
        self.rank = comm.rank if comm else 0
        self.session_len, self.max_batch_size = session_len, max_batch_size
        self.handle = _l.default_handle(device)
        c = _l.TmLlamaConfig(cfg.head_num, cfg.kv_head_num, cfg.size_per_head, cfg.inter_size, cfg.num_layer,
                             cfg.vocab_size, cfg.norm_eps, cfg.rope_theta, cfg.quant_policy, cfg.group_size, self.tp,
                             self.rank, max_batch_size, session_len)
        self._m = C.c_void_p()
        _l.check(_l.lib.tm_llama_create(C.byref(self._m), self.handle.ptr, comm.ptr if comm else None, C.byref(c)),
                 "tm_llama_create")
        self._keep: List[object] = []   # tensors the C side points to
        self._layers = {}               # layer -> (tensors..., kv_scale), for save_workspace
        self._globals = None

    # -- weights -----------------------------------------------------------------------------
    def set_layer(self, l, attn_norm, ffn_norm, qkv: tm.LlamaDenseWeight, o: tm.LlamaDenseWeight,
                  w13: tm.LlamaDenseWeight, w2: tm.LlamaDenseWeight, kv_scale=(1.0, 0.0, 1.0, 0.0)):
        w = _l.TmLlamaLayerWeights()
        w.self_attn_norm, w.ffn_norm = attn_norm.data_ptr(), ffn_norm.data_ptr()
        w.qkv_qweight, w.qkv_scales_zeros = qkv.kernel.data_ptr(), qkv.scales_and_zeros.data_ptr()
        w.qkv_bias = 0 if qkv.bias is None else qkv.bias.data_ptr()
        w.o_qweight, w.o_scales_zeros = o.kernel.data_ptr(), o.scales_and_zeros.data_ptr()
        w.w13_qweight, w.w13_scales_zeros = w13.kernel.data_ptr(), w13.scales_and_zeros.data_ptr()
        w.w2_qweight, w.w2_scales_zeros = w2.kernel.data_ptr(), w2.scales_and_zeros.data_ptr()
        w.past_kv_scale = (C.c_float * 4)(*kv_scale)
        self._keep += [attn_norm, ffn_norm, qkv, o, w13, w2]
        self._layers[l] = (attn_norm, ffn_norm, qkv, o, w13, w2, tuple(kv_scale))
        _l.check(_l.lib.tm_llama_set_layer(self._m, l, C.byref(w)), "tm_llama_set_layer")

    def set_globals(self, tok_embeddings, output_norm, output_weight):
        self._keep += [tok_embeddings, output_norm, output_weight]
        self._globals = (tok_embeddings, output_norm, output_weight)
        _l.check(_l.lib.tm_llama_set_globals(self._m, tok_embeddings.data_ptr(), output_norm.data_ptr(),
                                             output_weight.data_ptr()), "tm_llama_set_globals")

    def random_init(self, seed: int = 0, kv_scale=(4.0 / 127, 0.0, 4.0 / 127, 0.0)):
        """Random-init weights of this architecture: every linear W ~ N(0, 0.02) AWQ-quantised (group
        128), norms 1, embeddings / lm-head ~ N(0, 0.02).  Each tensor-parallel rank draws its own
        slices (seeded by layer and rank); replicated tensors are seeded by layer only."""
        cfg, tp, dev = self.cfg, self.tp, torch.device("cuda", self.device)
        hid = cfg.hidden
        ones = torch.ones(hid, dtype=torch.float16, device=dev)
        for l in range(cfg.num_layer):
            g = torch.Generator(device=dev).manual_seed(seed * 1000003 + l * 131 + self.rank)
            qkv = awq.random_linear((cfg.head_num + 2 * cfg.kv_head_num) * 128 // tp, hid, g)
            o = awq.random_linear(hid, hid // tp, g)
            w13 = awq.random_linear(2 * cfg.inter_size // tp, hid, g)
            w2 = awq.random_linear(hid, cfg.inter_size // tp, g)
            self.set_layer(l, ones, ones, qkv, o, w13, w2, kv_scale)
        g = torch.Generator(device=dev).manual_seed(seed * 1000003 + 999983)
        emb = (torch.randn(cfg.vocab_size, hid, device=dev, generator=g) * 0.02).half()
        head = (torch.randn(cfg.vocab_size, hid, device=dev, generator=g) * 0.02).half()
        lo = cfg.vocab_size // tp * self.rank
        self.set_globals(emb, ones, head[lo: lo + cfg.vocab_size // tp].contiguous())

    # -- TurboMind workspace files -----------------------------------------------------------
    def save_workspace(self, path: str):
        """Write this rank's weights in the file layout of a TurboMind workspace (what
        lmdeploy/serve/turbomind/deploy.py exports for W4A16 and LlamaWeight::loadModel reads):
        raw little-endian tensors, one file each.  ``output.weight`` holds the whole vocabulary, so
        this helper is for tp == 1."""
        import os
        import numpy as np
        assert self.tp == 1, "save_workspace writes the un-sliced lm-head: tp == 1 only"
        os.makedirs(path, exist_ok=True)

        def dump(name, t):
            t.detach().contiguous().cpu().numpy().tofile(os.path.join(path, name))

        emb, norm, head = self._globals
        dump("tok_embeddings.weight", emb)
        dump("norm.weight", norm)
        dump("output.weight", head)
        for l, (an, fn, qkv, o, w13, w2, kv) in self._layers.items():
            dump(f"layers.{l}.attention_norm.weight", an)
            dump(f"layers.{l}.ffn_norm.weight", fn)
            for name, w in (("attention.w_qkv", qkv), ("attention.wo", o), ("feed_forward.w13", w13), ("feed_forward.w2", w2)):
                dump(f"layers.{l}.{name}.{self.rank}.qweight", w.kernel)
                dump(f"layers.{l}.{name}.{self.rank}.scales_zeros", w.scales_and_zeros)
            if qkv.bias is not None:
                dump(f"layers.{l}.attention.w_qkv.{self.rank}.bias", qkv.bias)
            np.asarray(kv, np.float32).tofile(os.path.join(path, f"layers.{l}.past_kv_scale.{self.rank}.weight"))

    def load_workspace(self, path: str):
        """Load every weight of this rank from a TurboMind workspace directory (tm_llama_load_workspace:
        the library reads the files and owns the device copies)."""
        _l.check(_l.lib.tm_llama_load_workspace(self._m, path.encode()), f"tm_llama_load_workspace({path})")

    # -- decode state ------------------------------------------------------------------------
    def new_state(self, batch: int, max_steps: int, start_step=None, forced_ids=None, keep_hidden=False,
                  keep_logits=False):
        return DecodeState(self, batch, max_steps, start_step, forced_ids, keep_hidden, keep_logits)

    def decode(self, state: "DecodeState", n_steps: int, use_graph: bool = True, stream=None):
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        _l.check(_l.lib.tm_llama_decode(self._m, C.byref(state.c), n_steps, int(use_graph), st), "tm_llama_decode")

    def prefill(self, state: "DecodeState", new_tokens, keep_hidden: bool = False, stream=None):
        """tm_llama_prefill: run ``new_tokens[b]`` (a list of ids per sequence, possibly empty) through all layers on top
        of the ``state.lengths[b]`` tokens already cached, leave their keys / values in the state's cache and advance
        ``state.lengths``.  Returns the normed last-layer output [token_num, hidden] when ``keep_hidden``."""
        import numpy as np
        dev = torch.device("cuda", self.device)
        lens = np.asarray([len(t) for t in new_tokens], np.int32)
        assert len(lens) == state.c.batch_size
        token_num, max_q = int(lens.sum()), int(lens.max(initial=0))
        ids = torch.tensor([i for t in new_tokens for i in t], dtype=torch.int32, device=dev)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
        hist = state.lengths.clone()
        ctx = hist + torch.from_numpy(lens).to(dev)
        hidden = torch.zeros((token_num, self.cfg.hidden), dtype=torch.float16, device=dev) if keep_hidden else None
        c = _l.TmLlamaPrefillState()
        c.batch_size, c.token_num, c.max_q_len = len(lens), token_num, max_q
        c.input_ids, c.cu_seqlens = ids.data_ptr(), cu.data_ptr()
        c.history_lengths, c.context_lengths = hist.data_ptr(), ctx.data_ptr()
        c.k_cache_ptrs, c.v_cache_ptrs = state.k_ptrs.data_ptr(), state.v_ptrs.data_ptr()
        c.hidden_out = 0 if hidden is None else hidden.data_ptr()
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        _l.check(_l.lib.tm_llama_prefill(self._m, C.byref(c), st), "tm_llama_prefill")
        state.lengths.copy_(ctx)
        torch.cuda.current_stream().synchronize()   # ids / cu / hist / ctx are released when this returns
        return hidden

    def check_status(self, stream=None) -> None:
        """tm_llama_check_status: synchronise the stream and raise if a kernel of this model recorded a fault
        (a bounded wait that gave up, a prefill past session_len)."""
        st = torch.cuda.current_stream().cuda_stream if stream is None else stream
        w = C.c_uint(0)
        rc = _l.lib.tm_llama_check_status(self._m, st, C.byref(w))
        if rc != _l.TM_OK:
            raise _l.TmError(rc, f"tm_llama_check_status: device status word 0x{w.value:x}")

    def last_launches(self) -> int:
        return int(_l.lib.tm_llama_last_launches(self._m))

    def close(self):
        if self._m:
            _l.lib.tm_llama_destroy(self._m)
            self._m = C.c_void_p()


class DecodeState:
    """Device buffers of ``tm_llama_decode_state`` (per-sequence KV slabs
    ``[num_layer][kv_heads / tp][session_len][128]``, step-major id buffers)."""

    def __init__(self, model: LlamaModel, batch, max_steps, start_step, forced_ids, keep_hidden, keep_logits):
        cfg, dev = model.cfg, torch.device("cuda", model.device)
        kvh = cfg.kv_head_num // model.tp
        dt = torch.int8 if cfg.quant_policy & 4 else torch.float16
        shape = (batch, cfg.num_layer, kvh, model.session_len, 128)
        self.k_cache = torch.zeros(shape, dtype=dt, device=dev)
        self.v_cache = torch.zeros(shape, dtype=dt, device=dev)
        self.k_ptrs = torch.tensor([self.k_cache[b].data_ptr() for b in range(batch)], dtype=torch.int64, device=dev)
        self.v_ptrs = torch.tensor([self.v_cache[b].data_ptr() for b in range(batch)], dtype=torch.int64, device=dev)
        self.lengths = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.step = torch.zeros(1, dtype=torch.int32, device=dev)
        self.output_ids = torch.full((max_steps, batch), -1, dtype=torch.int32, device=dev)
        self.start_step = None if start_step is None else torch.as_tensor(start_step, dtype=torch.int32).to(dev)
        self.forced_ids = None if forced_ids is None else torch.as_tensor(forced_ids, dtype=torch.int32).to(dev).contiguous()
        self.hidden = torch.zeros(batch, cfg.hidden, dtype=torch.float16, device=dev) if keep_hidden else None
        self.logits = torch.zeros(batch, cfg.vocab_size, dtype=torch.float32, device=dev) if keep_logits else None
        c = _l.TmLlamaDecodeState()
        c.batch_size, c.max_steps = batch, max_steps
        c.k_cache_ptrs, c.v_cache_ptrs = self.k_ptrs.data_ptr(), self.v_ptrs.data_ptr()
        c.sequence_lengths, c.step, c.output_ids = self.lengths.data_ptr(), self.step.data_ptr(), self.output_ids.data_ptr()
        c.start_step = 0 if self.start_step is None else self.start_step.data_ptr()
        c.forced_ids = 0 if self.forced_ids is None else self.forced_ids.data_ptr()
        c.hidden_out = 0 if self.hidden is None else self.hidden.data_ptr()
        c.logits_out = 0 if self.logits is None else self.logits.data_ptr()
        self.c = c


# -- tensor-parallel slicing of full (un-sharded) weights -------------------------------------------

def tp_column_index(cfg: LlamaConfig, tp: int, rank: int):
    """Output-feature indices each rank owns, as the reference slices them
    (LlamaDecoderLayerWeight.cc:49-77, deploy.py:251-260 `merge_qkv`, :668-670 `tp_m_s4`):
    qkv -> this rank's q heads | k heads | v heads; w13 -> a contiguous run of interleaved
    (gate, up) pairs; o / w2 are split along their INPUT features (rows of the [K, N] weight)."""
    import numpy as np
    d = cfg.size_per_head
    hq, hkv = cfg.head_num // tp, cfg.kv_head_num // tp
    q = np.arange(rank * hq * d, (rank + 1) * hq * d)
    k = cfg.head_num * d + np.arange(rank * hkv * d, (rank + 1) * hkv * d)
    v = (cfg.head_num + cfg.kv_head_num) * d + np.arange(rank * hkv * d, (rank + 1) * hkv * d)
    inter = cfg.inter_size // tp
    return dict(qkv_cols=np.concatenate([q, k, v]),
                o_rows=np.arange(rank * hq * d, (rank + 1) * hq * d),
                w13_cols=np.arange(rank * 2 * inter, (rank + 1) * 2 * inter),
                w2_rows=np.arange(rank * inter, (rank + 1) * inter),
                vocab_rows=np.arange(rank * (cfg.vocab_size // tp), (rank + 1) * (cfg.vocab_size // tp)))


# -- persistent-batch scheduler ------------------------------------------------------------------------------------
class Batch:
    """tm_batch (include/tm_b200.h): requests in, tokens out; a cache manager sized for the model is created with it.

    ``submit`` queues a request, ``step`` runs one scheduling round (intake + context decode + one decoder step + one
    draw), ``output`` returns the tokens generated so far for a session's latest request and its state."""

    QUEUED, RUNNING, FINISHED, FAILED = 0, 1, 2, 3

    def __init__(self, model: LlamaModel, max_batch_size: int, start_id: int = 1, end_id: int = 2, cache_max_entry_count: int = 0,
                 cache_chunk_size: int = 1, max_context_token_num: int = 0):
        cfg = model.cfg
        self.model = model
        self._cache = C.c_void_p()
        entries = cache_max_entry_count or max_batch_size
        _l.check(_l.lib.tm_cache_manager_create(C.byref(self._cache), cfg.num_layer, cfg.kv_head_num // model.tp, cfg.size_per_head,
                                                model.session_len, 8 if cfg.quant_policy & 4 else 16, entries, cache_chunk_size,
                                                model.device), "tm_cache_manager_create")
        self._b = C.c_void_p()
        _l.check(_l.lib.tm_batch_create(C.byref(self._b), model._m, self._cache, max_batch_size, model.session_len, start_id, end_id,
                                        max_context_token_num), "tm_batch_create")

    def submit(self, session_id: int, input_ids, request_output_len: int, start: bool = True, end: bool = True, top_k: int = 0,
               top_p: float = 0.0, temperature: float = 0.0, repetition_penalty: float = 0.0, random_seed: int = 0,
               ignore_eos: bool = False, stop_ids=(), bad_ids=(), step=None) -> int:
        ids = (C.c_int * max(1, len(input_ids)))(*[int(t) for t in input_ids])
        stops = (C.c_int * max(1, len(stop_ids)))(*[int(t) for t in stop_ids])
        bads = (C.c_int * max(1, len(bad_ids)))(*[int(t) for t in bad_ids])
        r = _l.TmRequest(session_id, int(start), int(end), ids, len(input_ids), request_output_len, top_k, top_p, temperature,
                         repetition_penalty, random_seed, int(ignore_eos), stops, len(stop_ids), bads, len(bad_ids),
                         0 if step is None else 1, 0 if step is None else int(step))
        return _l.lib.tm_batch_submit(self._b, C.byref(r))

    def step(self, use_graph: bool = False, stream=None) -> None:
        s = torch.cuda.current_stream().cuda_stream if stream is None else stream
        _l.check(_l.lib.tm_batch_step(self._b, C.c_void_p(s), int(use_graph)), "tm_batch_step")

    def output(self, session_id: int):
        n, state = C.c_size_t(0), C.c_int(0)
        _l.check(_l.lib.tm_batch_output(self._b, session_id, None, 0, C.byref(n), C.byref(state)), "tm_batch_output")
        buf = (C.c_int * max(1, n.value))()
        _l.check(_l.lib.tm_batch_output(self._b, session_id, buf, n.value, C.byref(n), C.byref(state)), "tm_batch_output")
        return list(buf[:n.value]), state.value

    def counts(self):
        a, p, s, t = C.c_int(0), C.c_int(0), C.c_ulonglong(0), C.c_ulonglong(0)
        _l.check(_l.lib.tm_batch_counts(self._b, C.byref(a), C.byref(p), C.byref(s), C.byref(t)), "tm_batch_counts")
        return dict(active=a.value, pending=p.value, steps=s.value, prefill_tokens=t.value)

    def forget(self, session_id: int) -> int:
        return _l.lib.tm_batch_forget(self._b, session_id)

    def has_session(self, session_id: int) -> bool:
        return bool(_l.lib.tm_cache_contains(self._cache, session_id))

    def run(self, max_rounds: int = 100000, use_graph: bool = False) -> None:
        """rounds until nothing is queued or running"""
        for _ in range(max_rounds):
            c = self.counts()
            if c["active"] == 0 and c["pending"] == 0:
                return
            self.step(use_graph)
        raise RuntimeError("scheduler did not drain")

    def close(self):
        if self._b:
            _l.lib.tm_batch_destroy(self._b)
            self._b = C.c_void_p()
        if self._cache:
            _l.lib.tm_cache_manager_destroy(self._cache)
            self._cache = C.c_void_p()
