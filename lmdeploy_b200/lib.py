"""ctypes binding of ``libtm_b200.so`` — the only way Python reaches the kernels.

There is no fallback: if the library is missing or a symbol of ``include/tm_b200.h`` is
absent, import of this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_lib", "libtm_b200.so")

TM_OK = 0
TM_ERR_INVALID_ARG = -1
TM_ERR_UNSUPPORTED = -2
TM_ERR_WORKSPACE = -3
TM_ERR_CUDA = -4
TM_ERR_DEVICE_TIMEOUT = -5
TM_ERR_NCCL = -6
TM_ERR_NOT_BUILT = -7
TM_ERR_IO = -8


class TmError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} ({status})")


def _preload_bundled_nccl() -> None:
    """One NCCL per process: when PyTorch's wheel ships its own libnccl.so.2 (nvidia.nccl), load that one before this
    library, whose NCCL dependency would otherwise bind the system copy under the same soname and leave a later
    ``import torch`` with an NCCL that lacks symbols it needs."""
    import importlib.util
    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        spec = None
    for d in (list(spec.submodule_search_locations) if spec and spec.submodule_search_locations else []):
        path = os.path.join(d, "lib", "libnccl.so.2")
        if os.path.exists(path):
            C.CDLL(path, mode=C.RTLD_GLOBAL)
            return


def _load() -> C.CDLL:
    _preload_bundled_nccl()
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m lmdeploy_b200.build` "
            "(there is no non-CUDA fallback)")
    return C.CDLL(LIB_PATH)


lib = _load()

_vp, _i, _sz, _u32p = C.c_void_p, C.c_int, C.c_size_t, C.c_void_p

class TmMmhaParams(C.Structure):
    """ctypes mirror of ``tm_mmha_params`` (include/tm_b200.h), field for field."""
    _fields_ = [
        ("out", C.c_void_p), ("q", C.c_void_p), ("q_bias", C.c_void_p), ("k", C.c_void_p), ("k_bias", C.c_void_p),
        ("v", C.c_void_p), ("v_bias", C.c_void_p),
        ("stride", C.c_int), ("batch_size", C.c_int), ("memory_max_len", C.c_int), ("num_heads", C.c_int),
        ("num_kv_heads", C.c_int), ("hidden_size_per_head", C.c_int), ("rotary_embedding_dim", C.c_int),
        ("timestep", C.c_int), ("inv_sqrt_dh", C.c_float), ("total_padding_tokens", C.c_void_p),
        ("int8_mode", C.c_int), ("attention_k_scale", C.c_float), ("attention_k_zp", C.c_float),
        ("attention_v_scale", C.c_float), ("attention_v_zp", C.c_float),
        ("finished", C.c_void_p), ("length_per_sample", C.c_void_p), ("k_cache_per_sample", C.c_void_p),
        ("v_cache_per_sample", C.c_void_p), ("kv_cache_per_sample_offset", C.c_size_t),
        ("max_position_embeddings", C.c_int), ("use_dynamic_ntk", C.c_int), ("use_logn_attn", C.c_int),
        ("rotary_embedding_base", C.c_float),
    ]


class TmSamplingParams(C.Structure):
    """ctypes mirror of ``tm_sampling_params`` (include/tm_b200.h), field for field."""
    _fields_ = [
        ("logits", C.c_void_p), ("ld", C.c_int), ("vocab_size", C.c_int), ("batch_size", C.c_int),
        ("output_ids", C.c_void_p), ("step", C.c_int), ("input_lengths", C.c_void_p), ("max_input_length", C.c_int),
        ("temperatures", C.c_void_p), ("repetition_penalties", C.c_void_p), ("min_lengths", C.c_void_p),
        ("sequence_lengths", C.c_void_p), ("end_ids", C.c_void_p), ("top_ks", C.c_void_p), ("max_top_k", C.c_int),
        ("top_ps", C.c_void_p), ("top_p", C.c_float), ("rng_states", C.c_void_p), ("uniforms", C.c_void_p),
        ("ids", C.c_void_p), ("sequence_lengths_out", C.c_void_p), ("finished", C.c_void_p), ("skip_decode", C.c_void_p),
        ("output_ids_stride", C.c_int),
    ]


class TmRequest(C.Structure):
    """ctypes mirror of ``tm_request``."""
    _fields_ = [("id", C.c_uint64), ("start_flag", C.c_int), ("end_flag", C.c_int), ("input_ids", C.POINTER(C.c_int)),
                ("input_length", C.c_int), ("request_output_len", C.c_int), ("top_k", C.c_int), ("top_p", C.c_float),
                ("temperature", C.c_float), ("repetition_penalty", C.c_float), ("random_seed", C.c_ulonglong),
                ("ignore_eos", C.c_int), ("stop_ids", C.POINTER(C.c_int)), ("stop_count", C.c_int),
                ("bad_ids", C.POINTER(C.c_int)), ("bad_count", C.c_int), ("rewind", C.c_int), ("step", C.c_int)]


class TmContextAttentionParams(C.Structure):
    """ctypes mirror of ``tm_context_attention_params`` (include/tm_b200.h), field for field."""
    _fields_ = [
        ("attn_out", C.c_void_p), ("query", C.c_void_p), ("key_cache", C.c_void_p), ("val_cache", C.c_void_p),
        ("cache_layer_offset", C.c_size_t), ("cu_seqlens", C.c_void_p), ("context_lengths", C.c_void_p),
        ("batch_size", C.c_int), ("head_num", C.c_int), ("kv_head_num", C.c_int), ("size_per_head", C.c_int),
        ("max_q_len", C.c_int), ("max_seq_len", C.c_int), ("quant_policy", C.c_int), ("kv_scale", C.c_float * 4),
        ("status_word", C.c_void_p),
    ]


class TmLlamaConfig(C.Structure):
    """ctypes mirror of ``tm_llama_config``."""
    _fields_ = [("head_num", C.c_int), ("kv_head_num", C.c_int), ("size_per_head", C.c_int), ("inter_size", C.c_int),
                ("num_layer", C.c_int), ("vocab_size", C.c_int), ("norm_eps", C.c_float), ("rope_theta", C.c_float),
                ("quant_policy", C.c_int), ("group_size", C.c_int), ("tensor_para_size", C.c_int),
                ("tensor_para_rank", C.c_int), ("max_batch_size", C.c_int), ("session_len", C.c_int)]


class TmLlamaWorkspaceInfo(C.Structure):
    """ctypes mirror of ``tm_llama_workspace_info``."""
    _fields_ = [("model_name", C.c_char * 64), ("weight_type", C.c_char * 16), ("start_id", C.c_int), ("end_id", C.c_int),
                ("rotary_embedding_dim", C.c_int), ("max_context_token_num", C.c_int), ("step_length", C.c_int),
                ("cache_max_entry_count", C.c_int), ("cache_chunk_size", C.c_int), ("use_context_fmha", C.c_int),
                ("attn_bias", C.c_int), ("max_position_embeddings", C.c_int), ("use_dynamic_ntk", C.c_int),
                ("use_logn_attn", C.c_int)]


class TmLlamaLayerWeights(C.Structure):
    """ctypes mirror of ``tm_llama_layer_weights``."""
    _fields_ = [(n, C.c_void_p) for n in (
        "self_attn_norm", "ffn_norm", "qkv_qweight", "qkv_scales_zeros", "qkv_bias", "o_qweight", "o_scales_zeros",
        "w13_qweight", "w13_scales_zeros", "w2_qweight", "w2_scales_zeros")] + [("past_kv_scale", C.c_float * 4)]


class TmLlamaDecodeState(C.Structure):
    """ctypes mirror of ``tm_llama_decode_state``."""
    _fields_ = [("batch_size", C.c_int), ("max_steps", C.c_int), ("k_cache_ptrs", C.c_void_p),
                ("v_cache_ptrs", C.c_void_p), ("sequence_lengths", C.c_void_p), ("start_step", C.c_void_p),
                ("forced_ids", C.c_void_p), ("output_ids", C.c_void_p), ("step", C.c_void_p),
                ("hidden_out", C.c_void_p), ("logits_out", C.c_void_p)]


class TmCacheSequence(C.Structure):
    """ctypes mirror of ``tm_cache_sequence``."""
    _fields_ = [("id", C.c_uint64), ("max_seq_len", C.c_size_t), ("cache_len", C.c_size_t), ("token_count", C.c_size_t),
                ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("timestamp", C.c_uint64)]


class TmLlamaPrefillState(C.Structure):
    """ctypes mirror of ``tm_llama_prefill_state``."""
    _fields_ = [("batch_size", C.c_int), ("token_num", C.c_int), ("max_q_len", C.c_int), ("input_ids", C.c_void_p),
                ("cu_seqlens", C.c_void_p), ("history_lengths", C.c_void_p), ("context_lengths", C.c_void_p),
                ("k_cache_ptrs", C.c_void_p), ("v_cache_ptrs", C.c_void_p), ("hidden_out", C.c_void_p)]


# name -> (restype, argtypes); must list every symbol declared in include/tm_b200.h
SIGNATURES = {
    "tm_create": (_i, [C.POINTER(_vp), _i]),
    "tm_destroy": (_i, [_vp]),
    "tm_handle_of_current_device": (_vp, []),
    "tm_status_string": (C.c_char_p, [_i]),
    "tm_last_cuda_error": (_i, [_vp]),
    "tm_check_device_status": (_i, [_vp, _vp, C.POINTER(C.c_uint)]),
    "tm_launch_count": (C.c_ulonglong, [_vp]),
    "tm_set_option": (_i, [_vp, C.c_char_p, _i]),
    "tm_gemm_s4_f16_workspace_bytes": (_sz, [_i, _i, _i]),
    "tm_gemm_s4_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "tm_gemm_s4_f16_noalloc": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "tm_reformat_s4_k_m8": (_i, [_u32p, _u32p, _i, _i, _vp]),
    "tm_convert_s4_k_m8": (_i, [_u32p, _vp, _vp, _u32p, _vp, _u32p, _i, _i, _i, _vp]),
    "tm_transpose_qk_s4_k_m8_hf": (_i, [_u32p, _u32p, _i, _i, _i, _vp]),
    "tm_fuse_w1_w3_s4_k_m8": (_i, [_u32p, _u32p, _i, _i, _vp]),
    "tm_dequantize_s4": (_i, [_vp, _u32p, _sz, _vp]),
    "tm_batch_create": (_i, [C.POINTER(_vp), _vp, _vp, _i, _i, _i, _i, _i]),
    "tm_batch_destroy": (_i, [_vp]),
    "tm_batch_submit": (_i, [_vp, C.POINTER(TmRequest)]),
    "tm_batch_step": (_i, [_vp, _vp, _i]),
    "tm_batch_output": (_i, [_vp, C.c_uint64, C.POINTER(C.c_int), _sz, C.POINTER(_sz), C.POINTER(_i)]),
    "tm_batch_forget": (_i, [_vp, C.c_uint64]),
    "tm_batch_counts": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)]),
    "tm_sampling_rng_state_bytes": (_sz, []),
    "tm_sampling_rng_init": (_i, [_vp, _i, _vp, C.c_ulonglong, _vp]),
    "tm_ban_bad_words": (_i, [_vp, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp]),
    "tm_stop_words_criterion": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _vp]),
    "tm_length_criterion": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "tm_sample_topk": (_i, [_vp, C.POINTER(TmSamplingParams), _vp]),
    "tm_sample_topp": (_i, [_vp, C.POINTER(TmSamplingParams), _vp]),
    "tm_top_p_decay": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "tm_lm_head_f16": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _vp]),
    "tm_mmha_decode": (_i, [_vp, C.POINTER(TmMmhaParams), _vp]),
    "tm_comm_unique_id": (_i, [_vp]),
    "tm_comm_create": (_i, [C.POINTER(_vp), _i, _i, _vp, _i]),
    "tm_comm_destroy": (_i, [_vp]),
    "tm_allreduce_sum_f16": (_i, [_vp, _vp, _sz, _vp]),
    "tm_allgather": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "tm_comm_p2p_export": (_i, [_vp, _sz, _vp]),
    "tm_comm_p2p_import": (_i, [_vp, _vp]),
    "tm_comm_set_option": (_i, [_vp, C.c_char_p, C.c_longlong]),
    "tm_comm_p2p_slot": (_vp, [_vp, _i]),
    "tm_comm_p2p_slot_bytes": (_sz, [_vp]),
    "tm_allreduce_add_residual_rmsnorm": (_i, [_vp, _i, _vp, _vp, _vp, C.c_float, _i, _i, _vp, _vp]),
    "tm_llama_create": (_i, [C.POINTER(_vp), _vp, _vp, C.POINTER(TmLlamaConfig)]),
    "tm_llama_destroy": (_i, [_vp]),
    "tm_llama_set_layer": (_i, [_vp, _i, C.POINTER(TmLlamaLayerWeights)]),
    "tm_llama_set_globals": (_i, [_vp, _vp, _vp, _vp]),
    "tm_llama_load_workspace": (_i, [_vp, C.c_char_p]),
    "tm_llama_read_config": (_i, [C.c_char_p, C.POINTER(TmLlamaConfig), C.POINTER(TmLlamaWorkspaceInfo)]),
    "tm_llama_decode": (_i, [_vp, C.POINTER(TmLlamaDecodeState), _i, _i, _vp]),
    "tm_llama_last_launches": (C.c_ulonglong, [_vp]),
    "tm_llama_check_status": (_i, [_vp, _vp, C.POINTER(C.c_uint)]),
    "tm_cache_manager_create": (_i, [C.POINTER(_vp), _sz, _sz, _sz, _sz, _sz, _sz, _sz, _i]),
    "tm_cache_manager_destroy": (_i, [_vp]),
    "tm_cache_create": (_i, [_vp, C.c_uint64, _vp, C.POINTER(TmCacheSequence)]),
    "tm_cache_fetch": (_i, [_vp, C.c_uint64, _vp, C.POINTER(TmCacheSequence)]),
    "tm_cache_update": (_i, [_vp, C.POINTER(TmCacheSequence), C.POINTER(C.c_int), _sz]),
    "tm_cache_tokens": (_i, [_vp, C.c_uint64, C.POINTER(C.c_int), _sz, C.POINTER(_sz)]),
    "tm_cache_erase": (_i, [_vp, C.c_uint64]),
    "tm_cache_contains": (_i, [_vp, C.c_uint64]),
    "tm_llama_prefill": (_i, [_vp, C.POINTER(TmLlamaPrefillState), _vp]),
    "tm_rmsnorm": (_i, [_vp, _vp, _vp, C.c_float, _i, _i, _vp]),
    "tm_add_residual_rmsnorm": (_i, [_vp, _vp, _vp, _vp, C.c_float, _i, _i, _vp]),
    "tm_add_fused_qkv_bias_transpose": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i,
                                             C.c_float, _i, _i, _i, _vp]),
    "tm_context_attention_last_status": (_i, [C.POINTER(C.c_uint)]),
    "tm_context_attention": (_i, [C.POINTER(TmContextAttentionParams), _vp]),
    "tm_extend_kv_cache": (_i, [_vp, _vp, _sz, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _vp, _i, C.POINTER(C.c_float)]),
    "tm_transpose_kv_cache": (_i, [_vp, _vp, _vp, _vp, _sz, _i, _vp, _i, _i, _i, _i, _i, _vp, _i, C.POINTER(C.c_float)]),
}


def _bind():
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args


_bind()


def status_string(status: int) -> str:
    return lib.tm_status_string(status).decode()


def check(status: int, where: str) -> None:
    if status != TM_OK:
        raise TmError(status, where)


class Handle:
    """Per-device state (tm_create / tm_destroy)."""

    def __init__(self, device: int = 0):
        self._h = _vp()
        check(lib.tm_create(C.byref(self._h), device), "tm_create")
        self.device = device

    @property
    def ptr(self):
        return self._h

    def launch_count(self) -> int:
        return int(lib.tm_launch_count(self._h))

    def set_option(self, name: str, value: int) -> None:
        """tuning knob of this handle (see tm_set_option in include/tm_b200.h)"""
        check(lib.tm_set_option(self._h, name.encode(), int(value)), f"tm_set_option({name})")

    def check_device_status(self, stream: int = 0) -> None:
        w = C.c_uint(0)
        st = lib.tm_check_device_status(self._h, _vp(stream), C.byref(w))
        if st != TM_OK:
            raise TmError(st, f"device status word 0x{w.value:x}, cudaError {lib.tm_last_cuda_error(self._h)}")

    def close(self):
        if self._h:
            lib.tm_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_handles = {}


def default_handle(device: int = 0) -> Handle:
    if device not in _handles:
        _handles[device] = Handle(device)
    return _handles[device]
