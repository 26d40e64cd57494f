"""Host-side mirror of the TurboMind operator surface on the quantized decode path.

Same names, argument order and meaning as lmdeploy v0.0.9:

* ``GemmS4F16.Run``            src/turbomind/kernels/gemm_s_f16/gemm_s4_f16.h:41-51
* ``LlamaDenseWeight`` / ``WeightType``   src/turbomind/models/llama/LlamaDenseWeight.h:28-63
* ``LlamaLinear.forward``      src/turbomind/models/llama/LlamaLinear.h:28-42
* ``masked_multihead_attention`` + ``Masked_multihead_attention_params``
                               src/turbomind/kernels/decoder_masked_multihead_attention.h:50-133
* ``invokeRootMeanSquareNorm`` src/turbomind/models/llama/llama_kernels.cu:69-79
* ``invokeFusedAddBiasResidualRMSNorm``  src/turbomind/models/llama/llama_decoder_kernels.cu:147-160
* ``transpose_qk_s4_k_m8`` / ``fuse_w1_w3_s4_k_m8`` / ``convert_s4_k_m8`` / ``dequantize_s4``
                               the ``_turbomind`` helpers of src/turbomind/python/bind.cpp:414-465

Tensors are torch CUDA tensors (device memory + streams are torch's job, nothing else);
every call goes through the C ABI of ``libtm_b200.so`` on the current torch stream.
Errors that the reference reports by throwing ``std::runtime_error`` / ``FT_CHECK`` surface
as :class:`lmdeploy_b200.lib.TmError`.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as _l


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("tm_b200 operators take CUDA tensors only (there is no CPU path)")
        if t is not None and not t.is_contiguous():
            raise ValueError("tm_b200 operators take contiguous tensors")


class WeightType(enum.IntEnum):
    kFP32 = 0
    kFP16 = 1
    kFP8 = 2
    kINT8 = 3
    kINT4 = 4


@dataclass
class LlamaDenseWeight:
    input_dims: int
    output_dims: int
    kernel: torch.Tensor                     # int4: int32 [K, N/8] in the runtime layout
    type: WeightType
    bias: Optional[torch.Tensor] = None
    scales_and_zeros: Optional[torch.Tensor] = None   # half [K/g, N, 2] = {64 + z, s}
    group_size: int = 128


class GemmS4F16:
    kGemm = 0
    kFusedSiluFfn = 1

    def __init__(self, device: Optional[int] = None):
        self.device = torch.cuda.current_device() if device is None else device
        self.handle = _l.default_handle(self.device)

    def Run(self, C_out, A, B, Q, m, n, k, group_size, type, algo_id=-1, stream=None):
        """C[n, m] = B[n, k] . dequant(A, Q)^T  (m = output features, n = tokens)."""
        _need_cuda(C_out, A, B, Q)
        st = _stream() if stream is None else C.c_void_p(stream)
        s = _l.lib.tm_gemm_s4_f16(self.handle.ptr, _ptr(C_out), _ptr(A), _ptr(B), _ptr(Q), int(m), int(n), int(k),
                                  int(group_size), int(type), None, 0, st)
        _l.check(s, "GemmS4F16.Run")


class LlamaLinear:
    kGemm = 0
    kFusedSiluFfn = 1

    def __init__(self, device: Optional[int] = None):
        self.gemm_s4_f16_ = GemmS4F16(device)

    def forward(self, output_data, input_data, batch_size, weight: LlamaDenseWeight, type=0):
        if weight.type == WeightType.kINT4:
            if input_data.dtype != torch.float16:
                raise NotImplementedError("int4 weights need half activations")  # LlamaLinear.h:64,78-80
            self.gemm_s4_f16_.Run(output_data, weight.kernel, input_data, weight.scales_and_zeros, weight.output_dims,
                                  batch_size, weight.input_dims, weight.group_size,
                                  GemmS4F16.kFusedSiluFfn if type == self.kFusedSiluFfn else GemmS4F16.kGemm, -1)
        else:
            raise NotImplementedError("only the int4 (W4A16) path is built; fp16 linears are out of scope")


# ---- `_turbomind` format helpers (bind.cpp:414-465): (src, dst, ...) argument order kept ----

def transpose_qk_s4_k_m8(src, dst, m, k, size_per_head):
    _need_cuda(src, dst)
    _l.check(_l.lib.tm_transpose_qk_s4_k_m8_hf(_ptr(dst), _ptr(src), m, k, size_per_head, _stream()),
             "transpose_qk_s4_k_m8")


def fuse_w1_w3_s4_k_m8(src, dst, m, k):
    _need_cuda(src, dst)
    _l.check(_l.lib.tm_fuse_w1_w3_s4_k_m8(_ptr(dst), _ptr(src), m, k, _stream()), "fuse_w1_w3_s4_k_m8")


def convert_s4_k_m8(A_dst, Q_dst, ws, A_src, scales, qzeros, m, k, group_size):
    _need_cuda(A_dst, Q_dst, ws, A_src, scales, qzeros)
    _l.check(_l.lib.tm_convert_s4_k_m8(_ptr(A_dst), _ptr(Q_dst), _ptr(ws), _ptr(A_src), _ptr(scales), _ptr(qzeros),
                                       m, k, group_size, _stream()), "convert_s4_k_m8")


def dequantize_s4(src, dst):
    _need_cuda(src, dst)
    if src.numel() * 8 != dst.numel():
        raise ValueError("dst must hold 8 halves per source word")  # bind.cpp:462
    _l.check(_l.lib.tm_dequantize_s4(_ptr(dst), _ptr(src), src.numel(), _stream()), "dequantize_s4")


# ---- decode attention -----------------------------------------------------------------------

QUANT_POLICY_CACHE_KV_INT8 = 0x04  # QuantPolicy::kCacheKVInt8, src/turbomind/models/llama/llama_utils.h:12-20


@dataclass
class Masked_multihead_attention_params:
    """The fields ``fusedQKV_masked_attention_dispatch`` fills
    (LlamaDecoderSelfAttentionLayer.cc:87-161); tensors instead of raw pointers.  ``q``, ``k``,
    ``v`` are views into one fused ``[batch, stride]`` half buffer."""
    out: torch.Tensor = None
    q: torch.Tensor = None
    k: torch.Tensor = None
    v: torch.Tensor = None
    q_bias: Optional[torch.Tensor] = None
    k_bias: Optional[torch.Tensor] = None
    v_bias: Optional[torch.Tensor] = None
    stride: int = 0
    batch_size: int = 0
    memory_max_len: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    hidden_size_per_head: int = 128
    rotary_embedding_dim: int = 128
    rotary_embedding_base: float = 10000.0
    max_position_embeddings: int = 0
    use_dynamic_ntk: bool = False
    use_logn_attn: bool = False
    timestep: int = 0
    inv_sqrt_dh: float = 0.0
    total_padding_tokens: Optional[torch.Tensor] = None   # int32 [batch]
    finished: Optional[torch.Tensor] = None               # bool [batch]
    length_per_sample: torch.Tensor = None                # int32 [batch]
    k_cache_per_sample: torch.Tensor = None               # int64 [batch] device array of base pointers
    v_cache_per_sample: torch.Tensor = None
    kv_cache_per_sample_offset: int = 0
    int8_mode: int = 0
    attention_k_scale: float = 0.0
    attention_k_zp: float = 0.0
    attention_v_scale: float = 0.0
    attention_v_zp: float = 0.0


def masked_multihead_attention(params: Masked_multihead_attention_params, stream=None, handle=None):
    p = params
    _need_cuda(p.out, p.length_per_sample, p.k_cache_per_sample, p.v_cache_per_sample, p.total_padding_tokens,
               p.finished)
    for t in (p.q, p.k, p.v):
        if t is None or not t.is_cuda:
            raise ValueError("q, k, v must be CUDA tensors")
    c = _l.TmMmhaParams()
    c.out, c.q, c.k, c.v = p.out.data_ptr(), p.q.data_ptr(), p.k.data_ptr(), p.v.data_ptr()
    c.q_bias = 0 if p.q_bias is None else p.q_bias.data_ptr()
    c.k_bias = 0 if p.k_bias is None else p.k_bias.data_ptr()
    c.v_bias = 0 if p.v_bias is None else p.v_bias.data_ptr()
    c.stride, c.batch_size, c.memory_max_len = p.stride, p.batch_size, p.memory_max_len
    c.num_heads, c.num_kv_heads, c.hidden_size_per_head = p.num_heads, p.num_kv_heads, p.hidden_size_per_head
    c.rotary_embedding_dim, c.timestep, c.inv_sqrt_dh = p.rotary_embedding_dim, p.timestep, p.inv_sqrt_dh
    c.total_padding_tokens = 0 if p.total_padding_tokens is None else p.total_padding_tokens.data_ptr()
    c.int8_mode = p.int8_mode
    c.attention_k_scale, c.attention_k_zp = p.attention_k_scale, p.attention_k_zp
    c.attention_v_scale, c.attention_v_zp = p.attention_v_scale, p.attention_v_zp
    c.finished = 0 if p.finished is None else p.finished.data_ptr()
    c.length_per_sample = p.length_per_sample.data_ptr()
    c.k_cache_per_sample, c.v_cache_per_sample = p.k_cache_per_sample.data_ptr(), p.v_cache_per_sample.data_ptr()
    c.kv_cache_per_sample_offset = p.kv_cache_per_sample_offset
    c.max_position_embeddings, c.use_dynamic_ntk, c.use_logn_attn = (p.max_position_embeddings, int(p.use_dynamic_ntk),
                                                                      int(p.use_logn_attn))
    c.rotary_embedding_base = p.rotary_embedding_base
    h = handle or _l.default_handle(p.out.device.index)
    st = _stream() if stream is None else C.c_void_p(stream)
    _l.check(_l.lib.tm_mmha_decode(h.ptr, C.byref(c), st), "masked_multihead_attention")


def invokeRootMeanSquareNorm(out, input, scale, eps, m, n, stream=None):
    _need_cuda(out, input, scale)
    st = _stream() if stream is None else C.c_void_p(stream)
    _l.check(_l.lib.tm_rmsnorm(_ptr(out), _ptr(input), _ptr(scale), eps, m, n, st), "invokeRootMeanSquareNorm")


def invokeFusedAddBiasResidualRMSNorm(residual, in_out, bias, scale, eps, batch_size, n_dims, stream=None):
    _need_cuda(residual, in_out, bias, scale)
    st = _stream() if stream is None else C.c_void_p(stream)
    _l.check(_l.lib.tm_add_residual_rmsnorm(_ptr(residual), _ptr(in_out), _ptr(bias), _ptr(scale), eps, batch_size,
                                            n_dims, st), "invokeFusedAddBiasResidualRMSNorm")


# ----------------------------------------------------------------------------------------------
# prefill-side writers around the KV cache (src/turbomind/kernels/unfused_attention_kernels.h:66-86,
# src/turbomind/models/llama/llama_kernels.h:36-68): same names and argument order as the reference

def _kv_scale(kv_scale):
    if kv_scale is None:
        return None
    vals = [float(v) for v in kv_scale]
    if len(vals) != 4:
        raise ValueError("kv_scale holds k_scale, k_zp, v_scale, v_zp")
    return (C.c_float * 4)(*vals)


def invokeAddFusedQKVBiasTranspose(q_buf, k_buf, v_buf, QKV, qkv_bias, padding_offset, history_length, input_length,
                                   batch_size, seq_len, token_num, head_num, kv_head_num, size_per_head,
                                   rotary_embedding_dim, rotary_embedding_base, max_position_embeddings, use_dynamic_ntk,
                                   use_logn_attn, stream=None):
    _need_cuda(q_buf, k_buf, v_buf, QKV, qkv_bias, padding_offset, history_length, input_length)
    st = _stream() if stream is None else C.c_void_p(stream)
    _l.check(_l.lib.tm_add_fused_qkv_bias_transpose(
        _ptr(q_buf), _ptr(k_buf), _ptr(v_buf), _ptr(QKV), _ptr(qkv_bias), _ptr(padding_offset), _ptr(history_length),
        _ptr(input_length), batch_size, seq_len, token_num, head_num, kv_head_num, size_per_head, rotary_embedding_dim,
        rotary_embedding_base, max_position_embeddings, int(use_dynamic_ntk), int(use_logn_attn), st),
        "invokeAddFusedQKVBiasTranspose")


def invokeExtendKVCache(k_dst, v_dst, dst_offset, k_src, v_src, local_batch_size, query_length, max_q_len, history_length,
                        max_seq_len, size_per_head, local_head_num, stream=None, quant=0, kv_scale=None):
    """k_dst / v_dst: int64 device tensors holding one cache base pointer per sequence."""
    _need_cuda(k_dst, v_dst, k_src, v_src, query_length, history_length)
    st = _stream() if stream is None else C.c_void_p(stream)
    _l.check(_l.lib.tm_extend_kv_cache(_ptr(k_dst), _ptr(v_dst), dst_offset, _ptr(k_src), _ptr(v_src), local_batch_size,
                                       _ptr(query_length), max_q_len, _ptr(history_length), max_seq_len, size_per_head,
                                       local_head_num, st, quant, _kv_scale(kv_scale)), "invokeExtendKVCache")


def invokeTransposeKVCache(key_cache_trans, val_cache_trans, key_cache, val_cache, src_offset, batch_size, key_length,
                           max_kv_len, max_seq_len, size_per_head, head_num, head_n_rep, stream=None, quant=0,
                           kv_scale=None):
    _need_cuda(key_cache_trans, val_cache_trans, key_cache, val_cache, key_length)
    st = _stream() if stream is None else C.c_void_p(stream)
    _l.check(_l.lib.tm_transpose_kv_cache(_ptr(key_cache_trans), _ptr(val_cache_trans), _ptr(key_cache), _ptr(val_cache),
                                          src_offset, batch_size, _ptr(key_length), max_kv_len, max_seq_len, size_per_head,
                                          head_num, head_n_rep, st, quant, _kv_scale(kv_scale)), "invokeTransposeKVCache")


def fusedMultiHeadAttention(attn_out, query, key_cache_ptrs, val_cache_ptrs, cache_layer_offset, cu_seqlens, context_lengths,
                            batch_size, max_q_len, max_seq_len, head_num, kv_head_num, size_per_head=128, quant_policy=0,
                            kv_scale=None, stream=None):
    """LlamaContextAttentionLayer<T>::fusedMultiHeadAttention (src/turbomind/models/llama/LlamaContextAttentionLayer.cc:
    257-313) with the layer's members passed explicitly: causal attention of the new tokens over the cache in place,
    attn_out [token_num, head_num * size_per_head] packed by cu_seqlens."""
    _need_cuda(attn_out, query, key_cache_ptrs, val_cache_ptrs, cu_seqlens, context_lengths)
    a = _l.TmContextAttentionParams()
    a.attn_out, a.query = attn_out.data_ptr(), query.data_ptr()
    a.key_cache, a.val_cache, a.cache_layer_offset = key_cache_ptrs.data_ptr(), val_cache_ptrs.data_ptr(), cache_layer_offset
    a.cu_seqlens, a.context_lengths = cu_seqlens.data_ptr(), context_lengths.data_ptr()
    a.batch_size, a.head_num, a.kv_head_num, a.size_per_head = batch_size, head_num, kv_head_num, size_per_head
    a.max_q_len, a.max_seq_len, a.quant_policy = max_q_len, max_seq_len, quant_policy
    if kv_scale is not None:
        a.kv_scale = _kv_scale(kv_scale)
    st = _stream() if stream is None else C.c_void_p(stream)
    _l.check(_l.lib.tm_context_attention(C.byref(a), st), "fusedMultiHeadAttention")
