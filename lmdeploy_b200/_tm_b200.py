"""Stand-in for the ``_turbomind`` extension module on the int4 format path: the helper functions that
src/turbomind/python/bind.cpp:414-465 exports to lmdeploy/serve/turbomind/deploy.py (same names, same argument order,
torch CUDA tensors, current stream), served by ``libtm_b200.so``.  In deploy.py the line

    import _turbomind as _tm        becomes        from lmdeploy_b200 import _tm_b200 as _tm

and nothing else changes (deploy.py:626-670 only calls the four functions below).
"""
from .turbomind import convert_s4_k_m8, dequantize_s4, fuse_w1_w3_s4_k_m8, transpose_qk_s4_k_m8  # noqa: F401

__all__ = ["transpose_qk_s4_k_m8", "fuse_w1_w3_s4_k_m8", "convert_s4_k_m8", "dequantize_s4"]
