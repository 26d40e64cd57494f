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


class TmError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {status_string(status)} ({status})")


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m lmdeploy_b200.build` "
            "(there is no non-CUDA fallback)")
    return C.CDLL(LIB_PATH)


lib = _load()

_vp, _i, _sz, _u32p = C.c_void_p, C.c_int, C.c_size_t, C.c_void_p

# name -> (restype, argtypes); must list every symbol declared in include/tm_b200.h
SIGNATURES = {
    "tm_create": (_i, [C.POINTER(_vp), _i]),
    "tm_destroy": (_i, [_vp]),
    "tm_status_string": (C.c_char_p, [_i]),
    "tm_last_cuda_error": (_i, [_vp]),
    "tm_check_device_status": (_i, [_vp, _vp, C.POINTER(C.c_uint)]),
    "tm_launch_count": (C.c_ulonglong, [_vp]),
    "tm_gemm_s4_f16_workspace_bytes": (_sz, [_i, _i, _i]),
    "tm_gemm_s4_f16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "tm_reformat_s4_k_m8": (_i, [_u32p, _u32p, _i, _i, _vp]),
    "tm_convert_s4_k_m8": (_i, [_u32p, _vp, _vp, _u32p, _vp, _u32p, _i, _i, _i, _vp]),
    "tm_transpose_qk_s4_k_m8_hf": (_i, [_u32p, _u32p, _i, _i, _i, _vp]),
    "tm_fuse_w1_w3_s4_k_m8": (_i, [_u32p, _u32p, _i, _i, _vp]),
    "tm_dequantize_s4": (_i, [_vp, _u32p, _sz, _vp]),
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

    def check_device_status(self, stream: int = 0) -> None:
        w = C.c_uint(0)
        st = lib.tm_check_device_status(self._h, _vp(stream), C.byref(w))
        if st != TM_OK:
            raise TmError(st, f"device status word 0x{w.value:x}")

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
