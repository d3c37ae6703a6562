"""ctypes binding of libtkb200.so (the C ABI declared in include/tkb200.h).

The library is built in-tree by `python -m thunderkittens_b200.build`.  There is no fallback: if the
shared object is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtkb200.so")

OK, ERR_INVALID_ARG, ERR_BAD_ALIGNMENT, ERR_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_CAPACITY = range(7)
NVFP4_SPEC, NVFP4_KERNEL_IEEE, NVFP4_KERNEL_FAST = 0, 1, 2
GEMM_DEFAULT, GEMM_PAIR_N256, GEMM_SINGLE_N256, GEMM_PAIR_N128, GEMM_SINGLE_N128, GEMM_SKINNY, GEMM_SKINNY_PREFETCH, GEMM_PAIR_M512_N256 = range(8)


class TkbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"tkb200 error {code}: {message}")
        self.code = code


_vp, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
_SIGNATURES = {
    "tkb_version": ([], _i),
    "tkb_last_error": ([], C.c_char_p),
    "tkb_set_wait_limit_cycles": ([C.c_longlong], _i),
    "tkb_device_status": ([_vp, C.POINTER(_i)], _i),
    "tkb_nvfp4_quantize": ([_vp, _i64, _vp, _vp, _vp, _i, _i, _i, _i, _vp], _i),
    "tkb_nvfp4_quantize_with_amax": ([_vp, _i64, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp], _i),
    "tkb_absmax_bf16": ([_vp, _i64, _i, _i, _vp, _vp], _i),
    "tkb_mxfp8_quantize": ([_vp, _i64, _vp, _vp, _i, _i, _vp], _i),
    "tkb_fp32_to_fp4x2": ([_vp, _vp, _sz, _vp], _i),
    "tkb_fp4x2_to_fp32": ([_vp, _vp, _sz, _vp], _i),
    "tkb_nvfp4_gemm": ([_vp] * 7 + [_i64, _i, _i, _i, _vp], _i),
    "tkb_nvfp4_gemm_ex": ([_vp] * 7 + [_i64, _i, _i, _i, _i, _vp], _i),
    "tkb_nvfp4_gemm_skinny_static": ([_vp] * 7 + [_i64, _i, _i, _i, _vp], _i),
    "tkb_mxfp8_gemm": ([_vp] * 5 + [_i64, _i, _i, _i, _vp], _i),
    "tkb_mxfp8_gemm_ex": ([_vp] * 5 + [_i64, _i, _i, _i, _i, _vp], _i),
    "tkb_bf16_gemm": ([_vp, _i64, _vp, _i64, _vp, _i64, _i, _i, _i, _vp], _i),
    "tkb_gemm_set_profile_buffer": ([_vp], _i),
    "tkb_dev_alloc": ([_sz, C.POINTER(_vp)], _i),
    "tkb_dev_free": ([_vp], _i),
    "tkb_ipc_export": ([_vp, _vp], _i),
    "tkb_ipc_open": ([_vp, C.POINTER(_vp)], _i),
    "tkb_ipc_close": ([_vp], _i),
    "tkb_signal_peers": ([C.POINTER(_vp), _i, _i, _i, C.c_uint, _i, _vp], _i),
    "tkb_wait_flags": ([_vp, _i, _i, C.c_uint, _vp], _i),
    "tkb_amax_allreduce": ([C.POINTER(_vp), _i, _i, C.c_uint, _vp, _vp, _vp], _i),
    "tkb_all_to_all": ([C.POINTER(_vp), _vp, _sz, _i, _i, _i, C.POINTER(_vp), _i, C.c_uint, _vp], _i),
    "tkb_all_to_all_4d": ([C.POINTER(_vp), _vp, C.POINTER(C.c_longlong), _i, _i, _i, _i, _i, C.POINTER(_vp), _i, C.c_uint, _vp], _i),
    "tkb_rs_maps_create": ([_vp, C.POINTER(_vp)], _i),
    "tkb_rs_maps_destroy": ([_vp], _i),
    "tkb_gemm_rs_nvfp4": ([_vp, C.c_uint, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp], _i),
    "tkb_ag_copy_create": ([_i, _i, C.POINTER(_vp)], _i),
    "tkb_ag_copy_destroy": ([_vp], _i),
    "tkb_ag_graph_create": ([_vp, C.c_uint, _i, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp), _i64, _i, _i,
                             C.POINTER(_vp)], _i),
    "tkb_ag_graph_launch": ([_vp, _vp], _i),
    "tkb_ag_graph_destroy": ([_vp], _i),
    "tkb_ag_linear_nvfp4": ([_vp, C.c_uint, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp], _i),
    "tkb_ag_gemm_nvfp4": ([C.POINTER(_vp), C.POINTER(_vp), _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, _i, C.POINTER(_vp), C.POINTER(_vp), _vp,
                           C.c_uint, _i, _vp], _i),
    "tkb_debug_ag_schedule": ([_i, _i, _i, _i, _i, _i, _i, C.POINTER(C.c_longlong), _i], _i),
    "tkb_debug_ag_schedule_parts": ([_i, _i, _i, _i, _i, _i, _i, _i, C.POINTER(C.c_longlong), _i], _i),
    "tkb_nvfp4_quantize_sharded": ([_vp, _i64, _vp, _vp, _vp, _i, _i, _i, _i, C.POINTER(_vp), _i, _i, C.c_uint, _vp], _i),
    "tkb_nvfp4_quantize_rows": ([_vp, _i64, _vp, _vp, _vp, _i, _i, _i, _vp], _i),
    "tkb_moe_route": ([_vp, _i, _i, _i, _vp, _vp, _vp], _i),
    "tkb_moe_schedule": ([_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp], _i),
    "tkb_moe_dispatch_gemm": ([C.POINTER(_vp), _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, C.c_uint,
                               _i, _i, _i, _i, _i, _i, _i, _vp], _i),
    "tkb_moe_layer_nvfp4": ([_vp, C.c_uint, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp], _i),
    "tkb_moe_combine": ([C.POINTER(_vp), _i64, _vp, _vp, _vp, _i, _i, _i, _i, _vp], _i),
    "tkb_fp8_gemm": ([_vp, _i64, _vp, _i64, _vp, _i64, _i, _i, _i, _vp], _i),
    "tkb_fp8_gemm_ex": ([_vp, _i64, _vp, _i64, _vp, _i64, _i, _i, _i, _i, _vp], _i),
    "tkb_nvfp4_gemm_quant": ([_vp] * 10 + [_i, _i, _i, _i, _vp], _i),
    "tkb_bf16_gemm_ex": ([_vp, _i64, _vp, _i64, _vp, _i64, _i, _i, _i, _i, _vp], _i),
}

class AgState(C.Structure):
    """Mirror of tkb_ag_state (include/tkb200.h)."""
    _fields_ = [("rank", _i), ("world", _i), ("M", _i), ("K", _i),
                ("codes", (_vp * 8) * 2), ("scales", (_vp * 8) * 2), ("arrived", (_vp * 8) * 2), ("slots", (_vp * 8) * 2),
                ("done", _vp * 8), ("amax", _vp), ("sg", _vp), ("exit_counter", _vp),
                ("copy", _vp), ("epoch_counter", _vp)]


class RsState(C.Structure):
    """Mirror of tkb_rs_state (include/tkb200.h)."""
    _fields_ = [("rank", _i), ("world", _i), ("M", _i), ("N", _i), ("out", _vp * 8), ("flags", _vp * 8), ("maps", _vp)]


class MoeState(C.Structure):
    """Mirror of tkb_moe_state (include/tkb200.h)."""
    _fields_ = [(n, _i) for n in ("rank", "world", "T", "H", "I", "E", "top_k", "cap_rows")] + \
               [("xq_rows", (_vp * 8) * 2), ("slots", (_vp * 8) * 2), ("experts_all", (_vp * 8) * 2),
                ("Y", _vp * 8), ("flags", _vp * 8), ("counters", _vp * 8)] + \
               [(n, _vp) for n in ("codes", "scales", "experts_local", "weights", "counts", "padded", "pull_idx", "block_expert", "num_blocks",
                                   "comb_idx", "arrived", "sg")]


_lib = None


def lib() -> C.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m thunderkittens_b200.build` (no CPU fallback exists)")
        L = C.CDLL(LIB_PATH)
        for name, (argtypes, restype) in _SIGNATURES.items():
            if not hasattr(L, name):
                continue   # optional entry points are bound where they are declared
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = L
    return _lib


def bind(name: str, argtypes, restype=_i):
    fn = getattr(lib(), name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def check(code: int) -> None:
    if code != OK:
        raise TkbError(code, lib().tkb_last_error().decode())


def device_status(stream: int = 0) -> int:
    st = C.c_int(0)
    check(lib().tkb_device_status(stream, C.byref(st)))
    return st.value
