"""CPU ORACLE — test infrastructure only.

numpy-facing wrappers over oracle/tk_oracle.cpp (the C++ restatement of the reference arithmetic),
over the CUDA-toolkit host codecs (nv_host_codecs.cpp) and, when it has been built, over the
reference's own naive GEMM kernels compiled for the host (oracle/_ref).  Only tests, the smoke
check and the benchmark's CPU-baseline leg may import this package; the product never does.

bf16 tensors travel as uint16 numpy arrays (bit patterns), fp4x2/e4m3/e8m0 as uint8.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


def _load(path):
    return C.CDLL(path)


_lib = None
_nvh = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        L = _load(_build.build_oracle())
        L.tko_num_threads.restype = C.c_int
        L.tko_absmax_bf16.restype = C.c_float
        L.tko_absmax_bf16.argtypes = [_u16p, C.c_size_t]
        L.tko_scale_swizzle_idx.restype = C.c_size_t
        L.tko_scale_swizzle_idx.argtypes = [C.c_int] * 3
        for n, a, b in [("tko_f32_to_bf16", _f32p, _u16p), ("tko_bf16_to_f32", _u16p, _f32p),
                        ("tko_f32_to_e4m3", _f32p, _u8p), ("tko_e4m3_to_f32", _u8p, _f32p),
                        ("tko_f32_to_e8m0", _f32p, _u8p), ("tko_e8m0_to_f32", _u8p, _f32p),
                        ("tko_fp32_to_fp4x2", _f32p, _u8p), ("tko_fp4x2_to_fp32", _u8p, _f32p)]:
            getattr(L, n).argtypes = [a, b, C.c_size_t]
            getattr(L, n).restype = None
        L.tko_fill_uniform_f32.argtypes = [_f32p, C.c_size_t, C.c_uint64, C.c_float, C.c_float]
        L.tko_nvfp4_quantize.argtypes = [_u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, _u8p, _u8p, _f32p]
        L.tko_mxfp8_quantize.argtypes = [_u16p, C.c_int, C.c_int, _u8p, _u8p]
        L.tko_nvfp4_gemm.argtypes = [_u8p, _u8p, _f32p, _u8p, _u8p, _f32p, _u16p] + [C.c_int] * 5
        L.tko_nvfp4_gemm_f32.argtypes = [_u8p, _u8p, _f32p, _u8p, _u8p, _f32p, _f32p] + [C.c_int] * 4
        L.tko_mxfp8_gemm.argtypes = [_u8p, _u8p, _u8p, _u8p, _u16p] + [C.c_int] * 5
        L.tko_bf16_gemm.argtypes = [_u16p, _u16p, _u16p] + [C.c_int] * 5
        L.tko_fp8_gemm.argtypes = [_u8p, _u8p, _u16p] + [C.c_int] * 5
        L.tko_moe_route.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _i32p, _f32p]
        L.tko_moe_schedule.restype = C.c_int
        L.tko_moe_schedule.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p,
                                       C.c_void_p, C.c_int]
        L.tko_moe_combine.argtypes = [_u16p, _i32p, _f32p, C.c_int, C.c_int, C.c_int, _u16p]
        _lib = L
    return _lib


def nvhost():
    """CUDA-toolkit host conversions (pins the codecs)."""
    global _nvh
    if _nvh is None:
        L = _load(_build.build_nv_codecs())
        for n, a, b in [("nvh_f32_to_e4m3", _f32p, _u8p), ("nvh_e4m3_to_f32", _u8p, _f32p),
                        ("nvh_f32_to_e8m0", _f32p, _u8p), ("nvh_e8m0_to_f32", _u8p, _f32p),
                        ("nvh_fp32_to_fp4x2", _f32p, _u8p), ("nvh_fp4x2_to_fp32", _u8p, _f32p),
                        ("nvh_f32_to_bf16", _f32p, _u16p)]:
            getattr(L, n).argtypes = [a, b, C.c_size_t]
            getattr(L, n).restype = None
        _nvh = L
    return _nvh


def ref_host():
    """The reference's own common.cuh kernels compiled for the host, or None if not built."""
    global _ref
    if _ref is None:
        p = _build.build_ref()
        if p is None:
            return None
        L = _load(p)
        vp = C.c_void_p
        L.tkref_nvfp4_gemm.argtypes = [_u8p, _u8p, _f32p, _u8p, _u8p, _f32p, _u16p] + [C.c_int] * 3
        L.tkref_mxfp8_gemm.argtypes = [_u8p, _u8p, _u8p, _u8p, _u16p] + [C.c_int] * 3
        L.tkref_bf16_gemm.argtypes = [_u16p, _u16p, _u16p] + [C.c_int] * 3
        L.tkref_fp8_gemm.argtypes = [_u8p, _u8p, _u16p] + [C.c_int] * 3
        L.tkref_fill_uniform_f32.argtypes = [_f32p, C.c_size_t, C.c_uint64, C.c_float, C.c_float]
        L.tkref_scale_swizzle_idx.restype = C.c_int
        L.tkref_scale_swizzle_idx.argtypes = [C.c_int] * 3
        del vp
        _ref = L
    return _ref


# ----------------------------------------------------------------------------- helpers ----
def num_threads() -> int:
    return lib().tko_num_threads()


def set_num_threads(n: int) -> None:
    """OpenMP threads of the oracle and of the reference host build (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().tko_set_num_threads(int(n))
    r = ref_host()
    if r is not None and hasattr(r, "tkref_set_num_threads"):
        r.tkref_set_num_threads(int(n))


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().tko_f32_to_bf16(x.reshape(-1), out.reshape(-1), x.size)
    return out


def bf16_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    return (x.astype(np.uint32) << 16).view(np.float32)


def _conv(fn, x, in_dt, out_dt, out_shape=None):
    x = np.ascontiguousarray(x, in_dt)
    out = np.empty(out_shape if out_shape is not None else x.shape, out_dt)
    fn(x.reshape(-1), out.reshape(-1), x.size)
    return out


def f32_to_e4m3(x): return _conv(lib().tko_f32_to_e4m3, x, np.float32, np.uint8)
def e4m3_to_f32(x): return _conv(lib().tko_e4m3_to_f32, x, np.uint8, np.float32)
def f32_to_e8m0(x): return _conv(lib().tko_f32_to_e8m0, x, np.float32, np.uint8)
def e8m0_to_f32(x): return _conv(lib().tko_e8m0_to_f32, x, np.uint8, np.float32)


def fp32_to_fp4x2(x: np.ndarray) -> np.ndarray:
    """(..., 2n) float32 -> (..., n) uint8, element 2i in the low nibble."""
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape[:-1] + (x.shape[-1] // 2,), np.uint8)
    lib().tko_fp32_to_fp4x2(x.reshape(-1), out.reshape(-1), out.size)
    return out


def fp4x2_to_fp32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint8)
    out = np.empty(x.shape[:-1] + (x.shape[-1] * 2,), np.float32)
    lib().tko_fp4x2_to_fp32(x.reshape(-1), out.reshape(-1), x.size)
    return out


def fill_uniform(n: int, seed: int, lo: float, hi: float) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().tko_fill_uniform_f32(out, n, seed, lo, hi)
    return out


def scale_swizzle_idx(row: int, k_block: int, k_blocks: int) -> int:
    return lib().tko_scale_swizzle_idx(row, k_block, k_blocks)


def swizzle_scales(sc_rowmajor: np.ndarray) -> np.ndarray:
    """(M, KB) uint8 row-major scales -> (ceil(M/128), KB/4, 512) swizzled chunks (pad = 0)."""
    M, KB = sc_rowmajor.shape
    Mp = (M + 127) // 128 * 128
    out = np.zeros((Mp // 128, KB // 4, 512), np.uint8)
    r = np.arange(M)[:, None]
    kb = np.arange(KB)[None, :]
    out[r // 128, kb // 4, (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4] = sc_rowmajor
    return out


def unswizzle_scales(sc: np.ndarray, M: int) -> np.ndarray:
    """Inverse of swizzle_scales: (ceil(M/128), KB/4, 512) -> (M, KB)."""
    KB = sc.shape[1] * 4
    r = np.arange(M)[:, None]
    kb = np.arange(KB)[None, :]
    return sc.reshape(sc.shape[0], sc.shape[1], 512)[r // 128, kb // 4, (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4]


def absmax_bf16(A: np.ndarray) -> float:
    A = np.ascontiguousarray(A, np.uint16)
    return float(lib().tko_absmax_bf16(A.reshape(-1), A.size))


def nvfp4_quantize(A_bf16: np.ndarray, scale_2d: bool = False, assoc: str = "kernel", amax: float | None = None):
    """Returns (codes (M,K/2) u8, scales (ceil(M/128),K/64,512) u8 e4m3, sg float32[1])."""
    A = np.ascontiguousarray(A_bf16, np.uint16)
    M, K = A.shape
    assert K % 64 == 0
    codes = np.empty((M, K // 2), np.uint8)
    sc = np.empty(((M + 127) // 128, K // 64, 512), np.uint8)
    sg = np.empty(1, np.float32)
    lib().tko_nvfp4_quantize(A, M, K, int(scale_2d), {"kernel": 0, "spec": 1}[assoc],
                             -1.0 if amax is None else float(amax), codes, sc, sg)
    return codes, sc, sg


def mxfp8_quantize(A_bf16: np.ndarray):
    """Returns (codes (M,K) u8 e4m3, scales (ceil(M/128),K/128,512) u8 e8m0)."""
    A = np.ascontiguousarray(A_bf16, np.uint16)
    M, K = A.shape
    assert K % 128 == 0
    codes = np.empty((M, K), np.uint8)
    sc = np.empty(((M + 127) // 128, K // 128, 512), np.uint8)
    lib().tko_mxfp8_quantize(A, M, K, codes, sc)
    return codes, sc


def nvfp4_gemm(A, A_sc, A_sg, B, B_sc, B_sg, row0: int = 0, nrows: int | None = None) -> np.ndarray:
    M, K = A.shape[0], A.shape[1] * 2
    N = B.shape[0]
    nrows = M - row0 if nrows is None else nrows
    D = np.empty((nrows, N), np.uint16)
    lib().tko_nvfp4_gemm(np.ascontiguousarray(A), np.ascontiguousarray(A_sc).reshape(-1), np.ascontiguousarray(A_sg, np.float32),
                         np.ascontiguousarray(B), np.ascontiguousarray(B_sc).reshape(-1), np.ascontiguousarray(B_sg, np.float32),
                         D, M, N, K, row0, nrows)
    return D


def nvfp4_gemm_f32(A, A_sc, A_sg, B, B_sc, B_sg, row0: int = 0, nrows: int | None = None) -> np.ndarray:
    """float64-accumulated dequantize-then-matmul, fp32 result (for the Frobenius gate)."""
    M, K = A.shape[0], A.shape[1] * 2
    N = B.shape[0]
    nrows = M - row0 if nrows is None else nrows
    D = np.empty((nrows, N), np.float32)
    lib().tko_nvfp4_gemm_f32(np.ascontiguousarray(A), np.ascontiguousarray(A_sc).reshape(-1), np.ascontiguousarray(A_sg, np.float32),
                             np.ascontiguousarray(B), np.ascontiguousarray(B_sc).reshape(-1), np.ascontiguousarray(B_sg, np.float32),
                             D, N, K, row0, nrows)
    return D


def mxfp8_gemm(A, A_sc, B, B_sc, row0: int = 0, nrows: int | None = None) -> np.ndarray:
    M, K = A.shape
    N = B.shape[0]
    nrows = M - row0 if nrows is None else nrows
    D = np.empty((nrows, N), np.uint16)
    lib().tko_mxfp8_gemm(np.ascontiguousarray(A), np.ascontiguousarray(A_sc).reshape(-1), np.ascontiguousarray(B),
                         np.ascontiguousarray(B_sc).reshape(-1), D, M, N, K, row0, nrows)
    return D


def bf16_gemm(A, B, row0: int = 0, nrows: int | None = None) -> np.ndarray:
    M, K = A.shape
    N = B.shape[0]
    nrows = M - row0 if nrows is None else nrows
    D = np.empty((nrows, N), np.uint16)
    lib().tko_bf16_gemm(np.ascontiguousarray(A, np.uint16), np.ascontiguousarray(B, np.uint16), D, M, N, K, row0, nrows)
    return D


def fp8_gemm(A, B, row0: int = 0, nrows: int | None = None) -> np.ndarray:
    """Dense e4m3 x e4m3 GEMM, fp32 accumulation in ascending k, bf16 out (tko_fp8_gemm)."""
    M, K = A.shape
    N = B.shape[0]
    nrows = M - row0 if nrows is None else nrows
    D = np.empty((nrows, N), np.uint16)
    lib().tko_fp8_gemm(np.ascontiguousarray(A, np.uint8), np.ascontiguousarray(B, np.uint8), D, M, N, K, row0, nrows)
    return D


def dequant_nvfp4(codes, sc, sg) -> np.ndarray:
    M = codes.shape[0]
    v = fp4x2_to_fp32(codes)
    s = e4m3_to_f32(unswizzle_scales(sc, M))
    return v * np.repeat(s, 16, axis=1) * np.float32(sg[0])


def dequant_mxfp8(codes, sc) -> np.ndarray:
    M = codes.shape[0]
    return e4m3_to_f32(codes) * np.repeat(e8m0_to_f32(unswizzle_scales(sc, M)), 32, axis=1)


def moe_route(logits: np.ndarray, top_k: int):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    experts = np.empty((T, top_k), np.int32)
    weights = np.empty((T, top_k), np.float32)
    lib().tko_moe_route(logits, T, E, top_k, experts, weights)
    return experts, weights


def moe_schedule(experts: np.ndarray, E: int, tokens_per_rank: int, e0: int, e1: int):
    experts = np.ascontiguousarray(experts, np.int32)
    T, top_k = experts.shape
    padded = np.empty(E, np.int32)
    max_rows = T * top_k + 128 * (e1 - e0)
    pull = np.empty((max_rows, 2), np.int32)
    slot = np.empty((T, top_k), np.int32)
    rows = lib().tko_moe_schedule(experts, T, E, top_k, tokens_per_rank, e0, e1, padded, pull.reshape(-1),
                                  slot.ctypes.data_as(C.c_void_p), max_rows)
    assert rows >= 0
    return padded, pull[:rows].copy(), slot


def moe_combine(Y_bf16: np.ndarray, slot_of: np.ndarray, weights: np.ndarray) -> np.ndarray:
    T, top_k = slot_of.shape
    I = Y_bf16.shape[1]
    out = np.empty((T, I), np.uint16)
    lib().tko_moe_combine(np.ascontiguousarray(Y_bf16, np.uint16), np.ascontiguousarray(slot_of, np.int32),
                          np.ascontiguousarray(weights, np.float32), T, top_k, I, out)
    return out
