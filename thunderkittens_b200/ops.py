"""Host-side mirror of the reference's per-kernel pybind modules (`_C`).

Same function names, argument order and in-place semantics as
  kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:828-833  (nvfp4_gemm, nvfp4_quantize, fp32_to_fp4x2, fp4x2_to_fp32)
  kernels/gemm/mxfp8_b200/mxfp8_b200_gemm.cu:621-624  (mxfp8_gemm, mxfp8_quantize)
so the reference's test_gemm.py / test_quantize.py scripts run against this module after
`import thunderkittens_b200.ops as _C`.  Tensors are torch CUDA tensors owned by the caller; checks
mirror the reference's TORCH_CHECKs (include/pyutils/torchutils.cuh:35-83) and raise RuntimeError.
Work is enqueued on torch's current stream; nothing synchronises.
"""
from __future__ import annotations

import torch

from . import _lib as L

_ARITH = {"spec": L.NVFP4_SPEC, "kernel_ieee": L.NVFP4_KERNEL_IEEE, "kernel_fast": L.NVFP4_KERNEL_FAST}
_CONFIG = {None: L.GEMM_DEFAULT, "default": L.GEMM_DEFAULT, "pair_n256": L.GEMM_PAIR_N256, "single_n256": L.GEMM_SINGLE_N256,
           "pair_n128": L.GEMM_PAIR_N128, "single_n128": L.GEMM_SINGLE_N128, "skinny": L.GEMM_SKINNY,
           "skinny_prefetch": L.GEMM_SKINNY_PREFETCH, "pair_m512_n256": L.GEMM_PAIR_M512_N256}

#: default NVFP4 arithmetic (see include/tkb200.h): the reference KERNEL's arithmetic, bit-exact with it on a B200;
#: "spec" is the reference's torch specification (IEEE), reproducible on a CPU
default_nvfp4_arithmetic = "kernel_fast"


def _chk(t: torch.Tensor, name: str, dtypes, ndim=None) -> None:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype not in dtypes:
        raise RuntimeError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if ndim is not None and t.dim() != ndim:
        raise RuntimeError(f"{name} must have {ndim} dimensions")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_FP4 = (torch.float4_e2m1fn_x2, torch.uint8)
_E4M3 = (torch.float8_e4m3fn, torch.uint8)
_E8M0 = (torch.uint8,) + ((torch.float8_e8m0fnu,) if hasattr(torch, "float8_e8m0fnu") else ())


def nvfp4_quantize(A_bf16, A_fp4x2, A_sc, A_sc_global, scale_2d: bool = False, arithmetic: str | None = None, amax=None) -> None:
    """A_bf16 (M,K) -> A_fp4x2 (M,K/2), A_sc (ceil(M/128),K/64,512) e4m3, A_sc_global (1,) fp32, in place."""
    _chk(A_bf16, "A_bf16", (torch.bfloat16,), 2)
    _chk(A_fp4x2, "A_fp4x2", _FP4, 2)
    _chk(A_sc, "A_sc", _E4M3)
    _chk(A_sc_global, "A_sc_global", (torch.float32,))
    M, K = A_bf16.shape
    if tuple(A_fp4x2.shape) != (M, K // 2):
        raise RuntimeError("A_fp4x2 must have shape (M, K/2)")
    if A_sc.numel() != ((M + 127) // 128) * (K // 64) * 512:
        raise RuntimeError("A_sc must have ceil(M/128) * (K/64) * 512 elements")
    mode = _ARITH[arithmetic or default_nvfp4_arithmetic]
    if amax is None:
        L.check(L.lib().tkb_nvfp4_quantize(A_bf16.data_ptr(), 0, A_fp4x2.data_ptr(), A_sc.data_ptr(), A_sc_global.data_ptr(), M, K,
                                           int(bool(scale_2d)), mode, _stream()))
    else:
        _chk(amax, "amax", (torch.float32,))
        L.check(L.lib().tkb_nvfp4_quantize_with_amax(A_bf16.data_ptr(), 0, A_fp4x2.data_ptr(), A_sc.data_ptr(), A_sc_global.data_ptr(),
                                                     amax.data_ptr(), M, K, int(bool(scale_2d)), mode, _stream()))


def absmax_bf16(A_bf16, out) -> None:
    _chk(A_bf16, "A_bf16", (torch.bfloat16,), 2)
    _chk(out, "out", (torch.float32,))
    M, K = A_bf16.shape
    L.check(L.lib().tkb_absmax_bf16(A_bf16.data_ptr(), 0, M, K, out.data_ptr(), _stream()))


def mxfp8_quantize(A_bf16, A_fp8, A_sc) -> None:
    _chk(A_bf16, "A_bf16", (torch.bfloat16,), 2)
    _chk(A_fp8, "A_fp8", _E4M3, 2)
    _chk(A_sc, "A_sc", _E8M0)
    M, K = A_bf16.shape
    if tuple(A_fp8.shape) != (M, K):
        raise RuntimeError("A_fp8 must have shape (M, K)")
    if A_sc.numel() != ((M + 127) // 128) * (K // 128) * 512:
        raise RuntimeError("A_sc must have ceil(M/128) * (K/128) * 512 elements")
    L.check(L.lib().tkb_mxfp8_quantize(A_bf16.data_ptr(), 0, A_fp8.data_ptr(), A_sc.data_ptr(), M, K, _stream()))


def fp32_to_fp4x2(A_fp32):
    _chk(A_fp32, "A_fp32", (torch.float32,), 2)
    out = torch.empty(A_fp32.shape[0], A_fp32.shape[1] // 2, dtype=torch.uint8, device=A_fp32.device).view(torch.float4_e2m1fn_x2)
    L.check(L.lib().tkb_fp32_to_fp4x2(A_fp32.data_ptr(), out.data_ptr(), out.numel(), _stream()))
    return out


def fp4x2_to_fp32(A_fp4x2):
    _chk(A_fp4x2, "A_fp4x2", _FP4, 2)
    out = torch.empty(A_fp4x2.shape[0], A_fp4x2.shape[1] * 2, dtype=torch.float32, device=A_fp4x2.device)
    L.check(L.lib().tkb_fp4x2_to_fp32(A_fp4x2.data_ptr(), out.data_ptr(), A_fp4x2.numel(), _stream()))
    return out


def nvfp4_gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D, config: str | None = None) -> None:
    """D (M,N) bf16 = dequant(A) @ dequant(B).T ; A (M,K/2), B (N,K/2) packed e2m1."""
    _chk(A, "A", _FP4, 2); _chk(B, "B", _FP4, 2)
    _chk(A_sc, "A_sc", _E4M3); _chk(B_sc, "B_sc", _E4M3)
    _chk(A_sc_global, "A_sc_global", (torch.float32,)); _chk(B_sc_global, "B_sc_global", (torch.float32,))
    _chk(D, "D", (torch.bfloat16,), 2)
    M, K2 = A.shape
    N = B.shape[0]
    if B.shape[1] != K2 or tuple(D.shape) != (M, N):
        raise RuntimeError("shape mismatch: A (M,K/2), B (N,K/2), D (M,N)")
    K = K2 * 2
    if A_sc.numel() != ((M + 127) // 128) * (K // 64) * 512 or B_sc.numel() != ((N + 127) // 128) * (K // 64) * 512:
        raise RuntimeError("scale tensors must have ceil(rows/128) * (K/64) * 512 elements")
    L.check(L.lib().tkb_nvfp4_gemm_ex(A.data_ptr(), A_sc.data_ptr(), A_sc_global.data_ptr(), B.data_ptr(), B_sc.data_ptr(),
                                      B_sc_global.data_ptr(), D.data_ptr(), 0, M, N, K, _CONFIG[config], _stream()))


def mxfp8_gemm(A, A_sc, B, B_sc, D, config: str | None = None) -> None:
    _chk(A, "A", _E4M3, 2); _chk(B, "B", _E4M3, 2)
    _chk(A_sc, "A_sc", _E8M0); _chk(B_sc, "B_sc", _E8M0)
    _chk(D, "D", (torch.bfloat16,), 2)
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or tuple(D.shape) != (M, N):
        raise RuntimeError("shape mismatch: A (M,K), B (N,K), D (M,N)")
    if A_sc.numel() != ((M + 127) // 128) * (K // 128) * 512 or B_sc.numel() != ((N + 127) // 128) * (K // 128) * 512:
        raise RuntimeError("scale tensors must have ceil(rows/128) * (K/128) * 512 elements")
    L.check(L.lib().tkb_mxfp8_gemm_ex(A.data_ptr(), A_sc.data_ptr(), B.data_ptr(), B_sc.data_ptr(), D.data_ptr(), 0, M, N, K,
                                      _CONFIG[config], _stream()))


def bf16_gemm(A, B, D, config: str | None = None) -> None:
    """D = A @ B.T with bf16 operands (the dense control; standalone-only in the reference)."""
    _chk(A, "A", (torch.bfloat16,), 2); _chk(B, "B", (torch.bfloat16,), 2); _chk(D, "D", (torch.bfloat16,), 2)
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or tuple(D.shape) != (M, N):
        raise RuntimeError("shape mismatch: A (M,K), B (N,K), D (M,N)")
    L.check(L.lib().tkb_bf16_gemm_ex(A.data_ptr(), 0, B.data_ptr(), 0, D.data_ptr(), 0, M, N, K, _CONFIG[config], _stream()))


def fp8_gemm(A, B, D, config: str | None = None) -> None:
    """D = A @ B.T with dense e4m3 operands (kernels/gemm/fp8_b200 in the reference; standalone-only there)."""
    e4m3 = (torch.uint8, torch.float8_e4m3fn)
    _chk(A, "A", e4m3, 2); _chk(B, "B", e4m3, 2); _chk(D, "D", (torch.bfloat16,), 2)
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or tuple(D.shape) != (M, N):
        raise RuntimeError("shape mismatch: A (M,K), B (N,K), D (M,N)")
    L.check(L.lib().tkb_fp8_gemm_ex(A.data_ptr(), 0, B.data_ptr(), 0, D.data_ptr(), 0, M, N, K, _CONFIG[config], _stream()))


def nvfp4_gemm_quant(A, A_sc, A_sg, B, B_sc, B_sg, out_amax, D_codes, D_sc, D_sg, arithmetic: str = "spec") -> None:
    """NVFP4 GEMM whose bf16 result is quantized to NVFP4 (with the caller's per-tensor amax) inside the epilogue."""
    M, K = A.shape[0], A.shape[1] * 2
    N = B.shape[0]
    if tuple(D_codes.shape) != (M, N // 2):
        raise RuntimeError("D_codes must have shape (M, N/2)")
    if arithmetic not in ("spec", "kernel_ieee"):
        raise RuntimeError("the fused epilogue offers the 'spec' and 'kernel_ieee' arithmetics")
    L.check(L.lib().tkb_nvfp4_gemm_quant(A.data_ptr(), A_sc.data_ptr(), A_sg.data_ptr(), B.data_ptr(), B_sc.data_ptr(), B_sg.data_ptr(),
                                         out_amax.data_ptr(), D_codes.data_ptr(), D_sc.data_ptr(), D_sg.data_ptr(), M, N, K, _ARITH[arithmetic], _stream()))
