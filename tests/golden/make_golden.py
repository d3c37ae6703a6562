"""Generates the committed golden fixtures in this folder from the REFERENCE's own Python specs.

Run once, in a container where the ThunderKittens tree is mounted (its location: environment variable TK_REFERENCE):

    python tests/golden/make_golden.py

What is imported from the reference, unmodified:
  kernels/gemm/nvfp4_b200/test_quantize.py : torch_nvfp4_quantize, torch_nvfp4_dequantize, scale_swizzle
  kernels/gemm/mxfp8_b200/test_quantize.py : torch_mxfp8_quantize, torch_mxfp8_dequantize, scale_swizzle
Both files do `from _C import ...` (their CUDA extension) at import time.  There is no GPU here, so a
stand-in `_C` module is registered first.  Its `fp32_to_fp4x2` / `fp4x2_to_fp32` call the CUDA toolkit's
HOST implementation of the very conversion the reference's CUDA helper uses
(`__nv_cvt_float2_to_fp4x2(.., __NV_E2M1, cudaRoundNearest)`, nvfp4_b200_gemm.cu:572) through
oracle/nv_host_codecs.cpp; the quantize/gemm entry points are never called by the specs.

Fixtures (all small):
  nvfp4_quantize_{1d,2d}.npz : bf16 input bits, codes, unswizzled + swizzled e4m3 scales, global scale
  mxfp8_quantize.npz         : spec run on randn input, and the reference's inverse-construction case
                               (random codes + random e8m0 -> bf16 -> quantize must return them)
The GPU box has no reference tree: tests only read the .npz files.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
# the ThunderKittens tree: $TK_REFERENCE, else a directory named `reference` beside this repository
REFERENCE = os.environ.get("TK_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference")

import oracle  # noqa: E402  (only for the toolkit host codecs)


def _fp32_to_fp4x2(t: torch.Tensor) -> torch.Tensor:
    x = np.ascontiguousarray(t.detach().cpu().numpy(), np.float32)
    out = np.empty((x.shape[0], x.shape[1] // 2), np.uint8)
    oracle.nvhost().nvh_fp32_to_fp4x2(x.reshape(-1), out.reshape(-1), out.size)
    return torch.from_numpy(out).view(torch.float4_e2m1fn_x2)


def _fp4x2_to_fp32(t: torch.Tensor) -> torch.Tensor:
    x = np.ascontiguousarray(t.view(torch.uint8).numpy())
    out = np.empty((x.shape[0], x.shape[1] * 2), np.float32)
    oracle.nvhost().nvh_fp4x2_to_fp32(x.reshape(-1), out.reshape(-1), x.size)
    return torch.from_numpy(out)


def _import_spec(path: str, name: str):
    stub = types.ModuleType("_C")
    stub.fp32_to_fp4x2 = _fp32_to_fp4x2
    stub.fp4x2_to_fp32 = _fp4x2_to_fp32
    for n in ("nvfp4_quantize", "nvfp4_gemm", "mxfp8_quantize", "mxfp8_gemm"):
        setattr(stub, n, None)
    sys.modules["_C"] = stub
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy().copy()
    if t.dtype in (torch.float8_e4m3fn, torch.float4_e2m1fn_x2):
        return t.view(torch.uint8).numpy().copy()
    return t.numpy().copy()


def main():
    nv = _import_spec(os.path.join(REFERENCE, "kernels/gemm/nvfp4_b200/test_quantize.py"), "ref_nvfp4_spec")
    mx = _import_spec(os.path.join(REFERENCE, "kernels/gemm/mxfp8_b200/test_quantize.py"), "ref_mxfp8_spec")

    g = torch.Generator().manual_seed(20240611)
    # N(0,1) with a few outliers and one all-zero 16-block / one all-zero row to hit the eps clamps
    A = torch.randn(256, 384, generator=g, dtype=torch.float32)
    A[torch.rand(256, 384, generator=g) < 0.01] *= 32.0
    A[5, 32:48] = 0.0
    A[17, :] = 0.0
    A = A.to(torch.bfloat16)
    for scale_2d in (False, True):
        codes, sc_un, sg = nv.torch_nvfp4_quantize(A, scale_2d)
        sc = nv.scale_swizzle(sc_un)
        deq = nv.torch_nvfp4_dequantize(codes, sc_un, sg)
        np.savez_compressed(os.path.join(HERE, f"nvfp4_quantize_{'2d' if scale_2d else '1d'}.npz"),
                            A_bf16=bits(A), codes=bits(codes), sc_unswizzled=bits(sc_un), sc=bits(sc),
                            sg=sg.numpy(), dequant=deq.numpy().astype(np.float32))

    # MXFP8: (a) spec on randn; (b) the reference's inverse construction (test_quantize.py:127-145)
    B = (torch.randn(256, 256, generator=g) * 3.0).to(torch.bfloat16)
    codes, sc_un = mx.torch_mxfp8_quantize(B)
    sc = mx.scale_swizzle(sc_un)
    fp8_ref = ((torch.rand(128, 256, generator=g) * 2 - 1) * 448).to(torch.float8_e4m3fn)
    sc_un_ref = torch.randint(127 - 20, 127 + 20, (128, 256 // 32), generator=g, dtype=torch.uint8)
    inv_bf16 = mx.torch_mxfp8_dequantize(fp8_ref, sc_un_ref).to(torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "mxfp8_quantize.npz"),
                        A_bf16=bits(B), codes=bits(codes), sc_unswizzled=sc_un.numpy(), sc=sc.numpy(),
                        inv_codes=bits(fp8_ref), inv_sc_unswizzled=sc_un_ref.numpy(),
                        inv_sc=mx.scale_swizzle(sc_un_ref).numpy(), inv_bf16=bits(inv_bf16))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
