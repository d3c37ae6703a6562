"""This library beside the reference's OWN GPU kernels (ThunderKittens kernels/gemm/nvfp4_b200 and mxfp8_b200,
compiled from the reference tree into oracle/_ref/tk_nvfp4 and tk_mxfp8 by oracle/build.py:build_ref_gpu).
Skipped when those objects are absent.  Codes, scales and per-tensor scales of the quantizers must be
bit-identical to the reference kernels' (NVFP4: the TKB_NVFP4_KERNEL_FAST arithmetic), GEMM outputs within the
GEMM tolerance (observed: identical).  Each reference module is loaded in a child process: both are named `_C`."""
import glob
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import sys, os, json, glob, importlib.util
ROOT, which = sys.argv[1], sys.argv[2]
sys.path.insert(0, ROOT)
import torch
import thunderkittens_b200.ops as ops
so = glob.glob(os.path.join(ROOT, "oracle", "_ref", f"tk_{which}", "_C*.so"))[0]
spec = importlib.util.spec_from_file_location("_C", so); ref = importlib.util.module_from_spec(spec); spec.loader.exec_module(ref)
dev = torch.device("cuda:0"); u8 = torch.uint8
out = []
for (M, N, K, s2d) in [(256, 256, 512, False), (1024, 1024, 1024, False), (2048, 512, 7168, True), (8192, 256, 8192, False)]:
    g = torch.Generator(device=dev).manual_seed(M + K)
    A = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    B = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    r = {"M": M, "N": N, "K": K, "scale_2d": s2d}
    if which == "nvfp4":
        def q_ref(X):
            c = torch.empty(X.shape[0], K // 2, dtype=torch.float4_e2m1fn_x2, device=dev); s = torch.empty(X.shape[0] // 128, K // 64, 512, dtype=torch.float8_e4m3fn, device=dev)
            gg = torch.empty(1, device=dev); ref.nvfp4_quantize(X, c, s, gg, s2d); return c, s, gg
        def q_own(X):
            c = torch.empty(X.shape[0], K // 2, dtype=u8, device=dev); s = torch.empty(X.shape[0] // 128, K // 64, 512, dtype=u8, device=dev)
            gg = torch.empty(1, device=dev); ops.nvfp4_quantize(X, c, s, gg, s2d, "kernel_fast"); return c, s, gg
        ra, rb, oa, ob = q_ref(A), q_ref(B), q_own(A), q_own(B)
        torch.cuda.synchronize()
        r["quant_diff"] = int((oa[0] != ra[0].view(u8)).sum() + (oa[1] != ra[1].view(u8)).sum() + (ob[0] != rb[0].view(u8)).sum() + (ob[1] != rb[1].view(u8)).sum())
        r["sg_equal"] = bool(oa[2].item() == ra[2].item() and ob[2].item() == rb[2].item())
        Dr = torch.zeros(M, N, dtype=torch.bfloat16, device=dev); Do = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        ref.nvfp4_gemm(*ra, *rb, Dr); ops.nvfp4_gemm(*oa, *ob, Do, "pair_n256")
    else:
        def q_ref(X):
            c = torch.empty(X.shape[0], K, dtype=torch.float8_e4m3fn, device=dev); s = torch.empty(X.shape[0] // 128, K // 128, 32, 16, dtype=u8, device=dev)
            ref.mxfp8_quantize(X, c, s); return c, s
        def q_own(X):
            c = torch.empty(X.shape[0], K, dtype=u8, device=dev); s = torch.empty(X.shape[0] // 128, K // 128, 512, dtype=u8, device=dev)
            ops.mxfp8_quantize(X, c, s); return c, s
        ra, rb, oa, ob = q_ref(A), q_ref(B), q_own(A), q_own(B)
        torch.cuda.synchronize()
        r["quant_diff"] = int((oa[0] != ra[0].view(u8)).sum() + (oa[1].view(-1) != ra[1].view(-1)).sum() + (ob[0] != rb[0].view(u8)).sum() + (ob[1].view(-1) != rb[1].view(-1)).sum())
        r["sg_equal"] = True
        Dr = torch.zeros(M, N, dtype=torch.bfloat16, device=dev); Do = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        ref.mxfp8_gemm(*ra, *rb, Dr); ops.mxfp8_gemm(*oa, *ob, Do, "pair_n256")
    torch.cuda.synchronize()
    d = (Dr.float() - Do.float())
    r["gemm_rel_fro"] = float(d.norm() / Dr.float().norm())
    r["gemm_identical"] = bool(torch.equal(Dr, Do))
    out.append(r)
print("RESULT " + json.dumps(out))
'''


@pytest.mark.parametrize("which", ["nvfp4", "mxfp8"])
def test_against_reference_gpu_kernels(cuda, lib, which):
    if not glob.glob(os.path.join(ROOT, "oracle", "_ref", f"tk_{which}", "_C*.so")):
        pytest.skip("reference GPU kernels not built (oracle/build.py:build_ref_gpu needs the reference tree)")
    r = subprocess.run([sys.executable, "-c", CHILD, ROOT, which], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    for case in json.loads(line[7:]):
        assert case["quant_diff"] == 0, case
        assert case["sg_equal"], case
        assert case["gemm_rel_fro"] <= 1e-3, case
