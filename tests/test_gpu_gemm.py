"""GPU parity of the tcgen05 GEMMs (through the C ABI) against the CPU oracle, which restates the
reference's naive GEMM kernels (kernels/gemm/common.cuh) bit-for-bit.

Tolerance: the reference accumulates sequentially in fp32; the tensor core accumulates the same
exact products in another order, so results differ only where the final bf16 rounding falls the
other way.  Gates: relative Frobenius error <= 1e-3 against the oracle's bf16 result, and at most
2 bf16 ulp on every element that is not a near-cancellation (|ref| >= 1% of the rms)."""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import randn_bf16, bf16_bits, to_dev_u8, rel_fro, bf16_ulp_diff

pytestmark = pytest.mark.gpu

CONFIGS = ["pair_n256", "single_n256", "pair_n128", "single_n128"]


def _ops():
    import thunderkittens_b200.ops as ops
    return ops


def _check(D_gpu_bits, D_ref_bits, what):
    from thunderkittens_b200 import _lib
    assert _lib.device_status() == 0, "a device-side wait timed out"
    d, r = O.bf16_to_f32(D_gpu_bits), O.bf16_to_f32(D_ref_bits)
    assert np.isfinite(d).all(), f"{what}: non-finite output"
    err = rel_fro(d, r)
    rms = np.sqrt((r.astype(np.float64) ** 2).mean())
    big = np.abs(r) >= 0.01 * rms
    ulp = bf16_ulp_diff(D_gpu_bits, D_ref_bits)
    max_ulp = int(ulp[big].max()) if big.any() else 0
    assert err <= 1e-3, f"{what}: relative Frobenius error {err:.3e}"
    assert max_ulp <= 2, f"{what}: {max_ulp} bf16 ulp"
    return err, max_ulp


def _nvfp4_case(cuda, M, N, K, config, seed=0):
    ops = _ops()
    A = randn_bf16((M, K), seed=seed + 1)
    B = randn_bf16((N, K), seed=seed + 2, std=0.02)
    ac, asc, asg = O.nvfp4_quantize(bf16_bits(A))
    bc, bsc, bsg = O.nvfp4_quantize(bf16_bits(B))
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.nvfp4_gemm(to_dev_u8(ac, cuda), to_dev_u8(asc, cuda), torch.from_numpy(asg).to(cuda), to_dev_u8(bc, cuda), to_dev_u8(bsc, cuda),
                   torch.from_numpy(bsg).to(cuda), D, config)
    torch.cuda.synchronize()
    return bf16_bits(D), (ac, asc, asg, bc, bsc, bsg)


@pytest.mark.parametrize("config", CONFIGS)
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (256, 256, 1024), (512, 768, 2048), (130, 200, 320), (1024, 1024, 1024)])
def test_nvfp4_gemm_vs_oracle(cuda, lib, config, M, N, K):
    D, q = _nvfp4_case(cuda, M, N, K, config, seed=M + N + K)
    ref = O.nvfp4_gemm(*q)
    _check(D, ref, f"nvfp4 {M}x{N}x{K} {config}")


@pytest.mark.parametrize("config", CONFIGS)
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (256, 256, 1024), (512, 768, 2048), (130, 200, 384), (1024, 1024, 1024)])
def test_mxfp8_gemm_vs_oracle(cuda, lib, config, M, N, K):
    ops = _ops()
    A = randn_bf16((M, K), seed=M + 1, outlier_frac=0.01)
    B = randn_bf16((N, K), seed=N + 2, outlier_frac=0.01)
    ac, asc = O.mxfp8_quantize(bf16_bits(A))
    bc, bsc = O.mxfp8_quantize(bf16_bits(B))
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.mxfp8_gemm(to_dev_u8(ac, cuda), to_dev_u8(asc, cuda), to_dev_u8(bc, cuda), to_dev_u8(bsc, cuda), D, config)
    torch.cuda.synchronize()
    _check(bf16_bits(D), O.mxfp8_gemm(ac, asc, bc, bsc), f"mxfp8 {M}x{N}x{K} {config}")


@pytest.mark.parametrize("config", CONFIGS + ["pair_m512_n256"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 256, 1024), (512, 768, 2048), (130, 200, 72), (1024, 1024, 1024)])
def test_bf16_gemm_vs_oracle(cuda, lib, config, M, N, K):
    ops = _ops()
    A = randn_bf16((M, K), seed=M + 3)
    B = randn_bf16((N, K), seed=N + 4)
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.bf16_gemm(A.to(cuda), B.to(cuda), D, config)
    torch.cuda.synchronize()
    _check(bf16_bits(D), O.bf16_gemm(bf16_bits(A), bf16_bits(B)), f"bf16 {M}x{N}x{K} {config}")


def test_nvfp4_gemm_many_tiles_default_config(cuda, lib):
    """More tiles than clusters (persistent loop, accumulator hand-over) with the default configuration;
    a row slab is checked against the oracle."""
    M, N, K = 4096, 4096, 1024
    D, q = _nvfp4_case(cuda, M, N, K, None, seed=77)
    ac, asc, asg, bc, bsc, bsg = q
    for r0 in (0, 2048 + 128, 4096 - 64):
        ref = O.nvfp4_gemm(ac, asc, asg, bc, bsc, bsg, row0=r0, nrows=64)
        _check(D[r0:r0 + 64], ref, f"nvfp4 4096 slab {r0}")


def test_full_size_gemm_properties(cuda, lib):
    """8192^3 (headline size): GPU quantize + GEMM, checked through (a) row slabs against the oracle fed
    with the GPU's own codes and (b) linearity in the per-tensor scale."""
    ops = _ops()
    from tests.test_gpu_quantize import gpu_nvfp4_quantize  # noqa: F401
    M = N = K = 8192
    g = torch.Generator(device=cuda).manual_seed(11)
    A = torch.randn(M, K, generator=g, device=cuda).to(torch.bfloat16)
    B = (torch.randn(N, K, generator=g, device=cuda) * 0.02).to(torch.bfloat16)
    def q(X):
        codes = torch.empty(X.shape[0], K // 2, dtype=torch.uint8, device=cuda)
        sc = torch.empty(X.shape[0] // 128, K // 64, 512, dtype=torch.uint8, device=cuda)
        sg = torch.empty(1, dtype=torch.float32, device=cuda)
        ops.nvfp4_quantize(X, codes, sc, sg, False, "spec")
        return codes, sc, sg
    ac, asc, asg = q(A)
    bc, bsc, bsg = q(B)
    D = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    ops.nvfp4_gemm(ac, asc, asg, bc, bsc, bsg, D)
    torch.cuda.synchronize()
    hq = [t.cpu().numpy() for t in (ac, asc, asg, bc, bsc, bsg)]
    for r0 in (0, 8192 - 16):
        ref = O.nvfp4_gemm(*hq, row0=r0, nrows=16)
        _check(bf16_bits(D[r0:r0 + 16]), ref, f"nvfp4 8192 slab {r0}")
    # linearity: scaling A's per-tensor scale by 2 scales D by exactly 2 (power of two, no rounding change)
    D2 = torch.empty_like(D)
    ops.nvfp4_gemm(ac, asc, asg * 2, bc, bsc, bsg, D2)
    torch.cuda.synchronize()
    assert torch.equal(D2[:512].float(), D[:512].float() * 2)
    # MXFP8 at the same size, slab check
    def q8(X):
        codes = torch.empty(X.shape[0], K, dtype=torch.uint8, device=cuda)
        sc = torch.empty(X.shape[0] // 128, K // 128, 512, dtype=torch.uint8, device=cuda)
        ops.mxfp8_quantize(X, codes, sc)
        return codes, sc
    a8, a8s = q8(A)
    b8, b8s = q8(B)
    ops.mxfp8_gemm(a8, a8s, b8, b8s, D)
    torch.cuda.synchronize()
    h8 = [t.cpu().numpy() for t in (a8, a8s, b8, b8s)]
    ref = O.mxfp8_gemm(*h8, row0=4096, nrows=16)
    _check(bf16_bits(D[4096:4096 + 16]), ref, "mxfp8 8192 slab")


def test_gemm_argument_errors(cuda, lib):
    ops = _ops()
    from thunderkittens_b200._lib import TkbError
    A = torch.zeros(256, 100, dtype=torch.bfloat16, device=cuda)   # K % 8 != 0
    with pytest.raises((TkbError, RuntimeError)):
        ops.bf16_gemm(A, A, torch.zeros(256, 256, dtype=torch.bfloat16, device=cuda))
    with pytest.raises(RuntimeError):
        ops.bf16_gemm(A.cpu(), A.cpu(), torch.zeros(256, 256, dtype=torch.bfloat16))
