"""The oracle's GEMM restatement against the reference's own naive GEMM kernels
(kernels/gemm/common.cuh) compiled for the host by oracle/build.py (oracle/_ref)."""
import numpy as np
import pytest

import oracle as O


@pytest.fixture(scope="module")
def ref():
    r = O.ref_host()
    if r is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    return r


def _inputs(M, N, K, seed):
    rng = np.random.default_rng(seed)
    A = O.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    B = O.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    return A, B


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (256, 192, 512), (130, 72, 64)])
def test_nvfp4_gemm_bit_exact_vs_reference_kernel(ref, M, N, K):
    A, B = _inputs(M, N, K, 11)
    ac, asc, asg = O.nvfp4_quantize(A)
    bc, bsc, bsg = O.nvfp4_quantize(B)
    D = O.nvfp4_gemm(ac, asc, asg, bc, bsc, bsg)
    Dr = np.empty((M, N), np.uint16)
    ref.tkref_nvfp4_gemm(ac, asc.reshape(-1), asg, bc, bsc.reshape(-1), bsg, Dr, M, N, K)
    assert np.array_equal(D, Dr)


@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (256, 192, 512)])
def test_mxfp8_gemm_bit_exact_vs_reference_kernel(ref, M, N, K):
    A, B = _inputs(M, N, K, 12)
    ac, asc = O.mxfp8_quantize(A)
    bc, bsc = O.mxfp8_quantize(B)
    D = O.mxfp8_gemm(ac, asc, bc, bsc)
    Dr = np.empty((M, N), np.uint16)
    ref.tkref_mxfp8_gemm(ac, asc.reshape(-1), bc, bsc.reshape(-1), Dr, M, N, K)
    assert np.array_equal(D, Dr)


def test_bf16_gemm_bit_exact_vs_reference_kernel(ref):
    A, B = _inputs(96, 80, 200, 13)
    D = O.bf16_gemm(A, B)
    Dr = np.empty((96, 80), np.uint16)
    ref.tkref_bf16_gemm(A, B, Dr, 96, 80, 200)
    assert np.array_equal(D, Dr)


def test_fp8_gemm_bit_exact_vs_reference_kernel(ref):
    rng = np.random.default_rng(16)
    A = O.f32_to_e4m3(rng.standard_normal((96, 256)).astype(np.float32))
    B = O.f32_to_e4m3((rng.standard_normal((80, 256)) * 0.5).astype(np.float32))
    D = O.fp8_gemm(A, B)
    Dr = np.empty((96, 80), np.uint16)
    ref.tkref_fp8_gemm(A, B, Dr, 96, 80, 256)
    assert np.array_equal(D, Dr)


def test_slab_equals_full(ref):
    A, B = _inputs(256, 128, 256, 14)
    ac, asc, asg = O.nvfp4_quantize(A)
    bc, bsc, bsg = O.nvfp4_quantize(B)
    full = O.nvfp4_gemm(ac, asc, asg, bc, bsc, bsg)
    slab = O.nvfp4_gemm(ac, asc, asg, bc, bsc, bsg, row0=130, nrows=17)
    assert np.array_equal(full[130:147], slab)


def test_fill_and_swizzle_index_match_reference(ref):
    a = O.fill_uniform(4096, 2024, -1.0, 1.0)
    b = np.empty(4096, np.float32)
    ref.tkref_fill_uniform_f32(b, 4096, 2024, -1.0, 1.0)
    assert np.array_equal(a, b)
    for r in range(0, 300, 7):
        for kb in range(16):
            assert O.scale_swizzle_idx(r, kb, 16) == ref.tkref_scale_swizzle_idx(r, kb, 16)


def test_gemm_matches_float64_dequant_matmul():
    A, B = _inputs(128, 128, 512, 15)
    ac, asc, asg = O.nvfp4_quantize(A)
    bc, bsc, bsg = O.nvfp4_quantize(B)
    D = O.bf16_to_f32(O.nvfp4_gemm(ac, asc, asg, bc, bsc, bsg))
    ref64 = O.dequant_nvfp4(ac, asc, asg).astype(np.float64) @ O.dequant_nvfp4(bc, bsc, bsg).astype(np.float64).T
    assert np.linalg.norm(D - ref64) / np.linalg.norm(ref64) < 3e-3   # bf16 output rounding dominates
    D32 = O.nvfp4_gemm_f32(ac, asc, asg, bc, bsc, bsg)
    assert np.linalg.norm(D32 - ref64) / np.linalg.norm(ref64) < 1e-6
