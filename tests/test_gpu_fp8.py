"""Dense e4m3 GEMM (tkb_fp8_gemm) against the oracle (tko_fp8_gemm, pinned to the reference's naive kernel)."""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import bf16_bits
from tests.test_gpu_gemm import _check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,cfg", [(256, 256, 256, None), (512, 384, 1024, None), (1024, 1024, 1024, "single_n128"), (130, 72, 144, None),
                                       (256, 512, 2048, "pair_n128"), (384, 256, 512, "single_n256")])
def test_fp8_gemm_matches_oracle(cuda, lib, M, N, K, cfg):
    import thunderkittens_b200.ops as ops
    rng = np.random.default_rng(M + N + K)
    A = O.f32_to_e4m3(rng.standard_normal((M, K)).astype(np.float32))
    B = O.f32_to_e4m3((rng.standard_normal((N, K)) * 0.5).astype(np.float32))
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.fp8_gemm(torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda), D, cfg)
    torch.cuda.synchronize()
    _check(bf16_bits(D), O.fp8_gemm(A, B), f"fp8 {M}x{N}x{K} {cfg}")


@pytest.mark.parametrize("M,N,K", [(1024, 512, 512), (600, 264, 272), (2048, 2048, 1024)])
def test_fp8_gemm_tall_tile(cuda, lib, M, N, K):
    """The 512 x 256 cluster tile of the dense kinds (two 128-row halves of A per CTA), forced, including ragged edges."""
    import thunderkittens_b200.ops as ops
    rng = np.random.default_rng(M + N + K + 1)
    A = O.f32_to_e4m3(rng.standard_normal((M, K)).astype(np.float32))
    B = O.f32_to_e4m3((rng.standard_normal((N, K)) * 0.5).astype(np.float32))
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.fp8_gemm(torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda), D, "pair_m512_n256")
    torch.cuda.synchronize()
    _check(bf16_bits(D), O.fp8_gemm(A, B), f"fp8 tall {M}x{N}x{K}")
