"""NVFP4 GEMM with the quantizing epilogue: bit-identical to GEMM -> bf16 -> quantize with the same amax."""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import randn_bf16, bf16_bits, to_dev_u8

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("arith", ["spec", "kernel_ieee"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 384, 1024), (300, 256, 512), (1024, 1024, 2048)])
def test_quantizing_epilogue_equals_gemm_then_quantize(cuda, lib, M, N, K, arith):
    import thunderkittens_b200.ops as ops
    u8 = torch.uint8
    aq = O.nvfp4_quantize(bf16_bits(randn_bf16((M, K), seed=M + 1)), False, "spec")
    bq = O.nvfp4_quantize(bf16_bits(randn_bf16((N, K), seed=N + 2, std=0.05)), False, "spec")
    a = [to_dev_u8(aq[0], cuda), to_dev_u8(aq[1], cuda), torch.from_numpy(aq[2]).to(cuda)]
    b = [to_dev_u8(bq[0], cuda), to_dev_u8(bq[1], cuda), torch.from_numpy(bq[2]).to(cuda)]
    D = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    ops.nvfp4_gemm(*a, *b, D, "pair_n256")
    amax = torch.empty(1, dtype=torch.float32, device=cuda)
    ops.absmax_bf16(D, amax)
    rows128 = (M + 127) // 128
    rc = torch.empty(M, N // 2, dtype=u8, device=cuda); rs = torch.zeros(rows128, N // 64, 512, dtype=u8, device=cuda); rg = torch.empty(1, device=cuda)
    ops.nvfp4_quantize(D, rc, rs, rg, False, arith, amax=amax)
    fc = torch.full((M, N // 2), 0xEE, dtype=u8, device=cuda); fs = torch.full((rows128, N // 64, 512), 0xEE, dtype=u8, device=cuda); fg = torch.empty(1, device=cuda)
    ops.nvfp4_gemm_quant(*a, *b, amax, fc, fs, fg, arith)
    torch.cuda.synchronize()
    assert torch.equal(fc, rc), int((fc != rc).sum())
    assert torch.equal(fs, rs), int((fs != rs).sum())
    assert fg.item() == rg.item()
