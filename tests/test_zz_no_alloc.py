"""The allocation-free door to the skinny-M NVFP4 GEMM (tkb_nvfp4_gemm_skinny_static).

Who needs it: a host program that is not allowed to allocate device memory at the moment it calls the library — a
serving runtime that reserves all of its memory when it starts, or a plug-in whose execute hook forbids
cudaMalloc.  The regular entry point allocates a per-device context and stream-K scratch
on first use; this one keeps its scratch in an array that is part of the library image and therefore only serves
M <= 16.  The test drives both entry points through the C ABI with the same operands and expects the same result
(the tolerance is the one of the other GEMM tests), twice in a row with different activations so that whatever the
first call left in the shared array cannot leak into the second.  Collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from tests.util import randn_bf16, bf16_bits, to_dev_u8
from tests.test_gpu_gemm import _check

pytestmark = pytest.mark.gpu


def _quantized_activation(cuda, M, K, seed):
    import thunderkittens_b200.ops as ops
    X = randn_bf16((M, K), seed=seed).to(cuda)
    xc = torch.empty(M, K // 2, dtype=torch.uint8, device=cuda)
    xs = torch.empty(1, K // 64, 512, dtype=torch.uint8, device=cuda)
    xg = torch.empty(1, dtype=torch.float32, device=cuda)
    ops.nvfp4_quantize(X, xc, xs, xg, False, "spec")
    return xc, xs, xg


def test_static_scratch_entry_matches_regular_entry(cuda, lib):
    from thunderkittens_b200 import _lib
    M, N, K = 16, 512, 8192          # 4 weight slabs x 32 K-blocks over 128 CTAs: every slab is split, partials are used
    wq = O.nvfp4_quantize(bf16_bits(randn_bf16((N, K), seed=41, std=0.02)))
    wc, ws, wg = to_dev_u8(wq[0], cuda), to_dev_u8(wq[1], cuda), torch.from_numpy(wq[2]).to(cuda)
    stream = torch.cuda.current_stream().cuda_stream
    for call, seed in enumerate((51, 52)):                       # two calls in a row, different activations
        xc, xs, xg = _quantized_activation(cuda, M, K, seed)
        d_static = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
        d_regular = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
        rc = lib.tkb_nvfp4_gemm_skinny_static(xc.data_ptr(), xs.data_ptr(), xg.data_ptr(), wc.data_ptr(), ws.data_ptr(), wg.data_ptr(),
                                              d_static.data_ptr(), 0, M, N, K, stream)
        assert rc == 0, lib.tkb_last_error()
        rc = lib.tkb_nvfp4_gemm_ex(xc.data_ptr(), xs.data_ptr(), xg.data_ptr(), wc.data_ptr(), ws.data_ptr(), wg.data_ptr(),
                                   d_regular.data_ptr(), 0, M, N, K, _lib.GEMM_SKINNY, stream)
        assert rc == 0, lib.tkb_last_error()
        torch.cuda.synchronize()
        _check(bf16_bits(d_static), bf16_bits(d_regular), f"static vs regular, call {call}")
        # and both agree with the oracle
        ref = O.nvfp4_gemm(xc.cpu().numpy(), xs.cpu().numpy(), xg.cpu().numpy(), *wq)
        _check(bf16_bits(d_static), ref, f"static vs oracle, call {call}")


def test_static_scratch_entry_rejects_large_m(cuda, lib):
    z = torch.zeros(4096, dtype=torch.uint8, device=cuda)
    f = torch.zeros(1, dtype=torch.float32, device=cuda)
    rc = lib.tkb_nvfp4_gemm_skinny_static(z.data_ptr(), z.data_ptr(), f.data_ptr(), z.data_ptr(), z.data_ptr(), f.data_ptr(), z.data_ptr(),
                                          0, 17, 128, 64, None)
    assert rc == 1
    assert b"1..16" in lib.tkb_last_error()
