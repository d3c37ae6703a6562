"""GPU parity of the skinny-M (decode) NVFP4 GEMM against the CPU oracle.  The reference kernel cannot run
M < 256, so for these shapes the oracle's restatement of the reference arithmetic is the specification
(parity unpinned against the reference itself)."""
import numpy as np
import pytest
import torch

import oracle as O
from tests.util import randn_bf16, bf16_bits, to_dev_u8
from tests.test_gpu_gemm import _check

pytestmark = pytest.mark.gpu


def _ops():
    import thunderkittens_b200.ops as ops
    return ops


def _weights(N, K, seed):
    W = randn_bf16((N, K), seed=seed, std=0.02)
    return O.nvfp4_quantize(bf16_bits(W))


def _run(cuda, X, wq, config="skinny"):
    ops = _ops()
    M, K = X.shape
    wc, wsc, wsg = wq
    N = wc.shape[0]
    Xd = X.to(cuda)
    xc = torch.empty(M, K // 2, dtype=torch.uint8, device=cuda)
    xsc = torch.empty(1, K // 64, 512, dtype=torch.uint8, device=cuda)
    xsg = torch.empty(1, dtype=torch.float32, device=cuda)
    ops.nvfp4_quantize(Xd, xc, xsc, xsg, False, "spec")          # activations quantized on the fly
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.nvfp4_gemm(xc, xsc, xsg, to_dev_u8(wc, cuda), to_dev_u8(wsc, cuda), torch.from_numpy(wsg).to(cuda), D, config)
    torch.cuda.synchronize()
    # the activation codes come from the GPU quantizer (default arithmetic); its parity has its own tests
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    assert np.array_equal(xc.cpu().numpy(), xq[0]) and np.array_equal(xsc.cpu().numpy(), xq[1]) and xsg.item() == xq[2][0]
    return bf16_bits(D)


@pytest.mark.parametrize("M", [1, 16, 17, 64, 128])
@pytest.mark.parametrize("N,K", [(256, 8192), (1000, 320), (3072, 1024), (128, 256)])
def test_decode_vs_oracle(cuda, lib, M, N, K):
    X = randn_bf16((M, K), seed=M * 3 + N)
    wq = _weights(N, K, seed=N + K)
    D = _run(cuda, X, wq)
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    _check(D, O.nvfp4_gemm(*xq, *wq), f"decode {M}x{N}x{K}")


def test_decode_default_dispatch_and_general_kernel_agree(cuda, lib):
    X = randn_bf16((128, 1024), seed=4)
    wq = _weights(512, 1024, seed=5)
    d_skinny = _run(cuda, X, wq, None)          # default config picks the skinny kernel for M <= 128
    d_general = _run(cuda, X, wq, "pair_n256")  # the general kernel with zero-filled rows
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    ref = O.nvfp4_gemm(*xq, *wq)
    _check(d_skinny, ref, "skinny")
    _check(d_general, ref, "general")


def test_decode_repeated_calls_reuse_scratch(cuda, lib):
    X = randn_bf16((16, 8192), seed=6)
    wq = _weights(512, 8192, seed=7)            # 4 slabs x 32 K-blocks over 128 CTAs: every slab is split
    first = _run(cuda, X, wq)
    for _ in range(9):                          # walks the scratch ring and the epoch more than once
        again = _run(cuda, X, wq)
        assert np.array_equal(first, again)
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    _check(first, O.nvfp4_gemm(*xq, *wq), "decode repeat")


@pytest.mark.parametrize("M", [1, 16, 128])
def test_decode_full_size(cuda, lib, M):
    """N=28672, K=8192 (the decode configuration): all columns of a few activation rows against the oracle."""
    N, K = 28672, 8192
    g = torch.Generator().manual_seed(5)
    W = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    wq = O.nvfp4_quantize(bf16_bits(W))
    X = randn_bf16((M, K), seed=6)
    D = _run(cuda, X, wq)
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    rows = min(M, 4)
    ref = O.nvfp4_gemm(*xq, *wq, row0=M - rows, nrows=rows)
    _check(D[M - rows:], ref, f"decode full M={M}")


@pytest.mark.parametrize("config", ["skinny", "skinny_prefetch"])
def test_decode_weights_quantized_right_before(cuda, lib, config):
    """Weights quantized ON THE DEVICE by the launch that directly precedes the skinny GEMM in the same stream.  With the
    default config the GEMM reads nothing before that launch has finished, so the result must be right; the prefetching
    config is only legal when the weights were complete earlier, which the extra synchronisation below provides."""
    ops = _ops()
    M, N, K = 16, 4096, 8192
    X, W = randn_bf16((M, K), seed=11), randn_bf16((N, K), seed=12, std=0.02)
    xq, wq = O.nvfp4_quantize(bf16_bits(X), False, "spec"), O.nvfp4_quantize(bf16_bits(W), False, "spec")
    xc, xs, xg = to_dev_u8(xq[0], cuda), to_dev_u8(xq[1], cuda), torch.from_numpy(xq[2]).to(cuda)
    Wd = W.to(cuda)
    wc = torch.zeros(N, K // 2, dtype=torch.uint8, device=cuda); ws = torch.zeros(N // 128, K // 64, 512, dtype=torch.uint8, device=cuda)
    wg = torch.zeros(1, dtype=torch.float32, device=cuda)
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    torch.cuda.synchronize()
    for _ in range(3):
        wc.zero_(); ws.zero_()
        ops.nvfp4_quantize(Wd, wc, ws, wg, False, "spec")
        if config == "skinny_prefetch":
            torch.cuda.synchronize()             # the contract of the prefetching config: weights complete beforehand
        ops.nvfp4_gemm(xc, xs, xg, wc, ws, wg, D, config)
        torch.cuda.synchronize()
        _check(bf16_bits(D), O.nvfp4_gemm(*xq, *wq), f"decode after device-side weight quantize ({config})")


@pytest.mark.parametrize("M", [1, 16, 33, 128])
def test_decode_mid_size_is_repeatable(cuda, lib, M):
    """N = 8192, K = 8192: every CTA's share of the stream-K split starts and ends inside a weight slab, so every slab is
    finished from partial tiles.  Three runs: the flags must come back by themselves, and the result must be the same bit
    for bit every time (partial tiles are always added in the same order)."""
    N, K = 8192, 8192
    wq = _weights(N, K, seed=77)
    X = randn_bf16((M, K), seed=78 + M)
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    rows = min(M, 3)
    ref = O.nvfp4_gemm(*xq, *wq, row0=M - rows, nrows=rows)
    first = None
    for _ in range(3):
        D = _run(cuda, X, wq)
        _check(D[M - rows:], ref, f"decode mid size M={M}")
        assert not np.isnan(O.bf16_to_f32(D)).any()
        if first is None:
            first = D
        assert np.array_equal(first, D)
