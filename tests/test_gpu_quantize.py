"""GPU parity of the quantize kernels (through the C ABI) against the CPU oracle and the golden
vectors.  Codes, scales and per-tensor scales must be bit-exact."""
import os

import numpy as np
import pytest
import torch

import oracle as O
from tests.util import randn_bf16, bf16_bits, bits_to_bf16, u8

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _ops():
    import thunderkittens_b200.ops as ops
    return ops


def gpu_nvfp4_quantize(A, scale_2d=False, arithmetic="spec", amax=None):
    ops = _ops()
    M, K = A.shape
    codes = torch.full((M, K // 2), 0xAA, dtype=torch.uint8, device=A.device)
    sc = torch.full(((M + 127) // 128, K // 64, 512), 0xAA, dtype=torch.uint8, device=A.device)
    sg = torch.full((1,), -1.0, dtype=torch.float32, device=A.device)
    ops.nvfp4_quantize(A, codes, sc, sg, scale_2d, arithmetic, amax)
    torch.cuda.synchronize()
    from thunderkittens_b200 import _lib
    assert _lib.device_status() == 0
    return u8(codes), u8(sc), sg.cpu().numpy()


def gpu_mxfp8_quantize(A):
    ops = _ops()
    M, K = A.shape
    codes = torch.full((M, K), 0xAA, dtype=torch.uint8, device=A.device)
    sc = torch.full(((M + 127) // 128, K // 128, 512), 0xAA, dtype=torch.uint8, device=A.device)
    ops.mxfp8_quantize(A, codes, sc)
    torch.cuda.synchronize()
    return u8(codes), u8(sc)


@pytest.mark.parametrize("tag,scale_2d", [("1d", False), ("2d", True)])
def test_nvfp4_golden(cuda, lib, tag, scale_2d):
    g = np.load(os.path.join(GOLD, f"nvfp4_quantize_{tag}.npz"))
    A = bits_to_bf16(g["A_bf16"], cuda)
    codes, sc, sg = gpu_nvfp4_quantize(A, scale_2d, "spec")
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(sc, g["sc"])
    assert sg[0] == g["sg"][0]


# the last two 1-D cases take the tile-per-CTA kernel (more than two 128 x 128 tiles per SM, K % 128 == 0), one with a ragged last row block
@pytest.mark.parametrize("M,K", [(128, 128), (1, 64), (16, 8192), (130, 192), (1024, 1024), (2048, 7168), (2100, 4096)])
@pytest.mark.parametrize("arith,assoc", [("spec", "spec"), ("kernel_ieee", "kernel")])
@pytest.mark.parametrize("scale_2d", [False, True])
def test_nvfp4_vs_oracle(cuda, lib, M, K, arith, assoc, scale_2d):
    if scale_2d and M % 16:
        pytest.skip("2-D scaling needs whole 16-row blocks")
    A = randn_bf16((M, K), seed=M * 7 + K, outlier_frac=0.01)
    rc, rs, rg = O.nvfp4_quantize(bf16_bits(A), scale_2d, assoc)
    codes, sc, sg = gpu_nvfp4_quantize(A.to(cuda), scale_2d, arith)
    assert sg[0] == rg[0]
    assert np.array_equal(sc, rs), f"{(sc != rs).sum()} scale bytes differ"
    assert np.array_equal(codes, rc), f"{(codes != rc).sum()} code bytes differ"


def test_nvfp4_with_supplied_amax_equals_full_tensor(cuda, lib):
    ops = _ops()
    A = randn_bf16((512, 256), seed=5)
    full_c, full_s, full_g = O.nvfp4_quantize(bf16_bits(A))
    Ad = A.to(cuda)
    amax = torch.zeros(1, dtype=torch.float32, device=cuda)
    ops.absmax_bf16(Ad, amax)
    torch.cuda.synchronize()
    assert float(amax.item()) == O.absmax_bf16(bf16_bits(A))
    for r0 in (0, 128, 256, 384):     # four row shards quantized on their own with the global amax
        c, s, g = gpu_nvfp4_quantize(Ad[r0:r0 + 128].contiguous(), False, "spec", amax)
        assert np.array_equal(c, full_c[r0:r0 + 128])
        assert np.array_equal(s[0], full_s[r0 // 128])
        assert g[0] == full_g[0]


def test_nvfp4_repeated_calls_reuse_scratch_cleanly(cuda, lib):
    A = randn_bf16((256, 256), seed=9).to(cuda)
    B = (randn_bf16((256, 256), seed=10) * 0.01).to(cuda)
    a1 = gpu_nvfp4_quantize(A)
    for _ in range(300):           # more calls than scratch slots
        b = gpu_nvfp4_quantize(B)
    a2 = gpu_nvfp4_quantize(A)
    assert all(np.array_equal(x, y) for x, y in zip(a1, a2))
    rb = O.nvfp4_quantize(bf16_bits(B.cpu()))
    assert all(np.array_equal(x, y) for x, y in zip(b, rb))


def test_nvfp4_tile_kernel_matches_register_tile_kernel(cuda, lib):
    """Large tensors take the tile-per-CTA kernel; a sub-tensor view (row pitch larger than K) of the same data must give the
    same bytes, and so must repeated calls (the scratch slot of the grid barrier is handed back clean)."""
    big = randn_bf16((2304, 4352), seed=77, outlier_frac=0.01).to(cuda)
    A = big[:, :4096]                                 # lda = 4352, K = 4096
    ref = O.nvfp4_quantize(bf16_bits(A.cpu().contiguous()), False, "spec")
    _ops()
    for _ in range(3):
        codes = torch.empty(2304, 2048, dtype=torch.uint8, device=cuda)
        sc = torch.empty(18, 64, 512, dtype=torch.uint8, device=cuda)
        sg = torch.empty(1, dtype=torch.float32, device=cuda)
        from thunderkittens_b200 import _lib as L
        L.check(L.lib().tkb_nvfp4_quantize(A.data_ptr(), 4352, codes.data_ptr(), sc.data_ptr(), sg.data_ptr(), 2304, 4096, 0, L.NVFP4_SPEC,
                                           torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert L.device_status() == 0
        assert np.array_equal(u8(codes), ref[0]) and np.array_equal(u8(sc), ref[1]) and float(sg.item()) == ref[2][0]


def test_nvfp4_fast_mode_close_to_ieee(cuda, lib):
    A = randn_bf16((1024, 1024), seed=21).to(cuda)
    c0, s0, g0 = gpu_nvfp4_quantize(A, False, "kernel_ieee")
    c1, s1, g1 = gpu_nvfp4_quantize(A, False, "kernel_fast")
    assert abs(float(g0[0]) - float(g1[0])) <= 4 * np.spacing(np.float32(g0[0]))
    assert (s0 != s1).mean() < 0.02 and (c0 != c1).mean() < 0.02


def test_nvfp4_zero_and_edge_inputs(cuda, lib):
    Z = torch.zeros(128, 128, dtype=torch.bfloat16, device=cuda)
    for arith, assoc in (("spec", "spec"), ("kernel_ieee", "kernel")):
        c, s, g = gpu_nvfp4_quantize(Z, False, arith)
        rc, rs, rg = O.nvfp4_quantize(np.zeros((128, 128), np.uint16), False, assoc)
        assert not c.any() and not s.any() and g[0] == rg[0]     # spec: 1/(2688/1e-12); kernel order: 0
    A = randn_bf16((128, 128), seed=3)
    A[0, 0] = 3.0e38     # near bf16 max
    rc, rs, rg = O.nvfp4_quantize(bf16_bits(A))
    c, s, g = gpu_nvfp4_quantize(A.to(cuda))
    assert np.array_equal(c, rc) and np.array_equal(s, rs) and g[0] == rg[0]


def test_mxfp8_golden(cuda, lib):
    g = np.load(os.path.join(GOLD, "mxfp8_quantize.npz"))
    codes, sc = gpu_mxfp8_quantize(bits_to_bf16(g["A_bf16"], cuda))
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(sc.reshape(g["sc"].shape), g["sc"])
    codes, sc = gpu_mxfp8_quantize(bits_to_bf16(g["inv_bf16"], cuda))
    assert np.array_equal(sc.reshape(g["inv_sc"].shape), g["inv_sc"])
    assert np.array_equal(O.e4m3_to_f32(codes), O.e4m3_to_f32(g["inv_codes"]))


# the last two take the tile-per-CTA kernel (two or more 128 x 128 tiles per SM), one of them with a ragged last row block
@pytest.mark.parametrize("M,K", [(128, 128), (1, 128), (130, 384), (1024, 1024), (2048, 7168), (2100, 4096)])
def test_mxfp8_vs_oracle(cuda, lib, M, K):
    A = randn_bf16((M, K), seed=M + K, outlier_frac=0.01)
    rc, rs = O.mxfp8_quantize(bf16_bits(A))
    codes, sc = gpu_mxfp8_quantize(A.to(cuda))
    assert np.array_equal(sc, rs)
    assert np.array_equal(codes, rc)


def test_fp4_pack_unpack(cuda, lib):
    ops = _ops()
    x = (torch.randn(64, 256, generator=torch.Generator().manual_seed(1)) * 3).to(cuda)
    packed = ops.fp32_to_fp4x2(x)
    torch.cuda.synchronize()
    assert np.array_equal(u8(packed), O.fp32_to_fp4x2(x.cpu().numpy()))
    back = ops.fp4x2_to_fp32(packed)
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy(), O.fp4x2_to_fp32(u8(packed)))


def test_full_size_quantize_properties(cuda, lib):
    """8192 x 8192 (the GEMM operand size of the headline configs): row slabs against the oracle with the
    global amax, and the reconstruction error of the dequantised tensor."""
    g = torch.Generator(device=cuda).manual_seed(7)
    A = torch.randn(8192, 8192, generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16)
    codes, sc, sg = gpu_nvfp4_quantize(A)
    amax = float(A.abs().max().float().item())
    for r0 in (0, 4096 + 128, 8192 - 128):
        slab = bf16_bits(A[r0:r0 + 128])
        rc, rs, rg = O.nvfp4_quantize(slab, False, "spec", amax=amax)
        assert np.array_equal(codes[r0:r0 + 128], rc)
        assert np.array_equal(sc[r0 // 128], rs[0])
        assert sg[0] == rg[0]
    mc, ms = gpu_mxfp8_quantize(A)
    for r0 in (0, 8192 - 128):
        rc, rs = O.mxfp8_quantize(bf16_bits(A[r0:r0 + 128]))
        assert np.array_equal(mc[r0:r0 + 128], rc) and np.array_equal(ms[r0 // 128], rs[0])
    # reconstruction error of the whole tensor stays at the format's level (e4m3: 3 mantissa bits; e2m1: 1)
    a32 = A[:1024].float().cpu().numpy()
    d8 = O.dequant_mxfp8(mc[:1024], ms[:8])
    assert np.linalg.norm(d8 - a32) / np.linalg.norm(a32) < 0.04
    d4 = O.dequant_nvfp4(codes[:1024], sc[:8], sg)
    assert np.linalg.norm(d4 - a32) / np.linalg.norm(a32) < 0.15


def test_argument_errors(cuda, lib):
    ops = _ops()
    from thunderkittens_b200._lib import TkbError
    A = torch.zeros(128, 96, dtype=torch.bfloat16, device=cuda)      # K not a multiple of 64
    with pytest.raises((TkbError, RuntimeError)):
        ops.nvfp4_quantize(A, torch.zeros(128, 48, dtype=torch.uint8, device=cuda), torch.zeros(1, 1, 512, dtype=torch.uint8, device=cuda),
                           torch.zeros(1, device=cuda), False)
    with pytest.raises(RuntimeError):
        ops.mxfp8_quantize(torch.zeros(128, 128, dtype=torch.float32, device=cuda), torch.zeros(128, 128, dtype=torch.uint8, device=cuda),
                           torch.zeros(1, 1, 512, dtype=torch.uint8, device=cuda))


@pytest.mark.parametrize("M,K", [(1, 8192), (5, 2112), (16, 1024), (16, 8192), (3, 64), (16, 7168)])
@pytest.mark.parametrize("arith,assoc", [("spec", "spec"), ("kernel_ieee", "kernel")])
def test_nvfp4_small_activation_kernel_vs_oracle(cuda, lib, M, K, arith, assoc):
    """M <= 16, K <= 8192 takes the thread-block-cluster kernel (amax through distributed shared memory)."""
    A = randn_bf16((M, K), seed=M * 11 + K, outlier_frac=0.01)
    rc, rs, rg = O.nvfp4_quantize(bf16_bits(A), False, assoc)
    codes, sc, sg = gpu_nvfp4_quantize(A.to(cuda), False, arith)
    assert sg[0] == rg[0]
    assert np.array_equal(sc, rs), f"{(sc != rs).sum()} scale bytes differ"
    assert np.array_equal(codes, rc), f"{(codes != rc).sum()} code bytes differ"


@pytest.mark.parametrize("M,K", [(1, 8192), (16, 8192), (7, 4160)])
def test_nvfp4_small_activation_kernel_fast_arithmetic_equals_general_kernel(cuda, lib, M, K):
    """The fast-math arithmetic has no CPU restatement: the cluster kernel must equal the general kernel, which is reached
    by supplying the amax (and which is bit-identical to the reference's own kernel)."""
    ops = _ops()
    A = randn_bf16((M, K), seed=M + K, outlier_frac=0.01).to(cuda)
    amax = torch.zeros(1, dtype=torch.float32, device=cuda)
    ops.absmax_bf16(A, amax)
    a = gpu_nvfp4_quantize(A, False, "kernel_fast")
    b = gpu_nvfp4_quantize(A, False, "kernel_fast", amax)
    assert a[2][0] == b[2][0] and np.array_equal(a[1], b[1]) and np.array_equal(a[0], b[0])
