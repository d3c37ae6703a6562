"""The oracle against the committed golden vectors, which were produced by importing the reference's
own torch specifications (tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest

import oracle as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("tag,scale_2d", [("1d", False), ("2d", True)])
def test_nvfp4_quantize_matches_reference_spec(tag, scale_2d):
    g = np.load(os.path.join(GOLD, f"nvfp4_quantize_{tag}.npz"))
    codes, sc, sg = O.nvfp4_quantize(g["A_bf16"], scale_2d, assoc="spec")
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(sc, g["sc"])
    assert sg[0] == g["sg"][0]
    assert np.array_equal(O.unswizzle_scales(sc, g["A_bf16"].shape[0]), g["sc_unswizzled"])
    assert np.array_equal(O.dequant_nvfp4(codes, sc, sg), g["dequant"])


def test_nvfp4_kernel_association_differs_only_in_rounding():
    # The reference kernel forms sg_dec = amax/2688 first (nvfp4_b200_gemm.cu:420-422); the torch spec forms
    # sg_enc = 2688/amax first.  The two agree except where a rounding tie falls the other way.
    g = np.load(os.path.join(GOLD, "nvfp4_quantize_1d.npz"))
    c0, s0, g0 = O.nvfp4_quantize(g["A_bf16"], False, assoc="spec")
    c1, s1, g1 = O.nvfp4_quantize(g["A_bf16"], False, assoc="kernel")
    assert abs(float(g0[0]) - float(g1[0])) <= 2 * np.spacing(np.float32(g0[0]))
    assert (s0 != s1).mean() < 0.02
    d0, d1 = O.dequant_nvfp4(c0, s0, g0), O.dequant_nvfp4(c1, s1, g1)
    a = O.bf16_to_f32(g["A_bf16"])
    assert abs(np.abs(d0 - a).mean() - np.abs(d1 - a).mean()) < 1e-3 * np.abs(a).mean()


def test_mxfp8_quantize_matches_reference_spec():
    g = np.load(os.path.join(GOLD, "mxfp8_quantize.npz"))
    codes, sc = O.mxfp8_quantize(g["A_bf16"])
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(sc.reshape(g["sc"].shape), g["sc"])
    assert np.array_equal(O.unswizzle_scales(sc, g["A_bf16"].shape[0]), g["sc_unswizzled"])


def test_mxfp8_inverse_construction():
    # random codes + random e8m0 -> bf16 -> quantize returns them (mxfp8_b200/test_quantize.py:127-145)
    g = np.load(os.path.join(GOLD, "mxfp8_quantize.npz"))
    codes, sc = O.mxfp8_quantize(g["inv_bf16"])
    assert np.array_equal(sc.reshape(g["inv_sc"].shape), g["inv_sc"])
    # -0 and +0 codes dequantise to the same bf16 zero; compare values
    assert np.array_equal(O.e4m3_to_f32(codes), O.e4m3_to_f32(g["inv_codes"]))


def test_ragged_rows_pad_scales_with_zero():
    rng = np.random.default_rng(3)
    A = O.f32_to_bf16(rng.standard_normal((130, 128)).astype(np.float32))
    codes, sc, sg = O.nvfp4_quantize(A)
    assert sc.shape == (2, 2, 512)
    un = O.unswizzle_scales(sc, 256)
    assert (un[130:] == 0).all() and (un[:130] != 0).any()
    full, scf, sgf = O.nvfp4_quantize(np.vstack([A, np.zeros((126, 128), np.uint16)]))
    assert np.array_equal(full[:130], codes) and np.array_equal(scf, sc) and sgf[0] == sg[0]


def test_all_zero_input():
    A = np.zeros((128, 128), np.uint16)
    codes, sc, sg = O.nvfp4_quantize(A)
    assert not codes.any() and not sc.any() and sg[0] == 0.0
    codes, sc = O.mxfp8_quantize(A)
    assert not codes.any() and (O.unswizzle_scales(sc, 128) == 88).all()   # 2^-39, the 1e-12 clamp rounded up
