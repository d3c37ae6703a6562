"""The oracle's hand-written narrow-float codecs against the CUDA toolkit's host conversions
(cuda_fp4.h / cuda_fp8.h / cuda_bf16.h) — the functions the reference kernels call."""
import numpy as np

import oracle as O


def _values():
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 2**32, size=1_000_000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    special = np.array([0.0, -0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.25, -2.5, 2**-10, 2**-9, 2**-6,
                        448.0, 449.0, 463.9, 464.0, 480.0, 1e9, np.inf, -np.inf, np.nan, 1e-12, 1e-38, 1e-45,
                        2.0**-126, 2.0**-127, 2.0**127], np.float32)
    grid = np.linspace(-8, 8, 100001, dtype=np.float32)
    normal = np.concatenate([(rng.standard_normal(300000) * s).astype(np.float32) for s in (1e-3, 1.0, 100.0)])
    return np.concatenate([bits, special, grid, normal])


def _nv(fn, x, out_dtype, n_out=None):
    out = np.empty(x.size if n_out is None else n_out, out_dtype)
    fn(np.ascontiguousarray(x), out, x.size if n_out is None else n_out)
    return out


def test_e4m3_encode_matches_toolkit():
    x = _values()
    assert np.array_equal(O.f32_to_e4m3(x), _nv(O.nvhost().nvh_f32_to_e4m3, x, np.uint8))


def test_e8m0_encode_matches_toolkit():
    x = _values()
    assert np.array_equal(O.f32_to_e8m0(x), _nv(O.nvhost().nvh_f32_to_e8m0, x, np.uint8))


def test_e2m1_encode_matches_toolkit():
    x = _values()
    x = x[: x.size // 2 * 2]
    assert np.array_equal(O.fp32_to_fp4x2(x), _nv(O.nvhost().nvh_fp32_to_fp4x2, x, np.uint8, x.size // 2))


def test_bf16_encode_matches_toolkit():
    x = _values()
    assert np.array_equal(O.f32_to_bf16(x), _nv(O.nvhost().nvh_f32_to_bf16, x, np.uint16))


def test_decoders_match_toolkit():
    b = np.arange(256, dtype=np.uint8)
    nv = O.nvhost()
    out = np.empty(256, np.float32); nv.nvh_e4m3_to_f32(b, out, 256)
    assert np.array_equal(O.e4m3_to_f32(b), out, equal_nan=True)
    out = np.empty(256, np.float32); nv.nvh_e8m0_to_f32(b, out, 256)
    assert np.array_equal(O.e8m0_to_f32(b), out, equal_nan=True)
    out = np.empty(512, np.float32); nv.nvh_fp4x2_to_fp32(b, out, 256)
    assert np.array_equal(O.fp4x2_to_fp32(b), out)


def test_nibble_order():
    # element 2i in the low nibble (kernels/gemm/common.cuh:195-212): {2.4, -5.1} -> 0xF4
    assert O.fp32_to_fp4x2(np.array([2.4, -5.1], np.float32))[0] == 0xF4


def test_scale_swizzle_roundtrip_and_formula():
    rng = np.random.default_rng(1)
    sc = rng.integers(0, 256, size=(300, 24), dtype=np.uint8)
    sw = O.swizzle_scales(sc)
    assert sw.shape == (3, 6, 512)
    assert np.array_equal(O.unswizzle_scales(sw, 300), sc)
    flat = sw.reshape(-1)
    for r, kb in [(0, 0), (31, 3), (32, 0), (127, 23), (128, 5), (299, 23)]:
        assert flat[O.scale_swizzle_idx(r, kb, 24)] == sc[r, kb]
