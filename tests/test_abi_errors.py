"""Error behaviour of the C ABI that does not depend on a device: argument checks come before any CUDA call, so a bad
call is answered with the same code and message with or without a GPU (the reference answers these with TORCH_CHECK
exceptions: include/pyutils/torchutils.cuh:35-83).  EVERY call below fails validation; none reaches a kernel launch,
so the made-up (16-byte aligned, never dereferenced) addresses are safe on a machine that has a GPU too."""
import ctypes

import pytest

from thunderkittens_b200 import _lib

P = 0x7F0000001000          # an aligned address that is never dereferenced
ODD = P + 4                 # a misaligned one
INVALID, ALIGN = 1, 2


def _msg(lib):
    return lib.tkb_last_error().decode()


def test_gemm_argument_errors(lib):
    f = lib.tkb_nvfp4_gemm
    assert f(None, P, P, P, P, P, P, 0, 256, 256, 256, None) == INVALID and "null" in _msg(lib)
    assert f(P, P, P, P, P, P, P, 0, 0, 256, 256, None) == INVALID and "positive" in _msg(lib)
    assert f(P, P, P, P, P, P, P, 0, 256, 256, 100, None) == INVALID and "multiple of 64" in _msg(lib)
    assert f(P, P, P, P, P, P, P, 0, 256, 252, 256, None) == INVALID and "multiple of 8" in _msg(lib)
    assert f(P, P, P, P, P, P, P, 100, 256, 256, 256, None) == ALIGN          # ldd < N
    assert f(ODD, P, P, P, P, P, P, 0, 256, 256, 256, None) == ALIGN
    assert f(P, None, P, P, P, P, P, 0, 256, 256, 256, None) == INVALID and "scale" in _msg(lib)
    assert f(P, P, None, P, P, P, P, 0, 256, 256, 256, None) == INVALID and "per-tensor" in _msg(lib)
    assert lib.tkb_nvfp4_gemm_ex(P, P, P, P, P, P, P, 0, 256, 256, 256, 99, None) == INVALID and "config" in _msg(lib)
    assert lib.tkb_nvfp4_gemm_ex(P, P, P, P, P, P, P, 0, 256, 256, 256, _lib.GEMM_SKINNY if hasattr(_lib, "GEMM_SKINNY") else 5, None) == INVALID
    assert lib.tkb_mxfp8_gemm(P, P, P, P, P, 0, 256, 256, 192, None) == INVALID and "multiple of 128" in _msg(lib)
    assert lib.tkb_bf16_gemm(P, 64, P, 0, P, 0, 256, 256, 128, None) == INVALID      # lda < K
    assert lib.tkb_fp8_gemm(P, 0, P, 0, P, 0, 256, 256, 72, None) == INVALID and "multiple of 16" in _msg(lib)


def test_quantize_argument_errors(lib):
    assert lib.tkb_nvfp4_quantize(None, 0, P, P, P, 128, 128, 0, 0, None) == INVALID
    assert lib.tkb_nvfp4_quantize(P, 0, P, P, P, 128, 100, 0, 0, None) == INVALID and "multiple of 64" in _msg(lib)
    assert lib.tkb_nvfp4_quantize(P, 0, P, P, P, 128, 128, 0, 7, None) == INVALID and "arithmetic" in _msg(lib)
    assert lib.tkb_nvfp4_quantize(P, 120, P, P, P, 128, 128, 0, 0, None) == ALIGN          # lda < K
    assert lib.tkb_nvfp4_quantize(P, 0, ODD, P, P, 128, 128, 0, 0, None) == ALIGN
    assert lib.tkb_nvfp4_quantize_with_amax(P, 0, P, P, P, None, 128, 128, 0, 0, None) == INVALID
    assert lib.tkb_mxfp8_quantize(P, 0, P, P, 128, 192, None) == INVALID and "multiple of 128" in _msg(lib)
    assert lib.tkb_mxfp8_quantize(P, 0, P, ODD, 128, 128, None) == ALIGN
    assert lib.tkb_absmax_bf16(P, 0, 0, 128, P, None) == INVALID
    assert lib.tkb_fp32_to_fp4x2(None, P, 16, None) == INVALID
    slots = (ctypes.c_void_p * 8)(*([P] * 8))
    f = lib.tkb_nvfp4_quantize_sharded
    assert f(P, 0, P, P, P, 128, 128, 0, 0, slots, 9, 0, 1, None) == INVALID           # world > 8
    assert f(P, 0, P, P, P, 128, 128, 2, 0, slots, 2, 0, 1, None) == INVALID and "layout" in _msg(lib)
    assert f(P, 0, P, P, P, 128, 128, 0, 0, None, 2, 0, 1, None) == INVALID             # no slot table
    assert f(P, 0, P, P, P, 128, 128, 0, 0, slots, 2, 0, 0, None) == INVALID            # epoch 0


def test_skinny_static_rejects_sizes_beyond_its_scratch(lib):
    f = lib.tkb_nvfp4_gemm_skinny_static
    assert f(P, P, P, P, P, P, P, 0, 17, 1024, 1024, None) == INVALID and "1..16" in _msg(lib)
    assert f(P, P, P, P, P, P, P, 0, 16, 1024, 1000, None) == INVALID
    assert f(ODD, P, P, P, P, P, P, 0, 16, 1024, 1024, None) == ALIGN


def test_multi_gpu_argument_errors(lib):
    arr = (ctypes.c_void_p * 8)(*([P] * 8))
    f = lib.tkb_ag_gemm_nvfp4
    assert f(None, arr, P, P, P, P, P, 0, 1024, 256, 1024, 0, 2, arr, None, None, 1, 4, None) == INVALID
    assert f(arr, arr, P, P, P, P, P, 0, 1024, 256, 1024, 0, 9, arr, None, None, 1, 4, None) == INVALID and "world" in _msg(lib)
    assert f(arr, arr, P, P, P, P, P, 0, 1000, 256, 1024, 0, 2, arr, None, None, 1, 4, None) == INVALID and "256 * world" in _msg(lib)
    assert lib.tkb_all_to_all(arr, P, 24, 0, 0, 2, arr, 0, 1, None) == ALIGN              # chunk size not a multiple of 16
    assert lib.tkb_all_to_all(arr, P, 0, 0, 0, 2, arr, 0, 1, None) == INVALID
    assert lib.tkb_wait_flags(None, 2, 0, 1, None) == INVALID
    assert lib.tkb_signal_peers(arr, 9, 0, 0, 1, 0, None) == INVALID
    assert lib.tkb_amax_allreduce(arr, 2, 2, 1, P, P, None) == INVALID                    # rank out of range
    assert lib.tkb_moe_route(P, 128, 48, 4, P, P, None) == INVALID and "multiple of 32" in _msg(lib)
    assert lib.tkb_moe_schedule(P, 128, 2, 30, 4, 0, P, P, P, P, P, P, 1024, None) == INVALID     # E % world
    assert lib.tkb_moe_dispatch_gemm(arr, P, P, P, P, P, P, P, 0, P, P, P, P, P, 1, 1000, 256, 4, 1024, 0, 2, 4, None) == INVALID
    assert lib.tkb_ag_linear_nvfp4(None, 1, P, P, P, P, P, 0, 256, 4, 0, None) == INVALID
    assert lib.tkb_moe_layer_nvfp4(None, 1, P, P, P, P, P, P, 4, 0, None) == INVALID


def test_no_device_is_an_error_not_a_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    # arguments that pass validation: the first CUDA call fails and nothing else happens
    assert lib.tkb_mxfp8_quantize(P, 0, P, P, 128, 128, None) == 3 and "cuda" in _msg(lib).lower()
    assert lib.tkb_nvfp4_gemm(P, P, P, P, P, P, P, 0, 256, 256, 256, None) == 3
    st = ctypes.c_int(0)
    assert lib.tkb_device_status(None, ctypes.byref(st)) == 3
