"""The C-ABI library loads without a GPU, exports every symbol include/tkb200.h declares, and fails
loudly (error code + message, no fallback) when no device is present."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tkb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tkb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for s in ["tkb_nvfp4_gemm", "tkb_nvfp4_quantize", "tkb_mxfp8_gemm", "tkb_mxfp8_quantize", "tkb_bf16_gemm",
              "tkb_fp32_to_fp4x2", "tkb_fp4x2_to_fp32"]:
        assert s in syms


def test_library_exports_every_declared_symbol(lib):
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} declared in include/tkb200.h but not exported"


def test_no_cpu_fallback_without_device(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    rc = lib.tkb_mxfp8_quantize(None, 0, None, None, 128, 128, None)
    assert rc != 0
    assert len(lib.tkb_last_error()) > 0


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "thunderkittens_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text and "tk_oracle" not in text, f


def test_ctypes_mirrors_of_the_state_structs_match_the_header(lib):
    """thunderkittens_b200/_lib.py mirrors tkb_ag_state and tkb_moe_state by hand: size and every member offset must
    equal what the C compiler laid out (tkb_debug_struct_layout)."""
    from thunderkittens_b200 import _lib
    f = lib.tkb_debug_struct_layout
    f.argtypes = [ctypes.c_int, ctypes.c_int]
    f.restype = ctypes.c_int
    for which, mirror in ((0, _lib.AgState), (1, _lib.MoeState), (2, _lib.RsState)):
        assert f(which, 0) == ctypes.sizeof(mirror)
        for i, (name, *_rest) in enumerate(mirror._fields_, start=1):
            assert f(which, i) == getattr(mirror, name).offset, (mirror.__name__, name)
        assert f(which, len(mirror._fields_) + 1) == -1      # the mirror lists every member
