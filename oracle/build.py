"""Build recipes for the CPU oracle (test infrastructure only; never imported by the product).

  python oracle/build.py            # builds everything that can be built on this machine

Outputs
  oracle/_build/libtkoracle.so   the C++ restatement (tk_oracle.cpp)
  oracle/_build/libnvhost.so     CUDA-toolkit host conversions (nv_host_codecs.cpp)
  oracle/_ref/libtkref_host.so   the reference's own kernels/gemm/common.cuh kernel bodies compiled
                                 for the host (only when the reference tree is present; the built
                                 object is git-ignored and travels with the working copy)
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")
REF_OUT = os.path.join(HERE, "_ref")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
# the ThunderKittens tree: $TK_REFERENCE, else a directory named `reference` beside this repository
REFERENCE = os.environ.get("TK_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

CXXFLAGS = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", "-std=c++17"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError("oracle build failed: " + cmd[-1])


def build_oracle() -> str:
    os.makedirs(BUILD, exist_ok=True)
    src = os.path.join(HERE, "tk_oracle.cpp")
    out = os.path.join(BUILD, "libtkoracle.so")
    if not _newer(out, [src, __file__]):
        _run(["g++", *CXXFLAGS, src, "-o", out])
    return out


def build_nv_codecs() -> str:
    os.makedirs(BUILD, exist_ok=True)
    src = os.path.join(HERE, "nv_host_codecs.cpp")
    out = os.path.join(BUILD, "libnvhost.so")
    if not _newer(out, [src, __file__]):
        _run(["g++", "-O2", "-shared", "-fPIC", "-std=c++17", "-I", os.path.join(CUDA_HOME, "include"), src, "-o", out])
    return out


def build_ref() -> str | None:
    """Compile the reference's kernels/gemm/common.cuh for the host.  Returns None when the
    reference tree is absent and no prebuilt object exists."""
    out = os.path.join(REF_OUT, "libtkref_host.so")
    common = os.path.join(REFERENCE, "kernels", "gemm", "common.cuh")
    if not os.path.exists(common):
        return out if os.path.exists(out) else None
    os.makedirs(REF_OUT, exist_ok=True)
    driver = os.path.join(HERE, "ref_host.cpp")
    shim = os.path.join(HERE, "ref_shim", "kittens.cuh")
    if _newer(out, [driver, shim, common, __file__]):
        return out
    # The launch syntax `kernel<<<grid, block>>>(args)` only appears in launcher wrappers that the
    # host driver never calls; strip it so that g++ can parse the file.  Kernel bodies are untouched.
    text = open(common).read()
    stripped = re.sub(r"<<<[^>]*>>>", "", text)
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:     # the stripped copy of the reference header never stays in this tree
        gen = os.path.join(tmp, "common_host.cuh")
        with open(gen, "w") as f:
            f.write(stripped)
        _run(["g++", "-O2", "-march=x86-64-v3", "-ffp-contract=fast", "-fopenmp", "-shared", "-fPIC", "-std=c++20",
              "-x", "c++", "-I", os.path.join(HERE, "ref_shim"), "-I", os.path.join(CUDA_HOME, "include"),
              f'-DREF_COMMON_CUH="{gen}"', driver, "-o", out])
    return out


def build_ref_gpu(which: str = "nvfp4") -> str | None:
    """Compile the reference's own GPU kernels (nvfp4_b200 or mxfp8_b200: GEMM + quantizer) as the PyTorch extension the
    reference's Makefile describes (kernels/common.mk `CONFIG := pytorch`, kernels/gemm/<dir>/Makefile), straight from the
    reference tree with one nvcc command.  Output: oracle/_ref/tk_<which>/_C<ext>.so (git-ignored).  Used on the GPU box to
    compare quantizer outputs bit-for-bit with the reference kernel and to time the reference beside this library.
    Single-GPU use only: the reference kernels issue TMA loads with cluster multicast."""
    import sysconfig
    srcdir = os.path.join(REFERENCE, "kernels", "gemm", f"{which}_b200")
    src = os.path.join(srcdir, f"{which}_b200_gemm.cu")
    outdir = os.path.join(REF_OUT, f"tk_{which}")
    out = os.path.join(outdir, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if _newer(out, [src, __file__]):
        return out
    os.makedirs(outdir, exist_ok=True)
    from torch.utils.cpp_extension import include_paths, library_paths
    import pybind11
    cmd = ["nvcc", "-std=c++20", "-O3", "--use_fast_math", "--expt-extended-lambda", "--expt-relaxed-constexpr",
           "-forward-unknown-to-host-compiler", "-Xcompiler=-Wno-psabi", "-Xcompiler=-fno-strict-aliasing", "-DNDEBUG", "-lineinfo",
           "-DKITTENS_BLACKWELL", "-gencode", "arch=compute_100a,code=sm_100a", "-DTORCH_COMPILE", "-shared", "-fPIC",
           "-diag-suppress", "3189", "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
           "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-DTORCH_EXTENSION_NAME=_C", "-I", os.path.join(REFERENCE, "include"), "-I", os.path.join(REFERENCE, "prototype"),
           "-I", sysconfig.get_path("include"), "-I", pybind11.get_include()]
    for pth in include_paths():
        cmd += ["-I", pth]
    for pth in library_paths() + [os.path.join(CUDA_HOME, "lib64", "stubs")]:
        cmd += ["-L", pth]
    cmd += ["-ltorch_python", "-ltorch_cuda", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-lc10", "-lcuda", "-lcudart_static", "-lrt",
            "-lpthread", "-ldl", src, "-o", out]
    _run(cmd)
    return out


def build_ref_standalone(which: str = "bf16") -> str | None:
    """Compile one of the reference's standalone GEMM benchmarks (kernels/gemm/bf16_b200 or fp8_b200: a kernel plus a main()
    that times it at 1024^3 ... 16384^3 and checks it against the reference's naive kernel) the way the reference's Makefile does
    (kernels/common.mk `CONFIG := standalone`, GPU := B200), straight from the reference tree with one nvcc command.  Output:
    oracle/_ref/tk_<which>/<which>_b200_gemm.out (git-ignored).  Used on a single-GPU box to time the reference beside this
    library; single-GPU use only (the reference kernels issue TMA loads with cluster multicast)."""
    srcdir = os.path.join(REFERENCE, "kernels", "gemm", f"{which}_b200")
    src = os.path.join(srcdir, f"{which}_b200_gemm.cu")
    outdir = os.path.join(REF_OUT, f"tk_{which}")
    out = os.path.join(outdir, f"{which}_b200_gemm.out")
    if not os.path.exists(src):
        return out if os.path.exists(out) else None
    if _newer(out, [src, __file__]):
        return out
    os.makedirs(outdir, exist_ok=True)
    _run(["nvcc", src, "-std=c++20", "-O3", "--use_fast_math", "-lrt", "-lpthread", "-ldl", "-lcuda", "-lcudadevrt", "-lcudart_static",
          "--expt-extended-lambda", "--expt-relaxed-constexpr", "-forward-unknown-to-host-compiler", "-Xcompiler=-Wno-psabi",
          "-Xcompiler=-fno-strict-aliasing", "-I", os.path.join(REFERENCE, "include"), "-I", os.path.join(REFERENCE, "prototype"),
          "-DNDEBUG", "-lineinfo", "-DKITTENS_BLACKWELL", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out])
    return out


def build_all() -> dict:
    return {"oracle": build_oracle(), "nvhost": build_nv_codecs(), "ref": build_ref()}


if __name__ == "__main__":
    for k, v in build_all().items():
        print(k, "->", v)
