"""GEMM + reduce-scatter (NVFP4): world size 1 in-process (the reduce-add epilogue against the plain GEMM), world size 2+
as child processes when the machine has the GPUs."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle as O
from tests.util import randn_bf16, bf16_bits, to_dev_u8
from tests.test_gpu_gemm import _check

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_gemm_rs_world1(cuda, lib):
    """One rank: every tile is added into this rank's zeroed rows, so the result equals the plain GEMM's."""
    from thunderkittens_b200 import parallel, _lib
    M, N, K = 512, 384, 1024
    aq = O.nvfp4_quantize(bf16_bits(randn_bf16((M, K), seed=1)), False, "spec")
    bq = O.nvfp4_quantize(bf16_bits(randn_bf16((N, K), seed=2, std=0.05)), False, "spec")
    op = parallel.GemmReduceScatterNVFP4(M, N, 0, 1)
    for _ in range(2):
        out = op(to_dev_u8(aq[0], cuda), to_dev_u8(aq[1], cuda), torch.from_numpy(aq[2]).to(cuda),
                 to_dev_u8(bq[0], cuda), to_dev_u8(bq[1], cuda), torch.from_numpy(bq[2]).to(cuda))
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        _check(bf16_bits(out), O.nvfp4_gemm(*aq, *bq), "gemm_rs world=1")
    op.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gemm_rs_multi_gpu(cuda, lib, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29700 + world), os.path.join(ROOT, "tests", "mp_rs_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    sys.stdout.write(r.stdout[-4000:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("PASS") == world
