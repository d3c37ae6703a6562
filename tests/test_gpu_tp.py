"""Tensor-parallel all-gather GEMM (NVFP4): world size 1 in-process, world size 2+ as child processes
(one per GPU, torchrun) when the machine has the GPUs."""
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


def test_ag_gemm_world1(cuda, lib):
    """The all-gather variant of the kernel with a single rank: no comm CTAs, same result as the plain GEMM."""
    from thunderkittens_b200 import parallel
    M, K, N = 1024, 1024, 512
    X = randn_bf16((M, K), seed=1)
    wq = O.nvfp4_quantize(bf16_bits(randn_bf16((N, K), seed=2, std=0.02)))
    op = parallel.AllGatherMatmulNVFP4(M, K, 0, 1, arithmetic="spec")
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    for _ in range(3):
        op(X.to(cuda), to_dev_u8(wq[0], cuda), to_dev_u8(wq[1], cuda), torch.from_numpy(wq[2]).to(cuda), D)
    torch.cuda.synchronize()
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    _check(bf16_bits(D), O.nvfp4_gemm(*xq, *wq), "ag world=1")
    op.close()


def _run_workers(world, gather, size):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TKB_TEST_TP_CE="1" if gather == "copy_engines" else "0",
               TKB_TEST_TP_PUSH="1" if gather == "push_warps" else "0", TKB_TEST_TP_SIZE=size)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29500 + world), os.path.join(ROOT, "tests", "mp_tp_worker.py")],
                       capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    sys.stdout.write(r.stdout[-6000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PASS") == world


@pytest.mark.parametrize("gather", ["comm_ctas", "copy_engines", "push_warps"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ag_gemm_multi_gpu(cuda, lib, world, gather):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_workers(world, gather, "small")


@pytest.mark.parametrize("gather", ["comm_ctas", "copy_engines", "push_warps"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ag_gemm_multi_gpu_benchmark_size(cuda, lib, world, gather):
    """M = 8192, N = 28672, K = 8192 with the benchmark's gather settings: gathered operand bit-exact, D on slabs of every shard."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_workers(world, gather, "c4")
