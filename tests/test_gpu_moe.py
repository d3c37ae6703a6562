"""MoE layer (routing, device-side schedule, dispatch fused with the grouped NVFP4 expert GEMM, combine):
world size 1 in-process; world size 2+ as child processes when the GPUs are there.  The combine step and the
routing have no counterpart in the reference (parity unpinned): the oracle's restatement is the specification."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("comm_sms", [4, 0])        # dispatch by CTAs of the GEMM kernel / by the gather kernel on all SMs
@pytest.mark.parametrize("T,H,I,E,top_k", [(512, 512, 256, 32, 4), (1024, 1024, 512, 64, 8), (256, 256, 128, 32, 1)])
def test_moe_layer_world1(cuda, lib, T, H, I, E, top_k, comm_sms):
    from tests.moe_common import run_and_check
    ok, layer = run_and_check(cuda, 0, 1, T, H, I, E, top_k, iters=3, comm_sms=comm_sms)
    layer.close()
    assert ok


def test_moe_capacity_overflow_is_reported(cuda, lib):
    from thunderkittens_b200 import parallel, _lib
    from tests.moe_common import make_problem
    import oracle as O
    from tests.util import bf16_bits, to_dev_u8
    T, H, I, E, k = 256, 256, 128, 32, 4
    layer = parallel.MoELayerNVFP4(T, H, I, E, k, 0, 1, cap_rows=128)      # far too small
    X, logits, W = make_problem(T, H, I, E)
    wq = O.nvfp4_quantize(bf16_bits(W.reshape(E * I, H)))
    layer.forward(logits.to(cuda), X.to(cuda), to_dev_u8(wq[0], cuda), to_dev_u8(wq[1], cuda), torch.from_numpy(wq[2]).to(cuda))
    torch.cuda.synchronize()
    assert _lib.device_status() == _lib.ERR_CAPACITY
    layer.close()


def _run_workers(world, size, comm):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TKB_TEST_MOE_SIZE=size, TKB_TEST_MOE_COMM=str(comm))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29600 + world), os.path.join(ROOT, "tests", "mp_moe_worker.py")],
                       capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    sys.stdout.write(r.stdout[-6000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("PASS") == world


@pytest.mark.parametrize("comm", [4, 0])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_moe_layer_multi_gpu(cuda, lib, world, comm):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_workers(world, "small", comm)


@pytest.mark.parametrize("comm", [32, 0])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_moe_layer_multi_gpu_benchmark_size(cuda, lib, world, comm):
    """16384 tokens, hidden 7168, 128 experts, intermediate 2048, top-8 with the benchmark's dispatch settings."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_workers(world, "c5", comm)
