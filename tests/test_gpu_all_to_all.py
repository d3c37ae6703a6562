"""General 4-D all-to-all (tkb_all_to_all_4d / parallel.tk_all_to_all) against the definition in the reference kernel
(all_to_all.cu:63-89): world size 1 in-process (every axis pair; the result is the input), world size 2+ as child processes."""
import itertools
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("scatter,gather", [p for p in itertools.permutations(range(4), 2)])
def test_all_to_all_world1_is_identity(cuda, lib, scatter, gather):
    from thunderkittens_b200 import parallel, _lib
    x = parallel.TKParallelTensor((2, 3, 16, 64), torch.bfloat16, 0, 1, False)
    y = parallel.TKParallelTensor((2, 3, 16, 64), torch.bfloat16, 0, 1, False)
    bar = parallel.TKParallelTensor((2,), torch.int32, 0, 1, False)
    x.data_.copy_(torch.randn(2, 3, 16, 64, device=cuda).to(torch.bfloat16))
    for _ in range(2):
        y.data_.zero_()
        parallel.tk_all_to_all(y, x, bar, scatter, gather)
        torch.cuda.synchronize()
        assert _lib.device_status() == 0 and torch.equal(y.data_, x.data_)
    for t in (x, y, bar):
        t.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_to_all_multi_gpu(cuda, lib, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29700 + world), os.path.join(ROOT, "tests", "mp_a2a_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    sys.stdout.write(r.stdout[-3000:])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("PASS") == world
