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


@pytest.mark.parametrize("comm_sms", [4, 0])
def test_reference_shaped_moe_dispatch_gemm_world1(cuda, lib, comm_sms):
    """parallel.moe_dispatch_gemm with the reference's argument list and a schedule built on the host the way the reference's
    benchmark builds it (moe_dispatch_gemm/benchmark.py:112-149: experts drawn per token, counts padded to 128, rows of an
    expert segment in ring order of the source ranks, (-1, -1) padding)."""
    import numpy as np
    import oracle as O
    from thunderkittens_b200 import parallel, _lib
    from tests.util import bf16_bits, to_dev_u8, randn_bf16, rel_fro
    T, H, I, E, k = 384, 512, 256, 8, 2
    rng = np.random.default_rng(5)
    chosen = np.stack([rng.choice(E, size=k, replace=False) for _ in range(T)]).astype(np.int32)
    counts = np.bincount(chosen.reshape(-1), minlength=E).astype(np.int32)
    padded = (counts + 127) // 128 * 128
    rows = int(padded.sum())
    start = np.concatenate([[0], np.cumsum(padded[:-1])]).astype(np.int64)
    pull = np.full((rows, 2), -1, np.int32)
    fill = start.copy()
    for tok in range(T):                     # one rank: the ring starts and ends at rank 0
        for e in chosen[tok]:
            pull[fill[e]] = (0, tok)
            fill[e] += 1
    X = randn_bf16((T, H), seed=21)
    W = randn_bf16((E * I, H), seed=22, std=0.02)
    wq = O.nvfp4_quantize(bf16_bits(W))
    pre = parallel.TKParallelTensor((T, H), torch.bfloat16, 0, 1)
    pre.data_.copy_(X)
    state = parallel.MoEDispatchGemmState(T, H, I, E, rows, 0, 1)
    state.arithmetic = _lib.NVFP4_SPEC
    out = torch.full((rows, I), float("nan"), dtype=torch.bfloat16, device=cuda)
    for _ in range(2):
        parallel.moe_dispatch_gemm(pre, None, (to_dev_u8(wq[0], cuda), to_dev_u8(wq[1], cuda), torch.from_numpy(wq[2]).to(cuda)), out,
                                   torch.from_numpy(padded).to(cuda), torch.from_numpy(pull).to(cuda), state, comm_sms, rows)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
    x_sc_rows = O.unswizzle_scales(xq[1], T)
    w_sc_rows = O.unswizzle_scales(wq[1], E * I)
    got = bf16_bits(out)
    for e in range(E):
        n = int(padded[e])
        if n == 0:
            continue
        seg = pull[start[e]:start[e] + n]
        valid = seg[:, 0] >= 0
        tok = np.where(valid, seg[:, 1], 0)
        a_codes = np.where(valid[:, None], xq[0][tok], 0).astype(np.uint8)
        a_sc = O.swizzle_scales(np.where(valid[:, None], x_sc_rows[tok], 0).astype(np.uint8))
        ref = O.nvfp4_gemm(a_codes, a_sc, xq[2], wq[0][e * I:(e + 1) * I], O.swizzle_scales(w_sc_rows[e * I:(e + 1) * I]), wq[2])
        err = rel_fro(O.bf16_to_f32(got[start[e]:start[e] + n]), O.bf16_to_f32(ref))
        assert err <= 1e-3, f"expert {e}: relative Frobenius error {err:.2e}"
    state.close(); pre.close()
