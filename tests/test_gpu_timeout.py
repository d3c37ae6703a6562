"""A bounded device-side wait that runs out: the kernel gives up, the host reads TKB_ERR_TIMEOUT, the context stays usable.

The waits are made to run out the harmless way: a flag that nothing ever raises, with the wait limit lowered to about a
millisecond (tkb_set_wait_limit_cycles).  Nothing faults, traps or hangs; every kernel involved returns by itself.
The reference's waits are unbounded (include/ops/thread/util/sync.cuh:311-318)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle as O
from tests.util import randn_bf16, bf16_bits, to_dev_u8
from tests.test_gpu_gemm import _check

pytestmark = pytest.mark.gpu
SHORT = 2_000_000        # clock cycles: about a millisecond


def _gemm_still_right(cuda):
    import thunderkittens_b200.ops as ops
    M, N, K = 256, 256, 512
    aq = O.nvfp4_quantize(bf16_bits(randn_bf16((M, K), seed=1)), False, "spec")
    bq = O.nvfp4_quantize(bf16_bits(randn_bf16((N, K), seed=2, std=0.02)), False, "spec")
    D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
    ops.nvfp4_gemm(to_dev_u8(aq[0], cuda), to_dev_u8(aq[1], cuda), torch.from_numpy(aq[2]).to(cuda),
                   to_dev_u8(bq[0], cuda), to_dev_u8(bq[1], cuda), torch.from_numpy(bq[2]).to(cuda), D)
    torch.cuda.synchronize()
    _check(bf16_bits(D), O.nvfp4_gemm(*aq, *bq), "gemm after a timeout")


def test_wait_flags_runs_out_and_is_reported(cuda, lib):
    from thunderkittens_b200 import _lib
    flags = torch.zeros(4, dtype=torch.int32, device=cuda)
    assert _lib.device_status() == 0
    assert lib.tkb_set_wait_limit_cycles(SHORT) == 0
    try:
        assert lib.tkb_wait_flags(flags.data_ptr(), 4, -1, 1, torch.cuda.current_stream().cuda_stream) == 0      # nobody raises these flags
        torch.cuda.synchronize()
        assert _lib.device_status() == _lib.ERR_TIMEOUT
        assert _lib.device_status() == 0              # reading the status clears it
    finally:
        assert lib.tkb_set_wait_limit_cycles(0) == 0
    _gemm_still_right(cuda)


def test_gemm_kernel_gives_up_on_rows_that_never_arrive(cuda, lib):
    """The all-gather GEMM as rank 0 of a world of 2 whose peer never delivers its rows: the kernel multiplies its own rows,
    its producer then waits (about a millisecond) for the arrival flags of the peer's rows, gives up, lets its in-flight
    copies land, frees tensor memory and returns with TKB_ERR_TIMEOUT."""
    from thunderkittens_b200 import _lib
    M, N, K = 512, 256, 512
    u8 = torch.uint8
    codes = torch.zeros(M, K // 2, dtype=u8, device=cuda); scales = torch.zeros(M // 128, K // 64, 512, dtype=u8, device=cuda)
    arrived = torch.zeros(M // 64, dtype=torch.int32, device=cuda)
    sg = torch.ones(1, dtype=torch.float32, device=cuda)
    wc = torch.zeros(N, K // 2, dtype=u8, device=cuda); ws = torch.zeros(N // 128, K // 64, 512, dtype=u8, device=cuda)
    D = torch.zeros(M, N, dtype=torch.bfloat16, device=cuda)
    vp2 = ctypes.c_void_p * 2
    # both "ranks" point at this GPU's buffers; only the flags matter: nothing ever raises the ones of rank 1's rows
    pc, ps, pa = vp2(codes.data_ptr(), codes.data_ptr()), vp2(scales.data_ptr(), scales.data_ptr()), vp2(arrived.data_ptr(), arrived.data_ptr())
    assert _lib.device_status() == 0
    assert lib.tkb_set_wait_limit_cycles(SHORT) == 0
    try:
        rc = lib.tkb_ag_gemm_nvfp4(pc, ps, sg.data_ptr(), wc.data_ptr(), ws.data_ptr(), sg.data_ptr(), D.data_ptr(), 0, M, N, K, 0, 2, pa,
                                   None, None, 1, 0, torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.tkb_last_error()
        torch.cuda.synchronize()
        assert _lib.device_status() == _lib.ERR_TIMEOUT
    finally:
        assert lib.tkb_set_wait_limit_cycles(0) == 0
    _gemm_still_right(cuda)
    assert _lib.device_status() == 0
