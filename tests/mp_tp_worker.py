"""Worker for the multi-GPU all-gather GEMM test (one process per GPU, launched by torchrun).
Writes "PASS" / "FAIL ..." per rank to stdout; exit code 0 only if the rank's checks passed."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle as O  # noqa: E402
from tests.util import bf16_bits, to_dev_u8, rel_fro, bf16_ulp_diff  # noqa: E402


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from thunderkittens_b200 import parallel, _lib
    M, K, N = 512 * world, 1024, 256 * world
    n_local = N // world
    rows = M // world
    g = torch.Generator().manual_seed(1234)
    W = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    wq = O.nvfp4_quantize(bf16_bits(W[rank * n_local:(rank + 1) * n_local]))
    Wd, Wsc, Wsg = to_dev_u8(wq[0], dev), to_dev_u8(wq[1], dev), torch.from_numpy(wq[2]).to(dev)
    ce = os.environ.get("TKB_TEST_TP_CE", "0") == "1"       # gather by copy engines instead of comm CTAs
    op = parallel.AllGatherMatmulNVFP4(M, K, local, world, num_comm_sms=4, arithmetic="spec", copy_engines=ce)
    ok = True
    for it in range(6):      # several calls: both buffer sets, acknowledgements, growing epochs
        X = (torch.randn(M, K, generator=g) * (1.0 + it)).to(torch.bfloat16)
        D = torch.full((M, n_local), float("nan"), dtype=torch.bfloat16, device=dev)
        # both host paths on alternating calls: the single library call (epoch hand-shake inside the kernels) and
        # the spelled-out sequence (separate wait / signal launches)
        (op if (it % 2 == 0 or ce) else op.step_by_step)(X[rank * rows:(rank + 1) * rows].to(dev), Wd, Wsc, Wsg, D)
        torch.cuda.synchronize()
        st = _lib.device_status()
        xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")        # quantize(full X): what the shards must add up to
        ref = O.nvfp4_gemm(*xq, *wq)
        got = bf16_bits(D)
        err = rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(ref))
        codes_ok = np.array_equal(op.codes[(it + 1) % 2].data_.cpu().numpy(), xq[0])
        scales_ok = np.array_equal(op.scales[(it + 1) % 2].data_.cpu().numpy(), xq[1])
        ulp = int(bf16_ulp_diff(got, ref)[np.abs(O.bf16_to_f32(ref)) > 1e-2 * np.abs(O.bf16_to_f32(ref)).mean()].max())
        good = st == 0 and err <= 1e-3 and ulp <= 2 and codes_ok and scales_ok
        print(f"rank {rank} iter {it}: status={st} rel_fro={err:.2e} max_ulp={ulp} gathered_codes_bit_exact={codes_ok} scales={scales_ok}", flush=True)
        ok = ok and good
    dist.barrier()
    op.close()
    dist.destroy_process_group()
    print(f"rank {rank}: {'PASS' if ok else 'FAIL'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
