"""Worker for the multi-GPU GEMM + reduce-scatter test (one process per GPU, launched by torchrun).
Every rank quantizes its own K-slice of X and W with the oracle, runs the fused kernel, and compares its output rows with
the fp32 sum over the ranks of the oracle's per-rank products.  The kernel accumulates the ranks' bf16 tiles in bf16 and in
no fixed order (as the reference's kernel does), so the gate is a relative Frobenius error of 1e-2, not bit equality."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle as O  # noqa: E402
from tests.util import bf16_bits, to_dev_u8, rel_fro  # noqa: E402


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from thunderkittens_b200 import parallel, _lib
    M, N, k_local = 512 * world, 384, 512
    rows = M // world
    op = parallel.GemmReduceScatterNVFP4(M, N, local, world)
    ok = True
    for it in range(3):
        rng = np.random.default_rng(50 + it)                 # the same stream on every rank: all K-slices of both operands
        X = torch.from_numpy(rng.standard_normal((M, k_local * world), dtype=np.float32)).to(torch.bfloat16)
        W = torch.from_numpy(rng.standard_normal((N, k_local * world), dtype=np.float32) * np.float32(0.05)).to(torch.bfloat16)
        parts, mine = [], None
        for r in range(world):
            xq = O.nvfp4_quantize(bf16_bits(X[:, r * k_local:(r + 1) * k_local].contiguous()), False, "spec")
            wq = O.nvfp4_quantize(bf16_bits(W[:, r * k_local:(r + 1) * k_local].contiguous()), False, "spec")
            parts.append(O.bf16_to_f32(O.nvfp4_gemm(*xq, *wq, row0=rank * rows, nrows=rows)))
            if r == rank:
                mine = (xq, wq)
        ref = np.sum(parts, axis=0, dtype=np.float32)
        xq, wq = mine
        out = op(to_dev_u8(xq[0], dev), to_dev_u8(xq[1], dev), torch.from_numpy(xq[2]).to(dev),
                 to_dev_u8(wq[0], dev), to_dev_u8(wq[1], dev), torch.from_numpy(wq[2]).to(dev))
        torch.cuda.synchronize()
        st = _lib.device_status()
        err = rel_fro(out.float().cpu().numpy(), ref)
        good = st == 0 and err <= 1e-2
        print(f"rank {rank} iter {it}: status={st} rel_fro={err:.2e}", flush=True)
        ok = ok and good
        dist.barrier()
    op.close()
    dist.destroy_process_group()
    print(f"rank {rank}: {'PASS' if ok else 'FAIL'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
