"""Worker for the multi-GPU MoE test (one process per GPU, launched by torchrun).

Environment:
  TKB_TEST_MOE_SIZE  "small" (default): T = 256 * world, H = 512, I = 256, 16 * world experts, top-4, every stage against the oracle;
                     "c5": the benchmark's layer (16384 tokens, hidden 7168, 128 experts, intermediate 2048, top-8): routing,
                     schedule and combine map bit-exact, the grouped GEMM on the first and last rows of every expert segment.
  TKB_TEST_MOE_COMM  CTAs of the GEMM kernel that pull rows (default 4, "c5": 32); 0 = the gather kernel on all SMs.
Combine is checked bit for bit at every world size: the oracle gets the gathered expert outputs of all ranks and adds in the
same order with the same fused multiply-adds.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import oracle as O
    from tests.moe_common import run_and_check
    from tests.util import bf16_bits
    size = os.environ.get("TKB_TEST_MOE_SIZE", "small")
    if size == "c5":
        T, H, I, E, k, iters, edge, comm = 16384, 7168, 2048, 128, 8, 2, 4, 32
    else:
        T, H, I, E, k, iters, edge, comm = 256 * world, 512, 256, 16 * world, 4, 3, 0, 4
    comm = int(os.environ.get("TKB_TEST_MOE_COMM", comm))
    ok, layer = run_and_check(dev, rank, world, T, H, I, E, k, iters=iters, comm_sms=comm, edge=edge)
    # combine across ranks, bit for bit: the oracle's weighted sum over the gathered expert outputs of every rank
    Tl = T // world
    ys = [torch.empty_like(layer.Y.data_) for _ in range(world)]
    dist.all_gather(ys, layer.Y.data_.contiguous())
    Yall = np.concatenate([bf16_bits(y) for y in ys], axis=0)
    cap = layer.Y.data_.shape[0]
    comb = layer.comb_idx.cpu().numpy().reshape(Tl, k, 2)
    slot = (comb[..., 0].astype(np.int64) * cap + comb[..., 1]).astype(np.int32)
    ref = O.moe_combine(Yall, slot, layer.weights.cpu().numpy())
    comb_ok = np.array_equal(bf16_bits(layer.out), ref)
    print(f"rank {rank} [{size}, comm {comm}]: combine bit-exact against the oracle over the gathered outputs: {comb_ok}", flush=True)
    ok = ok and comb_ok
    dist.barrier()
    layer.close()
    dist.destroy_process_group()
    print(f"rank {rank}: {'PASS' if ok else 'FAIL'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
