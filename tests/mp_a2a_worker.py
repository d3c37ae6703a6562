"""Worker of the multi-GPU all-to-all test (one process per GPU, torchrun): every axis pair, checked element by element
against the definition in the reference kernel (all_to_all.cu:63-89) evaluated on the host from all ranks' inputs."""
import itertools
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def expected(inputs, rank, scatter, gather):
    """Output of `rank`: the rank-th part (along the scatter axis) of every rank's input, concatenated along the gather axis."""
    world = len(inputs)
    return torch.cat([torch.chunk(x, world, dim=scatter)[rank] for x in inputs], dim=gather)


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from thunderkittens_b200 import parallel, _lib
    shape = (2 * world, 3 * world, 4 * world, 8 * world)      # every axis divides by world; innermost part = 8 bf16 = 16 bytes
    ok = True
    for scatter, gather in itertools.permutations(range(4), 2):
        out_shape = list(shape); out_shape[scatter] //= world; out_shape[gather] *= world
        x = parallel.TKParallelTensor(shape, torch.bfloat16, local, world, False)
        y = parallel.TKParallelTensor(tuple(out_shape), torch.bfloat16, local, world, False)
        bar = parallel.TKParallelTensor((2 * world,), torch.int32, local, world, False)
        g = torch.Generator().manual_seed(1000 + 17 * scatter + gather)
        inputs = [torch.randn(shape, generator=g).to(torch.bfloat16) for _ in range(world)]     # the same on every rank
        x.data_.copy_(inputs[rank])
        dist.barrier()
        for it in range(2):
            parallel.tk_all_to_all(y, x, bar, scatter, gather)
            torch.cuda.synchronize()
            good = _lib.device_status() == 0 and torch.equal(y.data_.cpu(), expected(inputs, rank, scatter, gather))
            ok = ok and good
        dist.barrier()
        for t in (x, y, bar):
            t.close()
    print(f"rank {rank}: {'PASS' if ok else 'FAIL'}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
