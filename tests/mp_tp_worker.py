"""Worker for the multi-GPU all-gather GEMM test (one process per GPU, launched by torchrun).
Writes "PASS" / "FAIL ..." per rank to stdout; exit code 0 only if the rank's checks passed.

Environment:
  TKB_TEST_TP_SIZE  "small" (default): M = 512 * world, K = 1024, N = 256 * world, whole result against the oracle;
                    "c4": the tensor-parallel benchmark problem M = 8192, N = 28672, K = 8192 with the benchmark's gather
                    settings; the gathered codes and scales are compared bit for bit with the oracle's quantize(full X)
                    and D on row slabs that touch the first and the last rows of EVERY source shard.
  TKB_TEST_TP_CE    "1": gather by copy engines instead of comm CTAs.
  TKB_TEST_TP_PUSH  "1": gather by two push warps in every CTA of the GEMM kernel.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import oracle as O  # noqa: E402
from tests.util import bf16_bits, to_dev_u8, rel_fro, bf16_ulp_diff  # noqa: E402


def normal_bf16(rng, shape, std=1.0):
    return torch.from_numpy(rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).to(torch.bfloat16)


def check_rows(got_bits, ref_bits):
    ref = O.bf16_to_f32(ref_bits)
    err = rel_fro(O.bf16_to_f32(got_bits), ref)
    big = np.abs(ref) > 1e-2 * np.abs(ref).mean()
    ulp = int(bf16_ulp_diff(got_bits, ref_bits)[big].max()) if big.any() else 0
    return err, ulp


def main():
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from thunderkittens_b200 import parallel, _lib
    size = os.environ.get("TKB_TEST_TP_SIZE", "small")
    ce = os.environ.get("TKB_TEST_TP_CE", "0") == "1"       # gather by copy engines instead of comm CTAs
    push = os.environ.get("TKB_TEST_TP_PUSH", "0") == "1"   # gather by push warps in every CTA
    if size == "c4":
        M, K, N, comm, iters, edge = 8192, 8192, 28672, (8 if world <= 2 else 20), 3, 8
    else:
        M, K, N, comm, iters, edge = 512 * world, 1024, 256 * world, 4, 6, 0
    n_local = N // world
    rows = M // world
    rng = np.random.default_rng(1234)                       # the activations: the same stream on every rank
    wq = O.nvfp4_quantize(bf16_bits(normal_bf16(np.random.default_rng(4321 + rank), (n_local, K), 0.02)))    # this rank's weight shard
    Wd, Wsc, Wsg = to_dev_u8(wq[0], dev), to_dev_u8(wq[1], dev), torch.from_numpy(wq[2]).to(dev)
    op = parallel.AllGatherMatmulNVFP4(M, K, local, world, num_comm_sms=comm, arithmetic="spec", copy_engines=ce, push_warps=push)
    ok = True
    for it in range(iters):      # several calls: both buffer sets, acknowledgements, growing epochs
        X = normal_bf16(rng, (M, K), 1.0 + it)
        D = torch.full((M, n_local), float("nan"), dtype=torch.bfloat16, device=dev)
        # both host paths on alternating calls: the single library call (epoch hand-shake inside the kernels) and
        # the spelled-out sequence (separate wait / signal launches)
        (op if (it % 2 == 0 or ce) else op.step_by_step)(X[rank * rows:(rank + 1) * rows].to(dev), Wd, Wsc, Wsg, D)
        torch.cuda.synchronize()
        st = _lib.device_status()
        xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")        # quantize(full X): what the shards must add up to
        b = (it + 1) % 2
        codes_ok = np.array_equal(op.codes[b].data_.cpu().numpy(), xq[0])
        scales_ok = np.array_equal(op.scales[b].data_.cpu().numpy(), xq[1])
        if edge == 0:
            err, ulp = check_rows(bf16_bits(D), O.nvfp4_gemm(*xq, *wq))
            nan_free = True
        else:
            # the first and the last `edge` rows of every source shard, all of this rank's columns
            err, ulp = 0.0, 0
            for s in range(world):
                for r0 in (s * rows, (s + 1) * rows - edge):
                    e1, u1 = check_rows(bf16_bits(D[r0:r0 + edge]), O.nvfp4_gemm(*xq, *wq, row0=r0, nrows=edge))
                    err, ulp = max(err, e1), max(ulp, u1)
            nan_free = not bool(torch.isnan(D).any().item())        # every tile of D was written
        good = st == 0 and err <= 1e-3 and ulp <= 2 and codes_ok and scales_ok and nan_free
        print(f"rank {rank} iter {it} [{size}, {'copy engines' if ce else ('push warps' if push else 'comm CTAs')}]: status={st} rel_fro={err:.2e} max_ulp={ulp} "
              f"gathered_codes_bit_exact={codes_ok} scales={scales_ok} all_written={nan_free}", flush=True)
        ok = ok and good
    if ce:
        # the same step recorded as a CUDA graph of two calls and replayed twice (device-side epochs, both buffer sets)
        Xs = [normal_bf16(rng, (M, K), 0.5 + j) for j in range(2)]
        Xl = [x[rank * rows:(rank + 1) * rows].to(dev) for x in Xs]
        Ds = [torch.full((M, n_local), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        graph = op.capture([(Xl[j], Wd, Wsc, Wsg, Ds[j]) for j in range(2)])
        for rep in range(2):
            for d_ in Ds:
                d_.fill_(float("nan"))
            op.replay(graph)
            torch.cuda.synchronize()
            st = _lib.device_status()
            good = st == 0
            for j in range(2):
                xq = O.nvfp4_quantize(bf16_bits(Xs[j]), False, "spec")
                if edge == 0:
                    err, ulp = check_rows(bf16_bits(Ds[j]), O.nvfp4_gemm(*xq, *wq))
                else:
                    err, ulp = 0.0, 0
                    for s_ in range(world):
                        r0 = s_ * rows + (rows - edge if (s_ + j) % 2 else 0)
                        e1, u1 = check_rows(bf16_bits(Ds[j][r0:r0 + edge]), O.nvfp4_gemm(*xq, *wq, row0=r0, nrows=edge))
                        err, ulp = max(err, e1), max(ulp, u1)
                good = good and err <= 1e-3 and ulp <= 2 and not bool(torch.isnan(Ds[j]).any().item())
            print(f"rank {rank} graph replay {rep} [{size}]: status={st} ok={good}", flush=True)
            ok = ok and good
    dist.barrier()
    op.close()
    dist.destroy_process_group()
    print(f"rank {rank}: {'PASS' if ok else 'FAIL'}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
