"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of seeded synthetic input:

  N = 1   workload = MXFP8 GEMM M=N=K=8192 (bf16 ~N(0,1) with 1 % of entries x32, quantized to e4m3 with per-32
          UE8M0 scales, fp32 accumulate, bf16 out).  `value` = TFLOP/s of the GEMM with operands resident in HBM;
          `e2e` = the same FLOPs through the C-ABI calls a user makes, starting from bf16 matrices in pinned HOST
          memory: H2D copies, both quantize launches, the GEMM and the D2H copy of D are all inside the timed region.
  N > 1   workload = tensor-parallel NVFP4 GEMM M=8192 N=28672 K=8192 (weights N-sharded, activation rows sharded and
          all-gathered over NVLink inside the GEMM kernel), strong scaling; the line also carries the time of the same
          whole problem on one GPU.  `--workload moe` runs the expert-parallel MoE layer instead.
  `--case <kernel>` runs one kernel only (the commands of the ncu summaries under profiles/), `--workload tp_timeline`
  prints per-launch times and the kernels' wait counters of the tensor-parallel step.

`--impl reference` times the reference's CPU implementation of the same GEMM arithmetic — its own naive kernels from
kernels/gemm/common.cuh compiled for the host (oracle/_ref) when that build exists, otherwise the oracle's C++
restatement — on all host cores, on a bounded row slab of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 8192
FLOPS = 2.0 * M * N * K
NOMINAL = {"bf16": 2250.0, "fp8": 4500.0, "fp4": 9000.0, "hbm_gbs": 8000.0}


def measured_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks ------
class ClockSampler:
    """SM clock, power and throttle reasons through NVML (read-only), sampled DURING the timed region by the measuring
    thread itself: between the moment the timed loop has been enqueued and the moment its end event completes, while
    the GPU is still working through the queue.  Nothing is sampled while the host is launching: NVML queries take a
    driver lock that delays kernel launches (a background sampler at 0.5 ms made a two-launch step of the tensor-parallel
    loop about 100 us slower)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, nvml=None):
        self.index = index
        self.samples = []          # (sm_mhz, power_w, reasons_mask), all taken while the timed work was in flight
        self.idle_sample = None    # one sample after the region, used only if the region was too short to catch any
        self.max_mhz = None
        self._h = None
        try:
            if nvml is None:
                import pynvml as nvml
                nvml.nvmlInit()
            self._nv = nvml
            self._h = nvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(nvml.nvmlDeviceGetMaxClockInfo(self._h, nvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _read(self):
        nv = self._nv
        mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
        pw = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
        rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
            else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
        return (float(mhz), float(pw), int(rs))

    def poll_until(self, done, limit_s: float = 120.0) -> None:
        """Samples until done() is true (the end event of the timed loop has completed)."""
        if self._h is None:
            return
        t0 = time.time()
        try:
            while not done() and time.time() - t0 < limit_s:
                self.samples.append(self._read())
            self.idle_sample = self._read()
        except Exception:
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False

    def summary(self) -> dict:
        use = self.samples or ([self.idle_sample] if self.idle_sample else [])
        if not use:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mask = 0
        for _, _, r in use:
            mask |= r
        return {"sm_mhz": statistics.median(c for c, _, _ in use), "sm_min_mhz": min(c for c, _, _ in use), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(n for b, n in self.REASONS.items() if mask & b), "samples": len(self.samples),
                "power_w_max": max(p for _, p, _ in use),
                "when": "while the timed loop was executing on the GPU" if self.samples else "right after the timed loop (too short to sample)"}


# ----------------------------------------------------------------------------- CPU arm -----
def cpu_reference_gemm(steps: int, warmup: int, rows: int = 16):
    """Times the reference's CPU arithmetic for the N=1 workload on a `rows`-row slab (full N, full K)."""
    import numpy as np
    import oracle as O
    rng = np.random.default_rng(3)
    A = rng.standard_normal((rows, K)).astype(np.float32)
    A[rng.random((rows, K)) < 0.01] *= 32.0
    # B: 8192 x 8192 generated in blocks to keep peak memory modest
    B = rng.standard_normal((N, K)).astype(np.float32)
    B[rng.random((N, K)) < 0.01] *= 32.0
    ac, asc = O.mxfp8_quantize(O.f32_to_bf16(A))
    bc, bsc = O.mxfp8_quantize(O.f32_to_bf16(B))
    del A, B
    ref = O.ref_host()
    cores = O.num_threads()
    if ref is not None:
        kind = "reference"
        # the reference kernel indexes the scale tensor by row; give it a full 128-row block
        D = np.empty((rows, N), np.uint16)
        def run():
            ref.tkref_mxfp8_gemm(ac, asc.reshape(-1), bc, bsc.reshape(-1), D, rows, N, K)
    else:
        kind = "port"
        def run():
            O.mxfp8_gemm(ac, asc, bc, bsc, 0, rows)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    tflops = 2.0 * rows * N * K / dt * 1e-12
    return {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"{rows} of {M} output rows x full N={N} x full K={K} per step, {steps} steps ({dt:.2f} s/step)"}, dt


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, dt = cpu_reference_gemm(max(1, args.steps), max(0, min(args.warmup, 1)), rows=16)
    line = {"impl": "reference", "metric": "block-scaled GEMM throughput (MXFP8 8192^3)", "value": cb["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * (M / 16),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8 (e4m3 x ue8m0, fp32 acc)",
            "data": "synthetic", "config": {"workload": "MXFP8 GEMM M=N=K=8192, 1% x32 outliers", "timed": "CPU row slab"},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm -----
def synth(torch, dev, rows, cols, seed, std=1.0, outliers=0.0):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(rows, cols, generator=g, device=dev, dtype=torch.float32) * std
    if outliers > 0:
        mask = torch.rand(rows, cols, generator=g, device=dev) < outliers
        x = torch.where(mask, x * 32.0, x)
    return x.to(torch.bfloat16)


def event_time(torch, fn, steps, cooldown=0.5, sampler=None):
    """CUDA-event time per step on the current stream.  A 500 ms idle period precedes the timed loop, as in the
    reference's own protocol (kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:673-700), so the loop starts from the
    same thermal/power state every time."""
    s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    time.sleep(cooldown)
    s.record()
    for i in range(steps):
        fn(i)
    e.record()
    if sampler is not None:
        sampler.poll_until(e.query)       # clocks while the GPU works through the queue; the host launches are over
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e-3 / steps


def run_tp(args) -> None:
    """N > 1: tensor-parallel NVFP4 GEMM M=8192 N=28672 K=8192, weights column(N)-sharded, bf16 activation rows sharded
    and all-gathered (as NVFP4 codes + scales) over NVLink inside the GEMM kernel.  Strong scaling."""
    import torch
    import torch.distributed as dist
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib, parallel

    rank = int(os.environ.get("RANK", "0")); local_rank = int(os.environ.get("LOCAL_RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    Mt, Nt, Kt = 8192, 28672, 8192
    n_local, rows = Nt // world, Mt // world
    u8 = torch.uint8
    GROUPS = 3
    # comm CTAs: 20 at 4 and 8 GPUs leaves 64 CTA pairs, which divide the 896 / 448 output tiles of a rank into whole waves
    comm = args.comm_sms if args.comm_sms > 0 else (8 if world <= 2 else 20)
    op = parallel.AllGatherMatmulNVFP4(Mt, Kt, local_rank, world, num_comm_sms=comm, copy_engines=args.comm_sms < 0)   # --comm-sms -1: copy-engine gather
    sets = []
    amax_w = torch.zeros(1, dtype=torch.float32, device=dev)
    for gi in range(GROUPS):
        # weight shard: rows [rank*n_local, ...) of a seeded N(0, 0.02) matrix, quantized with the all-reduced amax
        W = synth(torch, dev, n_local, Kt, 800 + 10 * gi + rank, std=0.02)
        ops.absmax_bf16(W, amax_w)
        dist.all_reduce(amax_w, op=dist.ReduceOp.MAX)
        wc = torch.empty(n_local, Kt // 2, dtype=u8, device=dev); ws = torch.empty((n_local + 127) // 128, Kt // 64, 512, dtype=u8, device=dev)
        wg = torch.empty(1, dtype=torch.float32, device=dev)
        ops.nvfp4_quantize(W, wc, ws, wg, False, amax=amax_w)
        X = synth(torch, dev, rows, Kt, 700 + 10 * gi + rank)
        sets.append((X, wc, ws, wg, torch.empty(Mt, n_local, dtype=torch.bfloat16, device=dev)))
        del W
    hostX = sets[0][0].cpu().pin_memory()
    hostD = torch.empty(Mt, n_local, dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()

    def step(i):
        X, wc, ws, wg, D = sets[i % GROUPS]
        op(X, wc, ws, wg, D)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    cs = ClockSampler(local_rank)
    dt = event_time(torch, step, args.steps, sampler=cs)
    clocks = cs.summary()
    assert _lib.device_status() == 0, "a device-side wait timed out"
    t = torch.tensor([dt], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt = float(t.item())
    barrier()

    dX = torch.empty(rows, Kt, dtype=torch.bfloat16, device=dev)
    _, wc, ws, wg, D = sets[0]

    def e2e_step(i):
        dX.copy_(hostX, non_blocking=True)
        op(dX, wc, ws, wg, D)
        hostD.copy_(D, non_blocking=True)

    for i in range(2):
        e2e_step(i)
    barrier()
    dt_e2e = event_time(torch, e2e_step, max(3, min(args.steps, 10)))
    t = torch.tensor([dt_e2e], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt_e2e = float(t.item())
    barrier()
    # The same whole problem on ONE GPU (quantize of all 8192 activation rows + the full-N GEMM, no exchange), measured on
    # rank 0 while the other ranks idle: the T(1) of the strong-scaling curve.
    single = None
    if rank == 0 and not args.no_extra:
        del sets
        torch.cuda.empty_cache()
        Xf = synth(torch, dev, Mt, Kt, 700)
        Wf = synth(torch, dev, Nt, Kt, 800, std=0.02)
        wcf = torch.empty(Nt, Kt // 2, dtype=u8, device=dev); wsf = torch.empty(Nt // 128, Kt // 64, 512, dtype=u8, device=dev)
        wgf = torch.empty(1, dtype=torch.float32, device=dev)
        ops.nvfp4_quantize(Wf, wcf, wsf, wgf, False)
        del Wf
        xcf = torch.empty(Mt, Kt // 2, dtype=u8, device=dev); xsf = torch.empty(Mt // 128, Kt // 64, 512, dtype=u8, device=dev)
        xgf = torch.empty(1, dtype=torch.float32, device=dev)
        Df = [torch.empty(Mt, Nt, dtype=torch.bfloat16, device=dev) for _ in range(2)]

        def one_gpu(i):
            ops.nvfp4_quantize(Xf, xcf, xsf, xgf, False)
            ops.nvfp4_gemm(xcf, xsf, xgf, wcf, wsf, wgf, Df[i % 2])

        for i in range(3):
            one_gpu(i)
        t1 = event_time(torch, one_gpu, max(3, min(args.steps, 10)))
        single = {"ms_per_step": t1 * 1e3, "tflops": 2.0 * Mt * Nt * Kt / t1 * 1e-12,
                  "what": "tkb_nvfp4_quantize of the 8192 x 8192 activations + tkb_nvfp4_gemm with all 28672 weight rows on rank 0's GPU"}
        del Xf, wcf, wsf, xcf, xsf, Df
    barrier()
    if rank == 0:
        pk = measured_peaks()
        flops = 2.0 * Mt * Nt * Kt
        tf = flops / dt * 1e-12
        peak = 4.0 * pk["bf16_tflops"] * world
        nvl_bytes = (world - 1) / world * Mt * (Kt // 2 + Kt // 16)
        line = {
            "metric": "tensor-parallel NVFP4 GEMM throughput (M=8192 N=28672 K=8192)", "value": tf, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 x fp32, fp32 acc)", "data": "synthetic",
            "config": {"workload": "TP NVFP4 GEMM M=8192 N=28672 K=8192: weights N-sharded, bf16 activation rows sharded, per step two launches: "
                                   "quantize with the amax max-reduced over NVLink inside the kernel, then the NVFP4 all-gather over NVLink "
                                   "fused with the tcgen05 GEMM", "parallelism": f"tp{world}",
                       "l2": f"{GROUPS} rotating weight/activation/output sets", "comm_ctas": 0 if op.copy_engines else op.num_comm_sms,
                       "gather": "copy engines (peer cudaMemcpyAsync on a second stream)" if op.copy_engines else "comm CTAs of the GEMM kernel"},
            "roofline": {"bound": "tensor", "achieved": tf / world, "peak": 4.0 * pk["bf16_tflops"], "unit": "TFLOP/s per GPU",
                         "frac": tf / peak, "traffic": None, "kernel": "tkb::gemm_kernel<NVFP4, cta pair, N256, all-gather>",
                         "peak_source": f"4 x {pk['source']} cuBLAS bf16 burst (derived dense FP4 ceiling)",
                         "nvlink_bytes_in_per_gpu": nvl_bytes, "nvlink_time_at_770GBs_ms": nvl_bytes / 770e9 * 1e3},
            "e2e": {"value": flops / dt_e2e * 1e-12, "unit": "TFLOP/s", "h2d_bytes_per_step": rows * Kt * 2 * world,
                    "d2h_bytes_per_step": Mt * n_local * 2 * world, "ms_per_step": dt_e2e * 1e3,
                    "path": "pinned host bf16 shard -> H2D -> AllGatherMatmulNVFP4 -> D2H of the rank's output columns"},
            "gpu_launches": args.steps * 2 * world, "clocks": clocks, "single_gpu_same_problem": single,
            "scaling_note": "strong scaling of ONE problem: the 1-GPU time of this problem is single_gpu_same_problem.ms_per_step; the N=1 line of "
                            "this benchmark is a different workload (MXFP8 GEMM 8192^3, BASELINE configs[1]) and not the T(1) of this curve",
        }
        print(json.dumps(line), flush=True)
    op.close()
    dist.destroy_process_group()


def run_moe(args) -> None:
    """MoE layer (BASELINE configs[4]): 16384 tokens, hidden 7168, 128 experts, intermediate 2048, top-8 routing from a
    softmax over seeded N(0,1) logits, NVFP4 expert weights ~N(0,0.02), experts and tokens sharded over the ranks.
    A step = route -> schedule -> quantize -> dispatch fused with the grouped GEMM -> combine."""
    import torch
    import torch.distributed as dist
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib, parallel

    rank = int(os.environ.get("RANK", "0")); local_rank = int(os.environ.get("LOCAL_RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    T, H, I, E, k = 16384, 7168, 2048, 128, 8
    Tl, El = T // world, E // world
    u8 = torch.uint8
    layer = parallel.MoELayerNVFP4(T, H, I, E, k, local_rank, world, num_comm_sms=args.comm_sms if args.comm_sms > 0 else 32)
    amax_w = torch.zeros(1, dtype=torch.float32, device=dev)
    wc = torch.empty(El * I, H // 2, dtype=u8, device=dev); ws = torch.empty(El * I // 128, H // 64, 512, dtype=u8, device=dev)
    wg = torch.empty(1, dtype=torch.float32, device=dev)
    for e in range(El):       # expert by expert to keep the bf16 staging small
        W = synth(torch, dev, I, H, 1100 + rank * El + e, std=0.02)
        ops.absmax_bf16(W, amax_w)     # per-expert amax is fine for a benchmark; one common scale is used below
        if e == 0:
            common = amax_w.clone()
        else:
            common = torch.maximum(common, amax_w)
        del W
    if world > 1:
        dist.all_reduce(common, op=dist.ReduceOp.MAX)
    for e in range(El):
        W = synth(torch, dev, I, H, 1100 + rank * El + e, std=0.02)
        sg_tmp = torch.empty(1, dtype=torch.float32, device=dev)
        ops.nvfp4_quantize(W, wc[e * I:(e + 1) * I], ws[e * I // 128:(e + 1) * I // 128], wg, False, amax=common)
        del W
    sets = [(synth(torch, dev, Tl, E, 900 + 10 * gi + rank).float(), synth(torch, dev, Tl, H, 1000 + 10 * gi + rank)) for gi in range(3)]
    torch.cuda.synchronize()

    def step(i):
        lg, X = sets[i % 3]
        layer.forward(lg, X, wc, ws, wg)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    dt = event_time(torch, step, args.steps)
    st = _lib.device_status()
    if world > 1:
        t = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    rows = int(layer.num_blocks.item()) * 128
    if rank == 0:
        flops = 2.0 * T * k * H * I
        print(json.dumps({"metric": "MoE layer throughput (16384 tokens, H 7168, 128 experts, I 2048, top-8, NVFP4)", "value": flops / dt * 1e-12,
                          "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "ms_per_step": dt * 1e3, "scaling": "strong",
                          "device_status": st, "rank0_padded_rows": rows, "comm_ctas": layer.num_comm_sms,
                          "dispatch_bytes_in_per_gpu": (world - 1) / world * T * k / world * (H // 2 + H // 16),
                          "combine_bytes_in_per_gpu": (world - 1) / world * Tl * k * I * 2,
                          "config": {"workload": "MoE layer", "parallelism": f"ep{world}"}}), flush=True)
    barrier()
    layer.close()
    if world > 1:
        dist.destroy_process_group()


def run_tp_timeline(args) -> None:
    """Diagnostic for the tensor-parallel step (N > 1, torchrun): CUDA events around each of the two launches of a step
    inside a free-running loop, plus the kernels' own wait counters (tkb_gemm_set_profile_buffer) for the last step of
    the loop.  Prints one JSON line from rank 0 and one from rank world/2.  Not a benchmark line."""
    import ctypes
    import numpy as np
    import torch
    import torch.distributed as dist
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib as L, parallel

    rank = int(os.environ.get("RANK", "0")); local = int(os.environ.get("LOCAL_RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    Mt, Nt, Kt = 8192, 28672, 8192
    nl, rows = Nt // world, Mt // world
    lib, s = L.lib(), torch.cuda.current_stream().cuda_stream
    comm = args.comm_sms if args.comm_sms > 0 else (8 if world <= 2 else 20)
    op = parallel.AllGatherMatmulNVFP4(Mt, Kt, local, world, num_comm_sms=comm)
    X = synth(torch, dev, rows, Kt, 700 + rank)
    W = synth(torch, dev, nl, Kt, 800 + rank, std=0.02)
    u8 = torch.uint8
    wc = torch.empty(nl, Kt // 2, dtype=u8, device=dev); ws = torch.empty((nl + 127) // 128, Kt // 64, 512, dtype=u8, device=dev)
    wg = torch.empty(1, dtype=torch.float32, device=dev)
    ops.nvfp4_quantize(W, wc, ws, wg, False)
    D = torch.empty(Mt, nl, dtype=torch.bfloat16, device=dev)
    arith = ops._ARITH[ops.default_nvfp4_arithmetic]

    def two(ev=None):       # the two launches of tkb_ag_linear_nvfp4, issued one by one so that an event fits in between
        op.epoch += 1
        e, b = op.epoch, op.epoch % 2
        codes, scales = op.codes[b], op.scales[b]
        mc = codes.data_[rank * rows:(rank + 1) * rows]; ms = scales.data_[rank * rows // 128:(rank + 1) * rows // 128]
        if ev:
            ev[0].record()
        L.check(lib.tkb_nvfp4_quantize_sharded(X.data_ptr(), 0, mc.data_ptr(), ms.data_ptr(), op.sg.data_ptr(), rows, Kt, 0, arith,
                                               op.slots[b].peer_ptr_array(), world, rank, e, s))
        if ev:
            ev[1].record()
        L.check(lib.tkb_ag_gemm_nvfp4(codes.peer_ptr_array(), scales.peer_ptr_array(), op.sg.data_ptr(), wc.data_ptr(), ws.data_ptr(), wg.data_ptr(),
                                      D.data_ptr(), 0, Mt, nl, Kt, rank, world, op.arrived[b].peer_ptr_array(), op.flags.peer_ptr_array(),
                                      op.exit_counter.data_ptr(), e, op.num_comm_sms, s))
        if ev:
            ev[2].record()

    for _ in range(max(args.warmup, 3)):
        two()
    torch.cuda.synchronize(); dist.barrier()
    prof = torch.zeros(148 * 8, dtype=torch.int64, device=dev)
    setp = L.bind("tkb_gemm_set_profile_buffer", [ctypes.c_void_p])
    setp(prof.data_ptr())
    steps = max(args.steps, 4)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    for i in range(steps):
        two(evs[i])
    torch.cuda.synchronize()
    setp(None)
    q = np.array([evs[i][0].elapsed_time(evs[i][1]) for i in range(steps)]) * 1e3
    g = np.array([evs[i][1].elapsed_time(evs[i][2]) for i in range(steps)]) * 1e3
    pr = prof.cpu().numpy().reshape(148, 8)
    lead = pr[op.num_comm_sms::2]
    lead = lead[lead[:, 4] > 0]
    if len(lead) == 0:
        lead = np.zeros((1, 8), np.int64)
    med = lambda a: float(np.median(a))
    out = {"rank": rank, "n_gpus": world, "comm_ctas": op.num_comm_sms, "step_us": evs[0][0].elapsed_time(evs[-1][2]) * 1e3 / steps,
           "quantize_us_median_max": [med(q), float(q.max())], "ag_gemm_us_median_max": [med(g), float(g.max())],
           "cycles_of_last_step": {"mma_total": med(lead[:, 4]), "mma_waiting_for_operands": med(lead[:, 3]), "mma_waiting_for_drain": med(lead[:, 2]),
                                   "producer_waiting_for_remote_rows": med(lead[:, 7]), "comm_cta_total": med(pr[:op.num_comm_sms, 0]),
                                   "comm_cta_waiting_done_flags": med(pr[:op.num_comm_sms, 1]), "comm_cta_fence_and_flag": med(pr[:op.num_comm_sms, 2])},
           "device_status": L.device_status()}
    # The exchange alone: the same two launches with only 256 weight rows, so that the multiplying CTAs have next to
    # nothing to do and the fused kernel lasts as long as the pushes (bytes in per GPU: (world-1)/world * M * K * 0.5625).
    n_small = 256
    Ds = torch.empty(Mt, n_small, dtype=torch.bfloat16, device=dev)

    def push_only(ev):
        op.epoch += 1
        e, b = op.epoch, op.epoch % 2
        codes, scales = op.codes[b], op.scales[b]
        mc = codes.data_[rank * rows:(rank + 1) * rows]; ms = scales.data_[rank * rows // 128:(rank + 1) * rows // 128]
        L.check(lib.tkb_nvfp4_quantize_sharded(X.data_ptr(), 0, mc.data_ptr(), ms.data_ptr(), op.sg.data_ptr(), rows, Kt, 0, arith,
                                               op.slots[b].peer_ptr_array(), world, rank, e, s))
        ev[0].record()
        L.check(lib.tkb_ag_gemm_nvfp4(codes.peer_ptr_array(), scales.peer_ptr_array(), op.sg.data_ptr(), wc.data_ptr(), ws.data_ptr(), wg.data_ptr(),
                                      Ds.data_ptr(), 0, Mt, n_small, Kt, rank, world, op.arrived[b].peer_ptr_array(), op.flags.peer_ptr_array(),
                                      op.exit_counter.data_ptr(), e, op.num_comm_sms, s))
        ev[1].record()

    dist.barrier()
    pe = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(6)]
    for i in range(6):
        push_only(pe[i])
    torch.cuda.synchronize()
    pt = np.array([pe[i][0].elapsed_time(pe[i][1]) for i in range(2, 6)]) * 1e3
    bytes_in = (world - 1) / world * Mt * (Kt // 2 + Kt // 16)
    out["exchange_alone_us_median"] = med(pt)
    out["exchange_alone_gbs_in_per_gpu"] = bytes_in / (med(pt) * 1e-6) * 1e-9
    out["device_status"] = L.device_status()
    if rank in (0, world // 2):
        print(json.dumps(out), flush=True)
    dist.barrier()
    op.close()
    dist.destroy_process_group()


def run_ours(args) -> None:
    if args.workload == "moe":
        return run_moe(args)
    if args.workload == "tp_timeline":
        return run_tp_timeline(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return run_tp(args)
    import torch
    import torch.distributed as dist
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()   # fail loudly if the CUDA library is missing

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    u8 = torch.uint8
    GROUPS = 3   # rotating operand sets: 3 x (64 + 64 + 128 MiB) so every launch starts with a cold L2
    groups = []
    for gi in range(GROUPS):
        A = synth(torch, dev, M, K, 3 + 10 * gi + 100 * rank, outliers=0.01)
        B = synth(torch, dev, N, K, 4 + 10 * gi + 100 * rank, outliers=0.01)
        a = torch.empty(M, K, dtype=u8, device=dev); asc = torch.empty(M // 128, K // 128, 512, dtype=u8, device=dev)
        b = torch.empty(N, K, dtype=u8, device=dev); bsc = torch.empty(N // 128, K // 128, 512, dtype=u8, device=dev)
        ops.mxfp8_quantize(A, a, asc); ops.mxfp8_quantize(B, b, bsc)
        groups.append((a, asc, b, bsc, torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
        if gi == 0:
            hostA = A.cpu().pin_memory(); hostB = B.cpu().pin_memory()
        del A, B
    torch.cuda.synchronize()

    def step(i):
        ops.mxfp8_gemm(*groups[i % GROUPS])

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()
    cs = ClockSampler(local_rank)
    dt = event_time(torch, step, args.steps, sampler=cs)
    clocks = cs.summary()
    assert _lib.device_status() == 0, "a device-side wait timed out"
    if world > 1:
        t = torch.tensor([dt], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    barrier()

    # end to end: bf16 in pinned host memory -> H2D -> quantize x2 -> GEMM -> D2H
    dA = torch.empty(M, K, dtype=torch.bfloat16, device=dev); dB = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
    hostD = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    a, asc, b, bsc, D = groups[0]

    def e2e_step(i):
        dA.copy_(hostA, non_blocking=True); dB.copy_(hostB, non_blocking=True)
        ops.mxfp8_quantize(dA, a, asc); ops.mxfp8_quantize(dB, b, bsc)
        ops.mxfp8_gemm(a, asc, b, bsc, D)
        hostD.copy_(D, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    for i in range(2):
        e2e_step(i)
    barrier()
    dt_e2e = event_time(torch, e2e_step, e2e_steps)
    if world > 1:
        t = torch.tensor([dt_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt_e2e = float(t.item())

    # The same step as a user would stream it: copies on their own streams and two buffer sets, so the H2D copy of step
    # i+1 and the D2H copy of step i-1 overlap step i's kernels.  Every step still moves all of its bytes inside the
    # timed region.  The number is used only if the pipeline ran and its last results equal the device buffers.
    dt_e2e_serial, e2e_mode = dt_e2e, "serial: H2D, kernels and D2H of a step one after the other on one stream"
    if world == 1:
        try:
            main = torch.cuda.current_stream()
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            sets = [(dA, dB, groups[0], hostD), (torch.empty_like(dA), torch.empty_like(dB), groups[1], torch.empty_like(hostD).pin_memory())]
            ev_in = [torch.cuda.Event() for _ in range(2)]; ev_done = [torch.cuda.Event() for _ in range(2)]; ev_out = [torch.cuda.Event() for _ in range(2)]

            def piped_step(i):
                k = i % 2
                dAk, dBk, (a_, asc_, b_, bsc_, D_), hostDk = sets[k]
                s_in.wait_event(ev_done[k])              # the kernels of step i-2 have consumed this set's inputs
                with torch.cuda.stream(s_in):
                    dAk.copy_(hostA, non_blocking=True); dBk.copy_(hostB, non_blocking=True)
                    ev_in[k].record(s_in)
                main.wait_event(ev_in[k])
                main.wait_event(ev_out[k])               # this set's D has been copied out by step i-2
                ops.mxfp8_quantize(dAk, a_, asc_); ops.mxfp8_quantize(dBk, b_, bsc_)
                ops.mxfp8_gemm(a_, asc_, b_, bsc_, D_)
                ev_done[k].record(main)
                s_out.wait_event(ev_done[k])
                with torch.cuda.stream(s_out):
                    hostDk.copy_(D_, non_blocking=True)
                    ev_out[k].record(s_out)

            def piped_loop(steps):
                s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                time.sleep(0.5)
                s.record(main)
                for i in range(steps):
                    piped_step(i)
                main.wait_stream(s_in); main.wait_stream(s_out)      # the last D2H copies are inside the timed region
                e.record(main)
                torch.cuda.synchronize()
                return s.elapsed_time(e) * 1e-3 / steps

            piped_loop(2)
            dt_piped = piped_loop(e2e_steps)
            same = all(torch.equal(sets[k][3], sets[k][2][4].cpu()) for k in range(2))
            if same and 0.0 < dt_piped < dt_e2e_serial:
                dt_e2e = dt_piped
                e2e_mode = "pipelined: copies on their own streams, two buffer sets (H2D of step i+1 and D2H of step i-1 overlap step i's kernels)"
            del sets
        except Exception as ex:      # keep the serial number
            e2e_mode += f" (pipelined variant failed: {repr(ex)[:120]})"
        torch.cuda.synchronize()

    extras = {}
    if rank == 0 and not args.no_extra:
        extras = side_measurements(torch, ops, dev)
        if world == 1:
            torch.cuda.synchronize()
            extras["reference_gpu_kernels_8192"] = reference_gpu_kernels()

    if rank == 0:
        pk = measured_peaks()
        tflops = FLOPS / dt * 1e-12
        peak = 2.0 * pk["bf16_tflops"]
        line = {
            "metric": "block-scaled GEMM throughput (MXFP8 8192^3)", "value": tflops * world, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "mxfp8 (e4m3 x ue8m0, fp32 acc)", "data": "synthetic",
            "config": {"workload": "MXFP8 GEMM M=N=K=8192, bf16~N(0,1) with 1% x32 outliers, per-32 UE8M0 scales, bf16 out",
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas (no collective)",
                       "l2": f"{GROUPS} rotating operand sets of 256 MiB (> 126 MB L2)"},
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                         "traffic": MXFP8_GEMM_DRAM_BYTES, "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum, profiles/mxfp8_gemm_ncu.md)",
                         "algorithmic_bytes": 2 * M * K + 2 * (M // 128) * (K // 128) * 512 + M * N * 2,
                         "kernel": "tkb::gemm_kernel<MXFP8, cta pair, N256>",
                         "peak_source": f"2 x {pk['source']} cuBLAS bf16 burst {pk['bf16_tflops']} TFLOP/s (derived dense FP8 ceiling)",
                         "frac_of_nominal_4500": tflops / NOMINAL["fp8"]},
            "e2e": {"value": FLOPS / dt_e2e * 1e-12 * world, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * M * K * 2,
                    "d2h_bytes_per_step": M * N * 2, "ms_per_step": dt_e2e * 1e3, "serial_ms_per_step": dt_e2e_serial * 1e3, "mode": e2e_mode,
                    "path": "pinned host bf16 -> H2D -> tkb_mxfp8_quantize x2 -> tkb_mxfp8_gemm -> D2H"},
            "gpu_launches": args.steps, "clocks": clocks, "extra": extras,
        }
        if world == 1 and not args.no_extra:
            cb, _ = cpu_reference_gemm(3, 1, rows=16)
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the 8192^3 MXFP8 GEMM (ncu capture summarised in
# profiles/mxfp8_gemm_ncu.md): 348.0 MB read + 116.8 MB written.
MXFP8_GEMM_DRAM_BYTES = 464.8e6


# The reference's own GPU kernels (built from its tree into oracle/_ref/tk_<which> by oracle/build.py:build_ref_gpu) timed with
# the same protocol as this library's (CUDA events, 3 rotating operand sets, 500 ms idle first).  Runs in a child process: the
# reference's modules are both called `_C`.  Single-GPU only: the reference's kernel objects do not travel to multi-GPU runs.
REF_GPU_CHILD = r"""
import sys, os, json, glob, time, importlib.util
ROOT, which = sys.argv[1], sys.argv[2]
import torch
so = glob.glob(os.path.join(ROOT, "oracle", "_ref", f"tk_{which}", "_C*.so"))[0]
spec = importlib.util.spec_from_file_location("_C", so); ref = importlib.util.module_from_spec(spec); spec.loader.exec_module(ref)
dev = torch.device("cuda:0"); u8 = torch.uint8
M = N = K = 8192
def timed(fn, steps=10):
    for i in range(3): fn(i)
    s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(); time.sleep(0.5)
    s.record()
    for i in range(steps): fn(i)
    e.record(); torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / steps
sets = []
for gi in range(3):
    g = torch.Generator(device=dev).manual_seed(21 + gi)
    A = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
    B = (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    if which == "nvfp4":
        def q(X):
            c = torch.empty(X.shape[0], K // 2, dtype=torch.float4_e2m1fn_x2, device=dev); sc = torch.empty(X.shape[0] // 128, K // 64, 512, dtype=torch.float8_e4m3fn, device=dev)
            gg = torch.empty(1, device=dev); ref.nvfp4_quantize(X, c, sc, gg, False); return c, sc, gg
    else:
        def q(X):
            c = torch.empty(X.shape[0], K, dtype=torch.float8_e4m3fn, device=dev); sc = torch.empty(X.shape[0] // 128, K // 128, 32, 16, dtype=u8, device=dev)
            ref.mxfp8_quantize(X, c, sc); return c, sc
    sets.append((A, q(A), q(B), torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
    del B
torch.cuda.synchronize()
out = {}
if which == "nvfp4":
    out["gemm_us"] = timed(lambda i: ref.nvfp4_gemm(*sets[i % 3][1], *sets[i % 3][2], sets[i % 3][3]))
    out["quantize_us"] = timed(lambda i: ref.nvfp4_quantize(sets[i % 3][0], *sets[i % 3][1], False))
else:
    out["gemm_us"] = timed(lambda i: ref.mxfp8_gemm(*sets[i % 3][1], *sets[i % 3][2], sets[i % 3][3]))
    out["quantize_us"] = timed(lambda i: ref.mxfp8_quantize(sets[i % 3][0], *sets[i % 3][1]))
out["gemm_tflops"] = 2.0 * M * N * K / out["gemm_us"] * 1e-6
print("RESULT " + json.dumps(out))
"""


def reference_gpu_kernels() -> dict:
    """8192^3 GEMM and 8192 x 8192 quantize times of the reference's own sm_100a kernels, when they were built."""
    import glob
    import subprocess
    out = {}
    for which in ("nvfp4", "mxfp8"):
        if not glob.glob(os.path.join(ROOT, "oracle", "_ref", f"tk_{which}", "_C*.so")):
            out[which] = {"unavailable": "reference GPU kernels not built (oracle/build.py:build_ref_gpu needs the reference tree)"}
            continue
        try:
            r = subprocess.run([sys.executable, "-c", REF_GPU_CHILD, ROOT, which], capture_output=True, text=True, timeout=150)
            lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
            out[which] = json.loads(lines[-1][7:]) if r.returncode == 0 and lines else {"unavailable": (r.stderr or "no output")[-300:]}
        except Exception as e:      # a comparison aid: never fails the benchmark line
            out[which] = {"unavailable": repr(e)[:300]}
    return out


def side_measurements(torch, ops, dev) -> dict:
    """Other single-GPU rows of the path, timed the same way (CUDA events, rotating buffers)."""
    out = {}
    u8 = torch.uint8
    pk = measured_peaks()

    def quant4(X):
        r, k = X.shape
        c = torch.empty(r, k // 2, dtype=u8, device=dev); s = torch.empty((r + 127) // 128, k // 64, 512, dtype=u8, device=dev)
        g = torch.empty(1, dtype=torch.float32, device=dev)
        ops.nvfp4_quantize(X, c, s, g, False)
        return c, s, g

    try:
        gs = []
        for gi in range(3):
            A = synth(torch, dev, M, K, 21 + gi); B = synth(torch, dev, N, K, 31 + gi, std=0.02)
            gs.append((*quant4(A), *quant4(B), torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
            del A, B
        f = lambda i: ops.nvfp4_gemm(*gs[i % 3])
        for i in range(3):
            f(i)
        t = event_time(torch, f, 10)
        tf = FLOPS / t * 1e-12
        out["nvfp4_gemm_8192"] = {"tflops": tf, "us": t * 1e6, "frac_of_4x_measured_bf16": tf / (4 * pk["bf16_tflops"]),
                                  "frac_of_nominal_9000": tf / NOMINAL["fp4"]}
        del gs
        torch.cuda.empty_cache()
        gs = [(synth(torch, dev, M, K, 41 + gi), synth(torch, dev, N, K, 51 + gi), torch.empty(M, N, dtype=torch.bfloat16, device=dev)) for gi in range(3)]
        f = lambda i: ops.bf16_gemm(*gs[i % 3])
        for i in range(3):
            f(i)
        t = event_time(torch, f, 10)
        tf = FLOPS / t * 1e-12
        out["bf16_gemm_8192"] = {"tflops": tf, "us": t * 1e6, "frac_of_measured_bf16": tf / pk["bf16_tflops"]}
        # quantize kernels (HBM-bound)
        qs = [(g[0], torch.empty(M, K // 2, dtype=u8, device=dev), torch.empty(M // 128, K // 64, 512, dtype=u8, device=dev),
               torch.empty(1, dtype=torch.float32, device=dev)) for g in gs]
        f = lambda i: ops.nvfp4_quantize(*qs[i % 3], False)
        for i in range(3):
            f(i)
        t = event_time(torch, f, 10)
        out["nvfp4_quantize_8192x8192"] = {"us": t * 1e6, "gbs_two_pass_bytes": M * K * (2 + 2 + 0.5 + 1 / 16) / t * 1e-9,
                                           "gbs_one_pass_bytes": M * K * (2 + 0.5 + 1 / 16) / t * 1e-9}
        q8 = [(g[0], torch.empty(M, K, dtype=u8, device=dev), torch.empty(M // 128, K // 128, 512, dtype=u8, device=dev)) for g in gs]
        f = lambda i: ops.mxfp8_quantize(*q8[i % 3])
        for i in range(3):
            f(i)
        t = event_time(torch, f, 10)
        gbs = M * K * (2 + 1 + 1 / 32) / t * 1e-9
        out["mxfp8_quantize_8192x8192"] = {"us": t * 1e6, "gbs": gbs, "frac_of_measured_hbm": gbs / pk["hbm_gbs"]}
        del gs, qs, q8
        torch.cuda.empty_cache()
        # decode: activations quantized on the fly + skinny-M NVFP4 GEMM, weights N=28672 K=8192 (3 rotating copies)
        Nw, Kw = 28672, 8192
        ws = []
        for gi in range(3):
            W = synth(torch, dev, Nw, Kw, 61 + gi, std=0.02)
            ws.append(quant4(W))
            del W
        for Md in (1, 16, 128):
            X = synth(torch, dev, Md, Kw, 71 + Md)
            xc = torch.empty(Md, Kw // 2, dtype=u8, device=dev); xs = torch.empty(1, Kw // 64, 512, dtype=u8, device=dev)
            xg = torch.empty(1, dtype=torch.float32, device=dev)
            Dd = torch.empty(Md, Nw, dtype=torch.bfloat16, device=dev)
            def f(i):
                ops.nvfp4_quantize(X, xc, xs, xg, False)
                ops.nvfp4_gemm(xc, xs, xg, *ws[i % 3], Dd)
            for i in range(3):
                f(i)
            t = event_time(torch, f, 20)
            # the two launches take ~20 us of GPU time, less than it costs Python to enqueue them: replay them from a CUDA
            # graph (3 steps, one per weight copy) so that the GPU, not the host, is what is timed
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(3):
                    f(i)
            graph.replay()
            tg = event_time(torch, lambda i: graph.replay(), 10) / 3
            algo = Nw * Kw // 2 + Nw * Kw // 16 + 8 + Md * Kw * 2 + Md * Nw * 2
            out[f"decode_nvfp4_M{Md}"] = {"us": tg * 1e6, "us_eager_python": t * 1e6, "algorithmic_bytes": algo, "gbs": algo / tg * 1e-9,
                                          "frac_of_measured_hbm": algo / tg * 1e-9 / pk["hbm_gbs"],
                                          "frac_of_nominal_8000": algo / tg * 1e-9 / NOMINAL["hbm_gbs"],
                                          "launches_per_step": 2, "timed": "CUDA graph replay of 3 x (quantize + GEMM), cold weights"}
            del graph
    except Exception as e:   # side measurements never invalidate the headline line
        out["error"] = repr(e)
    return out


def run_case(args) -> None:
    """One kernel of the path, a few launches, nothing else: the command line used for ncu captures
    (python bench.py --case nvfp4_gemm --size 8192 --steps 3)."""
    import torch
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    u8 = torch.uint8
    m, n, k = args.size if args.m is None else args.m, args.size, args.size if args.k is None else args.k
    A = synth(torch, dev, m, k, 1, outliers=0.01 if "mxfp8" in args.case else 0.0)
    B = synth(torch, dev, n, k, 2, std=1.0 if "mxfp8" in args.case or "bf16" in args.case else 0.02)
    D = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    if args.case == "nvfp4_gemm" or args.case == "nvfp4_quantize":
        a = torch.empty(m, k // 2, dtype=u8, device=dev); asc = torch.empty((m + 127) // 128, k // 64, 512, dtype=u8, device=dev); ag = torch.empty(1, device=dev)
        b = torch.empty(n, k // 2, dtype=u8, device=dev); bsc = torch.empty((n + 127) // 128, k // 64, 512, dtype=u8, device=dev); bg = torch.empty(1, device=dev)
        ops.nvfp4_quantize(A, a, asc, ag, False); ops.nvfp4_quantize(B, b, bsc, bg, False)
        fn = (lambda: ops.nvfp4_gemm(a, asc, ag, b, bsc, bg, D, args.config)) if args.case == "nvfp4_gemm" else (lambda: ops.nvfp4_quantize(A, a, asc, ag, False))
    elif args.case == "mxfp8_gemm" or args.case == "mxfp8_quantize":
        a = torch.empty(m, k, dtype=u8, device=dev); asc = torch.empty((m + 127) // 128, k // 128, 512, dtype=u8, device=dev)
        b = torch.empty(n, k, dtype=u8, device=dev); bsc = torch.empty((n + 127) // 128, k // 128, 512, dtype=u8, device=dev)
        ops.mxfp8_quantize(A, a, asc); ops.mxfp8_quantize(B, b, bsc)
        fn = (lambda: ops.mxfp8_gemm(a, asc, b, bsc, D, args.config)) if args.case == "mxfp8_gemm" else (lambda: ops.mxfp8_quantize(A, a, asc))
    elif args.case == "decode":
        # skinny-M NVFP4 GEMM: activations (m rows) against weights [n, k]
        wc = torch.empty(n, k // 2, dtype=u8, device=dev); wsc = torch.empty((n + 127) // 128, k // 64, 512, dtype=u8, device=dev); wg = torch.empty(1, device=dev)
        ops.nvfp4_quantize(B, wc, wsc, wg, False)
        xc = torch.empty(m, k // 2, dtype=u8, device=dev); xs = torch.empty(1, k // 64, 512, dtype=u8, device=dev); xg = torch.empty(1, device=dev)
        ops.nvfp4_quantize(A, xc, xs, xg, False)
        fn = lambda: ops.nvfp4_gemm(xc, xs, xg, wc, wsc, wg, D)
    elif args.case == "bf16_gemm":
        fn = lambda: ops.bf16_gemm(A, B, D, args.config)
    else:
        raise SystemExit(f"unknown case {args.case}")
    for _ in range(max(args.warmup, 0)):
        fn()
    t = event_time(torch, lambda i: fn(), args.steps, cooldown=0.0)
    assert _lib.device_status() == 0
    print(json.dumps({"case": args.case, "m": m, "n": n, "k": k, "us": t * 1e6, "tflops": 2.0 * m * n * k / t * 1e-12}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, help="run a single kernel only (for profiling): nvfp4_gemm, mxfp8_gemm, bf16_gemm, nvfp4_quantize, mxfp8_quantize, decode")
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--m", type=int, default=None)
    ap.add_argument("--k", type=int, default=None)
    ap.add_argument("--config", default=None)
    ap.add_argument("--no-extra", action="store_true", help="skip the side measurements (other kernels of the path) and the CPU baseline leg")
    ap.add_argument("--workload", default="auto", choices=["auto", "moe", "tp_timeline"],
                    help="auto: N=1 MXFP8 GEMM, N>1 tensor-parallel NVFP4 GEMM; moe: the MoE layer; tp_timeline: per-launch timing and wait counters of the tensor-parallel step (diagnostic)")
    ap.add_argument("--comm-sms", type=int, default=0, help="CTAs of the multi-GPU kernels that move data over NVLink (0 = per-workload default)")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
