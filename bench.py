"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0).  The workload is the same at every N, so the per-N lines form one strong-scaling curve:

  NVFP4 tensor-parallel GEMM M=8192 N=28672 K=8192: weights (NVFP4, N(0, 0.02)) sharded by output column over the N GPUs,
  bf16 activation rows (N(0, 1)) sharded by row.  A step = every rank quantizes its rows to NVFP4 (the per-tensor amax is
  max-reduced over NVLink inside the quantize kernel), the codes and scales are all-gathered over NVLink while the
  tcgen05 GEMM already multiplies (own rows first), D[:, rank's columns] is written as bf16.  At N = 1 the same two
  launches run on one GPU without an exchange.  `value` = 2*M*N*K / step time, whole job, operands resident in HBM;
  `e2e` = the same step from bf16 rows in pinned HOST memory to the rank's output columns back in pinned host memory.
  `extra` carries the other rows of the path measured the same way: the MXFP8 / NVFP4 / BF16 / FP8 GEMMs at 8192^3, the
  quantizers, the skinny-M decode GEMM (HBM GB/s), and the expert-parallel MoE layer on the same N GPUs (`extra.moe`).

  `--case <kernel>` runs one kernel only (the commands of the ncu summaries under profiles/), `--workload tp_timeline`
  prints per-launch times and the kernels' wait counters of the tensor-parallel step, `--workload moe` the MoE layer alone.

`--impl reference` times the reference's CPU implementation of the same GEMM arithmetic (its own naive NVFP4 kernel from
kernels/gemm/common.cuh compiled for the host, oracle/_ref, when that build exists, otherwise the oracle's C++
restatement) on all host cores, each step a bounded row slab of the same workload.
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

M = N = K = 8192                      # the 8192^3 side measurements
FLOPS = 2.0 * M * N * K
TP_M, TP_N, TP_K = 8192, 28672, 8192  # the headline workload
TP_FLOPS = 2.0 * TP_M * TP_N * TP_K
NOMINAL = {"bf16": 2250.0, "fp8": 4500.0, "fp4": 9000.0, "hbm_gbs": 8000.0}
METRIC = "NVFP4 GEMM throughput (M=8192 N=28672 K=8192, tensor-parallel over the GPUs of the run)"
WORKLOAD = ("NVFP4 tensor-parallel GEMM M=8192 N=28672 K=8192: weights ~N(0,0.02) N-sharded, bf16 activations ~N(0,1) row-sharded, "
            "quantized on the fly, gathered over NVLink, bf16 out")
DTYPE = "nvfp4 (e2m1 x ue4m3 block scales x fp32 tensor scale, fp32 accumulate)"
CPU_SLAB_ROWS = 4

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel at N = 1 (the NVFP4 GEMM, M=8192 N=28672
# K=8192), from an ncu capture of `python bench.py --case nvfp4_gemm --m 8192 --size 28672 --k 8192`; None = not captured.
TP_GEMM_DRAM_BYTES = 735267584     # 302.7 MB read + 432.6 MB written (profiles/nvfp4_tp_gemm_ncu.md)


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
def cpu_reference_slab(steps: int, warmup: int, rows: int = CPU_SLAB_ROWS):
    """Times the reference's CPU arithmetic for the headline workload on a `rows`-row slab (all 28672 columns, full K)
    with every host core.  Returns (cpu_baseline dict, seconds per step)."""
    # torchrun exports OMP_NUM_THREADS=1; this leg is the only CPU work of its process and takes every core
    import numpy as np
    import oracle as O
    O.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(3)
    A = rng.standard_normal((128, TP_K), dtype=np.float32)           # a whole 128-row scale block; `rows` of it are multiplied
    aq = O.nvfp4_quantize(O.f32_to_bf16(A))
    B = (rng.standard_normal((TP_N, TP_K), dtype=np.float32) * np.float32(0.02))
    bq = O.nvfp4_quantize(O.f32_to_bf16(B))
    del A, B
    ref = O.ref_host()
    cores = O.num_threads()
    if ref is not None:
        kind = "reference"
        D = np.empty((rows, TP_N), np.uint16)
        a_codes, a_sc, a_sg = np.ascontiguousarray(aq[0][:rows]), np.ascontiguousarray(aq[1]).reshape(-1), np.ascontiguousarray(aq[2], np.float32)
        b_codes, b_sc, b_sg = np.ascontiguousarray(bq[0]), np.ascontiguousarray(bq[1]).reshape(-1), np.ascontiguousarray(bq[2], np.float32)

        def run():
            ref.tkref_nvfp4_gemm(a_codes, a_sc, a_sg, b_codes, b_sc, b_sg, D, rows, TP_N, TP_K)
    else:
        kind = "port"

        def run():
            O.nvfp4_gemm(*aq, *bq, 0, rows)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    tflops = 2.0 * rows * TP_N * TP_K / dt * 1e-12
    return {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"{rows} of {TP_M} output rows x all N={TP_N} columns x full K={TP_K} per step, {steps} steps ({dt:.2f} s/step), "
                      f"{'the reference kernel reference_nvfp4_gemm_kernel compiled for the host' if kind == 'reference' else 'C++ restatement'}"}, dt


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    cb, dt = cpu_reference_slab(steps, warmup)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "TFLOP/s", "n_gpus": max(args.gpus, world), "steps": steps,
            "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic", "config": {"workload": WORKLOAD},
            "timed": "CPU: each step multiplies a bounded row slab of the workload (cpu_baseline.sample); value = the slab's FLOPs / its time",
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


def event_time(torch, fn, steps, cooldown=0.5, sampler=None, host=None, barrier=None):
    """CUDA-event time per step on the current stream.  A 500 ms idle period precedes the timed loop, as in the
    reference's own protocol (kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:673-700), so the loop starts from the
    same thermal/power state every time.  `host`, if given, receives the host time spent enqueueing one step.
    `barrier` (multi-rank runs) is called right before the start event, after the idle period: the ranks' sleeps and
    set-up end milliseconds apart, and a rank that starts early would otherwise time its wait for the late ones as part
    of its first step (at 8 ranks a step is ~0.2 ms, so a few ms of skew over 20 steps is as large as the steps)."""
    s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    time.sleep(cooldown)
    if barrier is not None:
        barrier()
    s.record()
    t0 = time.perf_counter()
    for i in range(steps):
        fn(i)
    t1 = time.perf_counter()
    e.record()
    if host is not None:
        host.append((t1 - t0) / steps)
    if sampler is not None:
        sampler.poll_until(e.query)       # clocks while the GPU works through the queue; the host launches are over
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e-3 / steps


class Dist:
    """Rank bookkeeping; torch.distributed (NCCL) only when the run has more than one rank."""

    def __init__(self, torch):
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0")); self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def gather_settings(args, world):
    """--comm-sms: 0 = default (copy engines at N = 2, push warps from N = 3 on), -2 = two push warps in every CTA of the GEMM kernel, -1 = copy engines,
    k > 0 = k comm CTAs inside the GEMM kernel.  Returns (mode, comm CTAs)."""
    if world == 1:
        return "none", 0
    if args.comm_sms > 0:
        return "comm_ctas", args.comm_sms
    if args.comm_sms == -1:
        return "copy_engines", 0
    if args.comm_sms == -2:
        return "push_warps", 0
    # default: with two ranks a step is one 19 MB peer copy, which the copy engines move while every warp of every SM
    # multiplies (measured 0.394 against 0.414 ms); from three ranks on the copies get small and many, and the push warps win
    return ("copy_engines", 0) if world == 2 else ("push_warps", 0)


GATHER_TEXT = {"none": "none (one GPU)",
               "push_warps": "two push warps in every CTA of the GEMM kernel (plain 16-byte loads / peer stores, 16-row units, one arrival flag each)",
               "copy_engines": "copy engines: one peer cudaMemcpyAsync per destination for codes, scales and arrival flags",
               "comm_ctas": "comm CTAs of the GEMM kernel"}


def measure_tp(args, D_) -> dict:
    """The headline workload on the run's GPUs (see the module docstring)."""
    torch = D_.torch
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib, parallel
    rank, world, dev = D_.rank, D_.world, D_.dev
    n_local, rows = TP_N // world, TP_M // world
    u8 = torch.uint8
    GROUPS = 3
    mode, comm = gather_settings(args, world)
    ce = mode == "copy_engines"
    op = parallel.AllGatherMatmulNVFP4(TP_M, TP_K, D_.local_rank, world, num_comm_sms=max(comm, 2), copy_engines=ce, copy_streams=args.copy_streams,
                                       push_warps=mode == "push_warps")
    sets = []
    amax_w = torch.zeros(1, dtype=torch.float32, device=dev)
    for gi in range(GROUPS):
        # weight shard: rows [rank*n_local, ...) of a seeded N(0, 0.02) matrix, quantized with the all-reduced amax
        W = synth(torch, dev, n_local, TP_K, 800 + 10 * gi + rank, std=0.02)
        ops.absmax_bf16(W, amax_w)
        if world > 1:
            D_.dist.all_reduce(amax_w, op=D_.dist.ReduceOp.MAX)
        wc = torch.empty(n_local, TP_K // 2, dtype=u8, device=dev); ws = torch.empty((n_local + 127) // 128, TP_K // 64, 512, dtype=u8, device=dev)
        wg = torch.empty(1, dtype=torch.float32, device=dev)
        ops.nvfp4_quantize(W, wc, ws, wg, False, amax=amax_w)
        X = synth(torch, dev, rows, TP_K, 700 + 10 * gi + rank)
        sets.append((X, wc, ws, wg, torch.empty(TP_M, n_local, dtype=torch.bfloat16, device=dev)))
        del W
    hostX = sets[0][0].cpu().pin_memory()
    hostD = torch.empty(TP_M, n_local, dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()

    def step(i):
        X, wc, ws, wg, D = sets[i % GROUPS]
        op(X, wc, ws, wg, D)

    warm = max(args.warmup, 3)
    for i in range(warm):
        step(i)
    # With the copy-engine gather a step costs the host about thirty driver calls, more than the ~0.1 ms the GPUs need at
    # 8 ranks: the steps are therefore recorded once as a CUDA graph of 2 * GROUPS calls (both buffer sets x every operand
    # set) and replayed; what does not fill a whole graph is issued call by call.  Same kernels, same copies, same epochs.
    graph, per_graph = None, 2 * GROUPS
    if ce and not args.no_graph:
        graph = op.capture([sets[i % GROUPS] for i in range(per_graph)])
        op.replay(graph)
    D_.barrier()

    def run_steps(n):
        done = 0
        if graph is not None and (op.epoch + 1) % 2 == graph[2]:
            while n - done >= per_graph:
                op.replay(graph)
                done += per_graph
        for i in range(n - done):
            step(i)

    cs = ClockSampler(D_.local_rank)
    host = []
    dt = event_time(torch, lambda i: run_steps(args.steps) if i == 0 else None, args.steps, sampler=cs, host=host, barrier=D_.barrier)
    clocks = cs.summary()
    status = _lib.device_status()
    dt = D_.max(dt)
    D_.barrier()

    # per-launch breakdown of the same step (events between the launches of a step; a separate short loop so that the
    # events do not sit inside the timed region above)
    quant_us = gemm_us = None
    if world == 1:
        X, wc, ws, wg, D = sets[0]
        xc = torch.empty(TP_M, TP_K // 2, dtype=u8, device=dev); xs = torch.empty(TP_M // 128, TP_K // 64, 512, dtype=u8, device=dev)
        xg = torch.empty(1, dtype=torch.float32, device=dev)
        for i in range(3):
            ops.nvfp4_quantize(X, xc, xs, xg, False)
        quant_us = event_time(torch, lambda i: ops.nvfp4_quantize(sets[i % GROUPS][0], xc, xs, xg, False), 10, cooldown=0.1) * 1e6
        gemm_us = event_time(torch, lambda i: ops.nvfp4_gemm(xc, xs, xg, *sets[i % GROUPS][1:4], sets[i % GROUPS][4]), 10, cooldown=0.1) * 1e6
        del xc, xs, xg
    else:
        gemm_us = max(dt * 1e6 - 0.0, 0.0)      # at N > 1 the GEMM kernel spans the gather; the step time is its upper bound

    # end to end: pinned host rows -> H2D -> step -> D2H of this rank's output columns
    dX = torch.empty(rows, TP_K, dtype=torch.bfloat16, device=dev)
    _, wc, ws, wg, D = sets[0]

    def e2e_step(i):
        dX.copy_(hostX, non_blocking=True)
        op(dX, wc, ws, wg, D)
        hostD.copy_(D, non_blocking=True)

    for i in range(2):
        e2e_step(i)
    D_.barrier()
    dt_e2e = D_.max(event_time(torch, e2e_step, max(3, min(args.steps, 10)), barrier=D_.barrier))
    status |= _lib.device_status()
    D_.barrier()
    op.close()
    del sets, dX
    torch.cuda.empty_cache()
    return {"dt": dt, "dt_e2e": dt_e2e, "clocks": clocks, "status": status, "host_enqueue_us": statistics.median(host) * 1e6 if host else None,
            "quant_us": quant_us, "gemm_us": gemm_us, "graph": (f"{per_graph} steps per replayed CUDA graph" if graph is not None else None), "copy_engines": ce, "gather": mode, "comm_ctas": comm, "warmup": warm, "groups": GROUPS,
            "h2d": rows * TP_K * 2 * world, "d2h": TP_M * n_local * 2 * world}


def measure_moe(args, D_, steps: int) -> dict:
    """MoE layer: 16384 tokens, hidden 7168, 128 experts, intermediate 2048, top-8 routing from a softmax over seeded
    N(0,1) logits, NVFP4 expert weights ~N(0,0.02), experts and tokens sharded over the ranks.
    A step = route -> schedule -> quantize -> dispatch fused with the grouped GEMM -> combine."""
    torch = D_.torch
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib, parallel
    rank, world, dev = D_.rank, D_.world, D_.dev
    T, H, I, E, k = 16384, 7168, 2048, 128, 8
    Tl, El = T // world, E // world
    u8 = torch.uint8
    comm = 0 if args.moe_comm_sms < 0 else args.moe_comm_sms       # default: dispatch by the gather kernel on all SMs (1.44 against 1.72 ms on one GPU)
    layer = parallel.MoELayerNVFP4(T, H, I, E, k, D_.local_rank, world, num_comm_sms=comm)
    amax_w = torch.zeros(1, dtype=torch.float32, device=dev)
    wc = torch.empty(El * I, H // 2, dtype=u8, device=dev); ws = torch.empty(El * I // 128, H // 64, 512, dtype=u8, device=dev)
    wg = torch.empty(1, dtype=torch.float32, device=dev)
    common = torch.zeros(1, dtype=torch.float32, device=dev)
    for e in range(El):       # expert by expert to keep the bf16 staging small; one common per-tensor scale
        W = synth(torch, dev, I, H, 1100 + rank * El + e, std=0.02)
        ops.absmax_bf16(W, amax_w)
        common = torch.maximum(common, amax_w)
        del W
    if world > 1:
        D_.dist.all_reduce(common, op=D_.dist.ReduceOp.MAX)
    for e in range(El):
        W = synth(torch, dev, I, H, 1100 + rank * El + e, std=0.02)
        ops.nvfp4_quantize(W, wc[e * I:(e + 1) * I], ws[e * I // 128:(e + 1) * I // 128], wg, False, amax=common)
        del W
    sets = [(synth(torch, dev, Tl, E, 900 + 10 * gi + rank).float(), synth(torch, dev, Tl, H, 1000 + 10 * gi + rank)) for gi in range(3)]
    torch.cuda.synchronize()

    def step(i):
        lg, X = sets[i % 3]
        layer.forward(lg, X, wc, ws, wg)

    for i in range(3):
        step(i)
    D_.barrier()
    dt = D_.max(event_time(torch, step, steps, cooldown=0.2, barrier=D_.barrier))
    st = _lib.device_status()
    rows = int(layer.num_blocks.item()) * 128
    D_.barrier()
    layer.close()
    del wc, ws, sets
    torch.cuda.empty_cache()
    flops = 2.0 * T * k * H * I
    return {"metric": "MoE layer (16384 tokens, hidden 7168, 128 experts, intermediate 2048, top-8, NVFP4 up-projection + combine)",
            "ms_per_step": dt * 1e3, "tflops": flops / dt * 1e-12, "n_gpus": world, "steps": steps, "device_status": st, "comm_ctas": comm,
            "rank0_padded_rows": rows, "dispatch_bytes_in_per_gpu": (world - 1) / world * T * k / world * (H // 2 + H // 16),
            "combine_bytes_in_per_gpu": (world - 1) / world * Tl * k * I * 2,
            "parity": "routing and combine have no counterpart in the reference (unpinned); dispatch + grouped GEMM are checked against the oracle"}


def run_moe(args) -> None:
    import torch
    D_ = Dist(torch)
    out = measure_moe(args, D_, args.steps)
    if D_.rank == 0:
        print(json.dumps(out), flush=True)
    D_.close()


def run_ours(args) -> None:
    if args.workload == "moe":
        return run_moe(args)
    if args.workload == "tp_timeline":
        return run_tp_timeline(args)
    import torch
    from thunderkittens_b200 import _lib
    _lib.lib()   # fail loudly if the CUDA library is missing
    D_ = Dist(torch)
    rank, world = D_.rank, D_.world
    tp = measure_tp(args, D_)
    assert tp["status"] == 0, f"a device-side wait timed out or a capacity check failed (status {tp['status']})"
    extras = {}
    if not args.no_extra:
        try:
            extras["moe"] = measure_moe(args, D_, max(5, min(args.steps, 10)))
        except Exception as e:      # side measurements never invalidate the headline line
            extras["moe"] = {"error": repr(e)[:300]}
        if world == 1:
            import thunderkittens_b200.ops as ops
            extras.update(side_measurements(torch, ops, D_.dev))
            torch.cuda.synchronize()
            extras["reference_gpu_kernels_8192"] = reference_gpu_kernels()
    if rank == 0:
        pk = measured_peaks()
        dt, dt_e2e = tp["dt"], tp["dt_e2e"]
        tf = TP_FLOPS / dt * 1e-12
        peak = 4.0 * pk["bf16_tflops"]
        gemm_tf = TP_FLOPS / world / (tp["gemm_us"] * 1e-6) * 1e-12
        nvl_bytes = (world - 1) / world * TP_M * (TP_K // 2 + TP_K // 16)
        line = {
            "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": tp["warmup"],
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"tp{world}" if world > 1 else "single GPU",
                       "l2": f"{tp['groups']} rotating weight / activation / output sets (> 126 MB L2)",
                       "gather": (f"{tp['comm_ctas']} " if tp["gather"] == "comm_ctas" else "") + GATHER_TEXT[tp["gather"]],
                       "launches_per_step": "tkb_nvfp4_quantize_sharded + tkb_ag_gemm_nvfp4 (one call: tkb_ag_linear_nvfp4)"},
            "roofline": {"bound": "tensor", "achieved": gemm_tf, "peak": peak, "unit": "TFLOP/s per GPU", "frac": gemm_tf / peak,
                         "peak_derived": True, "peak_source": f"4 x {pk['source']} cuBLAS bf16 burst {pk['bf16_tflops']} TFLOP/s (derived dense-FP4 ceiling; "
                                                              "no FP4 figure is in the measured peaks)",
                         "frac_of_nominal_9000": gemm_tf / NOMINAL["fp4"],
                         "kernel": "tkb::gemm_kernel<NVFP4, cta pair, N256, all-gather>",
                         "kernel_us": tp["gemm_us"], "kernel_us_how": "CUDA events around 10 launches of the GEMM alone on the rotating sets" if world == 1
                         else "the step time (the GEMM kernel spans the gather): a lower bound on achieved",
                         "algorithmic_flops_per_launch": TP_FLOPS / world, "traffic": TP_GEMM_DRAM_BYTES if world == 1 else None,
                         "traffic_unit": "bytes per launch, dram__bytes_read.sum + dram__bytes_write.sum of an ncu capture of this kernel and shape",
                         "algorithmic_bytes": TP_M * TP_K // 2 + TP_N * TP_K // 2 + (TP_M + TP_N) * TP_K // 16 + TP_M * TP_N * 2,
                         "nvlink_bytes_in_per_gpu": nvl_bytes, "nvlink_time_at_770GBs_ms": nvl_bytes / 770e9 * 1e3},
            "e2e": {"value": TP_FLOPS / dt_e2e * 1e-12, "unit": "TFLOP/s", "h2d_bytes_per_step": tp["h2d"], "d2h_bytes_per_step": tp["d2h"],
                    "ms_per_step": dt_e2e * 1e3,
                    "path": "pinned host bf16 rows -> H2D -> AllGatherMatmulNVFP4 (tkb_ag_linear_nvfp4) -> D2H of the rank's output columns"},
            "gpu_launches": args.steps * 2 * world, "host_enqueue_us_per_step": tp["host_enqueue_us"], "cuda_graph": tp["graph"],
            "step_breakdown_us": {"quantize": tp["quant_us"], "gemm": tp["gemm_us"]} if world == 1 else None,
            "clocks": tp["clocks"], "extra": extras,
        }
        if world == 1 and not args.no_extra:
            cb, _ = cpu_reference_slab(3, 1)
            line["cpu_baseline"] = cb
        elif not args.no_extra:
            cb, _ = cpu_reference_slab(2, 1)
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
    D_.barrier()
    D_.close()


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
    # the reference's standalone bf16 / fp8 GEMM benchmarks: their own main() times 1024^3 ... 16384^3 (5 warm-up + 10 timed launches,
    # rotating operand groups, 500 ms idle first: the protocol this file mirrors); the 8192^3 figures are read from their output
    import re
    for which in ("bf16", "fp8"):
        exe = os.path.join(ROOT, "oracle", "_ref", f"tk_{which}", f"{which}_b200_gemm.out")
        if not os.path.exists(exe):
            out[which] = {"unavailable": "reference standalone benchmark not built (oracle/build.py:build_ref_standalone needs the reference tree)"}
            continue
        try:
            r = subprocess.run([exe], capture_output=True, text=True, timeout=240)
            m = re.search(r"M=8192 N=8192 K=8192.*?Average kernel execution time: ([0-9.eE+-]+) us.*?Achieved performance: ([0-9.eE+-]+) TFLOPs", r.stdout, re.S)
            out[which] = {"gemm_us": float(m.group(1)), "gemm_tflops": float(m.group(2))} if m else {"unavailable": (r.stdout + r.stderr)[-300:]}
        except Exception as e:
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
        # MXFP8 8192^3: bf16 ~N(0,1) with 1 % of entries x32, per-32 UE8M0 scales
        gs = []
        for gi in range(3):
            A = synth(torch, dev, M, K, 3 + 10 * gi, outliers=0.01); B = synth(torch, dev, N, K, 4 + 10 * gi, outliers=0.01)
            a = torch.empty(M, K, dtype=u8, device=dev); asc = torch.empty(M // 128, K // 128, 512, dtype=u8, device=dev)
            b = torch.empty(N, K, dtype=u8, device=dev); bsc = torch.empty(N // 128, K // 128, 512, dtype=u8, device=dev)
            ops.mxfp8_quantize(A, a, asc); ops.mxfp8_quantize(B, b, bsc)
            gs.append((a, asc, b, bsc, torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
            del A, B
        f = lambda i: ops.mxfp8_gemm(*gs[i % 3])
        for i in range(3):
            f(i)
        t = event_time(torch, f, 10)
        tf = FLOPS / t * 1e-12
        out["mxfp8_gemm_8192"] = {"tflops": tf, "us": t * 1e6, "frac_of_2x_measured_bf16": tf / (2 * pk["bf16_tflops"]),
                                  "frac_of_nominal_4500": tf / NOMINAL["fp8"]}
        # dense FP8 (e4m3) on the same codes
        f = lambda i: ops.fp8_gemm(gs[i % 3][0], gs[i % 3][2], gs[i % 3][4])
        for i in range(3):
            f(i)
        t = event_time(torch, f, 10)
        tf = FLOPS / t * 1e-12
        out["fp8_gemm_8192"] = {"tflops": tf, "us": t * 1e6, "frac_of_2x_measured_bf16": tf / (2 * pk["bf16_tflops"])}
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
                ops.nvfp4_gemm(xc, xs, xg, *ws[i % 3], Dd, "skinny_prefetch")   # static weights: may be loaded under the quantizer
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


def run_tp_timeline(args) -> None:
    """Diagnostic for the tensor-parallel step (N > 1, torchrun): per-step CUDA-event times of a free-running loop plus the
    GEMM kernel's own wait counters (tkb_gemm_set_profile_buffer) for the last step.  One JSON line from rank 0 and one
    from rank world/2.  Not a benchmark line."""
    import ctypes
    import numpy as np
    import torch
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib as L, parallel
    D_ = Dist(torch)
    rank, world, dev = D_.rank, D_.world, D_.dev
    nl, rows = TP_N // world, TP_M // world
    mode, comm = gather_settings(args, world)
    ce = mode == "copy_engines"
    op = parallel.AllGatherMatmulNVFP4(TP_M, TP_K, D_.local_rank, world, num_comm_sms=max(comm, 2), copy_engines=ce,
                                       copy_streams=args.copy_streams, push_warps=mode == "push_warps")
    X = synth(torch, dev, rows, TP_K, 700 + rank)
    W = synth(torch, dev, nl, TP_K, 800 + rank, std=0.02)
    u8 = torch.uint8
    wc = torch.empty(nl, TP_K // 2, dtype=u8, device=dev); ws = torch.empty((nl + 127) // 128, TP_K // 64, 512, dtype=u8, device=dev)
    wg = torch.empty(1, dtype=torch.float32, device=dev)
    ops.nvfp4_quantize(W, wc, ws, wg, False)
    del W
    D = torch.empty(TP_M, nl, dtype=torch.bfloat16, device=dev)
    for _ in range(max(args.warmup, 3)):
        op(X, wc, ws, wg, D)
    D_.barrier()
    prof = torch.zeros(160 * 8, dtype=torch.int64, device=dev)
    setp = L.bind("tkb_gemm_set_profile_buffer", [ctypes.c_void_p])
    steps = max(args.steps, 4)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record()
    for i in range(steps):
        if i == steps - 1:
            setp(prof.data_ptr())
        op(X, wc, ws, wg, D)
        evs[i + 1].record()
    torch.cuda.synchronize()
    setp(None)
    per = np.array([evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]) * 1e3
    pr = prof.cpu().numpy().reshape(160, 8)
    ncomm = op.num_comm_sms if mode == "comm_ctas" else 0
    lead = pr[ncomm::2]
    lead = lead[lead[:, 4] > 0]
    if len(lead) == 0:
        lead = np.zeros((1, 8), np.int64)
    med = lambda a: float(np.median(a))
    out = {"rank": rank, "n_gpus": world, "gather": mode if mode != "comm_ctas" else f"{ncomm} comm CTAs", "step_us_median_max": [med(per), float(per.max())],
           "cycles_of_last_step": {"mma_total": med(lead[:, 4]), "mma_waiting_for_operands": med(lead[:, 3]), "mma_waiting_for_drain": med(lead[:, 2]),
                                   "producer_waiting_for_remote_rows_median_max": [med(lead[:, 7]), float(lead[:, 7].max())],
                                   "push_warps_busy_median_max": ([med(pr[:148, 1][pr[:148, 1] > 0]), float(pr[:148, 1].max())] if mode == "push_warps" and (pr[:148, 1] > 0).any() else None)},
           "device_status": L.device_status()}
    if rank in (0, world // 2):
        print(json.dumps(out), flush=True)
    D_.barrier()
    op.close()
    D_.close()


def run_case(args) -> None:
    """One kernel of the path, a few launches, nothing else: the command line used for ncu captures
    (python bench.py --case nvfp4_gemm --size 8192 --steps 3)."""
    import torch
    import thunderkittens_b200.ops as ops
    from thunderkittens_b200 import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    u8 = torch.uint8
    m, n, k = args.size if args.m is None else args.m, args.size, args.size if args.k is None else args.k      # --size is N (and the default of M, K)
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
                    help="auto: the tensor-parallel NVFP4 GEMM (plus the side measurements); moe: the MoE layer alone; tp_timeline: per-launch timing and wait counters of the tensor-parallel step (diagnostic)")
    ap.add_argument("--comm-sms", type=int, default=0, help="gather of the tensor-parallel GEMM at N > 1: 0 = default (copy engines at N = 2, push warps beyond), -2 = push warps in every CTA of the GEMM kernel, -1 = copy engines, k > 0 = k comm CTAs inside the GEMM kernel")
    ap.add_argument("--no-graph", action="store_true", help="tensor-parallel step at N > 1 with the copy-engine gather: issue every step call by call instead of replaying a CUDA graph")
    ap.add_argument("--copy-streams", type=int, default=3, help="streams the copy-engine gather spreads its peer copies over (1..4)")
    ap.add_argument("--moe-comm-sms", type=int, default=-1, help="k > 0: k CTAs of the MoE GEMM kernel pull the token rows; 0 (default): dispatch by the gather kernel on all SMs")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
