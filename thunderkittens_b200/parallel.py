"""Single-node multi-GPU host layer: symmetric buffers and the collective-fused operators.

Mirrors the reference's Python-visible parallel API for this path:
  TKParallelTensor(shape, dtype, local_rank, local_world_size, multicast)   include/pyutils/parallel_tensor.cuh:320-336
  all_gather_matmul(A, B, C, barrier, num_comm_sms)                          kernels/parallel/ag_gemm/ag_gemm_b200.cu:280-305
One process per GPU (torchrun); `torch.distributed` must be initialised — it carries the 64-byte CUDA IPC
handles (the reference ships its own unix-socket broker for that).  Everything else — data, flags, the per-tensor
amax reduction, the gather of routing decisions — moves through kernels of libtkb200 over NVLink peer mappings.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.distributed as dist

from . import _lib as L
from . import ops

_DT_SIZE = {torch.uint8: 1, torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.int32: 4, torch.int: 4, torch.int64: 8}


class _RawCuda:
    """Minimal __cuda_array_interface__ carrier so torch can view memory owned by libtkb200."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class TKParallelTensor:
    """A tensor of the same shape on every rank of the node whose storage is mapped into every other rank.

    data_               torch view of the local storage
    local_rank_, local_world_size_
    peer_ptr(i)         device pointer of rank i's storage as seen from this rank
    The `multicast` argument is accepted for signature compatibility and ignored: nothing on this path uses
    an NVSwitch multicast object.
    """

    def __init__(self, shape, dtype, local_rank: int, local_world_size: int, multicast: bool = False, group=None):
        self.shape_ = tuple(int(s) for s in shape)
        self.dtype_ = dtype
        self.local_rank_ = int(local_rank)
        self.local_world_size_ = int(local_world_size)
        self.multicast_ = False
        self._group = group
        self.nbytes = int(math.prod(self.shape_)) * _DT_SIZE[dtype]
        ptr = C.c_void_p()
        L.check(L.lib().tkb_dev_alloc(max(self.nbytes, 16), C.byref(ptr)))
        self._ptr = ptr.value
        self.data_ = self._view()
        self._peer = [None] * self.local_world_size_
        self._peer[self.local_rank_] = self._ptr
        self._opened = []
        if self.local_world_size_ > 1:
            self._exchange()

    def _view(self) -> torch.Tensor:
        raw = torch.as_tensor(_RawCuda(self._ptr, self.nbytes), device=torch.device("cuda", torch.cuda.current_device()))
        return raw.view(self.dtype_).view(self.shape_)

    def _exchange(self) -> None:
        handle = (C.c_ubyte * 64)()
        L.check(L.lib().tkb_ipc_export(self._ptr, handle))
        handles = [None] * self.local_world_size_
        dist.all_gather_object(handles, bytes(handle), group=self._group)
        for r, h in enumerate(handles):
            if r == self.local_rank_:
                continue
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            p = C.c_void_p()
            L.check(L.lib().tkb_ipc_open(buf, C.byref(p)))
            self._peer[r] = p.value
            self._opened.append(p.value)

    def peer_ptr(self, rank: int) -> int:
        return self._peer[rank]

    def peer_ptr_array(self):
        arr = (C.c_void_p * self.local_world_size_)(*self._peer)
        return arr

    def close(self) -> None:
        if self._ptr is None:
            return
        torch.cuda.synchronize()
        for p in self._opened:
            L.lib().tkb_ipc_close(p)
        self._opened = []
        if self.local_world_size_ > 1:
            dist.barrier(group=self._group)     # nobody frees while a peer still has the mapping open
        self.data_ = None
        L.lib().tkb_dev_free(self._ptr)
        self._ptr = None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class AllGatherMatmulNVFP4:
    """Column-parallel linear layer with NVFP4 operands: every rank owns M/world activation rows (bf16) and
    N_local = N/world weight rows (already NVFP4).  One call =
        quantize into this rank's slice of the gathered buffers (the per-tensor amax is max-reduced over NVLink
        inside the quantize kernel) -> fused kernel that gathers the other ranks' slices while it multiplies.
    The gather is one of: `push_warps=True` — two extra warps in EVERY CTA of the GEMM kernel push a share of the slice
    (best from 3 ranks on); `copy_engines=True` — peer copies on library-owned streams, replayable as a CUDA graph
    (`capture` / `replay`; best at 2 ranks); otherwise `num_comm_sms` CTAs of the GEMM kernel push (the reference's
    scheme).  Two buffer sets alternate between calls; a set is written again only after every peer has finished
    with its previous contents (acknowledgement flags, or the amax exchange of the following step).
    """

    def __init__(self, M: int, K: int, local_rank: int, local_world_size: int, num_comm_sms: int = 8, group=None, arithmetic: str | None = None,
                 copy_engines: bool = False, copy_streams: int = 3, push_warps: bool = False):
        self.arithmetic = arithmetic      # NVFP4 quantizer arithmetic (None = ops.default_nvfp4_arithmetic)
        if M % (256 * local_world_size):
            raise RuntimeError("M must be a multiple of 256 * world size")
        if K % 64:
            raise RuntimeError("K must be a multiple of 64")
        self.M, self.K = M, K
        self.rank, self.world = local_rank, local_world_size
        self.group = group
        self.num_comm_sms = 0 if local_world_size == 1 else max(2, num_comm_sms - num_comm_sms % 2)
        mk = lambda shape, dt: TKParallelTensor(shape, dt, local_rank, local_world_size, False, group)
        self.codes = [mk((M, K // 2), torch.uint8) for _ in range(2)]
        self.scales = [mk((M // 128, K // 64, 512), torch.uint8) for _ in range(2)]
        # flags[0:world] = done (acknowledge) epochs; arrived[set] = arrival epochs of the row blocks, written by their owners
        self.flags = mk((local_world_size,), torch.int32)
        dev = self.flags.data_.device
        self.arrived = [mk((M // 8,), torch.int32) for _ in range(2)]      # arrival epochs: 4 or (push warps) 16 per 256 gathered rows in use
        self.slots = [mk((local_world_size,), torch.int64) for _ in range(2)]   # (epoch, amax bits) per rank, see tkb_amax_allreduce
        self.amax = torch.zeros(1, dtype=torch.float32, device=dev)
        self.sg = torch.zeros(1, dtype=torch.float32, device=dev)
        self.exit_counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch_counter = torch.zeros(1, dtype=torch.int32, device=dev)     # copy-engine gather: completed steps, kept by the kernels
        self.epoch = 0
        self.rows = M // local_world_size
        st = L.AgState()
        st.rank, st.world, st.M, st.K = local_rank, local_world_size, M, K
        for b in range(2):
            for i in range(local_world_size):
                st.codes[b][i] = self.codes[b].peer_ptr(i); st.scales[b][i] = self.scales[b].peer_ptr(i)
                st.arrived[b][i] = self.arrived[b].peer_ptr(i); st.slots[b][i] = self.slots[b].peer_ptr(i)
        for i in range(local_world_size):
            st.done[i] = self.flags.peer_ptr(i)
        st.amax, st.sg, st.exit_counter = self.amax.data_ptr(), self.sg.data_ptr(), self.exit_counter.data_ptr()
        st.epoch_counter = self.epoch_counter.data_ptr()
        self.copy_engines = bool(copy_engines) and local_world_size > 1 and not push_warps
        self.push_warps = bool(push_warps) and local_world_size > 1      # two push warps in every CTA of the GEMM kernel
        self._copy = None
        self._graphs = []
        if self.copy_engines:
            # the gather travels by peer copies on streams that the library owns
            h = C.c_void_p()
            L.check(L.lib().tkb_ag_copy_create(min(copy_streams, 4), max(1, self.rows // 64), C.byref(h)))
            self._copy = h.value
            st.copy = h.value
        self._state = st
        if local_world_size > 1:
            dist.barrier(group=group)

    def __call__(self, X_local: torch.Tensor, W: torch.Tensor, W_sc: torch.Tensor, W_sg: torch.Tensor, D: torch.Tensor) -> None:
        """One library call, two launches per step (tkb_ag_linear_nvfp4): the quantize kernel max-reduces the amax across
        the ranks itself and the GEMM kernel does the epoch hand-shake; `step_by_step` below spells the same step out
        with one entry point per phase."""
        if tuple(X_local.shape) != (self.rows, self.K) or X_local.dtype != torch.bfloat16 or not X_local.is_contiguous():
            raise RuntimeError("X_local must be a contiguous bf16 tensor of shape (M / world, K)")
        n_local = W.shape[0]
        if tuple(D.shape) != (self.M, n_local) or D.dtype != torch.bfloat16 or not D.is_contiguous():
            raise RuntimeError("D must be a contiguous bf16 tensor of shape (M, N_local)")
        self.epoch += 1
        arith = ops._ARITH[self.arithmetic or ops.default_nvfp4_arithmetic]
        L.check(L.lib().tkb_ag_linear_nvfp4(C.byref(self._state), self.epoch, X_local.data_ptr(), W.data_ptr(), W_sc.data_ptr(), W_sg.data_ptr(),
                                            D.data_ptr(), 0, n_local, -2 if self.push_warps else (-1 if self.copy_engines else self.num_comm_sms), arith, _stream()))

    def capture(self, steps):
        """Records len(steps) consecutive calls as one CUDA graph (copy-engine gather only).  `steps` is a list of
        (X_local, W, W_sc, W_sg, D) tuples of even length; the tensors must stay alive and in place.  Returns a handle for
        `replay`.  Every rank must capture and replay alike."""
        if not self.copy_engines:
            raise RuntimeError("capture needs the copy-engine gather (copy_engines=True, world > 1)")
        n = len(steps)
        arr = lambda k: (C.c_void_p * n)(*[s[k].data_ptr() for s in steps])
        h = C.c_void_p()
        arith = ops._ARITH[self.arithmetic or ops.default_nvfp4_arithmetic]
        n_local = steps[0][1].shape[0]
        first = self.epoch + 1
        L.check(L.lib().tkb_ag_graph_create(C.byref(self._state), first, n, arr(0), arr(1), arr(2), arr(3), arr(4), 0, n_local, arith, C.byref(h)))
        self._graphs.append(h.value)
        return (h.value, n, first % 2)

    def replay(self, graph) -> None:
        handle, n, parity = graph
        if (self.epoch + 1) % 2 != parity:
            raise RuntimeError("the graph was recorded starting on the other buffer set: issue one single call first")
        L.check(L.lib().tkb_ag_graph_launch(handle, _stream()))
        self.epoch += n

    def step_by_step(self, X_local: torch.Tensor, W: torch.Tensor, W_sc: torch.Tensor, W_sg: torch.Tensor, D: torch.Tensor) -> None:
        lib = L.lib()
        if tuple(X_local.shape) != (self.rows, self.K) or X_local.dtype != torch.bfloat16 or not X_local.is_contiguous():
            raise RuntimeError("X_local must be a contiguous bf16 tensor of shape (M / world, K)")
        n_local = W.shape[0]
        if tuple(D.shape) != (self.M, n_local) or D.dtype != torch.bfloat16 or not D.is_contiguous():
            raise RuntimeError("D must be a contiguous bf16 tensor of shape (M, N_local)")
        self.epoch += 1
        e, b, r, w, s = self.epoch, self.epoch % 2, self.rank, self.world, _stream()
        codes, scales = self.codes[b], self.scales[b]
        # set b was last used at epoch e-2: every peer's kernel of that epoch must be finished before its buffers are written again
        if w > 1 and e > 2:
            L.check(lib.tkb_wait_flags(self.flags.data_.data_ptr(), w, r, e - 2, s))
        ops.absmax_bf16(X_local, self.amax)
        if w > 1:
            L.check(lib.tkb_amax_allreduce(self.slots[b].peer_ptr_array(), w, r, e, self.amax.data_ptr(), self.amax.data_ptr(), s))
        my_codes = codes.data_[r * self.rows:(r + 1) * self.rows]
        my_scales = scales.data_[r * self.rows // 128:(r + 1) * self.rows // 128]
        ops.nvfp4_quantize(X_local, my_codes, my_scales, self.sg, False, self.arithmetic, amax=self.amax)
        L.check(lib.tkb_ag_gemm_nvfp4(codes.peer_ptr_array(), scales.peer_ptr_array(), self.sg.data_ptr(), W.data_ptr(), W_sc.data_ptr(),
                                      W_sg.data_ptr(), D.data_ptr(), 0, self.M, n_local, self.K, r, w, self.arrived[b].peer_ptr_array(),
                                      None, None, e, -2 if self.push_warps else self.num_comm_sms, s))
        if w > 1:
            L.check(lib.tkb_signal_peers(self.flags.peer_ptr_array(), w, r, r, e, 0, s))      # my kernel of epoch e is done

    def close(self) -> None:
        torch.cuda.synchronize()
        for g in self._graphs:
            L.lib().tkb_ag_graph_destroy(g)
        self._graphs = []
        if self._copy is not None:
            L.lib().tkb_ag_copy_destroy(self._copy)
            self._copy = None
        for t in self.codes + self.scales + self.arrived + self.slots + [self.flags]:
            t.close()


def all_gather_matmul(A: TKParallelTensor, W: torch.Tensor, W_sc: torch.Tensor, W_sg: torch.Tensor, C_out: torch.Tensor,
                      state: AllGatherMatmulNVFP4, num_comm_sms: int | None = None) -> None:
    """Reference-shaped entry: A is a bf16 TKParallelTensor of the FULL shape (M, K) whose rows
    [rank*M/world, (rank+1)*M/world) hold this rank's activations (ag_gemm/benchmark.py:55-63); the weight is
    this rank's NVFP4 shard instead of a bf16 matrix and `state` replaces the reference's barrier tensor."""
    r, rows = A.local_rank_, A.shape_[0] // A.local_world_size_
    if num_comm_sms is not None and A.local_world_size_ > 1:
        state.num_comm_sms = max(2, num_comm_sms - num_comm_sms % 2)
    state(A.data_[r * rows:(r + 1) * rows], W, W_sc, W_sg, C_out)


class MoELayerNVFP4:
    """Expert-parallel MoE layer with NVFP4 expert weights: route -> schedule -> quantize tokens -> dispatch fused
    with the grouped expert GEMM -> combine.  Rank r owns tokens [r*T/world, (r+1)*T/world) and experts
    [r*E/world, (r+1)*E/world); `W`, `W_sc`, `W_sg` are its stacked expert weights ([E/world * I, K/2] codes).

    One forward(logits_local, X_local) call enqueues everything on the current stream and returns
    out [T/world, I] bf16.  Nothing synchronises with the host; the row capacity of the operand buffers
    (`cap_rows`, default twice the balanced share) is checked on the device.
    """

    def __init__(self, T: int, H: int, I: int, E: int, top_k: int, local_rank: int, local_world_size: int, cap_rows: int | None = None,
                 num_comm_sms: int = 16, group=None):
        w, r = local_world_size, local_rank
        if T % w or E % w or H % 256 or I % 128:
            raise RuntimeError("need T and E divisible by world, H % 256 == 0, I % 128 == 0")
        self.T, self.H, self.I, self.E, self.top_k, self.rank, self.world, self.group = T, H, I, E, top_k, r, w, group
        self.arithmetic = L.NVFP4_KERNEL_FAST   # NVFP4 quantizer arithmetic of the tokens (L.NVFP4_SPEC is the CPU-reproducible one)
        self.Tl, self.El = T // w, E // w
        if cap_rows is None:
            cap_rows = 2 * (T * top_k // w) + 128 * self.El
        self.cap_rows = (cap_rows + 127) // 128 * 128
        self.num_comm_sms = num_comm_sms
        mk = lambda shape, dt: TKParallelTensor(shape, dt, r, w, False, group)
        u8, i32, f32 = torch.uint8, torch.int32, torch.float32
        # symmetric: quantized tokens (two sets), expert outputs, flags [ready(w), y_ready(w), done(w)]
        self.xq_rows = [mk((self.Tl, H // 2 + H // 16), u8) for _ in range(2)]     # per token: codes, then its scales
        self.Y = mk((self.cap_rows, I), torch.bfloat16)
        self.flags = mk((3 * w,), i32)
        # per parity of the call counter (a peer may run one call ahead, never two): amax all-reduce slots, everybody's
        # chosen experts (gathered by pushes) and the arrival counters of that gather
        self.slots = [mk((w,), torch.int64) for _ in range(2)]
        self.experts_all_sym = [mk((T, top_k), i32) for _ in range(2)]
        self.counters = mk((2 * w,), i32)
        dev = self.flags.data_.device
        z = lambda *shape, dt=i32: torch.zeros(*shape, dtype=dt, device=dev)
        self.codes = z(self.cap_rows, H // 2, dt=u8)
        self.scales = z(self.cap_rows // 128, H // 64, 512, dt=u8)
        self.experts_local = z(self.Tl, top_k)
        self.weights = z(self.Tl, top_k, dt=f32)
        self.counts, self.padded = z(E), z(E)
        self.pull_idx = z(self.cap_rows, 2)
        self.block_expert = z(self.cap_rows // 128)
        self.num_blocks = z(1)
        self.comb_idx = z(self.Tl * top_k, 2)
        self.arrived = z(self.cap_rows // 128)
        self.amax, self.sg = z(1, dt=f32), z(1, dt=f32)
        self.out = torch.empty(self.Tl, I, dtype=torch.bfloat16, device=dev)
        self.epoch = 0
        st = L.MoeState()
        st.rank, st.world, st.T, st.H, st.I, st.E, st.top_k, st.cap_rows = r, w, T, H, I, E, top_k, self.cap_rows
        for i in range(w):
            for b in range(2):
                st.xq_rows[b][i] = self.xq_rows[b].peer_ptr(i); st.slots[b][i] = self.slots[b].peer_ptr(i)
                st.experts_all[b][i] = self.experts_all_sym[b].peer_ptr(i)
            st.Y[i] = self.Y.peer_ptr(i); st.flags[i] = self.flags.peer_ptr(i); st.counters[i] = self.counters.peer_ptr(i)
        for name in ("codes", "scales", "experts_local", "weights", "counts", "padded", "pull_idx", "block_expert", "num_blocks", "comb_idx",
                     "arrived", "sg"):
            setattr(st, name, getattr(self, name).data_ptr())
        self._state = st
        if w > 1:
            dist.barrier(group=group)

    def forward(self, logits_local: torch.Tensor, X_local: torch.Tensor, W: torch.Tensor, W_sc: torch.Tensor, W_sg: torch.Tensor) -> torch.Tensor:
        """One library call per layer (tkb_moe_layer_nvfp4); `forward_step_by_step` spells the same sequence out."""
        if tuple(logits_local.shape) != (self.Tl, self.E) or logits_local.dtype != torch.float32 or not logits_local.is_contiguous():
            raise RuntimeError("logits_local must be a contiguous fp32 tensor of shape (T / world, E)")
        if tuple(X_local.shape) != (self.Tl, self.H) or X_local.dtype != torch.bfloat16 or not X_local.is_contiguous():
            raise RuntimeError("X_local must be a contiguous bf16 tensor of shape (T / world, H)")
        self.epoch += 1
        self.experts_all = self.experts_all_sym[self.epoch % 2].data_
        L.check(L.lib().tkb_moe_layer_nvfp4(C.byref(self._state), self.epoch, logits_local.data_ptr(), X_local.data_ptr(), W.data_ptr(),
                                            W_sc.data_ptr(), W_sg.data_ptr(), self.out.data_ptr(), self.num_comm_sms, self.arithmetic, _stream()))
        return self.out

    def forward_step_by_step(self, logits_local: torch.Tensor, X_local: torch.Tensor, W: torch.Tensor, W_sc: torch.Tensor, W_sg: torch.Tensor) -> torch.Tensor:
        lib, s = L.lib(), _stream()
        w, r = self.world, self.rank
        self.epoch += 1
        e, b = self.epoch, self.epoch % 2
        fl = self.flags.data_.data_ptr()
        # routing of my tokens, then everybody's choices
        L.check(lib.tkb_moe_route(logits_local.data_ptr(), self.Tl, self.E, self.top_k, self.experts_local.data_ptr(), self.weights.data_ptr(), s))
        # everything of parity b was last used at call e-2: all peers must be done with that call before it is overwritten
        if w > 1 and e > 2:
            L.check(lib.tkb_wait_flags(fl + 4 * 2 * w, w, r, e - 2, s))
        self.experts_all = self.experts_all_sym[b].data_
        L.check(lib.tkb_all_to_all(self.experts_all_sym[b].peer_ptr_array(), self.experts_local.data_ptr(), self.Tl * self.top_k * 4, 1, r, w,
                                   self.counters.peer_ptr_array(), b * w, (e + 1) // 2, s))
        L.check(lib.tkb_moe_schedule(self.experts_all.data_ptr(), self.T, self.top_k, self.E, w, r, self.counts.data_ptr(), self.padded.data_ptr(),
                                     self.pull_idx.data_ptr(), self.block_expert.data_ptr(), self.num_blocks.data_ptr(),
                                     self.comb_idx.data_ptr(), self.cap_rows, s))
        # quantize my tokens with the global amax into set b
        ops.absmax_bf16(X_local, self.amax)
        if w > 1:
            L.check(lib.tkb_amax_allreduce(self.slots[b].peer_ptr_array(), w, r, e, self.amax.data_ptr(), self.amax.data_ptr(), s))
        L.check(lib.tkb_nvfp4_quantize_rows(X_local.data_ptr(), 0, self.xq_rows[b].data_.data_ptr(), self.sg.data_ptr(), self.amax.data_ptr(),
                                            self.Tl, self.H, self.arithmetic, s))
        if w > 1:
            L.check(lib.tkb_signal_peers(self.flags.peer_ptr_array(), w, r, r, e, 0, s))
            # Y is rewritten below: every peer must have finished combining the previous layer call from it
            if e > 1:
                L.check(lib.tkb_wait_flags(fl + 4 * 2 * w, w, r, e - 1, s))
        L.check(lib.tkb_moe_dispatch_gemm(self.xq_rows[b].peer_ptr_array(), self.sg.data_ptr(),
                                          self.codes.data_ptr(), self.scales.data_ptr(), W.data_ptr(), W_sc.data_ptr(), W_sg.data_ptr(),
                                          self.Y.data_.data_ptr(), 0, self.pull_idx.data_ptr(), self.block_expert.data_ptr(),
                                          self.num_blocks.data_ptr(), fl, self.arrived.data_ptr(), e, self.H, self.I, self.El, self.cap_rows,
                                          r, w, self.num_comm_sms, s))
        if w > 1:
            L.check(lib.tkb_signal_peers(self.flags.peer_ptr_array(), w, r, w + r, e, 0, s))     # my Y rows are complete
            L.check(lib.tkb_wait_flags(fl + 4 * w, w, r, e, s))                                  # everybody's are
        L.check(lib.tkb_moe_combine(self.Y.peer_ptr_array(), 0, self.comb_idx.data_ptr(), self.weights.data_ptr(), self.out.data_ptr(),
                                    self.Tl, self.top_k, self.I, w, s))
        if w > 1:
            L.check(lib.tkb_signal_peers(self.flags.peer_ptr_array(), w, r, 2 * w + r, e, 0, s))  # done with peers' tokens and Y
        return self.out

    def close(self) -> None:
        for t in self.xq_rows + self.slots + self.experts_all_sym + [self.Y, self.flags, self.counters]:
            t.close()


def tk_all_to_all(output: TKParallelTensor, input: TKParallelTensor, barrier: TKParallelTensor, scatter_axis: int, gather_axis: int) -> None:
    """The reference's tk_all_to_all(output, input, barrier, scatter_axis, gather_axis) (all_to_all.cu:119-179): `input` is
    this rank's 4-D tensor, `output` has the scatter axis divided and the gather axis multiplied by the world size.
    `barrier` must be an int32 TKParallelTensor of at least 2 * world zero-initialised elements that is used for nothing
    else; the call counter lives on it."""
    w, r = input.local_world_size_, input.local_rank_
    if len(input.shape_) != 4 or len(output.shape_) != 4:
        raise RuntimeError("input and output must be 4-D")
    expect = list(input.shape_)
    if expect[scatter_axis] % w:
        raise RuntimeError("the scattered axis must divide by the world size")
    expect[scatter_axis] //= w
    expect[gather_axis] *= w
    if tuple(expect) != tuple(output.shape_) or input.dtype_ != output.dtype_:
        raise RuntimeError(f"output must have shape {tuple(expect)} and the input's dtype")
    if barrier.dtype_ != torch.int32 or barrier.data_.numel() < 2 * w:
        raise RuntimeError("barrier must be an int32 parallel tensor of at least 2 * world elements")
    epoch = getattr(barrier, "_tkb_epoch", 0) + 1
    barrier._tkb_epoch = epoch
    dims = (C.c_longlong * 4)(*input.shape_)
    L.check(L.lib().tkb_all_to_all_4d(output.peer_ptr_array(), input.data_.data_ptr(), dims, input.data_.element_size(), scatter_axis, gather_axis,
                                      r, w, barrier.peer_ptr_array(), 0, epoch, _stream()))


class MoEDispatchGemmState:
    """Buffers behind `moe_dispatch_gemm` (takes the place of the reference's `barrier` tensor): the quantized tokens of
    every rank (two alternating sets, symmetric), the amax exchange slots, the epoch flags, and this rank's operand
    staging for up to `cap_rows` dispatched rows."""

    def __init__(self, tokens_per_rank: int, H: int, I: int, experts_local: int, cap_rows: int, local_rank: int, local_world_size: int, group=None):
        w, r = local_world_size, local_rank
        if H % 256 or I % 128 or cap_rows % 128:
            raise RuntimeError("need H % 256 == 0, I % 128 == 0 and cap_rows % 128 == 0")
        self.Tl, self.H, self.I, self.El, self.cap_rows, self.rank, self.world, self.group = tokens_per_rank, H, I, experts_local, cap_rows, r, w, group
        mk = lambda shape, dt: TKParallelTensor(shape, dt, r, w, False, group)
        self.xq_rows = [mk((tokens_per_rank, H // 2 + H // 16), torch.uint8) for _ in range(2)]
        self.slots = [mk((w,), torch.int64) for _ in range(2)]
        self.flags = mk((3 * w,), torch.int32)          # [0, w) tokens quantized, [2w, 3w) call finished
        dev = self.flags.data_.device
        self.codes = torch.zeros(cap_rows, H // 2, dtype=torch.uint8, device=dev)
        self.scales = torch.zeros(cap_rows // 128, H // 64, 512, dtype=torch.uint8, device=dev)
        self.block_expert = torch.zeros(cap_rows // 128, dtype=torch.int32, device=dev)
        self.num_blocks = torch.zeros(1, dtype=torch.int32, device=dev)
        self.arrived = torch.zeros(cap_rows // 128, dtype=torch.int32, device=dev)
        self.sg = torch.zeros(1, dtype=torch.float32, device=dev)
        self.arithmetic = L.NVFP4_KERNEL_FAST
        self.epoch = 0
        if w > 1:
            dist.barrier(group=group)

    def close(self) -> None:
        for t in self.xq_rows + self.slots + [self.flags]:
            t.close()


def moe_dispatch_gemm(pre_tokens: TKParallelTensor, post_tokens, weights, outputs: torch.Tensor, padded_tokens_per_expert: torch.Tensor,
                      pull_dispatch_indices: torch.Tensor, barrier: MoEDispatchGemmState, num_comm_sms: int, num_padded_local_tokens: int) -> None:
    """The reference's entry (kernels/parallel/moe_dispatch_gemm/moe_dispatch_gemm_h100.cu:260-299) with its argument list and
    its host-built schedule: `padded_tokens_per_expert` int32[E] over ALL experts, `pull_dispatch_indices` int32[rows, 2] of
    (source rank, source row) per row of this rank's expert segments, (-1, -1) for padding (benchmark.py:112-149).
    Differences, all on the data side: `weights` is this rank's stacked expert weights as the NVFP4 triple (codes
    [E_local * I, H/2], scales, per-tensor scale) instead of a bf16 [E_local, H, I] tensor; the tokens of `pre_tokens`
    (bf16 [T/world, H], this rank's rows) are quantized to NVFP4 with the amax of all ranks before they travel;
    `post_tokens` (the reference's bf16 gather buffer) is not used and may be None; `barrier` is the state object above.
    outputs [num_padded_local_tokens, I] bf16.  num_comm_sms == 0 dispatches with the gather kernel on all SMs."""
    st = barrier
    lib, s = L.lib(), _stream()
    w, r = st.world, st.rank
    W, W_sc, W_sg = weights
    rows = int(num_padded_local_tokens)
    if rows % 128 or rows > st.cap_rows or rows < 128:
        raise RuntimeError("num_padded_local_tokens must be a positive multiple of 128 within the state's cap_rows")
    if tuple(outputs.shape) != (rows, st.I) or outputs.dtype != torch.bfloat16 or not outputs.is_contiguous():
        raise RuntimeError("outputs must be a contiguous bf16 tensor of shape (num_padded_local_tokens, I)")
    if pull_dispatch_indices.dtype != torch.int32 or tuple(pull_dispatch_indices.shape) != (rows, 2) or not pull_dispatch_indices.is_contiguous():
        raise RuntimeError("pull_dispatch_indices must be a contiguous int32 tensor of shape (num_padded_local_tokens, 2)")
    X = pre_tokens.data_
    st.epoch += 1
    e, b = st.epoch, st.epoch % 2
    fl = st.flags.data_.data_ptr()
    # the token set of parity b was last read by the peers' kernels of call e - 2
    if w > 1 and e > 2:
        L.check(lib.tkb_wait_flags(fl + 4 * 2 * w, w, r, e - 2, s))
    # local expert of every 128-row block, from the padded counts of this rank's experts (no host synchronisation)
    local = padded_tokens_per_expert[r * st.El:(r + 1) * st.El].to(torch.int64) // 128
    st.block_expert[:rows // 128] = torch.repeat_interleave(torch.arange(st.El, device=local.device, dtype=torch.int32), local, output_size=rows // 128)
    st.num_blocks.fill_(rows // 128)
    L.check(lib.tkb_nvfp4_quantize_sharded(X.data_ptr(), 0, st.xq_rows[b].data_.data_ptr(), None, st.sg.data_ptr(), st.Tl, st.H, 1, st.arithmetic,
                                           st.slots[b].peer_ptr_array(), w, r, e, s))
    if w > 1:
        L.check(lib.tkb_signal_peers(st.flags.peer_ptr_array(), w, r, r, e, 0, s))
    L.check(lib.tkb_moe_dispatch_gemm(st.xq_rows[b].peer_ptr_array(), st.sg.data_ptr(), st.codes.data_ptr(), st.scales.data_ptr(), W.data_ptr(),
                                      W_sc.data_ptr(), W_sg.data_ptr(), outputs.data_ptr(), 0, pull_dispatch_indices.data_ptr(),
                                      st.block_expert.data_ptr(), st.num_blocks.data_ptr(), fl, st.arrived.data_ptr(), e, st.H, st.I, st.El,
                                      rows, r, w, num_comm_sms, s))
    if w > 1:
        L.check(lib.tkb_signal_peers(st.flags.peer_ptr_array(), w, r, 2 * w + r, e, 0, s))       # done with the peers' tokens of this call


class GemmReduceScatterNVFP4:
    """Row-parallel linear layer with NVFP4 operands (the partner of AllGatherMatmulNVFP4; mirrors the reference's
    matmul_reduce_scatter, kernels/parallel/gemm_rs/gemm_rs_b200.cu:204-233): every rank holds a K-slice of the activations
    [M, K/world] and of the weights [N, K/world], both NVFP4, and receives rows [rank * M/world, (rank+1) * M/world) of their
    product summed over the ranks.  `out` is this rank's bf16 [M/world, N] result, valid after a call in stream order."""

    def __init__(self, M: int, N: int, local_rank: int, local_world_size: int, group=None):
        w = local_world_size
        if M % (256 * w) or N % 8:
            raise RuntimeError("M must be a multiple of 256 * world size and N of 8")
        self.M, self.N, self.rank, self.world = M, N, local_rank, w
        self._out = TKParallelTensor((M // w, N), torch.bfloat16, local_rank, w, False, group)
        self._flags = TKParallelTensor((2 * w,), torch.int32, local_rank, w, False, group)
        self.out = self._out.data_
        st = L.RsState()
        st.rank, st.world, st.M, st.N = local_rank, w, M, N
        for i in range(w):
            st.out[i] = self._out.peer_ptr(i); st.flags[i] = self._flags.peer_ptr(i)
        maps = C.c_void_p()
        L.check(L.lib().tkb_rs_maps_create(C.byref(st), C.byref(maps)))
        st.maps = maps.value
        self._state, self._maps, self.epoch = st, maps.value, 0
        if w > 1:
            dist.barrier(group=group)

    def __call__(self, A, A_sc, A_sg, B, B_sc, B_sg) -> torch.Tensor:
        k_local = A.shape[1] * 2
        if A.shape[0] != self.M or B.shape[0] != self.N or B.shape[1] != A.shape[1]:
            raise RuntimeError("A must be [M, K_local/2] and B [N, K_local/2] packed NVFP4 codes")
        self.epoch += 1
        L.check(L.lib().tkb_gemm_rs_nvfp4(C.byref(self._state), self.epoch, A.data_ptr(), A_sc.data_ptr(), A_sg.data_ptr(), B.data_ptr(),
                                          B_sc.data_ptr(), B_sg.data_ptr(), k_local, _stream()))
        return self.out

    def close(self) -> None:
        torch.cuda.synchronize()
        if self._maps is not None:
            L.lib().tkb_rs_maps_destroy(self._maps)
            self._maps = None
        self.out = None
        self._out.close(); self._flags.close()
