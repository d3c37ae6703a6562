"""World-size-2 tests of the multi-rank HOST logic on CPU (gloo): the sharding rules the tensor-parallel and
MoE paths rely on (checked with the oracle) and the symmetric-buffer handle exchange (with the CUDA library
replaced by a recording fake).  No GPU is involved."""
import ctypes
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class FakeLib:
    """Stands in for libtkb200 where the host code only moves handles around."""

    def __init__(self, rank):
        self.rank, self.next, self.closed = rank, 0x1000 * (rank + 1), []

    def tkb_dev_alloc(self, nbytes, out):
        out._obj.value = self.next
        self.next += 0x100
        return 0

    def tkb_ipc_export(self, ptr, handle):
        payload = (self.rank.to_bytes(8, "little") + int(ptr).to_bytes(8, "little")).ljust(64, b"\0")
        ctypes.memmove(handle, payload, 64)
        return 0

    def tkb_ipc_open(self, handle, out):
        raw = bytes(handle)
        owner, ptr = int.from_bytes(raw[:8], "little"), int.from_bytes(raw[8:16], "little")
        out._obj.value = (owner << 40) | ptr       # "address of rank `owner`'s buffer as seen from here"
        return 0

    def tkb_ipc_close(self, ptr):
        self.closed.append(ptr)
        return 0

    def tkb_dev_free(self, ptr):
        return 0

    def tkb_last_error(self):
        return b""

    # the single-call entry points: record what the host layer hands to the library
    def tkb_ag_linear_nvfp4(self, st, epoch, X, W, W_sc, W_sg, D, ldd, n_local, comm, arith, stream):
        self.calls = getattr(self, "calls", []) + [("ag_linear", int(epoch), int(n_local), int(comm), int(arith))]
        self.last_state = st._obj
        return 0

    def tkb_moe_layer_nvfp4(self, st, epoch, logits, X, W, W_sc, W_sg, out, comm, arith, stream):
        self.calls = getattr(self, "calls", []) + [("moe_layer", int(epoch), int(comm), int(arith))]
        self.last_state = st._obj
        return 0


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle as O
    res = {}
    # ---- 1. tensor parallel: shards quantized with the all-reduced amax equal quantize(full tensor)
    rng = np.random.default_rng(7)
    M, K = 256 * world, 256
    X = O.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32) * np.linspace(0.5, 3.0, M)[:, None].astype(np.float32))
    rows = M // world
    shard = X[rank * rows:(rank + 1) * rows]
    amax = torch.tensor([O.absmax_bf16(shard)], dtype=torch.float32)
    dist.all_reduce(amax, op=dist.ReduceOp.MAX)
    c, s, g = O.nvfp4_quantize(shard, False, "spec", amax=float(amax.item()))
    parts = [None] * world
    dist.all_gather_object(parts, (c, s, g))
    fc, fs, fg = O.nvfp4_quantize(X, False, "spec")
    res["tp_codes"] = np.array_equal(np.concatenate([p[0] for p in parts]), fc)
    res["tp_scales"] = np.array_equal(np.concatenate([p[1] for p in parts]), fs)
    res["tp_sg"] = all(p[2][0] == fg[0] for p in parts)
    # ---- 2. MoE: every (token, slot) pair lands in exactly one row of exactly one rank, and the combine map points at it
    T, E, k = 64 * world, 8 * world, 2
    logits = rng.standard_normal((T, E)).astype(np.float32)
    Tl, El = T // world, E // world
    my_exp, my_w = O.moe_route(logits[rank * Tl:(rank + 1) * Tl], k)
    gathered = [torch.zeros(Tl, k, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(my_exp))
    experts_all = torch.cat(gathered).numpy()
    res["moe_route_consistent"] = np.array_equal(experts_all, O.moe_route(logits, k)[0])
    padded, pull, slot = O.moe_schedule(experts_all, E, Tl, rank * El, (rank + 1) * El)
    pulls = [None] * world
    dist.all_gather_object(pulls, (pull, slot))
    seen = np.zeros((T, k), np.int32)
    ok_map = True
    for owner, (pl, sl) in enumerate(pulls):
        for t in range(T):
            for j in range(k):
                if sl[t, j] >= 0:
                    seen[t, j] += 1
                    ok_map = ok_map and tuple(pl[sl[t, j]]) == (t // Tl, t % Tl) and experts_all[t, j] // El == owner
    res["moe_cover_once"] = bool((seen == 1).all())
    res["moe_map"] = ok_map
    res["moe_padding"] = bool((padded % 128 == 0).all()) and pull.shape[0] == int(padded[rank * El:(rank + 1) * El].sum())
    # ---- 3. symmetric buffer handle exchange with a fake library
    from thunderkittens_b200 import _lib, parallel
    fake = FakeLib(rank)
    _lib.lib = lambda: fake
    _lib.check = lambda code: None
    parallel.TKParallelTensor._view = lambda self: torch.zeros(self.shape_, dtype=self.dtype_)
    t = parallel.TKParallelTensor((4, 8), torch.int32, rank, world)
    res["peer_table"] = [t.peer_ptr(r) for r in range(world)]
    res["own_ptr"] = t._ptr
    arr = t.peer_ptr_array()
    res["peer_array"] = [int(arr[i]) for i in range(world)]
    t.close.__func__   # exists
    # ---- 4. the layer objects hand complete peer tables to the single-call entry points
    parallel._stream = lambda: 0
    op = parallel.AllGatherMatmulNVFP4(256 * world, 256, rank, world, num_comm_sms=5)
    st = op._state
    ok = (st.rank, st.world, st.M, st.K) == (rank, world, 256 * world, 256) and op.num_comm_sms == 4      # rounded down to whole CTA pairs
    for b in range(2):
        for i in range(world):
            ok = ok and st.codes[b][i] == op.codes[b].peer_ptr(i) and st.scales[b][i] == op.scales[b].peer_ptr(i)
            ok = ok and st.arrived[b][i] == op.arrived[b].peer_ptr(i) and st.slots[b][i] == op.slots[b].peer_ptr(i)
    ok = ok and all(st.done[i] == op.flags.peer_ptr(i) for i in range(world)) and st.exit_counter == op.exit_counter.data_ptr()
    ok = ok and op.arrived[0].shape_ == (256 * world // 8,)
    Xl = torch.zeros(256, 256, dtype=torch.bfloat16); Wq = torch.zeros(128, 128, dtype=torch.uint8)
    Wsc = torch.zeros(1, 4, 512, dtype=torch.uint8); Wsg = torch.zeros(1); Dd = torch.zeros(256 * world, 128, dtype=torch.bfloat16)
    op(Xl, Wq, Wsc, Wsg, Dd); op(Xl, Wq, Wsc, Wsg, Dd)
    res["ag_calls"] = [c for c in fake.calls if c[0] == "ag_linear"]
    # the gather with push warps in every CTA of the GEMM travels as comm = -2, and needs no copy context
    op_push = parallel.AllGatherMatmulNVFP4(256 * world, 256, rank, world, push_warps=True)
    op_push(Xl, Wq, Wsc, Wsg, Dd)
    last = [c for c in fake.calls if c[0] == "ag_linear"][-1]
    res["ag_push"] = last[1] == 1 and last[3] == (-2 if world > 1 else 0) and op_push._copy is None and not op_push.copy_engines
    try:
        op(Xl[:100], Wq, Wsc, Wsg, Dd)
        ok = False
    except RuntimeError:
        pass
    res["ag_state"] = ok
    layer = parallel.MoELayerNVFP4(128 * world, 256, 128, 16 * world, 2, rank, world, num_comm_sms=6)
    ms = layer._state
    ok = (ms.rank, ms.world, ms.T, ms.H, ms.I, ms.E, ms.top_k, ms.cap_rows) == (rank, world, 128 * world, 256, 128, 16 * world, 2, layer.cap_rows)
    for i in range(world):
        for b in range(2):
            ok = ok and ms.xq_rows[b][i] == layer.xq_rows[b].peer_ptr(i) and ms.slots[b][i] == layer.slots[b].peer_ptr(i)
            ok = ok and ms.experts_all[b][i] == layer.experts_all_sym[b].peer_ptr(i)
        ok = ok and ms.Y[i] == layer.Y.peer_ptr(i) and ms.flags[i] == layer.flags.peer_ptr(i) and ms.counters[i] == layer.counters.peer_ptr(i)
    ok = ok and ms.codes == layer.codes.data_ptr() and ms.pull_idx == layer.pull_idx.data_ptr() and ms.sg == layer.sg.data_ptr()
    layer.forward(torch.zeros(128, 16 * world), torch.zeros(128, 256, dtype=torch.bfloat16), Wq, Wsc, Wsg)
    res["moe_calls"] = [c for c in fake.calls if c[0] == "moe_layer"]
    res["moe_state"] = ok and layer.cap_rows % 128 == 0
    q.put((rank, res))
    dist.barrier()
    dist.destroy_process_group()


def test_world2_host_logic_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        res = results[r]
        for key in ("tp_codes", "tp_scales", "tp_sg", "moe_route_consistent", "moe_cover_once", "moe_map", "moe_padding", "ag_state", "ag_push", "moe_state"):
            assert res[key], (r, key)
        assert [c[1] for c in res["ag_calls"]] == [1, 2] and all(c[2:4] == (128, 4) for c in res["ag_calls"])      # epochs grow by one per call
        assert [c[1] for c in res["moe_calls"]] == [1] and res["moe_calls"][0][2] == 6
        # rank r sees its own pointer for itself and "rank o's pointer" for the peer
        for o in range(world):
            expect = results[o]["own_ptr"] if o == r else ((o << 40) | results[o]["own_ptr"])
            assert res["peer_table"][o] == expect and res["peer_array"][o] == expect
