"""Shared MoE test logic: runs the layer on the calling rank and checks every stage against the CPU oracle."""
import numpy as np
import torch

import oracle as O
from tests.util import bf16_bits, to_dev_u8, rel_fro, bf16_ulp_diff


def make_problem(T, H, I, E, seed=0):
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g, dtype=torch.float32)
    W = (torch.randn(E, I, H, generator=g) * 0.02).to(torch.bfloat16)
    return X, logits, W


def make_problem_sharded(T, H, I, E, rank, world, seed=0):
    """The same kind of problem for sizes whose full weight tensor is too large to build on every rank: activations and
    logits are identical on all ranks (one seeded stream), the expert weights are generated for this rank's experts only."""
    rng = np.random.default_rng(seed)
    X = torch.from_numpy(rng.standard_normal((T, H), dtype=np.float32)).to(torch.bfloat16)
    logits = torch.from_numpy(rng.standard_normal((T, E), dtype=np.float32))
    El = E // world
    rw = np.random.default_rng(seed * 1000 + 17 + rank)
    Wl = torch.from_numpy(rw.standard_normal((El, I, H), dtype=np.float32) * np.float32(0.02)).to(torch.bfloat16)
    return X, logits, Wl


def run_and_check(dev, rank, world, T, H, I, E, top_k, iters=2, comm_sms=4, log=print, edge=0):
    """edge > 0: weights are generated per rank and the grouped GEMM is checked on the first and last `edge` rows of every
    expert segment only (sizes at which the whole product is too much for the CPU oracle)."""
    from thunderkittens_b200 import parallel, _lib
    Tl, El = T // world, E // world
    layer = parallel.MoELayerNVFP4(T, H, I, E, top_k, rank, world, num_comm_sms=comm_sms)
    layer.arithmetic = _lib.NVFP4_SPEC          # the CPU-reproducible quantizer arithmetic
    ok = True
    for it in range(iters):
        if edge > 0:
            X, logits, Wl = make_problem_sharded(T, H, I, E, rank, world, seed=100 + it)
            Wl = Wl.reshape(El * I, H)
        else:
            X, logits, W = make_problem(T, H, I, E, seed=100 + it)
            # this rank's stacked expert weights, quantized as one tensor
            Wl = W[rank * El:(rank + 1) * El].reshape(El * I, H)
        wq = O.nvfp4_quantize(bf16_bits(Wl))
        # both host paths of the layer on alternating calls: the single library call and the spelled-out sequence
        step = layer.forward if it % 2 == 0 else layer.forward_step_by_step
        out = step(logits[rank * Tl:(rank + 1) * Tl].contiguous().to(dev), X[rank * Tl:(rank + 1) * Tl].contiguous().to(dev),
                            to_dev_u8(wq[0], dev), to_dev_u8(wq[1], dev), torch.from_numpy(wq[2]).to(dev))
        torch.cuda.synchronize()
        st = _lib.device_status()
        # ---- oracle
        experts, weights = O.moe_route(logits.numpy(), top_k)
        padded, pull, slot = O.moe_schedule(experts, E, Tl, rank * El, (rank + 1) * El)
        g_exp = layer.experts_all.cpu().numpy()      # the gathered routing decisions of this call
        g_w = layer.weights.cpu().numpy()
        route_ok = np.array_equal(g_exp, experts) and np.allclose(g_w, weights[rank * Tl:(rank + 1) * Tl], rtol=1e-5, atol=1e-7)
        rows = pull.shape[0]
        sched_ok = (np.array_equal(layer.padded.cpu().numpy(), padded) and int(layer.num_blocks.item()) == rows // 128
                    and np.array_equal(layer.pull_idx.cpu().numpy()[:rows], pull))
        # combine map of my tokens: (owner rank, row on the owner)
        comb = layer.comb_idx.cpu().numpy().reshape(Tl, top_k, 2)
        comb_ok = True
        for owner in range(world):
            _, _, slot_o = O.moe_schedule(experts, E, Tl, owner * El, (owner + 1) * El)
            mine = slot_o[rank * Tl:(rank + 1) * Tl]
            sel = mine >= 0
            comb_ok = comb_ok and np.array_equal(comb[..., 0][sel], np.full(sel.sum(), owner)) and np.array_equal(comb[..., 1][sel], mine[sel])
        # grouped GEMM: per local expert, gather the quantized token rows and multiply on the CPU
        xq = O.nvfp4_quantize(bf16_bits(X), False, "spec")
        x_sc_rows = O.unswizzle_scales(xq[1], T)
        Y = bf16_bits(layer.Y.data_[:rows])
        w_sc_rows = O.unswizzle_scales(wq[1], El * I)
        gemm_ok, worst = True, 0.0
        start = 0
        for el in range(El):
            n = padded[rank * El + el]
            if n == 0:
                continue
            if edge > 0:
                # the first and the last `edge` rows of the segment (padded to a whole 128-row scale block for the oracle)
                sel = np.concatenate([np.arange(edge), np.arange(n - edge, n)])
                seg = np.full((128, 2), -1, pull.dtype)
                seg[:2 * edge] = pull[start + sel]
                got = Y[start + sel]
            else:
                seg = pull[start:start + n]
                got = Y[start:start + n]
            tok = np.where(seg[:, 0] >= 0, seg[:, 0] * Tl + seg[:, 1], 0)
            valid = seg[:, 0] >= 0
            a_codes = np.where(valid[:, None], xq[0][tok], 0).astype(np.uint8)
            a_sc = O.swizzle_scales(np.where(valid[:, None], x_sc_rows[tok], 0).astype(np.uint8))
            ref = O.nvfp4_gemm(a_codes, a_sc, xq[2], wq[0][el * I:(el + 1) * I], O.swizzle_scales(w_sc_rows[el * I:(el + 1) * I]), wq[2])
            if edge > 0:
                ref = ref[:2 * edge]
            err = rel_fro(O.bf16_to_f32(got), O.bf16_to_f32(ref))
            rr = O.bf16_to_f32(ref)
            big = np.abs(rr) > 1e-2 * np.sqrt((rr.astype(np.float64) ** 2).mean() + 1e-30)
            ulp = int(bf16_ulp_diff(got, ref)[big].max()) if big.any() else 0
            worst = max(worst, err)
            gemm_ok = gemm_ok and err <= 1e-3 and ulp <= 2
            start += n
        out_ok = True
        if world == 1:
            # combine: same fp32 fused multiply-adds in the same order -> bit-exact given the GPU's Y and weights
            ref_out = O.moe_combine(bf16_bits(layer.Y.data_[:max(rows, 1)]), slot, g_w)
            out_ok = np.array_equal(bf16_bits(out), ref_out)
        good = st == 0 and route_ok and sched_ok and comb_ok and gemm_ok and out_ok
        log(f"rank {rank} iter {it}: status={st} route={route_ok} schedule={sched_ok} combine_map={comb_ok} gemm={gemm_ok} (rel_fro {worst:.1e}) "
            f"combine_out={out_ok} rows={rows}")
        ok = ok and good
    return ok, layer
