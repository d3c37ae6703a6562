"""The oracle's MoE dispatch schedule against the reference's definition of it.

The reference builds the schedule in its benchmark script (kernels/parallel/moe_dispatch_gemm/benchmark.py:123-149):
per-expert counts padded to 128, one contiguous segment per local expert in expert order, and a pull list of
(source rank, source row) pairs filled by walking the source ranks as a ring that starts at the local rank, tokens in
ascending order inside a source, padding rows (-1, -1).  `reference_schedule` below restates that loop; the oracle
(and the device kernels checked against it) place the same rows in the same segments but in ascending global token
order, i.e. a permutation inside every segment.  The reference's own self-checks of a schedule (benchmark.py:151-166)
are applied to the oracle's output as well."""
import numpy as np
import pytest

import oracle as O


def reference_schedule(chosen, E, world, rank):
    """Restatement of benchmark.py:123-149 for one rank."""
    T, top_k = chosen.shape
    per_rank, e_per = T // world, E // world
    counts = np.bincount(chosen.reshape(-1), minlength=E).astype(np.int64)
    padded = (counts + 127) // 128 * 128
    e0, e1 = e_per * rank, e_per * (rank + 1)
    cursor = np.concatenate([[0], np.cumsum(padded[e0:e1 - 1])]).astype(np.int64)
    pull = np.full((int(padded[e0:e1].sum()), 2), -1, np.int64)
    for i in range(world):
        src = (i + rank) % world
        for tok in range(per_rank):
            for e in chosen[src * per_rank + tok]:
                if e0 <= e < e1:
                    le = e % e_per
                    pull[cursor[le]] = (src, tok)
                    cursor[le] += 1
    return counts, padded, pull


@pytest.mark.parametrize("T,E,top_k,world", [(256, 16, 2, 2), (512, 32, 4, 4), (1024, 64, 8, 8), (128, 8, 1, 1)])
def test_oracle_schedule_is_the_reference_schedule_up_to_order_inside_segments(T, E, top_k, world):
    rng = np.random.default_rng(T + E)
    # top_k distinct experts per token, as torch.multinomial without replacement gives the reference
    chosen = np.stack([rng.permutation(E)[:top_k] for _ in range(T)]).astype(np.int32)
    per_rank, e_per = T // world, E // world
    for rank in range(world):
        counts, padded_ref, pull_ref = reference_schedule(chosen, E, world, rank)
        padded, pull, slot = O.moe_schedule(chosen, E, per_rank, rank * e_per, (rank + 1) * e_per)
        assert np.array_equal(padded, padded_ref)
        assert pull.shape == pull_ref.shape
        start = 0
        for e in range(rank * e_per, (rank + 1) * e_per):
            n, npad = int(counts[e]), int(padded_ref[e])
            seg, seg_ref = pull[start:start + npad], pull_ref[start:start + npad]
            # same rows in the segment, padding at its end in both
            assert sorted(map(tuple, seg[:n].tolist())) == sorted(map(tuple, seg_ref[:n].tolist()))
            assert (seg[n:] == -1).all() and (seg_ref[n:] == -1).all()
            # the oracle's order: ascending global token; the reference's: ring of source ranks starting at `rank`
            glob = seg[:n, 0] * per_rank + seg[:n, 1]
            assert np.array_equal(glob, np.sort(glob))
            ring = (seg_ref[:n, 0] - rank) % world
            assert np.array_equal(ring, np.sort(ring))
            # the reference's self-checks (benchmark.py:151-166)
            assert seg[n:].sum() == (n - npad) * 2
            assert (seg[:n] >= 0).all() and (seg[:n, 1] < per_rank).all() and (glob < T).all()
            assert np.unique(glob).size == n
            for s, t in seg[:n]:
                assert e in chosen[s * per_rank + t]
            start += npad
        # the combine map points every routed pair of the tokens at the row that pulls it
        for t in range(T):
            for j in range(top_k):
                if slot[t, j] >= 0:
                    assert tuple(pull[slot[t, j]]) == (t // per_rank, t % per_rank) and chosen[t, j] // e_per == rank
