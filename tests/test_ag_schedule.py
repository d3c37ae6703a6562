"""Push schedule of the all-gather GEMM's comm CTAs, enumerated on the host by the library itself
(tkb_debug_ag_schedule walks the same integer arithmetic the kernel walks): for every rank, the pieces of all
comm CTAs together cover this rank's slice of the gathered codes and scales exactly once per destination,
stay inside the slice, keep 16-byte alignment, and raise every arrival flag exactly once."""
import ctypes

import numpy as np
import pytest


def _enumerate(lib, M, K, rank, world, comm_ctas, comm_idx, piece, parts=4):
    if parts == 4:
        fn = lambda out, cap: lib.tkb_debug_ag_schedule(M, K, rank, world, comm_ctas, comm_idx, piece, out, cap)
    else:
        fn = lambda out, cap: lib.tkb_debug_ag_schedule_parts(M, K, rank, world, comm_ctas, comm_idx, piece, parts, out, cap)
    n = fn(None, 0)
    assert n >= 0
    buf = (ctypes.c_longlong * (6 * max(n, 1)))()
    assert fn(buf, n) == n
    return np.frombuffer(buf, dtype=np.int64)[:6 * n].reshape(n, 6)


# parts = 4: dedicated comm CTAs; parts = 16: the push warps of every CTA of the kernel (148 CTAs on a B200)
@pytest.mark.parametrize("M,K,world,comm_ctas,parts", [(1024, 1024, 2, 4, 4), (2048, 1024, 4, 4, 4), (4096, 256, 8, 6, 4), (8192, 8192, 8, 16, 4),
                                                       (8192, 8192, 4, 8, 4), (8192, 8192, 2, 30, 4), (512, 64, 2, 2, 4),
                                                       (8192, 8192, 8, 148, 16), (8192, 1024, 4, 148, 16), (1024, 1024, 2, 148, 16),
                                                       (512, 64, 2, 148, 16), (2048, 256, 8, 18, 16)])
@pytest.mark.parametrize("piece", [16384, 1 << 30])        # the kernel moves whole spans (piece >= span)
def test_push_schedule_covers_every_byte_once(lib, M, K, world, comm_ctas, parts, piece):
    part_rows = 256 // parts
    rows = M // world
    k_bytes, sc_mblock = K // 2, (K // 64) * 512
    for rank in range(world):
        codes_lo, codes_hi = rank * rows * k_bytes, (rank + 1) * rows * k_bytes
        sc_lo, sc_hi = rank * (rows // 128) * sc_mblock, (rank + 1) * (rows // 128) * sc_mblock
        cover = {d: (np.zeros(codes_hi - codes_lo, np.uint8), np.zeros(sc_hi - sc_lo, np.uint8)) for d in range(world) if d != rank}
        flags = {d: np.zeros(M // part_rows, np.int32) for d in range(world) if d != rank}
        first_unit_dst = []
        for ci in range(comm_ctas):
            pcs = _enumerate(lib, M, K, rank, world, comm_ctas, ci, piece, parts)
            if len(pcs):
                first_unit_dst.append(int(pcs[0, 0]))
            unit_bytes = {}
            for dst, span, off, nbytes, flag, last in pcs:
                assert dst != rank and 0 <= dst < world
                assert nbytes > 0 and nbytes % 16 == 0 and off % 16 == 0 and nbytes <= piece
                lo, hi = (codes_lo, codes_hi) if span == 0 else (sc_lo, sc_hi)
                assert lo <= off and off + nbytes <= hi, "piece leaves this rank's slice"
                cover[dst][span][off - lo:off - lo + nbytes] += 1
                # the flag's rows: the codes of a unit must be exactly those rows
                if span == 0:
                    r0 = flag * part_rows
                    assert r0 * k_bytes <= off and off + nbytes <= (r0 + part_rows) * k_bytes
                else:
                    blk = flag // parts                                 # 256-row block: its two 128-row scale blocks
                    assert blk * 2 * sc_mblock <= off and off + nbytes <= (blk + 1) * 2 * sc_mblock
                unit_bytes[(dst, flag)] = unit_bytes.get((dst, flag), 0) + nbytes
                if last:
                    flags[dst][flag] += 1
                    assert unit_bytes[(dst, flag)] == part_rows * k_bytes + 2 * sc_mblock // parts
        for d, (c, s) in cover.items():
            assert (c == 1).all() and (s == 1).all(), f"rank {rank} -> {d}: bytes missed or sent twice"
            mine = np.zeros(M // part_rows, np.int32)
            mine[rank * rows // part_rows:(rank + 1) * rows // part_rows] = 1
            assert np.array_equal(flags[d], mine), "every part of the slice raises its flag exactly once per destination"
        # the first round of units serves the destinations that consume this rank's rows first (rank-1, rank-2, ...),
        # four of them at a time, alternating between them
        fan = min(4, world - 1)
        expect = [(rank + world - 1 - (ci % fan)) % world for ci in range(min(comm_ctas, fan * (rows // 256) * parts))]
        assert first_unit_dst[:len(expect)] == expect


def test_schedule_rejects_bad_arguments(lib):
    assert lib.tkb_debug_ag_schedule(1000, 1024, 0, 2, 4, 0, 16384, None, 0) < 0       # M not a multiple of 256 * world
    assert lib.tkb_debug_ag_schedule(1024, 1024, 0, 2, 4, 4, 16384, None, 0) < 0       # comm_idx out of range
    assert lib.tkb_debug_ag_schedule(1024, 1024, 0, 2, 4, 0, 100, None, 0) < 0         # piece size not a multiple of 16
    assert lib.tkb_debug_ag_schedule_parts(1024, 1024, 0, 2, 4, 0, 16384, 8, None, 0) < 0   # parts other than 4 or 16
