"""The work schedule of the CTA-pair GEMM kernel and the planner's arithmetic (csrc/schedule.cuh), compiled for the host:
every k block of every tile is computed exactly once, a cut tile has one head whose chain of slots reaches every piece, and
no pair ever waits for work that cannot have started."""
import ctypes as C

import numpy as np
import pytest

from test_numerics_host import hc  # noqa: F401  (the compiled host library)

WORK_TILE, WORK_WRITER, WORK_OWNER, NO_SLOT = 0, 1, 2, 0xFFFFFFFF


def items_of(hc, params, cut, pair, pairs):
    buf = np.zeros(8 * 64, np.uint32)
    n = hc.hc_schedule_items(np.asarray(params, np.uint32).ctypes.data_as(C.c_void_p), int(cut), pair, pairs, buf.ctypes.data_as(C.c_void_p), 64)
    assert 0 <= n <= 64
    return buf[: 8 * n].reshape(n, 8).tolist()


def plan(hc, rem, units, nkb, any_cut):
    hc.hc_plan_cut_tail.restype = C.c_uint64
    out = np.zeros(3, np.uint32)
    cost = hc.hc_plan_cut_tail(C.c_uint64(rem), C.c_uint64(units), nkb, int(any_cut), out.ctypes.data_as(C.c_void_p))
    return tuple(int(v) for v in out), int(cost)


@pytest.mark.parametrize("m_tiles,n_tiles,batches,nkb,units", [(4, 32, 1, 64, 74), (98, 1, 1, 36, 74), (2, 3, 1, 32, 74), (10, 8, 1, 16, 74),
                                                                (1, 1, 3, 16, 74), (4, 32, 1, 128, 74), (7, 11, 2, 24, 60), (5, 5, 1, 9, 8)])
def test_cut_tail_schedule_covers_every_k_block_once_and_cannot_deadlock(hc, m_tiles, n_tiles, batches, nkb, units):
    tiles = m_tiles * n_tiles * batches
    rem = tiles % units
    (head, piece, pieces), _ = plan(hc, rem, units, nkb, True)
    if head == 0:
        pytest.skip("no cut exists for this shape")
    assert 4 <= head < nkb and piece >= 2 and head + (pieces - 1) * piece < nkb <= head + pieces * piece and rem * pieces <= 224
    params = [m_tiles, n_tiles, batches, 1, 16, nkb, rem, head, piece, pieces]
    per_pair = [items_of(hc, params, True, pr, units) for pr in range(units)]
    covered, writer_of, readers = {}, {}, []
    for pr, items in enumerate(per_pair):
        for idx, (m0, n0, b, k0, k1, kind, slot, above) in enumerate(items):
            assert 0 <= k0 < k1 <= nkb
            covered.setdefault((m0, n0, b), []).append((k0, k1, kind, slot, above, pr, idx))
            if kind == WORK_WRITER:
                assert slot not in writer_of
                writer_of[slot] = (pr, idx)
            if kind != WORK_TILE and above != NO_SLOT:
                readers.append((pr, idx, above))
    assert len(covered) == tiles
    cut_tiles = 0
    for key, parts in covered.items():
        parts.sort()
        assert parts[0][0] == 0 and parts[-1][1] == nkb and all(a[1] == b[0] for a, b in zip(parts, parts[1:])), (key, parts)
        if len(parts) == 1:
            assert parts[0][2] == WORK_TILE
            continue
        cut_tiles += 1
        assert parts[0][2] == WORK_OWNER and all(q[2] == WORK_WRITER for q in parts[1:])
        # sums travel down the pieces: each piece reads the slot of the piece after it, the last piece reads none
        for q, nxt in zip(parts, parts[1:]):
            assert q[4] == nxt[3]
        assert parts[-1][4] == NO_SLOT
    assert cut_tiles == rem and len(writer_of) == rem * pieces
    # run it: a pair executes its items in order; an item that reads a slot finishes after the slot's writer has finished
    done, pos, progress = set(), [0] * units, True
    while progress:
        progress = False
        for pr in range(units):
            while pos[pr] < len(per_pair[pr]):
                kind, above = per_pair[pr][pos[pr]][5], per_pair[pr][pos[pr]][7]
                if kind != WORK_TILE and above != NO_SLOT and writer_of[above] not in done:
                    break
                done.add((pr, pos[pr]))
                pos[pr] += 1
                progress = True
    assert all(pos[pr] == len(per_pair[pr]) for pr in range(units)), "a pair waits for a slot nobody can write"
    # every slot is written by a pair that waits for nothing that has not started: a writer never follows an owner
    for pr, items in enumerate(per_pair):
        kinds = [it[5] for it in items]
        if WORK_OWNER in kinds:
            assert kinds[0] == WORK_OWNER and WORK_WRITER not in kinds
        # whole tiles come last
        assert kinds == sorted(kinds, key=lambda k: k == WORK_TILE)


@pytest.mark.parametrize("m_tiles,n_tiles,batches,split_k,pairs", [(32, 32, 1, 1, 74), (9, 1, 1, 8, 72), (3, 5, 4, 1, 7), (98, 1, 1, 1, 74)])
def test_plain_schedule_is_the_round_robin_over_the_raster(hc, m_tiles, n_tiles, batches, split_k, pairs):
    params = [m_tiles, n_tiles, batches, split_k, 16, 40, 0, 0, 0, 0]
    seen = set()
    for pr in range(pairs):
        for m0, n0, b, k0, k1, kind, slot, above in items_of(hc, params, False, pr, pairs):
            assert (m0, n0, b, k0) not in seen
            seen.add((m0, n0, b, k0))
            assert m0 % 128 == 0 and m0 // 128 < m_tiles and n0 < n_tiles and b < batches
    assert len(seen) == m_tiles * n_tiles * batches * split_k


def test_planner_numbers(hc):
    # the headline's share at eight GPUs: 54 tiles of 64 k blocks left over on 74 pairs -> heads of 48, one piece of 16
    assert plan(hc, 54, 74, 64, False) == ((48, 16, 1), 52)
    # eight images of the ResNet-shaped convolution: 24 tiles of 36 k blocks -> heads of 12 and two pieces of 12
    assert plan(hc, 24, 74, 36, False)[0] == (12, 12, 2)
    # nothing left over, or nobody left to help: no cut
    assert plan(hc, 0, 74, 64, True)[0] == (0, 0, 0) and plan(hc, 74, 74, 64, True)[0] == (0, 0, 0)
    # many short pieces cost their epilogues: 64 tiles on 74 pairs are not cut unless asked
    assert plan(hc, 64, 74, 64, False)[0] == (0, 0, 0) and plan(hc, 64, 74, 64, True)[0][0] > 0
    assert hc.hc_plan_raster_group(C.c_uint64(256), C.c_uint64(8192), 1) == 16      # fp8: 16 x 2 MiB
    assert hc.hc_plan_raster_group(C.c_uint64(256), C.c_uint64(8192), 2) == 8       # bf16: 16 x 4 MiB would not stay
    assert hc.hc_plan_raster_group(C.c_uint64(256), C.c_uint64(2304), 2) == 16      # the convolutions' K
    assert hc.hc_plan_raster_group(C.c_uint64(256), C.c_uint64(12288), 4) == 16     # 32-bit operands keep 16
