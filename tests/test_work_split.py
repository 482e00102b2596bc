"""Host logic of the persistent tensor-core decode kernels' work split (no GPU): every block of every row lands in exactly
one piece, pieces are cut at tile boundaries, the bookkeeping of a run's pieces (scratch slots, piece count, the piece a CTA
takes last) is consistent, and the two lists a plan carries (a single launch: at least 8 tiles per CTA; overlapping launches
of a whole-step call: at least 14) differ the way they are meant to."""
import ctypes as C

import numpy as np
import pytest

from kriya_rt_b200 import _native as N

SMS = 148


def split(ctx, block=16, runs_per_row=1, ctas=SMS, tp=4, min_tiles=8, window=0, cap=4096):
    ctx = np.asarray(ctx, dtype=np.int64)
    nb = (ctx + block - 1) // block
    indptr = np.concatenate([[0], np.cumsum(nb)]).astype(np.int32)
    last = np.where(ctx > 0, (ctx - 1) % block + 1, 0).astype(np.int32)
    rec = np.zeros((cap, 12), np.uint32)
    ptr = np.zeros(ctas + 1, np.uint32)
    n = N.cuda_lib().kriya_cuda_debug_work_split(indptr.ctypes.data, last.ctypes.data, len(ctx), block, runs_per_row, ctas, tp, min_tiles,
                                                 window, rec.ctypes.data, cap, ptr.ctypes.data)
    return int(n), rec[: max(n, 0)], ptr, indptr, nb


def check(ctx, runs_per_row, tp, min_tiles, window=0, block=16):
    n, rec, ptr, indptr, nb = split(ctx, block, runs_per_row, SMS, tp, min_tiles, window)
    assert n > 0
    assert ptr[0] == 0 and ptr[-1] == n and np.all(np.diff(ptr.astype(np.int64)) >= 0)
    ctx = np.asarray(ctx)
    slots_seen = set()
    for r in range(len(ctx)):
        first_tok = max(0, int(ctx[r]) - window) if window else 0
        b0 = min(first_tok // block, int(nb[r]))
        for h in range(runs_per_row):
            mine = rec[(rec[:, 0] == r) & (rec[:, 1] == h)]
            assert len(mine) >= 1
            assert np.all(mine[:, 6] == len(mine))  # piece count
            assert np.all(mine[:, 5] == mine[:, 5][0])  # the run's first slot
            assert sorted(mine[:, 4].tolist()) == list(range(int(mine[0, 5]), int(mine[0, 5]) + len(mine)))
            assert np.all(mine[:, 7] == indptr[r]) and np.all(mine[:, 8] == ctx[r])
            for s in mine[:, 4]:
                assert int(s) not in slots_seen
                slots_seen.add(int(s))
            order = mine[np.argsort(mine[:, 4])]
            if nb[r] == b0:
                assert len(order) == 1 and order[0, 2] == order[0, 3]
                continue
            assert order[0, 2] == b0 and order[-1, 3] == nb[r]
            for a, b in zip(order[:-1], order[1:]):
                assert a[3] == b[2] and a[3] % tp == 0  # contiguous, cut at a tile boundary
            assert np.all(order[:, 3] > order[:, 2])
    # a CTA whose list begins with the continuation of a run takes that piece last
    tiles_per_cta = []
    for k in range(SMS):
        lo, hi = int(ptr[k]), int(ptr[k + 1])
        if hi == lo:
            continue
        if hi - lo > 1:
            assert rec[lo, 4] == rec[lo, 5] or len(set(map(tuple, rec[lo:hi, :2]))) == 1
            for i in range(lo, hi - 1):
                assert rec[i, 4] == rec[i, 5] or i == hi - 1, (k, i)  # only the CTA's last record may be a continuation
        tiles_per_cta.append(sum(int((e + tp - 1) // tp - b // tp) for b, e in rec[lo:hi, 2:4] if e > b))
    return n, np.array(tiles_per_cta)


@pytest.mark.parametrize("min_tiles", [8, 14])
def test_benchmark_shape_split_covers_every_block_once(min_tiles):
    ctx = np.random.default_rng(2002).integers(512, 4097, size=32)
    n, tiles = check(ctx, 1, 4, min_tiles)
    total = int(sum((c + 63) // 64 for c in ctx))
    assert tiles.sum() >= total  # a tile cut between two pieces never happens, a tile shared by two rows cannot
    assert len(tiles) == min(SMS, max(1, -(-total // min_tiles)))
    assert tiles.max() - tiles.min() <= 2  # even streams


def test_the_list_for_overlapping_launches_uses_fewer_ctas_with_longer_streams():
    ctx = np.random.default_rng(2002).integers(512, 4097, size=32)
    _, t8 = check(ctx, 1, 4, 8)
    _, t14 = check(ctx, 1, 4, 14)
    assert len(t14) < len(t8) <= SMS
    assert t14.min() >= 13 and t8.min() >= 7


@pytest.mark.parametrize("runs_per_row,tp", [(1, 4), (2, 8), (2, 4), (3, 8)])
def test_ragged_and_empty_rows(runs_per_row, tp):
    ctx = np.array([0, 1, 15, 16, 17, 63, 64, 65, 1000, 0, 4096, 33])
    check(ctx, runs_per_row, tp, 8)
    check(ctx, runs_per_row, tp, 1)


def test_one_long_row_is_spread_over_every_cta():
    n, tiles = check(np.array([131072]), 1, 4, 8)
    assert len(tiles) == SMS and n == SMS


@pytest.mark.parametrize("window", [1, 100, 1024])
def test_sliding_window_rows_begin_at_the_windows_first_block(window):
    ctx = np.array([5, 100, 1023, 1024, 1025, 4000, 0])
    check(ctx, 1, 4, 8, window=window)
    check(ctx, 2, 8, 8, window=window)


def test_too_small_a_record_buffer_is_reported():
    n, *_ = split(np.full(32, 4096), cap=8)
    assert n == -1
