"""Host logic of the multi-GPU schemes on CPU ranks (gloo, world size 2): sequence assignment, KV-axis ranges and
the state gather.  Each rank evaluates its share with the CPU oracle; the merged result must equal the
single-rank evaluation."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _kv_split_worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from kriya_rt_b200 import sharding, workloads as W
    from oracle import c_oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        O.set_num_threads(1)
        shape, batch, data = W.config1(dtype=W.BF16)
        p = O.GqaParams(9, 3, 64, 16, 16, 1, float(np.float32(1.0) / np.sqrt(np.float32(64))), 0.0)
        nblk = np.diff(batch.page_indptr)
        b, e = sharding.kv_axis_ranges(nblk, world)[rank]
        m, l, o = O.decode_partial(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr, batch.page_indices,
                                   batch.last_page_len, b, e, p, W.BF16)
        m_all, l_all, o_all = sharding.gather_states(torch.from_numpy(m.reshape(-1)), torch.from_numpy(l.reshape(-1)),
                                                     torch.from_numpy(o.reshape(-1, 64)))
        merged = O.merge_states(m_all.numpy(), l_all.numpy(), o_all.numpy())
        _, whole = O.decode(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr, batch.page_indices,
                            batch.last_page_len, p, W.BF16)
        q.put((rank, float(np.abs(merged - whole.reshape(-1, 64)).max()), tuple(m_all.shape)))
    finally:
        dist.destroy_process_group()


def test_kv_axis_split_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_kv_split_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, shape in results:
        assert err < 1e-5 and shape == (2, 36)


def _seq_shard_worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    import torch.distributed as dist
    from kriya_rt_b200 import sharding, workloads as W
    from kriya_rt_b200.kv import PagedKvCacheManager
    from oracle import c_oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        O.set_num_threads(1)
        rng = np.random.default_rng(9)
        lengths = rng.integers(20, 400, size=11)
        mine = sharding.assign_sequences(lengths, world)[rank]
        # each rank owns a manager and a pool; sequences keep their global ids
        mgr = PagedKvCacheManager(256, 0, 16)
        for s in mine:
            mgr.allocate_sequence(int(s), (np.arange(int(lengths[s])) + 1000 * int(s)).astype(np.uint32))
        plan = mgr.build_schedule_plan([int(s) for s in mine], 8)
        # every sequence's K/V and q are a function of its global id, so any placement must give the same output
        Hq, Hkv, D = 4, 2, 64
        ck = np.zeros((256, 16, Hkv, D), np.uint16); cv = np.zeros((256, 16, Hkv, D), np.uint16)
        qs = np.zeros((len(mine), Hq, D), np.uint16)
        for i, s in enumerate(mine):
            r2 = np.random.default_rng(100 + int(s))
            L = int(lengths[s])
            k = W.normal16(r2, (L, Hkv, D), W.BF16); v = W.normal16(r2, (L, Hkv, D), W.BF16)
            qs[i] = W.normal16(r2, (Hq, D), W.BF16)
            blocks, _ = mgr.sequence_table(int(s))
            for t in range(L):
                ck[blocks[t // 16], t % 16] = k[t]; cv[blocks[t // 16], t % 16] = v[t]
        p = O.GqaParams(Hq, Hkv, D, 16, 16, 1, 0.125, 0.0)
        _, out = O.decode(qs, ck, cv, plan.page_indptr, plan.page_indices, plan.last_page_len, p, W.BF16)
        # gather (sequence id, checksum) pairs on every rank
        local = torch.zeros(len(lengths), dtype=torch.float64)
        for i, s in enumerate(mine):
            local[int(s)] = float(np.abs(out[i]).sum())
        dist.all_reduce(local)
        q.put((rank, local.numpy().tolist(), [int(s) for s in mine]))
    finally:
        dist.destroy_process_group()


def test_sequence_sharding_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_seq_shard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, sums0, mine0), (r1, sums1, mine1) = results
    assert sums0 == sums1 and all(s > 0 for s in sums0)  # every sequence was served by exactly one rank
    assert sorted(mine0 + mine1) == list(range(11)) and not set(mine0) & set(mine1)
    # single-rank evaluation gives the same per-sequence checksums
    from kriya_rt_b200 import sharding

    lengths = np.random.default_rng(9).integers(20, 400, size=11)
    loads = [sum(int(lengths[i]) for i in part) for part in sharding.assign_sequences(lengths, 2)]
    assert abs(loads[0] - loads[1]) <= int(lengths.max())


def test_kv_axis_ranges_tile_each_row():
    from kriya_rt_b200 import sharding

    nb = np.array([1, 7, 8, 9, 1024, 8192, 3])
    for ranks in (1, 2, 4, 8):
        parts = sharding.kv_axis_ranges(nb, ranks)
        assert np.array_equal(parts[0][0], np.zeros_like(nb)) and np.array_equal(parts[-1][1], nb)
        for a, b in zip(parts[:-1], parts[1:]):
            assert np.array_equal(a[1], b[0])
    t = sharding.local_block_table(list(range(100, 120)), 5, 9, [3, 1, 4, 2])
    assert t[5:9].tolist() == [3, 1, 4, 2] and t.sum() == 10
