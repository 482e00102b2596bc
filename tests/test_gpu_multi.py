"""KV-axis split of one long sequence across two GPUs with the real kernels: each rank holds only its block range in
its own pool, runs the partial-state decode, the states are all-gathered over NCCL and merged on every rank.
Needs two GPUs; skipped otherwise."""
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch.distributed as dist
    from kriya_rt_b200 import sharding, workloads as W
    from kriya_rt_b200.executor import CudaExecutor
    from oracle import c_oracle as O

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        Hq, Hkv, D, tokens = 16, 2, 128, 16384 + 5
        nb = (tokens + 15) // 16
        rng = np.random.default_rng(81)  # same stream on every rank: the full K/V exists on the host only
        k = W.normal16(rng, (nb, 16, Hkv, D), W.BF16); v = W.normal16(rng, (nb, 16, Hkv, D), W.BF16)
        q16 = W.normal16(rng, (1, Hq, D), W.BF16)
        b, e = sharding.kv_axis_ranges([nb], world)[rank]
        n_local = int(e[0] - b[0])
        pool_blocks = n_local + 7
        local_ids = np.random.default_rng(90 + rank).permutation(pool_blocks)[:n_local]
        ex = CudaExecutor(num_layers=1, num_kv_blocks=pool_blocks, block_size_tokens=16, num_q_heads=Hq, num_kv_heads=Hkv,
                          head_dim=D, device=rank, max_page_indices=nb)
        kview, vview = ex.layer_cache_views(0)
        ids = torch.from_numpy(local_ids.astype(np.int64)).cuda()
        kview[ids] = torch.from_numpy(k[int(b[0]):int(e[0])].view(np.int16)).cuda()
        vview[ids] = torch.from_numpy(v[int(b[0]):int(e[0])].view(np.int16)).cuda()
        table = sharding.local_block_table(np.zeros(nb), int(b[0]), int(e[0]), local_ids)
        qd = torch.from_numpy(q16.view(np.int16)).cuda()
        out = torch.zeros_like(qd)
        torch.cuda.synchronize()
        ex.plan_upload([0, nb], table, [tokens - (nb - 1) * 16], None, [tokens - 1])
        sharding.kv_split_decode(ex, 0, qd, b, e, out, ex.gqa_params())
        ex.sync()
        got = W.from_storage(out.cpu().numpy().view(np.uint16), W.BF16)
        p = O.GqaParams(Hq, Hkv, D, 16, 16, 1, float(np.float32(1.0) / np.sqrt(np.float32(D))), 0.0)
        _, ref = O.decode(q16, k, v, [0, nb], np.arange(nb), [tokens - (nb - 1) * 16], p, W.BF16)
        q.put((rank, float(np.abs(got - ref).max())))
        ex.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_axis_split_two_gpus_nccl():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in results:
        assert err <= 1e-2, (rank, err)
