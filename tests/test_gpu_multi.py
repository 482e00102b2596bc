"""KV-axis split of one long sequence across two GPUs through the C ABI: each rank (a process of its own) holds only its
block range in its own pool, exports its exchange buffer, maps the peer's, and runs kriya_cuda_kvsplit_decode - the
partial-state decode, the exchange over NVLink (peer stores, bounded wait) and the merge, with no collective library on
the data path.  The handles travel between the processes over a pipe.  Needs two GPUs; skipped otherwise.

A second test runs two contexts in ONE process, one thread's worth of calls per device: the kernels' per-device set-up
(shared-memory attribute) must hold on both devices."""
import sys
import traceback
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu


def _worker(rank, world, conns, result_q):
    """conns[rank]: this rank's end of a pipe to the parent, which gathers and redistributes the handles."""
    try:
        sys.path.insert(0, str(ROOT))
        sys.path.insert(0, str(ROOT / "tests"))
        from kriya_rt_b200 import sharding, workloads as W
        from kriya_rt_b200.executor import CudaExecutor
        from oracle import c_oracle as O

        torch.cuda.set_device(rank)
        Hq, Hkv, D, tokens = 16, 2, 128, 16384 + 5
        nb = (tokens + 15) // 16
        rng = np.random.default_rng(81)  # same stream on every rank: the full K/V exists on the host only
        k = W.normal16(rng, (nb, 16, Hkv, D), W.BF16); v = W.normal16(rng, (nb, 16, Hkv, D), W.BF16)
        layers = 3
        q16 = W.normal16(rng, (layers, 1, Hq, D), W.BF16)
        b, e = sharding.kv_axis_ranges([nb], world)[rank]
        n_local = int(e[0] - b[0])
        pool_blocks = n_local + 7
        local_ids = np.random.default_rng(90 + rank).permutation(pool_blocks)[:n_local]
        ex = CudaExecutor(num_layers=layers, num_kv_blocks=pool_blocks, block_size_tokens=16, num_q_heads=Hq, num_kv_heads=Hkv,
                          head_dim=D, device=rank, max_page_indices=nb)
        ids = torch.from_numpy(local_ids.astype(np.int64)).cuda()
        for layer in range(layers):  # every layer holds the same K/V; the queries differ per layer
            kview, vview = ex.layer_cache_views(layer)
            kview[ids] = torch.from_numpy(k[int(b[0]):int(e[0])].view(np.int16)).cuda()
            vview[ids] = torch.from_numpy(v[int(b[0]):int(e[0])].view(np.int16)).cuda()
        table = sharding.local_block_table(np.zeros(nb), int(b[0]), int(e[0]), local_ids)
        qd = torch.from_numpy(q16.view(np.int16)).cuda()
        out = torch.zeros_like(qd)
        torch.cuda.synchronize()
        # set-up: export, exchange the handles through the parent, map the peers
        conns[rank].send(ex.comm_export(1))
        handles = conns[rank].recv()
        ex.comm_init(rank, handles)
        ex.plan_upload([0, nb], table, [tokens - (nb - 1) * 16], None, [tokens - 1])
        ex.plan_set_ranges(b, e)
        gp = ex.gqa_params()
        ex.kvsplit_decode(0, qd[0], out[0], gp)       # one layer ...
        ex.sync()
        ex.kvsplit_decode_step(qd, out, gp)           # ... then all layers in one call (layer 0 again: same result)
        ex.sync()
        p = O.GqaParams(Hq, Hkv, D, 16, 16, 1, float(np.float32(1.0) / np.sqrt(np.float32(D))), 0.0)
        errs = []
        for layer in range(layers):
            _, ref = O.decode(q16[layer], k, v, [0, nb], np.arange(nb), [tokens - (nb - 1) * 16], p, W.BF16)
            got = W.from_storage(out[layer].cpu().numpy().view(np.uint16), W.BF16)
            errs.append(float(np.abs(got - ref).max()))
        conns[rank].send("done")
        conns[rank].recv()  # nobody tears its buffers down while a peer may still write to them
        ex.close()
        result_q.put((rank, "ok", max(errs)))
    except Exception:
        result_q.put((rank, "error", traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_kv_axis_split_two_gpus_through_the_c_abi():
    ctx = mp.get_context("spawn")
    world = 2
    result_q = ctx.Queue()
    pipes = [ctx.Pipe() for _ in range(world)]
    child_ends = [c for (_, c) in pipes]
    procs = [ctx.Process(target=_worker, args=(r, world, child_ends, result_q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        handles = []
        for parent_end, _ in pipes:
            assert parent_end.poll(120), "a rank never exported its handle"
            handles.append(parent_end.recv())
        for parent_end, _ in pipes:
            parent_end.send(handles)
        for parent_end, _ in pipes:
            if parent_end.poll(120):
                parent_end.recv()
        for parent_end, _ in pipes:
            parent_end.send("bye")
        results = [result_q.get(timeout=120) for _ in procs]
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()  # the exact child started above
    for p in procs:
        assert p.exitcode == 0
    for rank, status, payload in results:
        assert status == "ok", f"rank {rank}:\n{payload}"
        assert payload <= 1e-2, (rank, payload)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_contexts_on_two_devices_in_one_process():
    """One process, one context per device, the tensor-core decode kernels launched on both: a kernel attribute set for
    the first device must not be taken for set on the second."""
    sys.path.insert(0, str(ROOT / "tests"))
    from kriya_rt_b200 import workloads as W
    from kriya_rt_b200.executor import CudaExecutor
    from oracle import c_oracle as O

    shape = W.AttnShape("two", 16, 2, 128, W.BF16)
    ctx = np.array([3000, 17, 700])
    batch = W.make_decode_batch(shape, ctx, 512, seed=5)
    rng = np.random.default_rng(6)
    q16 = W.normal16(rng, (3, 16, 128), W.BF16)
    ck = W.normal16(rng, (512, 16, 2, 128), W.BF16); cv = W.normal16(rng, (512, 16, 2, 128), W.BF16)
    p = O.GqaParams(16, 2, 128, 16, 16, 1, float(np.float32(1.0) / np.sqrt(np.float32(128))), 0.0)
    _, ref = O.decode(q16, ck, cv, batch.page_indptr, batch.page_indices, batch.last_page_len, p, W.BF16)
    for path in (0, 3):
        for dev in (0, 1):
            torch.cuda.set_device(dev)
            ex = CudaExecutor(num_layers=1, num_kv_blocks=512, block_size_tokens=16, num_q_heads=16, num_kv_heads=2, head_dim=128,
                              device=dev)
            ex.set_decode_path(path)
            kview, vview = ex.layer_cache_views(0)
            kview.copy_(torch.from_numpy(ck.view(np.int16)).to(f"cuda:{dev}"))
            vview.copy_(torch.from_numpy(cv.view(np.int16)).to(f"cuda:{dev}"))
            q = torch.from_numpy(q16.view(np.int16)).to(f"cuda:{dev}")
            out = torch.zeros_like(q)
            torch.cuda.synchronize(dev)
            ex.upload_schedule_plan(batch, batch.positions)
            ex.paged_gqa_decode(0, q, out, ex.gqa_params())
            ex.sync()
            got = W.from_storage(out.cpu().numpy().view(np.uint16), W.BF16)
            assert np.abs(got - ref).max() <= 1e-2, (path, dev)
            ex.close()
    torch.cuda.set_device(0)
