"""Host-side sharding of the paged KV path across the GPUs of one box.

Two schemes, both new relative to the reference (which is single-GPU):

* by sequence - every GPU owns a pool, a bookkeeping manager and an executor; whole sequences are assigned to GPUs,
  longest first, so that attended tokens balance.  No collective is needed on the data path.
* along the KV axis - one very long sequence's block table is cut into contiguous ranges, one per GPU; each GPU runs
  the partial-state decode over its range, the (m, l, o) states are all-gathered and merged everywhere.

The functions here are plumbing only (integer ranges, tensor gathers); the arithmetic runs in the CUDA kernels.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def assign_sequences(lengths: Sequence[int], ranks: int) -> List[List[int]]:
    """Longest-processing-time assignment: returns, per rank, the indices of its sequences."""
    order = np.argsort(-np.asarray(lengths, dtype=np.int64), kind="stable")
    load = [0] * ranks
    out: List[List[int]] = [[] for _ in range(ranks)]
    for i in order:
        r = min(range(ranks), key=lambda j: (load[j], j))
        out[r].append(int(i))
        load[r] += int(lengths[i])
    return out


def kv_axis_ranges(blocks_per_row: Sequence[int], ranks: int) -> List[Tuple[np.ndarray, np.ndarray]]:
    """Cuts every row's logical blocks into `ranks` contiguous ranges of near-equal size.
    Returns, per rank, (blk_begin[rows], blk_end[rows]) as uint32 arrays; ranges of one row tile [0, blocks)."""
    nb = np.asarray(blocks_per_row, dtype=np.int64)
    out = []
    for r in range(ranks):
        out.append((((nb * r) // ranks).astype(np.uint32), ((nb * (r + 1)) // ranks).astype(np.uint32)))
    return out


def local_block_table(table: Sequence[int], begin: int, end: int, local_ids: Sequence[int]) -> np.ndarray:
    """A rank that stores only blocks [begin, end) of a row keeps them in its own pool under `local_ids`;
    this returns the rank's view of the row's table: its own range mapped to local ids, everything else 0
    (never read, because the partial decode is restricted to [begin, end))."""
    t = np.zeros(len(table), dtype=np.int32)
    t[begin:end] = np.asarray(local_ids, dtype=np.int32)[: end - begin]
    return t


def gather_states(m, l, o, group=None):
    """All-gathers per-rank partial softmax states.  m, l: [rows] tensors, o: [rows, D] (any device the process
    group supports: CUDA with NCCL, CPU with gloo).  Returns (m_all [ranks, rows], l_all, o_all [ranks, rows, D])."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    m_all = torch.empty((world,) + tuple(m.shape), dtype=m.dtype, device=m.device)
    l_all = torch.empty((world,) + tuple(l.shape), dtype=l.dtype, device=l.device)
    o_all = torch.empty((world,) + tuple(o.shape), dtype=o.dtype, device=o.device)
    for dst, src in ((m_all, m), (l_all, l), (o_all, o)):
        # views of one contiguous buffer: the gathered states land side by side, ready for the merge kernel
        dist.all_gather([dst[i] for i in range(world)], src.contiguous(), group=group)
    return m_all, l_all, o_all


def kv_split_decode(ex, layer: int, q, blk_begin, blk_end, out, gqa, group=None, scratch=None, rows_hint=None):
    """One KV-axis-split decode on this rank: partial state over [blk_begin, blk_end) of every row of the current
    plan, ONE all-gather of the packed (m, l, o) states, merge into `out` ([rows, Hq, D] in the storage dtype).
    Everything is queued on the executor's stream (the collective is ordered behind it by torch), so the host does
    not wait in between.  `scratch` may carry preallocated (local [R*(D+2)], gathered [world, R*(D+2)]) fp32 device
    tensors to keep the step path allocation-free.  With blk_begin = blk_end = None the ranges set by
    `ex.plan_set_ranges` are used and `rows_hint` gives the number of plan rows (default 1)."""
    import torch
    import torch.distributed as dist

    if blk_begin is None:  # ranges were set once for the plan (CudaExecutor.plan_set_ranges)
        R = ex.num_q_heads * int(rows_hint if rows_hint is not None else 1)
    else:
        R = ex.num_q_heads * int(len(blk_begin))
    D = ex.head_dim
    world = dist.get_world_size(group)
    if scratch is None:
        scratch = (torch.empty(R * (D + 2), device=q.device), torch.empty(world, R * (D + 2), device=q.device))
    local, gathered = scratch
    stream = torch.cuda.ExternalStream(ex.stream_ptr, device=q.device)
    with torch.cuda.stream(stream):
        ex.paged_gqa_decode_partial(layer, q, blk_begin, blk_end, local[:R], local[R:2 * R], local[2 * R:], gqa)
        dist.all_gather_into_tensor(gathered, local, group=group)
        ex.merge_packed_states(gathered, world, R, out)
    return out
