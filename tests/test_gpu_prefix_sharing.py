"""Radix prefix sharing with copy-on-write, end to end on the GPU (benchmark configuration 3 in small and at full size):
sequences share a prefix through the manager's radix cache, forks of a parent with a partly filled tail block trigger
copy-on-write pairs, the pairs are applied by the block-copy kernel, and decode attention runs over shared and private
blocks.  Bookkeeping is checked bit for bit, attention against the fp32 oracle."""
import numpy as np
import pytest
import torch

from kriya_rt_b200 import workloads as W
from kriya_rt_b200.kv import PagedKvCacheManager
from oracle import c_oracle as O
from oracle import kv_oracle as KO
from gpu_util import dev16, fill_cache, host16, make_executor, oracle_gqa, oracle_rope, read_cache

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_seq,prefix_len,suffix_lo,suffix_hi,nb", [(8, 256, 20, 90, 512), (64, 2048, 128, 512, 4096)])
def test_shared_prefix_cow_fork_then_decode(n_seq, prefix_len, suffix_lo, suffix_hi, nb):
    shape = W.AttnShape("qwen3b", 16, 2, 128, W.BF16, rope_theta=1e6)
    Hq, Hkv, D = 16, 2, 128
    rng = np.random.default_rng(3003)
    mgr, ora = PagedKvCacheManager(nb, 0, 16), KO.PagedKvCacheManager(nb, 0, 16)
    prefix = (np.arange(prefix_len) + 7).astype(np.uint32)
    suffix = rng.integers(suffix_lo, suffix_hi + 1, size=n_seq)
    for s in range(n_seq):
        toks = np.concatenate([prefix, (np.arange(suffix[s]) + 100000 * (s + 1)).astype(np.uint32)])
        assert mgr.allocate_sequence(s, toks) == ora.allocate_sequence(s, toks.tolist()) == (0 if s == 0 else prefix_len)
    shared = ora.sequences[0].logical_blocks[: prefix_len // 16]
    for b in shared:
        assert mgr.gpu_allocator.ref_count(b) == n_seq
    # a parent with a partly filled tail, forked: each child's first append must copy the tail block
    parent = 1000
    ptoks = np.concatenate([prefix, np.arange(8, dtype=np.uint32) + 900000])
    mgr.allocate_sequence(parent, ptoks); ora.allocate_sequence(parent, ptoks.tolist())
    children = list(range(1001, 1005))
    pairs = []
    for c in children:
        mgr.fork_sequence(parent, c); ora.fork_sequence(parent, c)
        got, exp = mgr.append_token_slot(c), ora.append_token_slot(c)
        assert got == exp and got[1] is not None
        pairs.append(got[1])
    # every running sequence reserves its next slot, as the scheduler does before a decode step
    for s in range(n_seq):
        assert mgr.append_token_slot(s) == ora.append_token_slot(s)
    ids = list(range(n_seq)) + children
    plan, oplan = mgr.build_schedule_plan(ids, 8), ora.build_schedule_plan(ids, 8)
    assert plan.page_indptr.tolist() == oplan.page_indptr and plan.page_indices.tolist() == oplan.page_indices
    assert plan.last_page_len.tolist() == oplan.last_page_len

    # cache contents: random everywhere (shared blocks are read by every sequence)
    ck = W.normal16(rng, (nb, 16, Hkv, D), W.BF16); cv = W.normal16(rng, (nb, 16, Hkv, D), W.BF16)
    ex = make_executor(shape, nb, rope_max_seq_len=4096)
    fill_cache(ex, 0, ck, cv)
    ex.kv_block_copy(pairs)                       # copy-on-write data movement
    ock, ocv = ck[None].copy(), cv[None].copy()
    O.block_copy(ock, ocv, 1, pairs)
    B = len(ids)
    positions = np.array([prefix_len + suffix[s] for s in range(n_seq)] + [prefix_len + 8] * len(children), np.uint32)
    q16 = W.normal16(rng, (B, Hq, D), W.BF16); k16 = W.normal16(rng, (B, Hkv, D), W.BF16); v16 = W.normal16(rng, (B, Hkv, D), W.BF16)
    q, k, v = dev16(q16), dev16(k16), dev16(v16)
    out = torch.zeros_like(q)
    torch.cuda.synchronize()
    ex.upload_schedule_plan(plan, positions)
    rp, gp = ex.rope_params(), ex.gqa_params()
    ex.append_decode(0, q, k, v, out, rp, gp)
    gk, gv = read_cache(ex, 0)
    oq = q16.copy()
    O.rope_kv_append(oq, k16, v16, ock[0], ocv[0], plan.page_indptr, plan.page_indices, plan.last_page_len, positions,
                     oracle_rope(rp), W.BF16, table=O.rope_table(4096, D, 1e6))
    assert np.array_equal(gk, ock[0]) and np.array_equal(gv, ocv[0])   # CoW copies + appended slots, bit for bit
    _, ref = O.decode(oq, ock[0], ocv[0], plan.page_indptr, plan.page_indices, plan.last_page_len, oracle_gqa(ex), W.BF16)
    assert np.abs(W.from_storage(host16(out), W.BF16) - ref).max() <= 1e-2
    # the shared prefix blocks were not written by anybody's append
    for b in shared:
        assert np.array_equal(gk[b], ck[b]) and np.array_equal(gv[b], cv[b])
    ex.close()
