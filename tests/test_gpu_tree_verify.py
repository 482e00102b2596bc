"""Speculative tree verification on the GPU (prefix through the decode kernel + draft-tree kernel) and in-place RoPE through the
C ABI, against the CPU restatement of bsr_paged_gqa_tree_verify / apply_rope_inplace."""
import numpy as np
import pytest
import torch

from kriya_rt_b200 import workloads as W
from kriya_rt_b200.kv import PagedKvCacheManager
from oracle import c_oracle as O
from gpu_util import TOL, dev16, fill_cache, host16, make_executor, oracle_rope

pytestmark = pytest.mark.gpu


def random_tree(rng, n):
    """Parent pointers of a random tree rooted at node 0; mask[i, j] = 1 when j is i or an ancestor of i; depth per node."""
    parent = np.full(n, -1, np.int64)
    depth = np.zeros(n, np.int64)
    mask = np.zeros((n, n), np.uint8)
    for i in range(n):
        if i:
            parent[i] = rng.integers(0, i)
            depth[i] = depth[parent[i]] + 1
        j = i
        while j >= 0:
            mask[i, j] = 1
            j = parent[j]
    return mask, depth


def run_case(shape, prefix_tokens, n_nodes, seed, num_blocks=192):
    Hq, Hkv, D, dt = shape.num_q_heads, shape.num_kv_heads, shape.head_dim, shape.dtype
    rng = np.random.default_rng(seed)
    mgr = PagedKvCacheManager(num_blocks, 0, 16)
    mgr.allocate_sequence(1, list(range(37)))  # so the prefix blocks are not 0..n
    if prefix_tokens:
        mgr.allocate_sequence(2, list(range(9000, 9000 + prefix_tokens)))
    ck = W.normal16(rng, (num_blocks, 16, Hkv, D), dt)
    cv = W.normal16(rng, (num_blocks, 16, Hkv, D), dt)
    tq = W.normal16(rng, (n_nodes, Hq, D), dt); tk = W.normal16(rng, (n_nodes, Hkv, D), dt); tv = W.normal16(rng, (n_nodes, Hkv, D), dt)
    mask, _ = random_tree(rng, n_nodes)
    ex = make_executor(shape, num_blocks, max_batch_rows=max(n_nodes, 32))
    fill_cache(ex, 0, ck, cv)
    tp = ex.tree_verify_params(n_nodes, prefix_tokens)
    table = np.zeros(0, np.int32)
    if prefix_tokens:
        plan = mgr.build_schedule_plan([2] * n_nodes, 8)  # one decode row per tree node, all over the prefix table
        ex.upload_schedule_plan(plan)
        table = np.asarray(mgr.sequence_table(2)[0], np.int32)
        assert tp.prefix_kv_blocks == table.size and tp.prefix_last_len == plan.last_page_len[0]
    dq, dk, dv = dev16(tq), dev16(tk), dev16(tv)
    out = torch.zeros_like(dq)
    torch.cuda.synchronize()
    ex.tree_verify(0, dq, dk, dv, mask, out, tp)
    ex.sync()
    got = W.from_storage(host16(out), dt)
    op = O.TreeParams(n_nodes, Hq, Hkv, D, 16, tp.prefix_kv_blocks, tp.prefix_last_len, tp.sm_scale)
    _, ref = O.tree_verify(tq, tk, tv, ck, cv, table, mask, op, dt)
    ex.close()
    return got, ref


@pytest.mark.parametrize("prefix_tokens", [0, 7, 16, 333, 2048])
def test_qwen_shape_tree_verify(prefix_tokens):
    shape = W.AttnShape("qwen3b", 16, 2, 128, W.BF16, rope_theta=1e6)
    got, ref = run_case(shape, prefix_tokens, 11, seed=prefix_tokens + 1)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= TOL[W.BF16]


@pytest.mark.parametrize("dtype", [W.FP16, W.BF16])
def test_smollm_shape_tree_verify_head_dim_64(dtype):
    shape = W.AttnShape("smol", 9, 3, 64, dtype)
    got, ref = run_case(shape, 200, 24, seed=5)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= TOL[dtype]


def test_largest_tree():
    shape = W.AttnShape("qwen1.5b", 12, 2, 128, W.BF16, rope_theta=1e6)
    got, ref = run_case(shape, 100, 128, seed=9)
    assert np.abs(got - ref).max() <= TOL[W.BF16]


def test_tree_verify_rejects_a_plan_that_is_not_the_prefix():
    shape = W.AttnShape("qwen3b", 16, 2, 128, W.BF16)
    ex = make_executor(shape, 64, max_batch_rows=32)
    mgr = PagedKvCacheManager(64, 0, 16)
    mgr.allocate_sequence(2, list(range(40)))
    ex.upload_schedule_plan(mgr.build_schedule_plan([2] * 3, 8))
    z = torch.zeros(4, 16, 128, dtype=torch.int16, device="cuda")
    kv = torch.zeros(4, 2, 128, dtype=torch.int16, device="cuda")
    with pytest.raises(Exception, match="one row per tree node"):
        ex.tree_verify(0, z, kv, kv, np.eye(4, dtype=np.uint8), z.clone(), ex.tree_verify_params(4, 40))
    with pytest.raises(Exception, match="does not describe the prefix"):
        ex.tree_verify(0, z[:3], kv[:3], kv[:3], np.eye(3, dtype=np.uint8), z[:3].clone(), ex.tree_verify_params(3, 33))
    ex.close()


@pytest.mark.parametrize("shape", [W.AttnShape("qwen3b", 16, 2, 128, W.BF16, rope_theta=1e6), W.AttnShape("smol", 9, 3, 64, W.FP16)])
def test_rope_inplace_matches_the_append_arithmetic(shape):
    """apply_rope_inplace uses the arithmetic of the fused append: q and k must equal the oracle's rotated q and the K rows the
    oracle's append writes to a cache, bit for bit (cos/sin table)."""
    Hq, Hkv, D, dt = shape.num_q_heads, shape.num_kv_heads, shape.head_dim, shape.dtype
    n = 11
    rng = np.random.default_rng(3)
    _, depth = random_tree(rng, n)
    positions = (500 + depth).astype(np.uint32)
    q = W.normal16(rng, (n, Hq, D), dt); k = W.normal16(rng, (n, Hkv, D), dt); v = W.normal16(rng, (n, Hkv, D), dt)
    ex = make_executor(shape, 64, max_batch_rows=32)
    mgr = PagedKvCacheManager(64, 0, 16)
    for s in range(n):
        mgr.allocate_sequence(s, [1000 * s + 1])
    plan = mgr.build_schedule_plan(list(range(n)), 8)
    ex.upload_schedule_plan(plan, positions)
    rp = ex.rope_params()
    dq, dk = dev16(q), dev16(k)
    torch.cuda.synchronize()
    ex.rope_inplace(dq, dk, n, rp)
    ex.sync()
    ok = np.zeros((64, 16, Hkv, D), np.uint16); ov = np.zeros_like(ok)
    oq = q.copy()
    O.rope_kv_append(oq, k, v, ok, ov, plan.page_indptr, plan.page_indices, plan.last_page_len, positions, oracle_rope(rp), dt,
                     table=O.rope_table(4096, D, shape.rope_theta))
    assert np.array_equal(host16(dq), oq)
    want_k = np.stack([ok[plan.page_indices[plan.page_indptr[r + 1] - 1], plan.last_page_len[r] - 1] for r in range(n)])
    assert np.array_equal(host16(dk), want_k)
    ex.close()
