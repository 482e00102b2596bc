"""Fused RoPE + KV append on the GPU, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest
import torch

from kriya_rt_b200 import workloads as W
from kriya_rt_b200.executor import InvalidExecutionInput
from oracle import c_oracle as O
from gpu_util import dev16, fill_cache, host16, make_executor, oracle_rope, read_cache

pytestmark = pytest.mark.gpu


def run_append(shape, batch, data, *, has_table, norm=False, max_seq_len=4096):
    ex = make_executor(shape, batch.num_blocks, rope_max_seq_len=max_seq_len)
    fill_cache(ex, 0, data["cache_k"], data["cache_v"])
    rp = ex.rope_params(has_table=has_table, apply_qk_norm=norm)
    q = dev16(data["q"]); k = dev16(data["k"]); v = dev16(data["v"])
    qw = kw = None
    qw_h = kw_h = None
    if norm:
        rng = np.random.default_rng(77)
        qw_h = W.to_storage(1.0 + 0.1 * rng.standard_normal(shape.head_dim).astype(np.float32), shape.dtype)
        kw_h = W.to_storage(1.0 + 0.1 * rng.standard_normal(shape.head_dim).astype(np.float32), shape.dtype)
        qw, kw = dev16(qw_h), dev16(kw_h)
    torch.cuda.synchronize()
    ex.upload_schedule_plan(batch, batch.positions)
    ex.rope_kv_append(0, q, k, v, batch.batch, rp, q_norm_w=qw, k_norm_w=kw)
    gk, gv = read_cache(ex, 0)
    gq = host16(q)
    # oracle
    oq = data["q"].copy(); ok = data["cache_k"].copy(); ov = data["cache_v"].copy()
    table = O.rope_table(max_seq_len, shape.head_dim, shape.rope_theta)
    O.rope_kv_append(oq, data["k"], data["v"], ok, ov, batch.page_indptr, batch.page_indices, batch.last_page_len,
                     batch.positions, oracle_rope(rp), shape.dtype, table=table, q_norm_w=qw_h, k_norm_w=kw_h)
    ex.close()
    return (gq, gk, gv), (oq, ok, ov)


@pytest.mark.parametrize("dtype", [W.BF16, W.FP16])
def test_append_with_table_is_bit_exact(dtype):
    shape, batch, data = W.config1(dtype=dtype)
    (gq, gk, gv), (oq, ok, ov) = run_append(shape, batch, data, has_table=True)
    assert np.array_equal(gq, oq)
    assert np.array_equal(gk, ok)  # whole pool: the new slots AND nothing else changed
    assert np.array_equal(gv, ov)
    # V slots hold the input bits
    for r in range(batch.batch):
        blk = batch.page_indices[batch.page_indptr[r + 1] - 1]
        assert np.array_equal(gv[blk, batch.last_page_len[r] - 1], data["v"][r])


@pytest.mark.parametrize("dtype", [W.BF16, W.FP16])
@pytest.mark.parametrize("head_dim,rotary_dim", [(64, 64), (64, 32), (128, 64), (256, 256), (256, 128), (128, 24)])
def test_append_head_dims_and_partial_rotary_are_bit_exact(dtype, head_dim, rotary_dim):
    """Rows of 64 / 128 / 256 values take the 16-byte kernel when the rotated part is a multiple of 16 values, anything
    else (here rotary_dim 24) the one-warp-per-row kernel; both have to leave the oracle's bits."""
    shape = W.AttnShape("dims", 8, 2, head_dim, dtype, rope_theta=1e4)
    ctx = np.array([1, 15, 16, 17, 100, 0, 33])
    nb = 64
    batch = W.make_decode_batch(shape, ctx, nb, seed=11)
    rng = np.random.default_rng(12)
    n = len(ctx)
    data = {"q": W.normal16(rng, (n, 8, head_dim), dtype), "k": W.normal16(rng, (n, 2, head_dim), dtype),
            "v": W.normal16(rng, (n, 2, head_dim), dtype),
            "cache_k": W.normal16(rng, (nb, 16, 2, head_dim), dtype), "cache_v": W.normal16(rng, (nb, 16, 2, head_dim), dtype)}
    ex = make_executor(shape, nb, rope_max_seq_len=512, rotary_dim=rotary_dim)
    fill_cache(ex, 0, data["cache_k"], data["cache_v"])
    rp = ex.rope_params(has_table=True)
    assert rp.rotary_dim == rotary_dim
    q = dev16(data["q"]); k = dev16(data["k"]); v = dev16(data["v"])
    torch.cuda.synchronize()
    ex.upload_schedule_plan(batch, batch.positions)
    ex.rope_kv_append(0, q, k, v, batch.batch, rp)
    gk, gv = read_cache(ex, 0)
    gq = host16(q)
    oq = data["q"].copy(); ok = data["cache_k"].copy(); ov = data["cache_v"].copy()
    table = O.rope_table(512, rotary_dim, shape.rope_theta)
    O.rope_kv_append(oq, data["k"], data["v"], ok, ov, batch.page_indptr, batch.page_indices, batch.last_page_len,
                     batch.positions, oracle_rope(rp), dtype, table=table)
    ex.close()
    assert np.array_equal(gq, oq) and np.array_equal(gk, ok) and np.array_equal(gv, ov)


def test_append_slot_mapping_qwen_shape():
    shape = W.AttnShape("qwen-small", 16, 2, 128, W.BF16, rope_theta=1e6)
    ctx = np.array([15, 16, 17, 31, 32, 511, 1000, 0])
    batch = W.make_decode_batch(shape, ctx, 256, seed=3)
    rng = np.random.default_rng(4)
    data = {"q": W.normal16(rng, (8, 16, 128), W.BF16), "k": W.normal16(rng, (8, 2, 128), W.BF16),
            "v": W.normal16(rng, (8, 2, 128), W.BF16),
            "cache_k": W.normal16(rng, (256, 16, 2, 128), W.BF16), "cache_v": W.normal16(rng, (256, 16, 2, 128), W.BF16)}
    (gq, gk, gv), (oq, ok, ov) = run_append(shape, batch, data, has_table=True)
    assert np.array_equal(gq, oq) and np.array_equal(gk, ok) and np.array_equal(gv, ov)


@pytest.mark.parametrize("dtype", [W.BF16, W.FP16])
def test_append_transcendental_path_within_reference_tolerance(dtype):
    """Positions beyond the table (or has_table = 0) use pow/cos/sin on the device; the reference holds the
    two paths to 1e-3 of each other (test_shader_compile.rs:2341-2354)."""
    shape, batch, data = W.config1(dtype=dtype)
    (gq, gk, gv), (oq, ok, ov) = run_append(shape, batch, data, has_table=False)
    ulp = 2.0 ** -8 if dtype == W.BF16 else 2.0 ** -11
    for g, o in ((gq, oq), (gk, ok)):
        gf, of = W.from_storage(g, dtype), W.from_storage(o, dtype)
        assert np.all(np.abs(gf - of) <= 1e-3 + 2 * ulp * np.abs(of))
    assert np.array_equal(gv, ov)


def test_append_with_qk_norm():
    shape, batch, data = W.config1(dtype=W.BF16)
    (gq, gk, gv), (oq, ok, ov) = run_append(shape, batch, data, has_table=True, norm=True)
    for g, o in ((gq, oq), (gk, ok)):
        gf, of = W.from_storage(g, W.BF16), W.from_storage(o, W.BF16)
        assert np.all(np.abs(gf - of) <= 1e-4 + 2.0 ** -7 * np.abs(of))  # rsqrt differs in the last bits
    assert np.array_equal(gv, ov)


def test_append_chunk_equals_per_token_rows():
    """Chunk form (table, prefix, count) against the oracle driven by the reference's per-token rows
    (build_parallel_prefill_layout, bsr_paged.rs:607-667)."""
    from kriya_rt_b200.kv import PagedKvCacheManager

    shape = W.AttnShape("qwen1p5-small", 12, 2, 128, W.BF16, rope_theta=1e6)
    mgr = PagedKvCacheManager(64, 0, 16)
    mgr.allocate_sequence(1, list(range(100)))   # occupy some blocks first so ids are not 0..n
    total, prefix, T = 150, 37, 70
    mgr.allocate_sequence(2, list(range(1000, 1000 + total)))
    rows = mgr.build_parallel_prefill_layout(2, prefix, T, 8)
    rng = np.random.default_rng(9)
    q = W.normal16(rng, (T, 12, 128), W.BF16); k = W.normal16(rng, (T, 2, 128), W.BF16); v = W.normal16(rng, (T, 2, 128), W.BF16)
    ck = W.normal16(rng, (64, 16, 2, 128), W.BF16); cv = W.normal16(rng, (64, 16, 2, 128), W.BF16)
    ex = make_executor(shape, 64)
    fill_cache(ex, 0, ck, cv)
    rp = ex.rope_params()
    dq, dk, dv = dev16(q), dev16(k), dev16(v)
    torch.cuda.synchronize()
    plan = mgr.build_prefix_schedule_plan(2, prefix + T, 8)
    ex.upload_schedule_plan(plan)
    ex.rope_kv_append_chunk(0, dq, dk, dv, prefix, T, rp)
    gk, gv = read_cache(ex, 0)
    oq, ok, ov = q.copy(), ck.copy(), cv.copy()
    O.rope_kv_append(oq, k, v, ok, ov, rows.page_indptr, rows.page_indices, rows.last_page_len,
                     np.arange(prefix, prefix + T), oracle_rope(rp), W.BF16, table=O.rope_table(4096, 128, 1e6))
    assert np.array_equal(host16(dq), oq) and np.array_equal(gk, ok) and np.array_equal(gv, ov)
    ex.close()


def test_plan_validation_errors_mirror_invalid_execution_input():
    shape, batch, data = W.config1()
    ex = make_executor(shape, 64, max_batch_rows=4, max_page_indices=64)
    with pytest.raises(InvalidExecutionInput, match="outside the pool"):
        ex.plan_upload([0, 1], [64], [1])
    with pytest.raises(InvalidExecutionInput, match="last_page_len"):
        ex.plan_upload([0, 1], [0], [17])
    with pytest.raises(InvalidExecutionInput, match="last_page_len"):
        ex.plan_upload([0, 1], [0], [0])
    with pytest.raises(InvalidExecutionInput, match="GPU buffer holds"):
        ex.plan_upload(list(range(6)), list(range(5)), [1] * 5)
    with pytest.raises(InvalidExecutionInput, match="GPU buffer holds"):
        ex.plan_upload([0, 65], list(range(64)) + [0], [1])
    with pytest.raises(InvalidExecutionInput, match="non-decreasing"):
        ex.plan_upload([0, 2, 1], [0, 1], [1, 1])
    with pytest.raises(InvalidExecutionInput, match="no plan"):
        ex.paged_gqa_decode(0, 1, 1, ex.gqa_params())
    ex.upload_schedule_plan(batch, batch.positions)
    q = dev16(data["q"])
    with pytest.raises(InvalidExecutionInput, match="seq_positions"):
        ex.rope_kv_append(0, q, q, q, 3, ex.rope_params())
    with pytest.raises(InvalidExecutionInput, match="layer"):
        ex.paged_gqa_decode(1, q, q, ex.gqa_params())
    with pytest.raises(InvalidExecutionInput, match="empty"):
        ex.rope_kv_append(0, q, q, q, 0, ex.rope_params())
    ex.close()
