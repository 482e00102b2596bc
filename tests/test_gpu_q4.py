"""Q4KvGroup32 cache (32 values -> 16 bytes of 4-bit codes + f16 scale + f16 min) on the GPU, through the C ABI, against
the CPU oracle: the append writes the oracle's bytes, and the decode over those bytes agrees with the oracle's decode."""
import numpy as np
import pytest
import torch

from kriya_rt_b200 import workloads as W
from kriya_rt_b200.executor import KV_Q4_GROUP32, CudaBackendError, CudaExecutor
from oracle import c_oracle as O
from gpu_util import TOL, dev16, host16, oracle_gqa, oracle_rope

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _oracle_q4():
    O.set_kv_format(True)
    yield
    O.set_kv_format(False)


def q4_pool(rng, nb, Hkv, D):
    """A pool of valid Q4 blocks, as the uint16 view [nb, 16, Hkv, D / 32 * 10] the oracle and the views share."""
    vals = rng.standard_normal((nb, 16, Hkv, D)).astype(np.float32)
    return O.q4kv_quantize(vals).view(np.uint16).reshape(nb, 16, Hkv, D // 32 * 10).copy()


def make_q4_executor(shape, nb, **kw):
    return CudaExecutor(num_layers=1, num_kv_blocks=nb, block_size_tokens=16, num_q_heads=shape.num_q_heads,
                        num_kv_heads=shape.num_kv_heads, head_dim=shape.head_dim, dtype=shape.dtype, rope_theta=shape.rope_theta,
                        kv_format=KV_Q4_GROUP32, **kw)


@pytest.mark.parametrize("Hq,Hkv,D,dtype", [(16, 2, 128, W.BF16), (8, 8, 64, W.FP16), (32, 8, 128, W.FP16)])
def test_q4_append_writes_the_oracles_bytes_and_decode_reads_them(Hq, Hkv, D, dtype):
    shape = W.AttnShape("q4", Hq, Hkv, D, dtype, rope_theta=1e6)
    ctx = np.array([15, 16, 17, 31, 700, 1, 2500, 0])
    nb = 320
    batch = W.make_decode_batch(shape, ctx, nb, seed=31)
    rng = np.random.default_rng(32)
    R = len(ctx)
    q = W.normal16(rng, (R, Hq, D), dtype); k = W.normal16(rng, (R, Hkv, D), dtype); v = W.normal16(rng, (R, Hkv, D), dtype)
    ck, cv = q4_pool(rng, nb, Hkv, D), q4_pool(rng, nb, Hkv, D)
    ex = make_q4_executor(shape, nb, rope_max_seq_len=4096)
    kview, vview = ex.layer_cache_views(0)
    assert tuple(kview.shape) == ck.shape
    kview.copy_(dev16(ck)); vview.copy_(dev16(cv))
    qd, kd, vd = dev16(q), dev16(k), dev16(v)
    out = torch.zeros_like(qd)
    torch.cuda.synchronize()
    rp = ex.rope_params(has_table=True)
    ex.upload_schedule_plan(batch, batch.positions)
    ex.rope_kv_append(0, qd, kd, vd, R, rp)
    ex.paged_gqa_decode(0, qd, out, ex.gqa_params())
    ex.sync()
    gk, gv = host16(kview), host16(vview)
    # oracle: the same append (quantising keys from the un-rounded rotated values), then decode over its pool
    oq = q.copy(); ok = ck.copy(); ov = cv.copy()
    table = O.rope_table(4096, D, shape.rope_theta)
    O.rope_kv_append(oq, k, v, ok, ov, batch.page_indptr, batch.page_indices, batch.last_page_len, batch.positions,
                     oracle_rope(rp), dtype, table=table)
    assert np.array_equal(host16(qd), oq)
    assert np.array_equal(gk, ok)  # the whole pool: the new rows' blocks and nothing else
    assert np.array_equal(gv, ov)
    _, ref = O.decode(oq, ok, ov, batch.page_indptr, batch.page_indices, batch.last_page_len, oracle_gqa(ex), dtype)
    got = W.from_storage(host16(out), dtype)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= TOL[dtype]
    ex.close()


def test_q4_round_trip_error_is_within_half_a_step():
    """Property of the stored format at any size: |dequant(quant(x)) - x| <= scale / 2 + the f16 rounding of scale and min."""
    rng = np.random.default_rng(33)
    x = rng.standard_normal(32 * 4096).astype(np.float32)
    b = O.q4kv_quantize(x)
    y = O.q4kv_dequantize(b)
    g = x.reshape(-1, 32)
    step = (g.max(1) - g.min(1)) / 15.0
    bound = (0.5 * step * (1 + 2.0 ** -10) + np.abs(g.min(1)) * 2.0 ** -11 + 15 * step * 2.0 ** -11 + 1e-6)[:, None]
    assert np.all(np.abs(y.reshape(-1, 32) - g) <= bound)


@pytest.mark.parametrize("Hq,Hkv,D,dtype", [(12, 2, 128, W.BF16), (9, 3, 64, W.FP16)])
def test_q4_chunked_prefill(Hq, Hkv, D, dtype):
    """A prompt goes through append_chunk (which quantises its K/V into the Q4 pool) and prefill in chunks; the attention
    reads the dequantised cache.  The pool's bytes equal the oracle's after every chunk and the outputs agree with the
    oracle's prefill over the same Q4 pool within twice the 16-bit bars (2e-2 bf16, 4e-3 fp16)."""
    from kriya_rt_b200.kv import PagedKvCacheManager

    shape = W.AttnShape("q4pf", Hq, Hkv, D, dtype, rope_theta=1e6)
    total, chunk, nb = 700, 256, 128
    mgr = PagedKvCacheManager(nb, 0, 16)
    mgr.allocate_sequence(1, list(range(50)))
    mgr.allocate_sequence(2, list(range(5000, 5000 + total)))
    table, _ = mgr.sequence_table(2)
    rng = np.random.default_rng(41)
    q = W.normal16(rng, (total, Hq, D), dtype); k = W.normal16(rng, (total, Hkv, D), dtype); v = W.normal16(rng, (total, Hkv, D), dtype)
    ck, cv = q4_pool(rng, nb, Hkv, D), q4_pool(rng, nb, Hkv, D)
    ex = make_q4_executor(shape, nb, max_query_tokens=chunk, rope_max_seq_len=4096)
    kview, vview = ex.layer_cache_views(0)
    kview.copy_(dev16(ck)); vview.copy_(dev16(cv))
    rp = ex.rope_params()
    ok, ov = ck.copy(), cv.copy()
    tab = O.rope_table(4096, D, shape.rope_theta)
    for start in range(0, total, chunk):
        n = min(chunk, total - start)
        gp = ex.gqa_params(max_query_tokens=n)
        dq, dk, dv = dev16(q[start:start + n]), dev16(k[start:start + n]), dev16(v[start:start + n])
        out = torch.zeros_like(dq)
        torch.cuda.synchronize()
        ex.upload_schedule_plan(mgr.build_prefix_schedule_plan(2, start + n, 8))
        ex.rope_kv_append_chunk(0, dq, dk, dv, start, n, rp)
        ex.paged_gqa_prefill(0, dq, out, start, n, gp)
        ex.sync()
        rows = mgr.build_parallel_prefill_layout(2, start, n, 8)
        oq = q[start:start + n].copy()
        O.rope_kv_append(oq, k[start:start + n], v[start:start + n], ok, ov, rows.page_indptr, rows.page_indices,
                         rows.last_page_len, np.arange(start, start + n), oracle_rope(rp), dtype, table=tab)
        assert np.array_equal(host16(dq), oq)
        assert np.array_equal(host16(kview), ok) and np.array_equal(host16(vview), ov)
        _, ref = O.prefill_causal(oq, ok, ov, np.asarray(table, np.int32), start, oracle_gqa(ex), dtype)
        got = W.from_storage(host16(out), dtype)
        assert np.isfinite(got).all()
        # the staging pools hold the dequantised values rounded to the storage type once more, the oracle attends over the
        # un-rounded fma(code, scale, min): twice the 16-bit bar (measured 1.1e-2 for bf16 on the first chunk)
        assert np.abs(got - ref).max() <= 2 * TOL[dtype], start
    ex.close()


def test_q4_context_refuses_what_it_does_not_cover():
    """Speculative tree verification reads the cache through the 16-bit decode kernel's state path: not built for Q4."""
    shape = W.AttnShape("q4", 16, 2, 128, W.BF16)
    ex = make_q4_executor(shape, 64)
    batch = W.make_decode_batch(shape, np.array([40, 40]), 64, seed=1)
    ex.upload_schedule_plan(batch, batch.positions)
    n = 2
    tq = torch.zeros((n, 16, 128), dtype=torch.int16, device="cuda")
    tk = torch.zeros((n, 2, 128), dtype=torch.int16, device="cuda")
    with pytest.raises(CudaBackendError) as e:
        ex.tree_verify(0, tq, tk, tk, np.tril(np.ones((n, n), np.uint8)), torch.zeros_like(tq), ex.tree_verify_params(n, 41))
    assert "16-bit cache" in str(e.value)
    ex.close()
