"""Chunked causal prefill on the GPU (tcgen05 kernel) through the C ABI, against the fp32 CPU oracle."""
import numpy as np
import pytest
import torch

from kriya_rt_b200 import workloads as W
from kriya_rt_b200.kv import PagedKvCacheManager
from oracle import c_oracle as O
from gpu_util import TOL, dev16, fill_cache, host16, make_executor, oracle_gqa, oracle_rope, read_cache

pytestmark = pytest.mark.gpu


def chunked_prefill(shape, total, chunk, num_blocks=256, seed=0, poison=True, other_seq_tokens=100, window=0):
    """Runs a whole prompt through append_chunk + prefill in chunks on the GPU and the same through the oracle.
    Returns (gpu_out f32 [total,Hq,D], oracle_out f32, gpu cache, oracle cache)."""
    Hq, Hkv, D, dt = shape.num_q_heads, shape.num_kv_heads, shape.head_dim, shape.dtype
    mgr = PagedKvCacheManager(num_blocks, 0, 16)
    if other_seq_tokens:
        mgr.allocate_sequence(1, list(range(other_seq_tokens)))  # so the prompt's blocks are not 0..n
    mgr.allocate_sequence(2, list(range(5000, 5000 + total)))
    table, _ = mgr.sequence_table(2)
    rng = np.random.default_rng(seed)
    q = W.normal16(rng, (total, Hq, D), dt); k = W.normal16(rng, (total, Hkv, D), dt); v = W.normal16(rng, (total, Hkv, D), dt)
    fillbits = (0x7FC1 if dt == W.BF16 else 0x7E01) if poison else 0
    ck = np.full((num_blocks, 16, Hkv, D), fillbits, np.uint16)
    cv = np.full((num_blocks, 16, Hkv, D), fillbits, np.uint16)
    ex = make_executor(shape, num_blocks, max_query_tokens=max(chunk, 64))
    ex.set_attention_window(window)
    fill_cache(ex, 0, ck, cv)
    rp, gp = ex.rope_params(), ex.gqa_params(max_query_tokens=chunk)
    outs = []
    ok, ov = ck.copy(), cv.copy()
    oouts = []
    tab = O.rope_table(4096, D, shape.rope_theta)
    for start in range(0, total, chunk):
        n = min(chunk, total - start)
        dq, dk, dv = dev16(q[start:start + n]), dev16(k[start:start + n]), dev16(v[start:start + n])
        out = torch.zeros_like(dq)
        torch.cuda.synchronize()
        plan = mgr.build_prefix_schedule_plan(2, start + n, 8)
        ex.upload_schedule_plan(plan)
        ex.rope_kv_append_chunk(0, dq, dk, dv, start, n, rp)
        ex.paged_gqa_prefill(0, dq, out, start, n, gp)
        ex.sync()
        outs.append(W.from_storage(host16(out), dt))
        # oracle: per-token rows as the reference lays them out
        rows = mgr.build_parallel_prefill_layout(2, start, n, 8)
        oq = q[start:start + n].copy()
        O.rope_kv_append(oq, k[start:start + n], v[start:start + n], ok, ov, rows.page_indptr, rows.page_indices,
                         rows.last_page_len, np.arange(start, start + n), oracle_rope(rp), dt, table=tab)
        assert np.array_equal(host16(dq), oq)
        O.set_attention_window(window)
        try:
            _, of = O.prefill_causal(oq, ok, ov, np.asarray(table, np.int32), start, oracle_gqa(ex), dt)
        finally:
            O.set_attention_window(0)
        oouts.append(of)
    gk, gv = read_cache(ex, 0)
    ex.close()
    return np.concatenate(outs), np.concatenate(oouts), (gk, gv), (ok, ov)


@pytest.mark.parametrize("total,chunk", [(16, 16), (130, 130), (700, 256), (1024, 512), (300, 77)])
def test_qwen15_shape_chunked_prefill(total, chunk):
    shape = W.AttnShape("qwen1.5b", 12, 2, 128, W.BF16, rope_theta=1e6)
    got, ref, (gk, gv), (ok, ov) = chunked_prefill(shape, total, chunk, seed=total)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= TOL[W.BF16]
    assert np.array_equal(gk, ok) and np.array_equal(gv, ov)  # the chunk's K/V landed bit-exactly


@pytest.mark.parametrize("dtype", [W.FP16, W.BF16])
def test_smollm_shape_head_dim_64(dtype):
    shape = W.AttnShape("smol", 9, 3, 64, dtype)
    got, ref, _, _ = chunked_prefill(shape, 333, 128, seed=7)
    assert np.isfinite(got).all()
    # P is rounded to the storage dtype before the P.V product, like the reference's tensor-core kernel
    # (paged_gqa_and_deltanet.metal:1386 stores P as half); the bar is still 2e-3 (fp16) / 1e-2 (bf16)
    assert np.abs(got - ref).max() <= TOL[dtype]


@pytest.mark.parametrize("window", [1, 100, 128, 300])
def test_sliding_window_prefill(window):
    """SlidingWindowCausal in the chunked prefill: every query attends its `window` most recent keys; KV tiles wholly in
    front of a query tile's windows are skipped, rows whose window begins behind a tile see nothing of it."""
    shape = W.AttnShape("pwin", 12, 2, 128, W.BF16, rope_theta=1e6)
    got, ref, (gk, gv), (ok, ov) = chunked_prefill(shape, 700, 256, seed=17, window=window)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= TOL[W.BF16]
    assert np.array_equal(gk, ok) and np.array_equal(gv, ov)


def test_reference_tiled_mma_prefill_case():
    """test_shader_compile.rs:1696-1881: T=16, Hq=2, Hkv=1, D=64, closed-form inputs, K/V given (no RoPE), tol 0.05."""
    T, Hq, Hkv, D = 16, 2, 1, 64
    f = np.float32
    q_f = np.array([(f(i % 17) - f(8.0)) * f(0.05) for i in range(T * Hq * D)], f)
    k_f = np.array([(f(i % 13) - f(6.0)) * f(0.06) for i in range(16 * Hkv * D)], f)
    v_f = np.array([(f(i % 11) - f(5.0)) * f(0.07) for i in range(16 * Hkv * D)], f)
    q = W.to_storage(q_f.reshape(T, Hq, D), W.BF16)
    ck = W.to_storage(k_f.reshape(1, 16, Hkv, D), W.BF16)
    cv = W.to_storage(v_f.reshape(1, 16, Hkv, D), W.BF16)
    expected = O.ref_test_causal_prefill(W.from_storage(q, W.BF16), W.from_storage(ck, W.BF16), W.from_storage(cv, W.BF16),
                                         Hq, Hkv, D, float(f(1.0) / np.sqrt(f(D))))
    shape = W.AttnShape("tsc", Hq, Hkv, D, W.BF16)
    ex = make_executor(shape, 1)
    fill_cache(ex, 0, ck, cv)
    dq = dev16(q)
    out = torch.zeros_like(dq)
    torch.cuda.synchronize()
    ex.plan_upload([0, 1], [0], [16])
    ex.paged_gqa_prefill(0, dq, out, 0, T, ex.gqa_params(max_query_tokens=T))
    ex.sync()
    assert np.abs(W.from_storage(host16(out), W.BF16).ravel() - expected).max() < 0.05
    ex.close()


def test_prefill_last_row_equals_decode():
    """Cross-check of the two attention kernels: the last query of a prefilled prompt sees exactly what a
    decode step at that position sees."""
    shape = W.AttnShape("x", 16, 2, 128, W.BF16)
    total = 517
    got, ref, (gk, gv), _ = chunked_prefill(shape, total, 517, seed=3, poison=False)
    assert np.abs(got[-1] - ref[-1]).max() <= 1e-2


def test_batched_prefill_three_sequences_one_launch():
    """Chunks of three sequences (different prefixes, ragged lengths) in one launch, each against the oracle."""
    shape = W.AttnShape("batch", 12, 2, 128, W.BF16, rope_theta=1e6)
    Hq, Hkv, D = 12, 2, 128
    nb = 256
    mgr = PagedKvCacheManager(nb, 0, 16)
    specs = [(300, 140, 160), (64, 0, 64), (517, 400, 117)]  # (total tokens so far, prefix, chunk length)
    rng = np.random.default_rng(91)
    ck = W.normal16(rng, (nb, 16, Hkv, D), W.BF16); cv = W.normal16(rng, (nb, 16, Hkv, D), W.BF16)
    for i, (total, _, _) in enumerate(specs):
        mgr.allocate_sequence(i, list(range(1000 * i, 1000 * i + total)))
    plan = mgr.build_schedule_plan([0, 1, 2], 8)
    counts = [c for _, _, c in specs]
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    q = W.normal16(rng, (sum(counts), Hq, D), W.BF16)
    ex = make_executor(shape, nb)
    fill_cache(ex, 0, ck, cv)
    dq = dev16(q)
    out = torch.zeros_like(dq)
    torch.cuda.synchronize()
    ex.upload_schedule_plan(plan)
    ex.paged_gqa_prefill_batch(0, dq, out, starts, [p for _, p, _ in specs], counts, ex.gqa_params(max_query_tokens=160))
    ex.sync()
    got = W.from_storage(host16(out), W.BF16)
    for i, (total, prefix, cnt) in enumerate(specs):
        table, _ = mgr.sequence_table(i)
        _, ref = O.prefill_causal(q[starts[i]:starts[i] + cnt], ck, cv, np.asarray(table, np.int32), prefix, oracle_gqa(ex), W.BF16)
        assert np.abs(got[starts[i]:starts[i] + cnt] - ref).max() <= 1e-2, i
    ex.close()


def test_batched_append_then_batched_prefill_three_sequences():
    """The chunk's K/V of several sequences appended in ONE launch (kriya_cuda_rope_kv_append_chunk_batch), then their
    attention in one launch: caches bit-exact against the oracle's per-token appends, outputs within the bar."""
    shape = W.AttnShape("batch2", 12, 2, 128, W.BF16, rope_theta=1e6)
    Hq, Hkv, D, nb = 12, 2, 128, 256
    mgr = PagedKvCacheManager(nb, 0, 16)
    specs = [(300, 140, 160), (64, 0, 64), (517, 400, 117)]  # (tokens after the chunk, prefix, chunk length)
    rng = np.random.default_rng(93)
    ck = W.normal16(rng, (nb, 16, Hkv, D), W.BF16); cv = W.normal16(rng, (nb, 16, Hkv, D), W.BF16)
    for i, (total, _, _) in enumerate(specs):
        mgr.allocate_sequence(i, list(range(1000 * i, 1000 * i + total)))
    plan = mgr.build_schedule_plan([0, 1, 2], 8)
    counts = [c for _, _, c in specs]
    prefixes = [p for _, p, _ in specs]
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    n_tok = sum(counts)
    q = W.normal16(rng, (n_tok, Hq, D), W.BF16); k = W.normal16(rng, (n_tok, Hkv, D), W.BF16); v = W.normal16(rng, (n_tok, Hkv, D), W.BF16)
    ex = make_executor(shape, nb, max_query_tokens=512)
    fill_cache(ex, 0, ck, cv)
    dq, dk, dv = dev16(q), dev16(k), dev16(v)
    out = torch.zeros_like(dq)
    torch.cuda.synchronize()
    ex.upload_schedule_plan(plan)
    rp = ex.rope_params()
    ex.rope_kv_append_chunk_batch(0, dq, dk, dv, starts, prefixes, counts, rp)
    ex.paged_gqa_prefill_batch(0, dq, out, starts, prefixes, counts, ex.gqa_params(max_query_tokens=160))
    ex.sync()
    got = W.from_storage(host16(out), W.BF16)
    gk, gv = read_cache(ex, 0)
    ok, ov = ck.copy(), cv.copy()
    tab = O.rope_table(4096, D, shape.rope_theta)
    for i, (total, prefix, cnt) in enumerate(specs):
        rows = mgr.build_parallel_prefill_layout(i, prefix, cnt, 8)
        sl = slice(int(starts[i]), int(starts[i]) + cnt)
        oq = q[sl].copy()
        O.rope_kv_append(oq, k[sl], v[sl], ok, ov, rows.page_indptr, rows.page_indices, rows.last_page_len,
                         np.arange(prefix, prefix + cnt), oracle_rope(rp), W.BF16, table=tab)
        assert np.array_equal(host16(dq)[sl], oq), i
        table, _ = mgr.sequence_table(i)
        _, ref = O.prefill_causal(oq, ok, ov, np.asarray(table, np.int32), prefix, oracle_gqa(ex), W.BF16)
        assert np.abs(got[sl] - ref).max() <= 1e-2, i
    assert np.array_equal(gk, ok) and np.array_equal(gv, ov)
    ex.close()


def test_config4_full_size_last_chunk_of_eight_prompts():
    """BASELINE config 4 at full size: eight 2048-token prompts (Hq 12, Hkv 2, D 128), the 512-token chunk at prefix 1536 of
    all of them in one launch.  Two prompts are compared row by row with the oracle; every prompt is checked through a
    size-independent property: the same launch repeated over relocated blocks (a different permutation of the pool with the
    cache contents moved along) must not change a single bit."""
    shape = W.AttnShape("c4", 12, 2, 128, W.BF16, rope_theta=1e6)
    Hq, Hkv, D = 12, 2, 128
    n_seq, total, chunk = 8, 2048, 512
    per = total // 16
    nb = n_seq * per + 64
    rng = np.random.default_rng(404)
    ck = W.normal16(rng, (nb, 16, Hkv, D), W.BF16); cv = W.normal16(rng, (nb, 16, Hkv, D), W.BF16)
    q = W.normal16(rng, (n_seq * chunk, Hq, D), W.BF16)
    starts = np.arange(n_seq) * chunk
    outs = []
    perm0 = None
    for trial in range(2):
        perm = np.random.default_rng(500 + trial).permutation(nb).astype(np.int32)
        if trial == 0:
            perm0, k_t, v_t = perm, ck, cv
        else:  # logical block j of the pool image moves from perm0[j] to perm[j]
            k_t, v_t = np.empty_like(ck), np.empty_like(cv)
            k_t[perm] = ck[perm0]
            v_t[perm] = cv[perm0]
        ex = make_executor(shape, nb, max_query_tokens=n_seq * chunk)
        fill_cache(ex, 0, k_t, v_t)
        ex.plan_upload(np.arange(n_seq + 1) * per, perm[: n_seq * per], [16] * n_seq)
        dq = dev16(q)
        out = torch.zeros_like(dq)
        torch.cuda.synchronize()
        ex.paged_gqa_prefill_batch(0, dq, out, starts, [total - chunk] * n_seq, [chunk] * n_seq, ex.gqa_params(max_query_tokens=chunk))
        ex.sync()
        outs.append(host16(out).copy())
        if trial == 0:
            got = W.from_storage(outs[0], W.BF16)
            for s in (0, n_seq - 1):
                table = perm[s * per:(s + 1) * per]
                _, ref = O.prefill_causal(q[starts[s]:starts[s] + chunk], ck, cv, table, total - chunk, oracle_gqa(ex), W.BF16)
                assert np.abs(got[starts[s]:starts[s] + chunk] - ref).max() <= 1e-2, s
        ex.close()
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("dtype,D,Hq,Hkv", [(W.BF16, 128, 12, 2), (W.FP16, 64, 9, 3)])
def test_few_tiles_are_cut_along_the_kv_axis_and_merged(dtype, D, Hq, Hkv, monkeypatch):
    """One request's chunk is a handful of CTAs: the launch cuts every query tile's keys into pieces, the pieces leave
    their states in scratch and a second kernel merges them.  Same result as the un-cut launch (KRIYA_PREFILL_SPLIT=0)
    within rounding, and all within the bar of the oracle; a cut launch counts two kernels.  Mode "1" is the library's own
    policy (it cuts the second chunk, whose four tiles have 10 to 12 KV tiles each), mode "3" forces three pieces."""
    shape = W.AttnShape("cut", Hq, Hkv, D, dtype, rope_theta=1e6)
    total, prefix_chunks = 1500, (0, 1100)  # prompt in two chunks: 1100 + 400 (ragged last query tile, prefix > 0)
    mgr = PagedKvCacheManager(256, 0, 16)
    mgr.allocate_sequence(1, list(range(37)))
    mgr.allocate_sequence(2, list(range(5000, 5000 + total)))
    table, _ = mgr.sequence_table(2)
    rng = np.random.default_rng(91)
    q = W.normal16(rng, (total, Hq, D), dtype); k = W.normal16(rng, (total, Hkv, D), dtype); v = W.normal16(rng, (total, Hkv, D), dtype)
    results = {}
    for mode in ("1", "0", "3"):
        monkeypatch.setenv("KRIYA_PREFILL_SPLIT", mode)
        ex = make_executor(shape, 256, max_query_tokens=1100)
        ck = np.full((256, 16, Hkv, D), 0x7FC1 if dtype == W.BF16 else 0x7E01, np.uint16)
        fill_cache(ex, 0, ck, ck)
        rp = ex.rope_params()
        outs, launches = [], []
        for start, n in ((0, 1100), (1100, 400)):
            gp = ex.gqa_params(max_query_tokens=n)
            dq, dk, dv = dev16(q[start:start + n]), dev16(k[start:start + n]), dev16(v[start:start + n])
            out = torch.zeros_like(dq)
            torch.cuda.synchronize()
            ex.upload_schedule_plan(mgr.build_prefix_schedule_plan(2, start + n, 8))
            ex.rope_kv_append_chunk(0, dq, dk, dv, start, n, rp)
            before = ex.launch_count
            ex.paged_gqa_prefill(0, dq, out, start, n, gp)
            ex.sync()
            launches.append(ex.launch_count - before)
            outs.append(W.from_storage(host16(out), dtype))
        results[mode] = (np.concatenate(outs), launches)
        if mode == "1":
            gk, gv = read_cache(ex, 0)
        ex.close()
    assert results["1"][1] == [1, 2] and results["0"][1] == [1, 1] and results["3"][1] == [2, 2]
    # oracle over the final cache (the appended K/V are bit-exact, checked elsewhere)
    tab = O.rope_table(4096, D, shape.rope_theta)
    ok = np.full((256, 16, Hkv, D), 0x7FC1 if dtype == W.BF16 else 0x7E01, np.uint16); ov = ok.copy()
    refs = []
    exo = make_executor(shape, 256, max_query_tokens=1100)
    for start, n in ((0, 1100), (1100, 400)):
        rows = mgr.build_parallel_prefill_layout(2, start, n, 8)
        oq = q[start:start + n].copy()
        O.rope_kv_append(oq, k[start:start + n], v[start:start + n], ok, ov, rows.page_indptr, rows.page_indices,
                         rows.last_page_len, np.arange(start, start + n), oracle_rope(exo.rope_params()), dtype, table=tab)
        _, of = O.prefill_causal(oq, ok, ov, np.asarray(table, np.int32), start, oracle_gqa(exo), dtype)
        refs.append(of)
    exo.close()
    ref = np.concatenate(refs)
    assert np.array_equal(gk, ok) and np.array_equal(gv, ov)
    for mode in ("1", "0", "3"):
        got = results[mode][0]
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= TOL[dtype], mode
    assert np.abs(results["1"][0] - results["0"][0]).max() <= TOL[dtype]
    assert np.abs(results["3"][0] - results["0"][0]).max() <= TOL[dtype]
