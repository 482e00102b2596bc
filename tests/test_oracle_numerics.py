"""Pins the C oracle's kernel math to the reference's own kernel tests.

The reference's GPU tests build inputs from closed-form expressions, compute the expected result with a
scalar CPU loop and assert a tolerance.  Here the inputs are regenerated from the same expressions, the CPU
loops are the restated ones (ko_ref_test_*), and the oracle's restatement of the shader math must agree with
them inside the reference's tolerance (and, since both are fp32 evaluations, far inside it)."""
import numpy as np
import pytest
import torch

from kriya_rt_b200 import workloads as W
from oracle import c_oracle as O


def gqa(Hq, Hkv, D, scale=None, splits=16, softcap=0.0):
    s = float(np.float32(1.0) / np.sqrt(np.float32(D))) if scale is None else scale
    return O.GqaParams(Hq, Hkv, D, 16, splits, 1, s, softcap)


def rope(Hq, Hkv, D, has_table=0, max_seq_len=4096, theta=10000.0, norm=0):
    return O.RopeParams(Hq, Hkv, D, D, 16, norm, 1e-6, theta, max_seq_len, has_table, 0, 0)


def test_bf16_rounding_matches_reference_definition_and_torch():
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 3,
                        np.array([0.0, -0.0, 1.0, 65504.0, 1e-40, 3.3895314e38, 0.00390625], np.float32)])
    mine = O.f32_to_16(x, O.BF16)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(mine, ref)  # RNE on finite values: same as quantizer.rs:19-24
    assert np.array_equal(mine, W.to_storage(x, W.BF16))
    assert np.array_equal(O.to_f32(mine, O.BF16), W.from_storage(mine, W.BF16))


def test_fp16_conversion_exhaustive_and_rne():
    allbits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    f = O.to_f32(allbits, O.FP16)
    ref = allbits.view(np.float16).astype(np.float32)
    assert np.array_equal(f.view(np.uint32)[~np.isnan(ref)], ref.view(np.uint32)[~np.isnan(ref)])
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 5, 200000),
                        np.array([65504.0, 65519.9, 65520.0, 1e9, 5.96e-8, 2.98e-8, 2.9802325e-8, 0.0, -0.0], np.float32)])
    x = x.astype(np.float32)
    with np.errstate(over="ignore"):
        assert np.array_equal(O.f32_to_16(x, O.FP16), x.astype(np.float16).view(np.uint16))


def test_paged_attention_3_tokens_matches_reference_cpu_loop():
    """test_shader_compile.rs:1037-1215: D=64, Hq=Hkv=1, three tokens appended one by one with
    transcendental RoPE, decode after each; expected = RoPE + softmax on the un-rounded f32 inputs; tol 0.01."""
    D, T = 64, 3
    f = np.float32
    q_raw = np.array([[f(t * 7 + d) * f(0.01) - f(0.2) for d in range(D)] for t in range(T)], f)
    k_raw = np.array([[f(t * 5 + d) * f(0.008) - f(0.15) for d in range(D)] for t in range(T)], f)
    v_raw = np.array([[f(t * 3 + d) * f(0.006) - f(0.1) for d in range(D)] for t in range(T)], f)
    ck = np.zeros((1, 16, 1, D), np.uint16)
    cv = np.zeros((1, 16, 1, D), np.uint16)
    out = None
    for t in range(T):
        q = O.f32_to_16(q_raw[t].reshape(1, 1, D), O.BF16)
        k = O.f32_to_16(k_raw[t].reshape(1, 1, D), O.BF16)
        v = O.f32_to_16(v_raw[t].reshape(1, 1, D), O.BF16)
        O.rope_kv_append(q, k, v, ck, cv, [0, 1], [0], [t + 1], [t], rope(1, 1, D, has_table=0), O.BF16)
        out, _ = O.decode(q, ck, cv, [0, 1], [0], [t + 1], gqa(1, 1, D, splits=1), O.BF16)
    expected = O.ref_test_rope_softmax_attention(q_raw, k_raw, v_raw)
    got = O.to_f32(out, O.BF16).reshape(D)
    assert np.abs(got - expected).max() < 0.01


def test_real_dimensions_decode_matches_reference_cpu_loop():
    """real_world_validation.rs:296-537: Hq=24, Hkv=8, D=128, 8 identity-mapped blocks; CPU loop runs on
    the un-rounded inputs; tol 0.05."""
    Hq, Hkv, D, NB = 24, 8, 128, 8
    f = np.float32
    q_f = ((np.arange(Hq * D, dtype=f) * f(0.01) - f(10.0)) * f(0.001)).astype(f)
    n = NB * 16 * Hkv * D
    k_f = ((np.arange(n, dtype=f) * f(0.008) - f(8.0)) * f(0.001)).astype(f)
    v_f = ((np.arange(n, dtype=f) * f(0.006) - f(6.0)) * f(0.001)).astype(f)
    expected = O.ref_test_online_decode(q_f, k_f, v_f, 1, Hq, Hkv, D, NB, 16)
    q = O.f32_to_16(q_f.reshape(1, Hq, D), O.BF16)
    ck = O.f32_to_16(k_f.reshape(NB, 16, Hkv, D), O.BF16)
    cv = O.f32_to_16(v_f.reshape(NB, 16, Hkv, D), O.BF16)
    out, outf = O.decode(q, ck, cv, [0, NB], list(range(NB)), [16], gqa(Hq, Hkv, D), O.BF16)
    assert np.abs(O.to_f32(out, O.BF16).ravel() - expected).max() <= 0.05
    # on identical (rounded) inputs the two fp32 evaluations agree to rounding noise
    exp_rounded = O.ref_test_online_decode(O.to_f32(q, O.BF16), O.to_f32(ck, O.BF16), O.to_f32(cv, O.BF16), 1, Hq, Hkv,
                                           D, NB, 16)
    assert np.abs(outf.ravel() - exp_rounded).max() < 2e-6


def test_causal_prefill_matches_reference_cpu_loop():
    """test_shader_compile.rs:1696-1881: T=16, Hq=2, Hkv=1, D=64, one block; CPU loop on rounded inputs; tol 0.05."""
    T, Hq, Hkv, D = 16, 2, 1, 64
    f = np.float32
    q_f = np.array([(f(i % 17) - f(8.0)) * f(0.05) for i in range(T * Hq * D)], f)
    k_f = np.array([(f(i % 13) - f(6.0)) * f(0.06) for i in range(16 * Hkv * D)], f)
    v_f = np.array([(f(i % 11) - f(5.0)) * f(0.07) for i in range(16 * Hkv * D)], f)
    q = O.f32_to_16(q_f.reshape(T, Hq, D), O.BF16)
    ck = O.f32_to_16(k_f.reshape(1, 16, Hkv, D), O.BF16)
    cv = O.f32_to_16(v_f.reshape(1, 16, Hkv, D), O.BF16)
    scale = float(f(1.0) / np.sqrt(f(D)))
    expected = O.ref_test_causal_prefill(O.to_f32(q, O.BF16), O.to_f32(ck, O.BF16), O.to_f32(cv, O.BF16), Hq, Hkv, D, scale)
    out, outf = O.prefill_causal(q, ck, cv, [0], 0, gqa(Hq, Hkv, D), O.BF16)
    assert np.abs(O.to_f32(out, O.BF16).ravel() - expected).max() < 0.05
    assert np.abs(outf.ravel() - expected).max() < 5e-6


def test_rope_table_matches_transcendental_path():
    """test_shader_compile.rs:2184-2355: table built as encoder.rs:1939-1950 vs pow/cos/sin in the kernel,
    D=64, positions {0,5,23,67}, inputs ((i%17)-8)*0.25, |diff| <= 1e-3 after bf16 rounding."""
    D, T = 64, 4
    init = O.f32_to_16(np.array([(np.float32(i % 17) - np.float32(8.0)) * np.float32(0.25) for i in range(T * D)],
                                np.float32).reshape(T, 1, D), O.BF16)
    table = O.rope_table(128, 64, 10000.0)
    pos = [0, 5, 23, 67]
    res = {}
    for has_table in (0, 1):
        q = init.copy()
        ck = np.zeros((T, 16, 1, D), np.uint16)
        cv = np.zeros((T, 16, 1, D), np.uint16)
        O.rope_kv_append(q, init.copy(), init.copy(), ck, cv, [0, 1, 2, 3, 4], [0, 1, 2, 3], [1, 1, 1, 1], pos,
                         rope(1, 1, D, has_table=has_table, max_seq_len=128), O.BF16, table=table)
        res[has_table] = (O.to_f32(q, O.BF16), O.to_f32(ck[:, 0], O.BF16), cv[:, 0].copy())
    assert np.abs(res[0][0] - res[1][0]).max() <= 1e-3
    assert np.abs(res[0][1] - res[1][1]).max() <= 1e-3
    assert np.array_equal(res[1][2].reshape(T, D), init.reshape(T, D))  # V is copied bit for bit
    # position 0 is the identity rotation
    assert np.array_equal(O.f32_to_16(res[1][0][0], O.BF16), init[0])


@pytest.mark.parametrize("dtype", [O.BF16, O.FP16])
def test_split_tiles_plus_reduce_equal_whole_row_decode(dtype):
    """Stage 1 over the reference's tiles (8 blocks each, with correct split slots) followed by the lse
    merge equals the one-tile-per-row evaluation; the reference never runs this on a GPU."""
    shape, batch, data = W.config1(dtype=dtype)
    p = gqa(shape.num_q_heads, shape.num_kv_heads, shape.head_dim, splits=16)
    whole, whole_f = O.decode(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr, batch.page_indices,
                              batch.last_page_len, p, dtype)
    tiles = batch.tiles
    split_idx = np.array([t[1] // 8 for t in tiles], np.uint32)
    final, pout, plse = O.decode_stage1(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr,
                                        batch.page_indices, batch.last_page_len, tiles, split_idx, p, dtype)
    nsplit = np.bincount(tiles[:, 0], minlength=batch.batch).astype(np.uint32)
    nsplit[nsplit <= 1] = 1
    O.split_k_reduce(pout, plse, nsplit, final, p, dtype)
    d = np.abs(O.to_f32(final, dtype) - whole_f).max()
    assert d < (2e-3 if dtype == O.FP16 else 1e-2)
    assert np.abs(O.to_f32(final, dtype) - O.to_f32(whole, dtype)).max() < (2e-3 if dtype == O.FP16 else 1e-2)


def test_kv_axis_partials_merge_to_whole_row():
    shape, batch, data = W.config1(dtype=O.BF16)
    p = gqa(shape.num_q_heads, shape.num_kv_heads, shape.head_dim)
    _, whole_f = O.decode(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr, batch.page_indices,
                          batch.last_page_len, p, O.BF16)
    nblk = np.diff(batch.page_indptr)
    parts = 4
    ms, ls, os_ = [], [], []
    for r in range(parts):
        b = (nblk * r) // parts
        e = (nblk * (r + 1)) // parts
        m, l, o = O.decode_partial(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr, batch.page_indices,
                                   batch.last_page_len, b, e, p, O.BF16)
        ms.append(m.reshape(-1)); ls.append(l.reshape(-1)); os_.append(o.reshape(-1, shape.head_dim))
    merged = O.merge_states(np.stack(ms), np.stack(ls), np.stack(os_))
    assert np.abs(merged - whole_f.reshape(-1, shape.head_dim)).max() < 1e-5


def test_decode_against_float64_softmax():
    """Independent check of the oracle itself: numpy float64 softmax attention on the same rounded inputs."""
    shape, batch, data = W.config1(dtype=O.BF16)
    Hq, Hkv, D = shape.num_q_heads, shape.num_kv_heads, shape.head_dim
    p = gqa(Hq, Hkv, D)
    _, outf = O.decode(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr, batch.page_indices,
                       batch.last_page_len, p, O.BF16)
    q = W.from_storage(data["q"], W.BF16).astype(np.float64)
    K = W.from_storage(data["cache_k"], W.BF16).astype(np.float64)
    V = W.from_storage(data["cache_v"], W.BF16).astype(np.float64)
    for r in range(batch.batch):
        blocks = batch.page_indices[batch.page_indptr[r]:batch.page_indptr[r + 1]]
        L = (len(blocks) - 1) * 16 + batch.last_page_len[r]
        k = K[blocks].reshape(-1, Hkv, D)[:L]
        v = V[blocks].reshape(-1, Hkv, D)[:L]
        for h in range(Hq):
            s = (k[:, h // (Hq // Hkv)] @ q[r, h]) * float(np.float32(p.sm_scale))
            w = np.exp(s - s.max()); w /= w.sum()
            assert np.abs(w @ v[:, h // (Hq // Hkv)] - outf[r, h]).max() < 1e-5


@pytest.mark.parametrize("window", [1, 7, 64, 1000])
def test_sliding_window_decode_and_prefill_against_float64_softmax(window):
    """SlidingWindowCausal (crates/kriya-core/src/descriptor.rs:63-70; the reference declares the mask, no kernel of its
    own reads it): the oracle's window - the last `window` keys of every query, the query's own position included -
    against numpy float64 softmax over exactly those keys, for decode rows and for the queries of a prefill chunk."""
    shape, batch, data = W.config1(dtype=O.BF16)
    Hq, Hkv, D = shape.num_q_heads, shape.num_kv_heads, shape.head_dim
    p = gqa(Hq, Hkv, D)
    q = W.from_storage(data["q"], W.BF16).astype(np.float64)
    K = W.from_storage(data["cache_k"], W.BF16).astype(np.float64)
    V = W.from_storage(data["cache_v"], W.BF16).astype(np.float64)
    scale = float(np.float32(p.sm_scale))

    def softmax_attend(qv, k, v):
        s = (k @ qv) * scale
        w = np.exp(s - s.max())
        return (w / w.sum()) @ v

    O.set_attention_window(window)
    try:
        _, outf = O.decode(data["q"], data["cache_k"], data["cache_v"], batch.page_indptr, batch.page_indices,
                           batch.last_page_len, p, O.BF16)
        table = batch.page_indices[batch.page_indptr[3]:batch.page_indptr[4]]
        prefix, n = 100, 40
        _, pf = O.prefill_causal(np.tile(data["q"][:1], (n, 1, 1)), data["cache_k"], data["cache_v"], table, prefix, p, O.BF16)
    finally:
        O.set_attention_window(0)
    for r in range(batch.batch):
        blocks = batch.page_indices[batch.page_indptr[r]:batch.page_indptr[r + 1]]
        L = (len(blocks) - 1) * 16 + batch.last_page_len[r]
        lo = max(L - window, 0)
        k = K[blocks].reshape(-1, Hkv, D)[lo:L]
        v = V[blocks].reshape(-1, Hkv, D)[lo:L]
        for h in range(Hq):
            g = h // (Hq // Hkv)
            assert np.abs(softmax_attend(q[r, h], k[:, g], v[:, g]) - outf[r, h]).max() < 1e-5
    kk = K[table].reshape(-1, Hkv, D)
    vv = V[table].reshape(-1, Hkv, D)
    for i in (0, 1, n - 1):
        hi = prefix + i + 1
        lo = max(hi - window, 0)
        for h in (0, Hq - 1):
            g = h // (Hq // Hkv)
            assert np.abs(softmax_attend(q[0, h], kk[lo:hi, g], vv[lo:hi, g]) - pf[i, h]).max() < 1e-5


def test_block_copy_and_slot_write_are_bytewise():
    rng = np.random.default_rng(5)
    ck = rng.integers(0, 65536, (3, 8, 16, 2, 64), dtype=np.uint16)
    cv = rng.integers(0, 65536, (3, 8, 16, 2, 64), dtype=np.uint16)
    k0, v0 = ck.copy(), cv.copy()
    O.block_copy(ck, cv, 3, [(1, 5), (2, 6)])
    assert np.array_equal(ck[:, 5], k0[:, 1]) and np.array_equal(cv[:, 6], v0[:, 2])
    untouched = [0, 1, 2, 3, 4, 7]
    assert np.array_equal(ck[:, untouched], k0[:, untouched]) and np.array_equal(cv[:, untouched], v0[:, untouched])
    sk = rng.integers(0, 65536, (4, 128), dtype=np.uint16)
    sv = rng.integers(0, 65536, (4, 128), dtype=np.uint16)
    O.slot_write(ck[0], cv[0], sk, sv, 16, [(2, 3, 7), (0, 4, 15)])
    assert np.array_equal(ck[0, 3, 7].ravel(), sk[2]) and np.array_equal(cv[0, 4, 15].ravel(), sv[0])


def test_tree_verify_with_a_chain_mask_is_causal_prefill():
    """A draft 'tree' that is a chain (mask lower-triangular) over a cached prefix is the causal prefill of those tokens: the two
    restatements (metal:1620-1729 and the prefill loop) must agree, which pins ko_tree_verify without a reference test."""
    from kriya_rt_b200 import workloads as W
    Hq, Hkv, D, dt = 6, 2, 64, W.BF16
    rng = np.random.default_rng(11)
    for prefix in (0, 5, 16, 77):
        n = 9
        nblk = (prefix + n + 15) // 16
        table = rng.permutation(12)[:nblk].astype(np.int32)
        ck = W.normal16(rng, (12, 16, Hkv, D), dt); cv = W.normal16(rng, (12, 16, Hkv, D), dt)
        q = W.normal16(rng, (n, Hq, D), dt); k = W.normal16(rng, (n, Hkv, D), dt); v = W.normal16(rng, (n, Hkv, D), dt)
        ck2, cv2 = ck.copy(), cv.copy()
        for i in range(n):  # the chunk's K/V at positions prefix + i
            pos = prefix + i
            ck2[table[pos // 16], pos % 16] = k[i]
            cv2[table[pos // 16], pos % 16] = v[i]
        gp = O.GqaParams(Hq, Hkv, D, 16, 16, n, 1.0 / np.sqrt(D), 0.0)
        _, want = O.prefill_causal(q, ck2, cv2, table, prefix, gp, dt)
        pb = (prefix + 15) // 16
        tp = O.TreeParams(n, Hq, Hkv, D, 16, pb, prefix - (pb - 1) * 16 if pb else 0, 1.0 / np.sqrt(D))
        _, got = O.tree_verify(q, k, v, ck, cv, table[:pb], np.tril(np.ones((n, n), np.uint8)), tp, dt)
        assert np.abs(got - want).max() <= 2e-6
