"""The compiled C++ manager (libkriya_kv.so through kriya_rt_b200.kv) against the reference's golden
expectations and, operation by operation, against the Python oracle: block ids, refcounts, generations,
copy-on-write pairs, error variants and every plan array must be identical."""
import json
from pathlib import Path

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from kriya_rt_b200 import kv as KV
from oracle import kv_oracle as KO
from kv_replay import replay

CASES = json.loads((Path(__file__).parent / "golden" / "kv_golden.json").read_text())["cases"]


class _NativeAllocator:
    def __init__(self, num_blocks, block_size):
        self._m = KV.PagedKvCacheManager(num_blocks, 0, block_size)

    def __getattr__(self, name):
        return getattr(self._m.gpu_allocator, name)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_native_matches_reference_unit_tests(case):
    replay(case, KV.PagedKvCacheManager, _NativeAllocator)


ERR = {KO.OutOfBlocks: KV.OutOfBlocks, KO.InvalidSequenceId: KV.InvalidSequenceId, KO.InvalidBlockId: KV.InvalidBlockId}


def _both(o_fn, n_fn):
    """Run the same call on oracle and native; results or error variants must agree."""
    try:
        o = o_fn()
        o_err = None
    except (KO.OutOfBlocks, KO.InvalidSequenceId, KO.InvalidBlockId) as e:
        o, o_err = None, e
    try:
        n = n_fn()
        n_err = None
    except KV.KvCacheError as e:
        n, n_err = None, e
    if o_err is None:
        assert n_err is None, f"native raised {n_err!r}, oracle returned {o!r}"
    else:
        assert isinstance(n_err, ERR[type(o_err)]), f"oracle raised {o_err!r}, native {n_err!r}"
        if isinstance(o_err, KO.OutOfBlocks):
            assert (n_err.requested, n_err.available) == (o_err.requested, o_err.available)
    return o, n


def _plans_equal(o, n):
    assert o.page_indptr == n.page_indptr.tolist()
    assert o.page_indices == n.page_indices.tolist()
    assert o.last_page_len == n.last_page_len.tolist()
    assert [tuple(t) for t in o.cta_work_tiles] == [tuple(int(x) for x in t) for t in n.cta_work_tiles]
    assert o.max_blocks_per_cta == n.max_blocks_per_cta


def _state_equal(o: KO.PagedKvCacheManager, n: KV.PagedKvCacheManager):
    assert o.gpu_allocator.num_free_blocks() == n.gpu_allocator.num_free_blocks()
    for b in range(o.gpu_allocator.total_blocks()):
        assert o.gpu_allocator.ref_count(b) == n.gpu_allocator.ref_count(b)
        assert o.gpu_allocator.get_generation(b) == n.gpu_allocator.get_generation(b)
    for sid, seq in o.sequences.items():
        blocks, total = n.sequence_table(sid)
        assert blocks == seq.logical_blocks and total == seq.total_tokens


op_strategy = st.lists(
    st.one_of(
        st.tuples(st.just("alloc"), st.integers(0, 7), st.integers(0, 3), st.integers(0, 40)),
        st.tuples(st.just("append"), st.integers(0, 7)),
        st.tuples(st.just("fork"), st.integers(0, 7), st.integers(0, 7)),
        st.tuples(st.just("free"), st.integers(0, 7)),
        st.tuples(st.just("plan"), st.lists(st.integers(0, 7), min_size=1, max_size=4), st.integers(0, 4)),
        st.tuples(st.just("prefix_plan"), st.integers(0, 7), st.integers(0, 45), st.integers(0, 3)),
        st.tuples(st.just("prefill"), st.integers(0, 7), st.integers(0, 20), st.integers(0, 20), st.integers(1, 3)),
        st.tuples(st.just("dedup"), st.integers(0, 7), st.integers(0, 20), st.integers(0, 20), st.integers(1, 3)),
        st.tuples(st.just("pos"), st.integers(0, 7), st.integers(0, 50)),
    ),
    min_size=1, max_size=60)


@settings(max_examples=150, deadline=None)
@given(ops=op_strategy, num_blocks=st.integers(1, 24), block_size=st.sampled_from([1, 4, 16]))
def test_random_operation_sequences_are_bit_identical(ops, num_blocks, block_size):
    o = KO.PagedKvCacheManager(num_blocks, 0, block_size)
    n = KV.PagedKvCacheManager(num_blocks, 0, block_size)
    # four prompt families that share prefixes, so radix hits, misses and first-token collisions all occur
    families = [list(range(100, 200)), list(range(100, 108)) + list(range(300, 400)),
                [100] + list(range(500, 600)), list(range(700, 800))]
    for op in ops:
        kind = op[0]
        if kind == "alloc":
            toks = families[op[2]][:op[3]]
            a, b = _both(lambda: o.allocate_sequence(op[1], toks), lambda: n.allocate_sequence(op[1], toks))
            assert a == b
        elif kind == "append":
            a, b = _both(lambda: o.append_token_slot(op[1]), lambda: n.append_token_slot(op[1]))
            assert a == b
        elif kind == "fork":
            _both(lambda: o.fork_sequence(op[1], op[2]), lambda: n.fork_sequence(op[1], op[2]))
        elif kind == "free":
            _both(lambda: o.free_sequence(op[1]), lambda: n.free_sequence(op[1]))
        elif kind == "plan":
            a, b = _both(lambda: o.build_schedule_plan(op[1], op[2]), lambda: n.build_schedule_plan(op[1], op[2]))
            if a is not None:
                _plans_equal(a, b)
        elif kind == "prefix_plan":
            a, b = _both(lambda: o.build_prefix_schedule_plan(op[1], op[2], op[3]),
                         lambda: n.build_prefix_schedule_plan(op[1], op[2], op[3]))
            if a is not None:
                _plans_equal(a, b)
        elif kind in ("prefill", "dedup"):
            fo = o.build_parallel_prefill_layout if kind == "prefill" else o.build_deduplicated_prefill_layout
            fn = n.build_parallel_prefill_layout if kind == "prefill" else n.build_deduplicated_prefill_layout
            a, b = _both(lambda: fo(op[1], op[2], op[3], op[4]), lambda: fn(op[1], op[2], op[3], op[4]))
            if a is not None:
                _plans_equal(a, b)
        elif kind == "pos":
            a, b = _both(lambda: o.block_for_position(op[1], op[2]), lambda: n.block_for_position(op[1], op[2]))
            assert a == b
        _state_equal(o, n)


def test_prefix_sharing_config_refcounts_and_cow_pairs():
    """The prefix-sharing benchmark shape in small: 8 sequences share a 4-block prefix through the radix
    cache (refcount 8), then forks of a parent with a partial tail each produce one copy-on-write pair."""
    for M in (KO.PagedKvCacheManager, KV.PagedKvCacheManager):
        m = M(256, 0, 16)
        prefix = list(range(1000, 1064))
        for s in range(8):
            matched = m.allocate_sequence(s, prefix + [5000 + 100 * s + i for i in range(20 + s)])
            assert matched == (0 if s == 0 else 64)
        blocks0 = m.sequences[0].logical_blocks if M is KO.PagedKvCacheManager else m.sequence_table(0)[0]
        for b in blocks0[:4]:
            assert m.gpu_allocator.ref_count(b) == 8
        m.allocate_sequence(100, prefix + list(range(9000, 9008)))  # 72 tokens: tail holds 8
        pairs = []
        for child in range(101, 105):
            m.fork_sequence(100, child)
            blk, cow = m.append_token_slot(child)
            assert cow is not None and cow[1] == blk
            pairs.append(cow)
        assert len({p[0] for p in pairs}) == 1 and len({p[1] for p in pairs}) == 4
        blk, cow = m.append_token_slot(100)  # parent's tail is private again after the children left it
        assert cow is None


def test_batched_append_equals_one_call_per_sequence():
    """kriya_kv_append_token_slots is the scheduler's loop in one native call: same blocks, same copy-on-write pairs,
    same manager state as append_token_slot per sequence (forked children with a shared partial tail included)."""
    from kriya_rt_b200.kv import PagedKvCacheManager

    def build():
        m = PagedKvCacheManager(64, 0, 16)
        m.allocate_sequence(1, list(range(40)))
        m.allocate_sequence(2, list(range(100, 132)))
        m.fork_sequence(1, 3)
        m.fork_sequence(1, 4)
        return m

    a, b = build(), build()
    ids = [3, 2, 4, 1]
    for _ in range(20):
        one = [a.append_token_slot(s) for s in ids]
        blocks, pairs = b.append_token_slots(ids)
        assert [blk for blk, _ in one] == list(blocks)
        assert [cow for _, cow in one if cow is not None] == pairs
        assert a.gpu_allocator.num_free_blocks() == b.gpu_allocator.num_free_blocks()
    for s in ids:
        assert a.sequence_table(s) == b.sequence_table(s)
