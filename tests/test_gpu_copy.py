"""Copy-on-write block copy and slot write on the GPU: bit-exact against the oracle's byte movers."""
import numpy as np
import pytest
import torch

from kriya_rt_b200 import workloads as W
from kriya_rt_b200.executor import InvalidExecutionInput
from kriya_rt_b200.kv import PagedKvCacheManager
from oracle import c_oracle as O
from gpu_util import dev16, fill_cache, make_executor, read_cache

pytestmark = pytest.mark.gpu


def test_cow_pairs_from_the_manager_copy_every_layer():
    shape = W.AttnShape("cow", 16, 2, 128, W.BF16)
    layers, nb = 3, 128
    mgr = PagedKvCacheManager(nb, 0, 16)
    mgr.allocate_sequence(100, list(range(64 + 8)))
    pairs = []
    for child in range(101, 109):
        mgr.fork_sequence(100, child)
        _blk, cow = mgr.append_token_slot(child)
        pairs.append(cow)
    assert all(p is not None for p in pairs)
    rng = np.random.default_rng(3)
    ck = rng.integers(0, 65536, (layers, nb, 16, 2, 128), dtype=np.uint16)
    cv = rng.integers(0, 65536, (layers, nb, 16, 2, 128), dtype=np.uint16)
    ex = make_executor(shape, nb, num_layers=layers)
    for l in range(layers):
        fill_cache(ex, l, ck[l], cv[l])
    ex.kv_block_copy(pairs)
    O.block_copy(ck, cv, layers, pairs)
    for l in range(layers):
        gk, gv = read_cache(ex, l)
        assert np.array_equal(gk, ck[l]) and np.array_equal(gv, cv[l])
    ex.close()


def test_chained_pairs_apply_in_order():
    shape = W.AttnShape("cow", 4, 2, 64, W.FP16)
    rng = np.random.default_rng(4)
    ck = rng.integers(0, 65536, (2, 16, 16, 2, 64), dtype=np.uint16)
    cv = rng.integers(0, 65536, (2, 16, 16, 2, 64), dtype=np.uint16)
    ex = make_executor(shape, 16, num_layers=2)
    for l in range(2):
        fill_cache(ex, l, ck[l], cv[l])
    # (10 -> 11) then (12 -> 10): block 10 is overwritten after it was read, block 11 must receive the old block 10
    pairs = [(0, 1), (1, 2), (2, 3), (5, 5), (7, 3), (3, 9), (10, 11), (12, 10)]
    ex.kv_block_copy(pairs)
    O.block_copy(ck, cv, 2, pairs)
    for l in range(2):
        gk, gv = read_cache(ex, l)
        assert np.array_equal(gk, ck[l]) and np.array_equal(gv, cv[l])
    with pytest.raises(InvalidExecutionInput, match="outside the pool"):
        ex.kv_block_copy([(0, 16)])
    ex.kv_block_copy([])
    ex.close()


def test_slot_write_commits_staged_rows():
    shape = W.AttnShape("spec", 16, 2, 128, W.BF16)
    rng = np.random.default_rng(5)
    ck = rng.integers(0, 65536, (32, 16, 2, 128), dtype=np.uint16)
    cv = rng.integers(0, 65536, (32, 16, 2, 128), dtype=np.uint16)
    sk = rng.integers(0, 65536, (16, 256), dtype=np.uint16)
    sv = rng.integers(0, 65536, (16, 256), dtype=np.uint16)
    ex = make_executor(shape, 32, num_layers=2)
    fill_cache(ex, 1, ck, cv)
    triples = [(3, 7, 0), (0, 31, 15), (15, 0, 8)]
    dsk, dsv = dev16(sk), dev16(sv)
    torch.cuda.synchronize()
    ex.kv_slot_write(1, dsk, dsv, triples)
    O.slot_write(ck, cv, sk, sv, 16, triples)
    gk, gv = read_cache(ex, 1)
    assert np.array_equal(gk, ck) and np.array_equal(gv, cv)
    g0k, g0v = read_cache(ex, 0)
    assert not g0k.any() and not g0v.any()  # other layers untouched (pool starts zeroed)
    ex.close()
