"""Pins the Python bookkeeping oracle to the reference's own unit-test expectations
(crates/kriya-kv/src/bsr_paged.rs:739-889, transcribed in tests/golden/kv_golden.json)."""
import json
from pathlib import Path

import pytest

from oracle import kv_oracle as KO
from kv_replay import replay

CASES = json.loads((Path(__file__).parent / "golden" / "kv_golden.json").read_text())["cases"]


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_reference_unit_tests(case):
    replay(case, KO.PagedKvCacheManager, KO.BlockAllocator)


def test_oracle_error_variants():
    m = KO.PagedKvCacheManager(2, 0, 4)
    with pytest.raises(KO.InvalidSequenceId):
        m.append_token_slot(9)
    with pytest.raises(KO.OutOfBlocks) as e:
        m.allocate_sequence(1, list(range(12)))
    assert (e.value.requested, e.value.available) == (3, 2)
    m.allocate_sequence(1, list(range(8)))
    with pytest.raises(KO.OutOfBlocks) as e:  # allocate_block reports (1, 0), bsr_paged.rs:89-93
        m.append_token_slot(1)
    assert (e.value.requested, e.value.available) == (1, 0)
    with pytest.raises(KO.InvalidBlockId):
        m.gpu_allocator.free_block(7)
    m.free_sequence(1)
    with pytest.raises(KO.InvalidBlockId):  # double free, bsr_paged.rs:130-132
        m.gpu_allocator.free_block(0)
    with pytest.raises(KO.InvalidSequenceId):
        m.build_prefix_schedule_plan(1, 1, 8)
