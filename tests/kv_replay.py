"""Replays one case of tests/golden/kv_golden.json against a manager implementation."""
import numpy as np


def replay(case, make_manager, make_allocator=None):
    if "allocator" in case:
        a = case["allocator"]
        alloc = make_allocator(a["num_blocks"], a["block_size"])
        b0 = None
        for op, expect in case["ops"]:
            if op == "num_free":
                assert alloc.num_free_blocks() == expect
            elif op == "allocate_block":
                b0 = alloc.allocate_block()
            elif op == "ref_count_b0":
                assert alloc.ref_count(b0) == expect
            elif op == "inc_ref_b0":
                alloc.inc_ref(b0)
            elif op == "free_block_b0":
                assert alloc.free_block(b0) is expect
            else:
                raise KeyError(op)
        return
    m = case["manager"]
    mgr = make_manager(m["num_blocks"], m["swap"], m["block_size"])
    for op in case["ops"]:
        name = op[0]
        if name == "allocate_sequence":
            matched = mgr.allocate_sequence(op[1], op[2])
            if op[3] is not None:
                assert matched == op[3], (case["name"], op)
        elif name == "allocate_sequence_range":
            mgr.allocate_sequence(op[1], list(range(op[2], op[3])))
        elif name == "num_free":
            assert mgr.gpu_allocator.num_free_blocks() == op[1], (case["name"], op)
        elif name == "fork_sequence":
            mgr.fork_sequence(op[1], op[2])
        elif name == "append_token_slot_cow_is_some":
            _blk, cow = mgr.append_token_slot(op[1])
            assert (cow is not None) is op[2]
        elif name == "append_token_slot_times":
            for _ in range(op[2]):
                mgr.append_token_slot(op[1])
        elif name == "free_sequence":
            mgr.free_sequence(op[1])
        elif name in ("parallel_prefill_layout", "dedup_prefill_layout", "prefix_plan", "schedule_plan"):
            if name == "parallel_prefill_layout":
                plan, exp = mgr.build_parallel_prefill_layout(op[1], op[2], op[3], op[4]), op[5]
            elif name == "dedup_prefill_layout":
                plan, exp = mgr.build_deduplicated_prefill_layout(op[1], op[2], op[3], op[4]), op[5]
            elif name == "prefix_plan":
                plan, exp = mgr.build_prefix_schedule_plan(op[1], op[2], op[3]), op[4]
            else:
                plan, exp = mgr.build_schedule_plan(op[1], op[2]), op[3]
            tiles = [tuple(int(x) for x in t) for t in plan.cta_work_tiles]
            for key, val in exp.items():
                if key in ("page_indptr", "page_indices", "last_page_len"):
                    assert list(np.asarray(getattr(plan, key)).tolist()) == val, (case["name"], key)
                elif key == "num_tiles":
                    assert len(tiles) == val
                elif key == "tile0_is_split_k":
                    assert tiles[0][3] == val
                elif key == "tile1_is_split_k":
                    assert tiles[1][3] == val
                elif key == "tile0_kv_block_count":
                    assert tiles[0][2] == val
                else:
                    raise KeyError(key)
        else:
            raise KeyError(name)
