"""Host-side mirror of the reference's `kriya-kv` manager API over the compiled C++ library.

Method names, argument meaning and error behaviour follow
`crates/kriya-kv/src/bsr_paged.rs` (`PagedKvCacheManager`, `BlockAllocator`), so tests written
against the Rust API read the same here.  All bookkeeping runs in `libkriya_kv.so`.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _native as N


class KvCacheError(Exception):
    """bsr_paged.rs:12-24"""


class OutOfBlocks(KvCacheError):
    def __init__(self, requested: int, available: int):
        super().__init__(f"Out of physical KV blocks on GPU: requested {requested}, available {available}")
        self.requested = requested
        self.available = available


class InvalidSequenceId(KvCacheError):
    pass


class InvalidBlockId(KvCacheError):
    pass


@dataclass
class FlashInferSchedulePlan:
    """bsr_paged.rs:274-321; arrays are numpy copies owned by the plan."""

    page_indptr: np.ndarray  # int32 [rows + 1]
    page_indices: np.ndarray  # int32
    last_page_len: np.ndarray  # int32 [rows]
    cta_work_tiles: np.ndarray  # uint32 [tiles, 4] = (request_idx, kv_block_start, kv_block_count, is_split_k)
    max_blocks_per_cta: int


def _copy(ptr, n, dtype):
    if n == 0:
        return np.zeros(0, dtype=dtype)
    return np.ctypeslib.as_array(ptr, shape=(n,)).astype(dtype, copy=True)


class _Allocator:
    """The `gpu_allocator` field of the manager (BlockAllocator accessors, bsr_paged.rs:69-152)."""

    def __init__(self, owner: "PagedKvCacheManager"):
        self._o = owner

    def num_free_blocks(self) -> int:
        return int(self._o._lib.kriya_kv_num_free_blocks(self._o._h))

    def total_blocks(self) -> int:
        return int(self._o._lib.kriya_kv_total_blocks(self._o._h))

    def block_size_tokens(self) -> int:
        return int(self._o._lib.kriya_kv_block_size_tokens(self._o._h))

    def ref_count(self, block_id: int) -> int:
        out = C.c_uint32()
        self._o._check(self._o._lib.kriya_kv_ref_count(self._o._h, block_id, C.byref(out)))
        return out.value

    def get_generation(self, block_id: int) -> int:
        out = C.c_uint64()
        self._o._check(self._o._lib.kriya_kv_generation(self._o._h, block_id, C.byref(out)))
        return out.value

    def allocate_block(self) -> int:
        out = C.c_uint32()
        self._o._check(self._o._lib.kriya_kv_allocate_block(self._o._h, C.byref(out)))
        return out.value

    def inc_ref(self, block_id: int) -> None:
        self._o._check(self._o._lib.kriya_kv_inc_ref(self._o._h, block_id))

    def free_block(self, block_id: int) -> bool:
        out = C.c_int32()
        self._o._check(self._o._lib.kriya_kv_free_block(self._o._h, block_id, C.byref(out)))
        return bool(out.value)


class PagedKvCacheManager:
    """bsr_paged.rs:325-733"""

    def __init__(self, num_gpu_blocks: int, num_cpu_swap_blocks: int, block_size_tokens: int):
        self._lib = N.kv_lib()
        self._h = self._lib.kriya_kv_create(num_gpu_blocks, num_cpu_swap_blocks, block_size_tokens)
        if not self._h:
            raise ValueError("block_size_tokens must be non-zero")
        self.gpu_allocator = _Allocator(self)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.kriya_kv_destroy(h)

    def _check(self, rc: int) -> None:
        if rc == 0:
            return
        info = N.KvErrorInfo()
        self._lib.kriya_kv_last_error(self._h, C.byref(info))
        if rc == -1:
            raise OutOfBlocks(int(info.requested), int(info.available))
        if rc == -2:
            raise InvalidSequenceId(int(info.id))
        if rc == -3:
            raise InvalidBlockId(int(info.id))
        raise KvCacheError(f"kriya_kv error {rc}")

    def allocate_sequence(self, seq_id: int, prompt_tokens: Sequence[int]) -> int:
        toks = np.ascontiguousarray(prompt_tokens, dtype=np.uint32)
        matched = C.c_size_t()
        self._check(self._lib.kriya_kv_allocate_sequence(
            self._h, seq_id, toks.ctypes.data_as(C.POINTER(C.c_uint32)), toks.size, C.byref(matched)))
        return matched.value

    def append_token_slot(self, seq_id: int) -> Tuple[int, Optional[Tuple[int, int]]]:
        blk, has, src, dst = C.c_uint32(), C.c_int32(), C.c_uint32(), C.c_uint32()
        self._check(self._lib.kriya_kv_append_token_slot(self._h, seq_id, C.byref(blk), C.byref(has), C.byref(src),
                                                         C.byref(dst)))
        return blk.value, ((src.value, dst.value) if has.value else None)

    def append_token_slots(self, seq_ids) -> Tuple[np.ndarray, List[Tuple[int, int]]]:
        """One append_token_slot per sequence, in order, in one native call (the scheduler's per-iteration loop,
        orca_engine.rs:267-278).  Returns (block per sequence, copy-on-write pairs)."""
        ids = np.ascontiguousarray(seq_ids, np.uint64)
        blocks = np.empty(ids.size, np.uint32)
        pairs = np.empty((max(ids.size, 1), 2), np.uint32)
        n_cow, done = C.c_size_t(), C.c_size_t()
        self._check(self._lib.kriya_kv_append_token_slots(self._h, ids.ctypes.data, ids.size, blocks.ctypes.data,
                                                          pairs.ctypes.data, C.byref(n_cow), C.byref(done)))
        return blocks, [(int(a), int(b)) for a, b in pairs[: n_cow.value]]

    def fork_sequence(self, parent_seq_id: int, child_seq_id: int) -> None:
        self._check(self._lib.kriya_kv_fork_sequence(self._h, parent_seq_id, child_seq_id))

    def free_sequence(self, seq_id: int) -> None:
        self._check(self._lib.kriya_kv_free_sequence(self._h, seq_id))

    def contains_sequence(self, seq_id: int) -> bool:
        return bool(self._lib.kriya_kv_contains_sequence(self._h, seq_id))

    def block_for_position(self, seq_id: int, position: int) -> Tuple[int, int]:
        blk, slot = C.c_uint32(), C.c_uint32()
        self._check(self._lib.kriya_kv_block_for_position(self._h, seq_id, position, C.byref(blk), C.byref(slot)))
        return blk.value, slot.value

    def sequence_table(self, seq_id: int) -> Tuple[List[int], int]:
        ptr, n, total = C.POINTER(C.c_uint32)(), C.c_size_t(), C.c_uint32()
        self._check(self._lib.kriya_kv_sequence_table(self._h, seq_id, C.byref(ptr), C.byref(n), C.byref(total)))
        return _copy(ptr, n.value, np.uint32).tolist(), total.value

    def _plan(self, view: N.KvPlanView) -> FlashInferSchedulePlan:
        tiles = np.zeros((view.cta_work_tiles_len, 4), dtype=np.uint32)
        if view.cta_work_tiles_len:
            raw = C.cast(view.cta_work_tiles, C.POINTER(C.c_uint32))
            tiles = np.ctypeslib.as_array(raw, shape=(view.cta_work_tiles_len, 4)).astype(np.uint32, copy=True)
        return FlashInferSchedulePlan(
            _copy(view.page_indptr, view.page_indptr_len, np.int32),
            _copy(view.page_indices, view.page_indices_len, np.int32),
            _copy(view.last_page_len, view.last_page_len_len, np.int32), tiles, int(view.max_blocks_per_cta))

    def build_schedule_plan(self, active_seq_ids: Sequence[int], max_blocks_per_cta: int) -> FlashInferSchedulePlan:
        ids = np.ascontiguousarray(active_seq_ids, dtype=np.uint64)
        view = N.KvPlanView()
        self._check(self._lib.kriya_kv_build_schedule_plan(self._h, ids.ctypes.data_as(C.POINTER(C.c_uint64)),
                                                           ids.size, max_blocks_per_cta, C.byref(view)))
        return self._plan(view)

    def build_prefix_schedule_plan(self, seq_id: int, prefix_tokens: int, max_blocks_per_cta: int):
        view = N.KvPlanView()
        self._check(self._lib.kriya_kv_build_prefix_schedule_plan(self._h, seq_id, prefix_tokens, max_blocks_per_cta,
                                                                  C.byref(view)))
        return self._plan(view)

    def build_parallel_prefill_layout(self, seq_id: int, prefix_tokens: int, num_tokens: int, max_blocks_per_cta: int):
        view = N.KvPlanView()
        self._check(self._lib.kriya_kv_build_parallel_prefill_layout(self._h, seq_id, prefix_tokens, num_tokens,
                                                                     max_blocks_per_cta, C.byref(view)))
        return self._plan(view)

    def build_deduplicated_prefill_layout(self, seq_id: int, prefix_tokens: int, num_tokens: int,
                                          max_blocks_per_cta: int):
        view = N.KvPlanView()
        self._check(self._lib.kriya_kv_build_deduplicated_prefill_layout(self._h, seq_id, prefix_tokens, num_tokens,
                                                                         max_blocks_per_cta, C.byref(view)))
        return self._plan(view)
