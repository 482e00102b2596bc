"""Bookkeeping oracle: a line-by-line Python restatement of the reference's `kriya-kv` crate.

TEST INFRASTRUCTURE ONLY.  The shipped host code (the C++ manager inside the native
library) never imports this module; the tests use it as the checker for block ids,
refcounts, generations, copy-on-write pairs and plan arrays, all of which must match
bit for bit.

Every method cites the lines of `crates/kriya-kv/src/bsr_paged.rs` it follows.  The
restatement is pinned by the literal arrays of that file's own unit tests
(`bsr_paged.rs:739-889`), replayed in `tests/test_kv_oracle_golden.py`.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class OutOfBlocks(Exception):
    """bsr_paged.rs:14-19"""

    def __init__(self, requested: int, available: int):
        super().__init__(f"Out of physical KV blocks on GPU: requested {requested}, available {available}")
        self.requested = requested
        self.available = available


class InvalidSequenceId(Exception):
    """bsr_paged.rs:20-21"""


class InvalidBlockId(Exception):
    """bsr_paged.rs:22-23"""


@dataclass
class PhysicalKvBlock:
    """bsr_paged.rs:27-38"""

    block_id: int
    ref_count: int = 0
    num_hashed_tokens: int = 0
    prefix_hash: Optional[int] = None
    generation: int = 0


class BlockAllocator:
    """bsr_paged.rs:41-153: FIFO free list, refcount, generation counter."""

    def __init__(self, num_blocks: int, block_size_tokens: int):
        self.block_size_tokens = block_size_tokens
        self.blocks = [PhysicalKvBlock(i) for i in range(num_blocks)]
        self.free_list = deque(range(num_blocks))  # bsr_paged.rs:59

    def num_free_blocks(self) -> int:
        return len(self.free_list)

    def total_blocks(self) -> int:
        return len(self.blocks)

    def allocate_block(self) -> int:  # bsr_paged.rs:85-101
        if not self.free_list:
            raise OutOfBlocks(1, 0)
        block_id = self.free_list.popleft()
        blk = self.blocks[block_id]
        blk.ref_count = 1
        blk.generation += 1
        blk.num_hashed_tokens = 0
        blk.prefix_hash = None
        return block_id

    def _get(self, block_id: int) -> PhysicalKvBlock:
        if block_id < 0 or block_id >= len(self.blocks):
            raise InvalidBlockId(block_id)
        return self.blocks[block_id]

    def get_generation(self, block_id: int) -> int:  # bsr_paged.rs:105-111
        return self._get(block_id).generation

    def inc_ref(self, block_id: int) -> None:  # bsr_paged.rs:114-121
        self._get(block_id).ref_count += 1

    def free_block(self, block_id: int) -> bool:  # bsr_paged.rs:124-143
        blk = self._get(block_id)
        if blk.ref_count == 0:
            raise InvalidBlockId(block_id)
        blk.ref_count -= 1
        if blk.ref_count == 0:
            blk.num_hashed_tokens = 0
            blk.prefix_hash = None
            self.free_list.append(block_id)
            return True
        return False

    def ref_count(self, block_id: int) -> int:  # bsr_paged.rs:146-152
        return self._get(block_id).ref_count


@dataclass
class RadixNode:
    """bsr_paged.rs:157-166"""

    block_tokens: List[int] = field(default_factory=list)
    physical_block_id: Optional[int] = None
    block_generation: int = 0
    children: Dict[int, "RadixNode"] = field(default_factory=dict)


class RadixPrefixCache:
    """bsr_paged.rs:170-253"""

    def __init__(self, block_size_tokens: int):
        self.root = RadixNode()
        self.block_size_tokens = block_size_tokens

    def match_prefix(self, prompt_tokens, alloc: BlockAllocator) -> Tuple[List[int], int]:  # bsr_paged.rs:185-215
        blk_sz = self.block_size_tokens
        matched: List[int] = []
        current = self.root
        offset = 0
        while offset + blk_sz <= len(prompt_tokens):
            chunk = list(prompt_tokens[offset : offset + blk_sz])
            child = current.children.get(chunk[0])
            if child is not None and child.block_tokens == chunk and child.physical_block_id is not None:
                phys = child.physical_block_id
                try:
                    gen = alloc.get_generation(phys)
                except InvalidBlockId:
                    gen = 0
                try:
                    rc = alloc.ref_count(phys)
                except InvalidBlockId:
                    rc = 0
                if gen == child.block_generation and rc > 0:
                    alloc.inc_ref(phys)
                    matched.append(phys)
                    current = child
                    offset += blk_sz
                    continue
            break
        return matched, offset

    def insert_prefix(self, tokens, physical_blocks, alloc: BlockAllocator) -> None:  # bsr_paged.rs:218-252
        blk_sz = self.block_size_tokens
        num_full = min(len(tokens) // blk_sz, len(physical_blocks))
        current = self.root
        for i in range(num_full):
            chunk = list(tokens[i * blk_sz : (i + 1) * blk_sz])
            phys = physical_blocks[i]
            try:
                gen = alloc.get_generation(phys)
            except InvalidBlockId:
                gen = 0
            node = current.children.get(chunk[0])
            if node is None:
                node = RadixNode(chunk, phys, gen, {})
                current.children[chunk[0]] = node
            if node.block_tokens == chunk:
                node.physical_block_id = phys
                node.block_generation = gen
                current = node
            else:
                break


@dataclass
class SequenceBlockTable:
    """bsr_paged.rs:256-271"""

    seq_id: int
    logical_blocks: List[int]
    total_tokens: int

    def last_page_len(self, block_size_tokens: int) -> int:
        rem = self.total_tokens % block_size_tokens
        if rem == 0 and self.total_tokens > 0:
            return block_size_tokens
        return rem


@dataclass
class Plan:
    """FlashInferSchedulePlan + BsrKvLayout (bsr_paged.rs:274-321); tiles are 4-tuples
    (request_idx, kv_block_start, kv_block_count, is_split_k) like CtaWorkTile."""

    page_indptr: List[int]
    page_indices: List[int]
    last_page_len: List[int]
    cta_work_tiles: List[Tuple[int, int, int, int]]
    max_blocks_per_cta: int


def _div_ceil(a: int, b: int) -> int:
    return -(-a // b)


class PagedKvCacheManager:
    """bsr_paged.rs:325-733"""

    def __init__(self, num_gpu_blocks: int, num_cpu_swap_blocks: int, block_size_tokens: int):
        self.gpu_allocator = BlockAllocator(num_gpu_blocks, block_size_tokens)
        self.radix_cache = RadixPrefixCache(block_size_tokens)
        self.sequences: Dict[int, SequenceBlockTable] = {}

    def allocate_sequence(self, seq_id: int, prompt_tokens) -> int:  # bsr_paged.rs:342-385
        blk_sz = self.gpu_allocator.block_size_tokens
        logical, matched_tokens = self.radix_cache.match_prefix(prompt_tokens, self.gpu_allocator)
        total_needed = _div_ceil(len(prompt_tokens), blk_sz)
        additional = max(total_needed - len(logical), 0)
        if self.gpu_allocator.num_free_blocks() < additional:
            for b in logical:
                try:
                    self.gpu_allocator.free_block(b)
                except InvalidBlockId:
                    pass
            raise OutOfBlocks(additional, self.gpu_allocator.num_free_blocks())
        for _ in range(additional):
            logical.append(self.gpu_allocator.allocate_block())
        self.radix_cache.insert_prefix(prompt_tokens, logical, self.gpu_allocator)
        self.sequences[seq_id] = SequenceBlockTable(seq_id, logical, len(prompt_tokens))
        return matched_tokens

    def append_token_slot(self, seq_id: int) -> Tuple[int, Optional[Tuple[int, int]]]:  # bsr_paged.rs:389-426
        blk_sz = self.gpu_allocator.block_size_tokens
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise InvalidSequenceId(seq_id)
        if seq.total_tokens % blk_sz == 0:
            new_blk = self.gpu_allocator.allocate_block()
            seq.logical_blocks.append(new_blk)
            seq.total_tokens += 1
            return new_blk, None
        if not seq.logical_blocks:
            raise InvalidSequenceId(seq_id)
        tail = seq.logical_blocks[-1]
        if self.gpu_allocator.ref_count(tail) > 1:
            fresh = self.gpu_allocator.allocate_block()  # allocate first ...
            self.gpu_allocator.free_block(tail)  # ... then drop the shared tail
            seq.logical_blocks[-1] = fresh
            seq.total_tokens += 1
            return fresh, (tail, fresh)
        seq.total_tokens += 1
        return tail, None

    def fork_sequence(self, parent_seq_id: int, child_seq_id: int) -> None:  # bsr_paged.rs:430-454
        parent = self.sequences.get(parent_seq_id)
        if parent is None:
            raise InvalidSequenceId(parent_seq_id)
        blocks = list(parent.logical_blocks)
        for b in blocks:
            self.gpu_allocator.inc_ref(b)
        self.sequences[child_seq_id] = SequenceBlockTable(child_seq_id, blocks, parent.total_tokens)

    def free_sequence(self, seq_id: int) -> None:  # bsr_paged.rs:457-467
        seq = self.sequences.pop(seq_id, None)
        if seq is None:
            raise InvalidSequenceId(seq_id)
        for b in seq.logical_blocks:
            self.gpu_allocator.free_block(b)

    def contains_sequence(self, seq_id: int) -> bool:  # bsr_paged.rs:471-473
        return seq_id in self.sequences

    def block_for_position(self, seq_id: int, position: int) -> Tuple[int, int]:  # bsr_paged.rs:477-493
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise InvalidSequenceId(seq_id)
        blk_sz = self.gpu_allocator.block_size_tokens
        idx, slot = position // blk_sz, position % blk_sz
        if idx >= len(seq.logical_blocks):
            raise InvalidSequenceId(seq_id)
        return seq.logical_blocks[idx], slot

    def build_schedule_plan(self, active_seq_ids, max_blocks_per_cta: int) -> Plan:  # bsr_paged.rs:497-544
        blk_sz = self.gpu_allocator.block_size_tokens
        max_blk = max(max_blocks_per_cta, 1)
        indptr, indices, last, tiles = [0], [], [], []
        for req_idx, seq_id in enumerate(active_seq_ids):
            seq = self.sequences.get(seq_id)
            if seq is None:
                raise InvalidSequenceId(seq_id)
            indices.extend(seq.logical_blocks)
            indptr.append(len(indices))
            last.append(seq.last_page_len(blk_sz))
            n = len(seq.logical_blocks)
            split = 1 if n > max_blk else 0
            for start in range(0, n, max_blk):
                tiles.append((req_idx, start, min(n - start, max_blk), split))
        return Plan(indptr, indices, last, tiles, max_blk)

    def build_prefix_schedule_plan(self, seq_id: int, prefix_tokens: int, max_blocks_per_cta: int) -> Plan:
        # bsr_paged.rs:550-594
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise InvalidSequenceId(seq_id)
        if prefix_tokens == 0 or prefix_tokens > seq.total_tokens:
            raise InvalidSequenceId(seq_id)
        blk_sz = self.gpu_allocator.block_size_tokens
        n = _div_ceil(prefix_tokens, blk_sz)
        max_blk = max(max_blocks_per_cta, 1)
        split = 1 if n > max_blk else 0
        tiles = [(0, start, min(n - start, max_blk), split) for start in range(0, n, max_blk)]
        rem = prefix_tokens % blk_sz
        return Plan([0, n], list(seq.logical_blocks[:n]), [blk_sz if rem == 0 else rem], tiles, max_blk)

    def _check_prefill_args(self, seq_id, prefix_tokens, num_tokens) -> SequenceBlockTable:
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise InvalidSequenceId(seq_id)
        if num_tokens == 0 or min(prefix_tokens + num_tokens, 0xFFFFFFFF) > seq.total_tokens:
            raise InvalidSequenceId(seq_id)
        return seq

    def build_parallel_prefill_layout(self, seq_id, prefix_tokens, num_tokens, max_blocks_per_cta) -> Plan:
        # bsr_paged.rs:607-667: one BSR row per query token, rows concatenated
        blk_sz = self.gpu_allocator.block_size_tokens
        seq = self._check_prefill_args(seq_id, prefix_tokens, num_tokens)
        indptr, indices = [0], []
        for i in range(num_tokens):
            need = _div_ceil(prefix_tokens + i + 1, blk_sz)
            if need > len(seq.logical_blocks):
                raise IndexError("slice end out of range")  # the Rust slice would panic here
            indices.extend(seq.logical_blocks[:need])
            indptr.append(len(indices))
        last = [((prefix_tokens + i) % blk_sz) + 1 for i in range(num_tokens)]
        tiles = []
        for i in range(num_tokens):
            n = _div_ceil(prefix_tokens + i + 1, blk_sz)
            tiles.append((0, 0, n, 1 if n > max_blocks_per_cta else 0))
        return Plan(indptr, indices, last, tiles, max_blocks_per_cta)

    def build_deduplicated_prefill_layout(self, seq_id, prefix_tokens, num_tokens, max_blocks_per_cta) -> Plan:
        # bsr_paged.rs:671-733: unique block list; indptr holds per-row block COUNTS
        blk_sz = self.gpu_allocator.block_size_tokens
        seq = self._check_prefill_args(seq_id, prefix_tokens, num_tokens)
        max_need = min(_div_ceil(prefix_tokens + num_tokens, blk_sz), len(seq.logical_blocks))
        indices = list(seq.logical_blocks[:max_need])
        indptr = [0] + [_div_ceil(prefix_tokens + i + 1, blk_sz) for i in range(num_tokens)]
        last = [((prefix_tokens + i) % blk_sz) + 1 for i in range(num_tokens)]
        tiles = []
        for i in range(num_tokens):
            n = _div_ceil(prefix_tokens + i + 1, blk_sz)
            tiles.append((0, 0, n, 1 if n > max_blocks_per_cta else 0))
        return Plan(indptr, indices, last, tiles, max_blocks_per_cta)
