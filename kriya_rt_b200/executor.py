"""Host-side mirror of the attention / KV ops of the reference executor over `libkriya_cuda.so`.

`CudaExecutor` stands where `MetalExecutor` (crates/kriya-backend-metal/src/encoder.rs) stands in the
reference: it owns the KV pool and the per-step plan buffers and exposes the ops of the hot path.
Every method is one call through the C ABI of `include/kriya_cuda.h`; device arrays are passed as raw
pointers (anything with `.data_ptr()` or an int), host arrays as numpy arrays.  There is no fallback:
a missing library or a missing GPU raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _native as N
from ._native import BsrGqaParams, RopeKvWriteParams, TreeVerifyParams

DTYPE_BF16, DTYPE_FP16 = 0, 1
KV_16BIT, KV_Q4_GROUP32 = 0, 1


class CudaBackendError(RuntimeError):
    """MetalError (encoder.rs:32-54) for this backend; `.code` is the kriya_cuda_status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


class InvalidExecutionInput(CudaBackendError):
    pass


def _ptr(x) -> Optional[int]:
    if x is None:
        return None
    if hasattr(x, "data_ptr"):
        return int(x.data_ptr())
    if isinstance(x, np.ndarray):
        return int(x.ctypes.data)
    return int(x)


class CudaExecutor:
    def __init__(self, *, num_layers: int, num_kv_blocks: int, block_size_tokens: int, num_q_heads: int,
                 num_kv_heads: int, head_dim: int, dtype: int = DTYPE_BF16, device: int = 0, rotary_dim: int = 0,
                 rope_theta: float = 10000.0, rope_max_seq_len: int = 0, max_batch_rows: int = 0,
                 max_page_indices: int = 0, max_tiles: int = 0, max_query_tokens: int = 0, kv_format: int = 0):
        self._lib = N.cuda_lib()
        self.cfg = N.CudaConfig(device, num_layers, num_kv_blocks, block_size_tokens, num_q_heads, num_kv_heads,
                                head_dim, dtype, rotary_dim, rope_theta, rope_max_seq_len, max_batch_rows,
                                max_page_indices, max_tiles, max_query_tokens, kv_format)
        h = C.c_void_p()
        rc = self._lib.kriya_cuda_ctx_create(C.byref(self.cfg), C.byref(h))
        if rc != 0:
            raise self._error(rc, None)
        self._h = h
        self.num_layers, self.num_kv_blocks, self.block_size_tokens = num_layers, num_kv_blocks, block_size_tokens
        self.num_q_heads, self.num_kv_heads, self.head_dim, self.dtype = num_q_heads, num_kv_heads, head_dim, dtype
        self.rotary_dim = rotary_dim or head_dim
        self.rope_theta = rope_theta
        self.rope_max_seq_len = rope_max_seq_len or 4096
        self.kv_format = kv_format

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.kriya_cuda_ctx_destroy(h)

    def __del__(self):
        self.close()

    def _error(self, rc: int, h) -> CudaBackendError:
        msg = self._lib.kriya_cuda_last_error(h)
        text = msg.decode() if msg else ""
        return (InvalidExecutionInput if rc == -2 else CudaBackendError)(rc, text)

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise self._error(rc, self._h)

    # ---- parameter blocks as the reference fills them (encoder.rs:4953-4966, 4990-4999) -------------
    def rope_params(self, *, apply_qk_norm: bool = False, rms_eps: float = 1e-6, has_table: bool = True,
                    rope_theta: Optional[float] = None, rotary_dim: Optional[int] = None) -> RopeKvWriteParams:
        return RopeKvWriteParams(self.num_q_heads, self.num_kv_heads, self.head_dim,
                                 self.rotary_dim if rotary_dim is None else rotary_dim, self.block_size_tokens,
                                 int(apply_qk_norm), rms_eps, self.rope_theta if rope_theta is None else rope_theta,
                                 self.rope_max_seq_len, int(has_table), 0, 0)

    def gqa_params(self, *, max_query_tokens: int = 1, sm_scale: Optional[float] = None,
                   logit_softcap: float = 0.0) -> BsrGqaParams:
        scale = float(np.float32(1.0) / np.sqrt(np.float32(self.head_dim))) if sm_scale is None else sm_scale
        return BsrGqaParams(self.num_q_heads, self.num_kv_heads, self.head_dim, self.block_size_tokens, 16,
                            max_query_tokens, scale, logit_softcap)

    # ---- context accessors -----------------------------------------------------------------------
    def layer_kv_byte_offset(self, layer: int) -> int:
        return int(self._lib.kriya_cuda_layer_kv_byte_offset(self._h, layer))

    def kv_pool_ptrs(self, layer: int):
        k, v = C.c_void_p(), C.c_void_p()
        self._check(self._lib.kriya_cuda_kv_pool_ptrs(self._h, layer, C.byref(k), C.byref(v)))
        return k.value, v.value

    def layer_cache_views(self, layer: int):
        """Zero-copy torch views (int16 bit patterns) of one layer's K and V pools,
        shaped [num_kv_blocks, block_size, Hkv, D].  For tests and for hosts that fill the cache themselves."""
        import torch

        k, v = self.kv_pool_ptrs(layer)
        shape = (self.num_kv_blocks, self.block_size_tokens, self.num_kv_heads, self.head_dim)
        if self.kv_format == KV_Q4_GROUP32:  # 20 bytes per 32 values, seen as 10 int16 words
            shape = shape[:3] + (self.head_dim // 32 * 10,)

        class _Raw:
            def __init__(self, ptr):
                self.__cuda_array_interface__ = {"shape": shape, "typestr": "<i2", "data": (ptr, False), "version": 3}

        dev = f"cuda:{self.cfg.device}"
        return torch.as_tensor(_Raw(k), device=dev), torch.as_tensor(_Raw(v), device=dev)

    @property
    def stream_ptr(self) -> int:
        return int(self._lib.kriya_cuda_stream(self._h))

    @property
    def launch_count(self) -> int:
        return int(self._lib.kriya_cuda_launch_count(self._h))

    def sync(self, timeout_ms: int = 0) -> None:
        self._check(self._lib.kriya_cuda_sync(self._h, timeout_ms))

    # ---- plan ------------------------------------------------------------------------------------
    def plan_upload(self, page_indptr, page_indices, last_page_len, cta_work_tiles=None, seq_positions=None) -> None:
        indptr = np.ascontiguousarray(page_indptr, dtype=np.int32)
        indices = np.ascontiguousarray(page_indices, dtype=np.int32)
        last = np.ascontiguousarray(last_page_len, dtype=np.int32)
        tiles = np.zeros((0, 4), np.uint32) if cta_work_tiles is None else np.ascontiguousarray(cta_work_tiles, np.uint32)
        pos = np.zeros(0, np.uint32) if seq_positions is None else np.ascontiguousarray(seq_positions, np.uint32)
        self._check(self._lib.kriya_cuda_plan_upload(
            self._h, indptr.ctypes.data, indptr.size, indices.ctypes.data, indices.size, last.ctypes.data, last.size,
            tiles.ctypes.data, tiles.shape[0], pos.ctypes.data, pos.size))

    def upload_schedule_plan(self, plan, seq_positions=None) -> None:
        """`plan` is a FlashInferSchedulePlan as the kv manager builds it."""
        self.plan_upload(plan.page_indptr, plan.page_indices, plan.last_page_len, plan.cta_work_tiles, seq_positions)

    # ---- ops -------------------------------------------------------------------------------------
    def rope_kv_append(self, layer: int, q_inout, k_in, v_in, num_tokens: int, params: RopeKvWriteParams,
                       q_norm_w=None, k_norm_w=None) -> None:
        self._check(self._lib.kriya_cuda_rope_kv_append(self._h, layer, _ptr(q_inout), _ptr(k_in), _ptr(v_in),
                                                        _ptr(q_norm_w), _ptr(k_norm_w), num_tokens, C.byref(params)))

    def rope_kv_append_chunk(self, layer: int, q_inout, k_in, v_in, prefix_tokens: int, num_tokens: int,
                             params: RopeKvWriteParams, q_norm_w=None, k_norm_w=None) -> None:
        self._check(self._lib.kriya_cuda_rope_kv_append_chunk(
            self._h, layer, _ptr(q_inout), _ptr(k_in), _ptr(v_in), _ptr(q_norm_w), _ptr(k_norm_w), prefix_tokens,
            num_tokens, C.byref(params)))

    def rope_kv_append_chunk_batch(self, layer: int, q_inout, k_in, v_in, q_start, prefix, count, params: RopeKvWriteParams,
                                   q_norm_w=None, k_norm_w=None) -> None:
        """Chunks of several sequences appended in one launch; plan row r is sequence r's table (as paged_gqa_prefill_batch)."""
        qs = np.ascontiguousarray(q_start, np.uint32)
        pf = np.ascontiguousarray(prefix, np.uint32)
        ct = np.ascontiguousarray(count, np.uint32)
        self._check(self._lib.kriya_cuda_rope_kv_append_chunk_batch(
            self._h, layer, _ptr(q_inout), _ptr(k_in), _ptr(v_in), _ptr(q_norm_w), _ptr(k_norm_w), qs.size, qs.ctypes.data,
            pf.ctypes.data, ct.ctypes.data, C.byref(params)))

    def rope_inplace(self, q_inout, k_inout, num_tokens: int, params: RopeKvWriteParams, q_norm_w=None,
                     k_norm_w=None) -> None:
        """apply_rope_inplace (paged_gqa_and_deltanet.metal:1738-1829): q and k rotated where they are, positions of the plan."""
        self._check(self._lib.kriya_cuda_rope_inplace(self._h, _ptr(q_inout), _ptr(k_inout), _ptr(q_norm_w), _ptr(k_norm_w),
                                                      num_tokens, C.byref(params)))

    def tree_verify_params(self, num_tree_nodes: int, prefix_tokens: int, sm_scale: Optional[float] = None) -> TreeVerifyParams:
        """TreeVerifyGqaParams for a prefix of `prefix_tokens` cached tokens (enc:3313-3326)."""
        bs = self.block_size_tokens
        blocks = (prefix_tokens + bs - 1) // bs
        last = prefix_tokens - (blocks - 1) * bs if blocks else 0
        scale = float(sm_scale) if sm_scale is not None else 1.0 / float(np.sqrt(self.head_dim))
        return TreeVerifyParams(num_tree_nodes, self.num_q_heads, self.num_kv_heads, self.head_dim, bs, blocks, last, scale)

    def tree_verify(self, layer: int, tree_q, tree_k, tree_v, tree_mask, tree_out, params: TreeVerifyParams) -> None:
        """bsr_paged_gqa_tree_verify (metal:1620-1729): the plan holds one row per tree node, each the prefix table."""
        mask = np.ascontiguousarray(tree_mask, np.uint8)
        if mask.size != params.num_tree_nodes ** 2:
            raise ValueError("tree_mask must hold num_tree_nodes x num_tree_nodes bytes")
        self._check(self._lib.kriya_cuda_tree_verify(self._h, layer, _ptr(tree_q), _ptr(tree_k), _ptr(tree_v),
                                                     mask.ctypes.data, _ptr(tree_out), C.byref(params)))

    def paged_gqa_decode(self, layer: int, q, out, params: BsrGqaParams) -> None:
        self._check(self._lib.kriya_cuda_paged_gqa_decode(self._h, layer, _ptr(q), _ptr(out), C.byref(params)))

    def paged_gqa_decode_partial(self, layer: int, q, blk_begin, blk_end, out_m, out_l, out_o,
                                 params: BsrGqaParams) -> None:
        b = None if blk_begin is None else np.ascontiguousarray(blk_begin, np.uint32)
        e = None if blk_end is None else np.ascontiguousarray(blk_end, np.uint32)
        self._check(self._lib.kriya_cuda_paged_gqa_decode_partial(
            self._h, layer, _ptr(q), _ptr(b), _ptr(e), _ptr(out_m), _ptr(out_l), _ptr(out_o), C.byref(params)))

    def plan_set_ranges(self, blk_begin, blk_end) -> None:
        """Block ranges for the partial-state decode of every layer of this plan (pass None ranges afterwards)."""
        b = np.ascontiguousarray(blk_begin, np.uint32)
        e = np.ascontiguousarray(blk_end, np.uint32)
        self._check(self._lib.kriya_cuda_plan_set_ranges(self._h, b.ctypes.data, e.ctypes.data))

    # ---- KV-axis split over several GPUs (kriya_comm.cu) -------------------------------------------------
    COMM_HANDLE_BYTES = 128

    def comm_export(self, max_rows: int = 1) -> bytes:
        """Allocates the exchange buffer and returns its handle (plain bytes, to be handed to every other rank)."""
        buf = C.create_string_buffer(self.COMM_HANDLE_BYTES)
        self._check(self._lib.kriya_cuda_comm_export(self._h, max_rows, buf))
        return buf.raw

    def comm_init(self, rank: int, handles: Sequence[bytes]) -> None:
        """`handles`: the handles of all ranks, ordered by rank (handles[rank] is this executor's own)."""
        blob = b"".join(bytes(h) for h in handles)
        if len(blob) != self.COMM_HANDLE_BYTES * len(handles):
            raise ValueError("every handle must hold COMM_HANDLE_BYTES bytes")
        self._check(self._lib.kriya_cuda_comm_init(self._h, len(handles), rank, C.c_char_p(blob)))

    def kvsplit_decode(self, layer: int, q, out, params: BsrGqaParams) -> None:
        """Partial decode over this rank's block ranges + exchange with the peers + merge, all on the executor's stream."""
        self._check(self._lib.kriya_cuda_kvsplit_decode(self._h, layer, _ptr(q), _ptr(out), C.byref(params)))

    def kvsplit_decode_step(self, q, out, params: BsrGqaParams) -> None:
        self._check(self._lib.kriya_cuda_kvsplit_decode_step(self._h, _ptr(q), _ptr(out), C.byref(params)))

    def merge_states(self, m, l, o, parts: int, rows_times_heads: int, out) -> None:
        self._check(self._lib.kriya_cuda_merge_states(self._h, _ptr(m), _ptr(l), _ptr(o), parts, rows_times_heads,
                                                      _ptr(out)))

    def merge_packed_states(self, packed, parts: int, rows_times_heads: int, out) -> None:
        """States gathered as one [parts, R*(D+2)] buffer, each part laid out [m | l | o]."""
        self._check(self._lib.kriya_cuda_merge_packed_states(self._h, _ptr(packed), parts, rows_times_heads, _ptr(out)))

    def paged_gqa_prefill(self, layer: int, q, out, prefix_tokens: int, num_tokens: int, params: BsrGqaParams) -> None:
        self._check(self._lib.kriya_cuda_paged_gqa_prefill(self._h, layer, _ptr(q), _ptr(out), prefix_tokens,
                                                           num_tokens, C.byref(params)))

    def paged_gqa_prefill_batch(self, layer: int, q, out, q_start, prefix, count, params: BsrGqaParams) -> None:
        """Chunks of several sequences in one launch; plan row r is sequence r's table."""
        qs = np.ascontiguousarray(q_start, np.uint32)
        pf = np.ascontiguousarray(prefix, np.uint32)
        ct = np.ascontiguousarray(count, np.uint32)
        self._check(self._lib.kriya_cuda_paged_gqa_prefill_batch(self._h, layer, _ptr(q), _ptr(out), qs.size, qs.ctypes.data,
                                                                 pf.ctypes.data, ct.ctypes.data, C.byref(params)))

    def kv_block_copy(self, pairs: Sequence) -> None:
        arr = np.ascontiguousarray(pairs, dtype=np.uint32).reshape(-1, 2)
        self._check(self._lib.kriya_cuda_kv_block_copy(self._h, arr.ctypes.data, arr.shape[0]))

    def kv_slot_write(self, layer: int, stage_k, stage_v, triples: Sequence) -> None:
        arr = np.ascontiguousarray(triples, dtype=np.uint32).reshape(-1, 3)
        self._check(self._lib.kriya_cuda_kv_slot_write(self._h, layer, _ptr(stage_k), _ptr(stage_v), arr.ctypes.data,
                                                       arr.shape[0]))

    def decode_layer_host(self, layer: int, q_host: np.ndarray, k_host: np.ndarray, v_host: np.ndarray,
                          out_host: np.ndarray, rope: RopeKvWriteParams, gqa: BsrGqaParams) -> None:
        rows = q_host.shape[0]
        self._check(self._lib.kriya_cuda_decode_layer_host(self._h, layer, _ptr(q_host), _ptr(k_host), _ptr(v_host),
                                                           _ptr(out_host), rows, C.byref(rope), C.byref(gqa)))

    def decode_step(self, q_inout, k_in, v_in, out, rows: int, rope: RopeKvWriteParams, gqa: BsrGqaParams) -> None:
        """All layers, device activations laid out [layers][rows][heads][D]."""
        self._check(self._lib.kriya_cuda_decode_step(self._h, _ptr(q_inout), _ptr(k_in), _ptr(v_in), _ptr(out), rows,
                                                     C.byref(rope), C.byref(gqa)))

    def decode_step_host(self, q_host, k_host, v_host, out_host, rows: int, rope: RopeKvWriteParams,
                         gqa: BsrGqaParams) -> None:
        """All layers, host activations (numpy arrays or pinned torch CPU tensors); waits for the result."""
        self._check(self._lib.kriya_cuda_decode_step_host(self._h, _ptr(q_host), _ptr(k_host), _ptr(v_host),
                                                          _ptr(out_host), rows, C.byref(rope), C.byref(gqa)))

    def decode_step_host_begin(self, q_host, k_host, v_host, out_host, rows: int, rope: RopeKvWriteParams,
                               gqa: BsrGqaParams) -> None:
        """Queues the whole step (copies in, layers, copies back) and returns; the host buffers stay untouched until
        decode_step_host_end().  The next step's plan may be built and uploaded in between: it queues behind this step."""
        self._check(self._lib.kriya_cuda_decode_step_host_begin(self._h, _ptr(q_host), _ptr(k_host), _ptr(v_host),
                                                                _ptr(out_host), rows, C.byref(rope), C.byref(gqa)))

    def decode_step_host_end(self, timeout_ms: int = 0) -> None:
        self._check(self._lib.kriya_cuda_decode_step_host_end(self._h, timeout_ms))

    def append_decode(self, layer: int, q, k_in, v_in, out, rope: RopeKvWriteParams, gqa: BsrGqaParams,
                      q_rope_out=None) -> None:
        """Append + decode of one layer in one launch; q is left un-rotated (see kriya_cuda_append_decode)."""
        self._check(self._lib.kriya_cuda_append_decode(self._h, layer, _ptr(q), _ptr(k_in), _ptr(v_in), _ptr(out),
                                                       _ptr(q_rope_out), C.byref(rope), C.byref(gqa)))

    def set_fused_append(self, mode) -> None:
        """1 / True: fused launches, consecutive layers may overlap at their edges (default); 0 / False: separate
        append and decode kernels; 3: fused, layers serialised (set-up may start early); 5: fused, a layer's activations
        wait for the previous layer while its cached K/V streams at once; 7: fused, ordinary launches."""
        self._check(self._lib.kriya_cuda_set_fused_append(self._h, int(mode)))

    def set_decode_path(self, path: int) -> None:
        """0 = by shape, 1 = CUDA-core decode kernel, 2 = a tensor-core decode kernel, 3 = the tensor-core kernel that
        copies one KV head at a time.  Upload the plan again afterwards."""
        self._check(self._lib.kriya_cuda_set_decode_path(self._h, path))

    def set_wait_limit_us(self, limit_us: int) -> None:
        """Limit of the bounded waits inside the tensor-core decode kernels (default 2 s)."""
        self._check(self._lib.kriya_cuda_set_wait_limit_us(self._h, limit_us))

    def selftest_wait_expiry(self) -> None:
        """Queues a kernel whose bounded wait runs out on purpose; the next sync() raises."""
        self._check(self._lib.kriya_cuda_selftest_wait_expiry(self._h))

    def set_attention_window(self, window_size: int) -> None:
        """SlidingWindowCausal { window_size } (descriptor.rs:63-70); 0 = plain causal.  Upload the plan again afterwards."""
        self._check(self._lib.kriya_cuda_set_attention_window(self._h, window_size))

    def timing_enable(self, enable: bool) -> None:
        self._check(self._lib.kriya_cuda_timing_enable(self._h, int(enable)))

    def timing_read(self, kind: int):
        """(launches, total_ms) of decode (kind 0) or append (kind 1) kernels since the last read."""
        n, ms = C.c_uint64(), C.c_double()
        self._check(self._lib.kriya_cuda_timing_read(self._h, kind, C.byref(n), C.byref(ms)))
        return n.value, ms.value
