"""ctypes bindings of the two native libraries.  Loading fails loudly when a library is missing."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "lib"


class NativeLibraryMissing(ImportError):
    pass


def _load(name: str) -> C.CDLL:
    path = _LIB_DIR / name
    if not path.exists():
        raise NativeLibraryMissing(
            f"{path} is missing: build it with `python -m kriya_rt_b200.build` (there is no fallback path)")
    return C.CDLL(str(path))


# ---- POD structs, byte-identical to the reference's #[repr(C)] types -------------------------------


class CtaWorkTile(C.Structure):  # crates/kriya-kv/src/bsr_paged.rs:285-297
    _fields_ = [("request_idx", C.c_uint32), ("kv_block_start", C.c_uint32), ("kv_block_count", C.c_uint32),
                ("is_split_k", C.c_uint32)]


class RopeKvWriteParams(C.Structure):  # crates/kriya-backend-metal/src/encoder.rs:159-174
    _fields_ = [("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("rotary_dim", C.c_uint32), ("block_size_tokens", C.c_uint32), ("apply_qk_norm", C.c_uint32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("max_seq_len", C.c_uint32),
                ("has_table", C.c_uint32), ("_pad0", C.c_uint32), ("_pad1", C.c_uint32)]


class BsrGqaParams(C.Structure):  # crates/kriya-backend-metal/src/encoder.rs:176-187
    _fields_ = [("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("block_size_tokens", C.c_uint32), ("max_split_k_tiles", C.c_uint32),
                ("max_query_tokens", C.c_uint32), ("sm_scale", C.c_float), ("logit_softcap", C.c_float)]


class TreeVerifyParams(C.Structure):  # crates/kriya-backend-metal/src/encoder.rs:189-200
    _fields_ = [("num_tree_nodes", C.c_uint32), ("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("block_size_tokens", C.c_uint32), ("prefix_kv_blocks", C.c_uint32),
                ("prefix_last_len", C.c_uint32), ("sm_scale", C.c_float)]


class KvPlanView(C.Structure):
    _fields_ = [("page_indptr", C.POINTER(C.c_int32)), ("page_indptr_len", C.c_size_t),
                ("page_indices", C.POINTER(C.c_int32)), ("page_indices_len", C.c_size_t),
                ("last_page_len", C.POINTER(C.c_int32)), ("last_page_len_len", C.c_size_t),
                ("cta_work_tiles", C.POINTER(CtaWorkTile)), ("cta_work_tiles_len", C.c_size_t),
                ("max_blocks_per_cta", C.c_uint32)]


class KvErrorInfo(C.Structure):
    _fields_ = [("code", C.c_int32), ("requested", C.c_uint64), ("available", C.c_uint64), ("id", C.c_uint64)]


class CudaConfig(C.Structure):
    _fields_ = [("device", C.c_int32), ("num_layers", C.c_uint32), ("num_kv_blocks", C.c_uint32),
                ("block_size_tokens", C.c_uint32), ("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("dtype", C.c_uint32), ("rotary_dim", C.c_uint32),
                ("rope_theta", C.c_float), ("rope_max_seq_len", C.c_uint32), ("max_batch_rows", C.c_uint32),
                ("max_page_indices", C.c_uint32), ("max_tiles", C.c_uint32), ("max_query_tokens", C.c_uint32),
                ("kv_format", C.c_uint32)]


assert C.sizeof(CtaWorkTile) == 16 and C.sizeof(RopeKvWriteParams) == 48 and C.sizeof(BsrGqaParams) == 32

KV_SYMBOLS = {
    "kriya_kv_create": (C.c_void_p, [C.c_uint32, C.c_uint32, C.c_uint32]),
    "kriya_kv_destroy": (None, [C.c_void_p]),
    "kriya_kv_last_error": (None, [C.c_void_p, C.POINTER(KvErrorInfo)]),
    "kriya_kv_num_free_blocks": (C.c_size_t, [C.c_void_p]),
    "kriya_kv_total_blocks": (C.c_size_t, [C.c_void_p]),
    "kriya_kv_block_size_tokens": (C.c_uint32, [C.c_void_p]),
    "kriya_kv_ref_count": (C.c_int32, [C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32)]),
    "kriya_kv_generation": (C.c_int32, [C.c_void_p, C.c_uint32, C.POINTER(C.c_uint64)]),
    "kriya_kv_allocate_block": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "kriya_kv_inc_ref": (C.c_int32, [C.c_void_p, C.c_uint32]),
    "kriya_kv_free_block": (C.c_int32, [C.c_void_p, C.c_uint32, C.POINTER(C.c_int32)]),
    "kriya_kv_allocate_sequence": (C.c_int32, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.c_size_t,
                                               C.POINTER(C.c_size_t)]),
    "kriya_kv_append_token_slot": (C.c_int32, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_int32),
                                               C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "kriya_kv_append_token_slots": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                                                C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "kriya_kv_fork_sequence": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint64]),
    "kriya_kv_free_sequence": (C.c_int32, [C.c_void_p, C.c_uint64]),
    "kriya_kv_contains_sequence": (C.c_int32, [C.c_void_p, C.c_uint64]),
    "kriya_kv_block_for_position": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint32, C.POINTER(C.c_uint32),
                                                C.POINTER(C.c_uint32)]),
    "kriya_kv_sequence_table": (C.c_int32, [C.c_void_p, C.c_uint64, C.POINTER(C.POINTER(C.c_uint32)),
                                            C.POINTER(C.c_size_t), C.POINTER(C.c_uint32)]),
    "kriya_kv_build_schedule_plan": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint64), C.c_size_t, C.c_uint32,
                                                 C.POINTER(KvPlanView)]),
    "kriya_kv_build_prefix_schedule_plan": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32,
                                                        C.POINTER(KvPlanView)]),
    "kriya_kv_build_parallel_prefill_layout": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32,
                                                           C.POINTER(KvPlanView)]),
    "kriya_kv_build_deduplicated_prefill_layout": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32,
                                                               C.c_uint32, C.POINTER(KvPlanView)]),
}

_VP = C.c_void_p
CUDA_SYMBOLS = {
    "kriya_cuda_ctx_create": (C.c_int32, [C.POINTER(CudaConfig), C.POINTER(C.c_void_p)]),
    "kriya_cuda_ctx_destroy": (None, [_VP]),
    "kriya_cuda_last_error": (C.c_char_p, [_VP]),
    "kriya_cuda_layer_kv_byte_offset": (C.c_uint64, [_VP, C.c_uint32]),
    "kriya_cuda_kv_pool_ptrs": (C.c_int32, [_VP, C.c_uint32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "kriya_cuda_stream": (C.c_void_p, [_VP]),
    "kriya_cuda_sync": (C.c_int32, [_VP, C.c_uint32]),
    "kriya_cuda_plan_upload": (C.c_int32, [_VP, _VP, C.c_size_t, _VP, C.c_size_t, _VP, C.c_size_t, _VP, C.c_size_t,
                                           _VP, C.c_size_t]),
    "kriya_cuda_rope_kv_append": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, _VP, _VP, C.c_uint32,
                                              C.POINTER(RopeKvWriteParams)]),
    "kriya_cuda_rope_kv_append_chunk": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, _VP, _VP, C.c_uint32, C.c_uint32,
                                                    C.POINTER(RopeKvWriteParams)]),
    "kriya_cuda_rope_kv_append_chunk_batch": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, _VP, _VP, C.c_uint32, _VP, _VP, _VP,
                                                          C.POINTER(RopeKvWriteParams)]),
    "kriya_cuda_paged_gqa_decode": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, C.POINTER(BsrGqaParams)]),
    "kriya_cuda_paged_gqa_decode_partial": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, _VP, _VP, _VP,
                                                        C.POINTER(BsrGqaParams)]),
    "kriya_cuda_plan_set_ranges": (C.c_int32, [_VP, _VP, _VP]),
    "kriya_cuda_merge_states": (C.c_int32, [_VP, _VP, _VP, _VP, C.c_uint32, C.c_uint32, _VP]),
    "kriya_cuda_merge_packed_states": (C.c_int32, [_VP, _VP, C.c_uint32, C.c_uint32, _VP]),
    "kriya_cuda_paged_gqa_prefill": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, C.c_uint32, C.c_uint32,
                                                 C.POINTER(BsrGqaParams)]),
    "kriya_cuda_paged_gqa_prefill_batch": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, C.c_uint32, _VP, _VP, _VP,
                                                       C.POINTER(BsrGqaParams)]),
    "kriya_cuda_kv_block_copy": (C.c_int32, [_VP, _VP, C.c_uint32]),
    "kriya_cuda_kv_slot_write": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, C.c_uint32]),
    "kriya_cuda_decode_layer_host": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, _VP, C.c_uint32,
                                                 C.POINTER(RopeKvWriteParams), C.POINTER(BsrGqaParams)]),
    "kriya_cuda_append_decode": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, _VP, _VP, C.POINTER(RopeKvWriteParams),
                                             C.POINTER(BsrGqaParams)]),
    "kriya_cuda_set_fused_append": (C.c_int32, [_VP, C.c_int32]),
    "kriya_cuda_decode_step": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_uint32, C.POINTER(RopeKvWriteParams),
                                           C.POINTER(BsrGqaParams)]),
    "kriya_cuda_decode_step_host": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_uint32, C.POINTER(RopeKvWriteParams),
                                                C.POINTER(BsrGqaParams)]),
    "kriya_cuda_decode_step_host_begin": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_uint32, C.POINTER(RopeKvWriteParams),
                                                C.POINTER(BsrGqaParams)]),
    "kriya_cuda_decode_step_host_end": (C.c_int32, [_VP, C.c_uint32]),
    "kriya_cuda_set_decode_path": (C.c_int32, [_VP, C.c_int32]),
    "kriya_cuda_set_attention_window": (C.c_int32, [_VP, C.c_uint32]),
    "kriya_cuda_set_wait_limit_us": (C.c_int32, [_VP, C.c_uint32]),
    "kriya_cuda_selftest_wait_expiry": (C.c_int32, [_VP]),
    "kriya_cuda_debug_work_split": (C.c_int64, [_VP, _VP, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                    C.c_uint32, _VP, C.c_uint32, _VP]),
    "kriya_cuda_timing_enable": (C.c_int32, [_VP, C.c_int32]),
    "kriya_cuda_timing_read": (C.c_int32, [_VP, C.c_uint32, C.POINTER(C.c_uint64), C.POINTER(C.c_double)]),
    "kriya_cuda_paged_gqa_decode_static": (C.c_int32, [C.c_int32, _VP, C.c_uint32, _VP, _VP, _VP, C.c_uint32, _VP, _VP,
                                                       _VP, _VP, C.c_uint32, _VP, C.POINTER(BsrGqaParams), C.c_char_p,
                                                       C.c_size_t]),
    "kriya_cuda_launch_count": (C.c_uint64, [_VP]),
    "kriya_cuda_comm_export": (C.c_int32, [_VP, C.c_uint32, _VP]),
    "kriya_cuda_comm_init": (C.c_int32, [_VP, C.c_uint32, C.c_uint32, _VP]),
    "kriya_cuda_kvsplit_decode": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, C.POINTER(BsrGqaParams)]),
    "kriya_cuda_kvsplit_decode_step": (C.c_int32, [_VP, _VP, _VP, C.POINTER(BsrGqaParams)]),
    "kriya_cuda_rope_inplace": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_uint32, C.POINTER(RopeKvWriteParams)]),
    "kriya_cuda_tree_verify": (C.c_int32, [_VP, C.c_uint32, _VP, _VP, _VP, _VP, _VP, C.POINTER(TreeVerifyParams)]),
}


def _bind(lib: C.CDLL, table) -> C.CDLL:
    for name, (restype, argtypes) in table.items():
        fn = getattr(lib, name)  # AttributeError when the library does not export it
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


_kv = None
_cuda = None


def kv_lib() -> C.CDLL:
    global _kv
    if _kv is None:
        _kv = _bind(_load("libkriya_kv.so"), KV_SYMBOLS)
    return _kv


def cuda_lib() -> C.CDLL:
    global _cuda
    if _cuda is None:
        _cuda = _bind(_load("libkriya_cuda.so"), CUDA_SYMBOLS)
    return _cuda
