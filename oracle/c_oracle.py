"""numpy-facing binding of `kriya_oracle.c` (TEST INFRASTRUCTURE ONLY, see the C file's header).

All arrays are host numpy arrays; 16-bit storage is carried as uint16 bit patterns.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "libkriya_oracle.so"
_SRC = _HERE / "kriya_oracle.c"

BF16, FP16 = 0, 1


class RopeParams(C.Structure):
    _fields_ = [("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("rotary_dim", C.c_uint32), ("block_size_tokens", C.c_uint32), ("apply_qk_norm", C.c_uint32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("max_seq_len", C.c_uint32),
                ("has_table", C.c_uint32), ("_pad0", C.c_uint32), ("_pad1", C.c_uint32)]


class GqaParams(C.Structure):
    _fields_ = [("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("block_size_tokens", C.c_uint32), ("max_split_k_tiles", C.c_uint32),
                ("max_query_tokens", C.c_uint32), ("sm_scale", C.c_float), ("logit_softcap", C.c_float)]


class TreeParams(C.Structure):
    _fields_ = [("num_tree_nodes", C.c_uint32), ("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("block_size_tokens", C.c_uint32), ("prefix_kv_blocks", C.c_uint32),
                ("prefix_last_len", C.c_uint32), ("sm_scale", C.c_float)]


def _cpu_stamp() -> str:
    """The library is built with -march=native, so it is only valid on the CPU model it was built on."""
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                import hashlib

                return hashlib.sha1(line.encode()).hexdigest()
    except OSError:
        pass
    return "unknown"


def build(force: bool = False) -> Path:
    """Compile the C oracle next to its source (gcc, OpenMP); rebuilt when the source or the host CPU changed."""
    stamp = _HERE / "libkriya_oracle.stamp"
    cur = _cpu_stamp()
    fresh = _SO.exists() and _SO.stat().st_mtime >= _SRC.stat().st_mtime and stamp.exists() and stamp.read_text() == cur
    if force or not fresh:
        subprocess.run(["gcc", "-O3", "-march=native", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-Wall",
                        str(_SRC), "-o", str(_SO), "-lm"], check=True)
        stamp.write_text(cur)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(str(build()))
        _lib.ko_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16
    return a


def num_threads() -> int:
    return int(lib().ko_num_threads())


def set_num_threads(n: int) -> None:
    lib().ko_set_num_threads(int(n))


def f32_to_16(x: np.ndarray, dtype: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().ko_f32_to_16(_p(x), _p(out), C.c_size_t(x.size), dtype)
    return out


def to_f32(x: np.ndarray, dtype: int) -> np.ndarray:
    x = _u16(x)
    out = np.empty(x.shape, dtype=np.float32)
    lib().ko_16_to_f32(_p(x), _p(out), C.c_size_t(x.size), dtype)
    return out


def rope_table(max_seq_len: int, rotary_dim: int, theta: float) -> np.ndarray:
    half = max(rotary_dim // 2, 1)
    t = np.empty((max_seq_len, half, 2), dtype=np.float32)
    lib().ko_rope_table(_p(t), C.c_uint32(max_seq_len), C.c_uint32(rotary_dim), C.c_float(theta))
    return t


def rope_kv_append(q_inout, k_in, v_in, cache_k, cache_v, indptr, indices, last_len, positions, params: RopeParams,
                   dtype: int, table=None, q_norm_w=None, k_norm_w=None) -> None:
    """In place on q_inout, cache_k, cache_v (uint16 arrays)."""
    for a in (q_inout, cache_k, cache_v):
        assert a.dtype == np.uint16 and a.flags.c_contiguous
    indptr = np.ascontiguousarray(indptr, np.int32)
    indices = np.ascontiguousarray(indices, np.int32)
    last_len = np.ascontiguousarray(last_len, np.int32)
    positions = np.ascontiguousarray(positions, np.uint32)
    lib().ko_rope_kv_append(_p(q_inout), _p(_u16(k_in)), _p(_u16(v_in)), _p(q_norm_w), _p(k_norm_w), _p(cache_k),
                            _p(cache_v), _p(indptr), _p(indices), _p(last_len), _p(positions),
                            C.c_uint32(positions.size), C.byref(params), _p(table), dtype)


Q4_GROUP, Q4_BLOCK_BYTES = 32, 20


def set_kv_format(q4: bool) -> None:
    """Cache format of every following append / decode / prefill call of the oracle: False = 16-bit pool, True =
    Q4KvGroup32 pool.  A Q4 pool is passed as a uint16 VIEW of its bytes (20-byte blocks in [block][token][head][d / 32]
    order), so that the wrappers' argument handling stays the same."""
    lib().ko_set_kv_format(C.c_int(1 if q4 else 0))


def q4kv_quantize(values: np.ndarray) -> np.ndarray:
    """f32 values (a multiple of 32 of them, flat order) -> Q4KvGroup32 bytes (20 per group of 32)."""
    v = np.ascontiguousarray(values, np.float32).ravel()
    assert v.size % Q4_GROUP == 0
    out = np.empty(v.size // Q4_GROUP * Q4_BLOCK_BYTES, np.uint8)
    lib().ko_q4kv_quantize(_p(v), C.c_uint32(v.size // Q4_GROUP), _p(out))
    return out


def q4kv_dequantize(blocks: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(blocks, np.uint8).ravel()
    assert b.size % Q4_BLOCK_BYTES == 0
    out = np.empty(b.size // Q4_BLOCK_BYTES * Q4_GROUP, np.float32)
    lib().ko_q4kv_dequantize(_p(b), C.c_uint32(b.size // Q4_BLOCK_BYTES), _p(out))
    return out


def set_attention_window(window_size: int) -> None:
    """Sliding-window causal mask for every following decode / prefill call of the oracle (0 = plain causal)."""
    lib().ko_set_attention_window(C.c_uint32(window_size))


def decode(q, cache_k, cache_v, indptr, indices, last_len, params: GqaParams, dtype: int):
    """Whole-row fp32 decode.  Returns (out16 uint16, out_f32)."""
    q = _u16(q)
    indptr = np.ascontiguousarray(indptr, np.int32)
    indices = np.ascontiguousarray(indices, np.int32)
    last_len = np.ascontiguousarray(last_len, np.int32)
    batch = indptr.size - 1
    out = np.empty(q.shape, np.uint16)
    outf = np.empty(q.shape, np.float32)
    lib().ko_decode(_p(q), _p(_u16(cache_k)), _p(_u16(cache_v)), _p(indptr), _p(indices), _p(last_len),
                    C.c_uint32(batch), _p(out), _p(outf), C.byref(params), dtype)
    return out, outf


def decode_stage1(q, cache_k, cache_v, indptr, indices, last_len, tiles, tile_split_idx, params: GqaParams,
                  dtype: int):
    """Per-tile stage 1 as the shader runs it.  Returns (final_out16, partial_out, partial_lse)."""
    q = _u16(q)
    indptr = np.ascontiguousarray(indptr, np.int32)
    indices = np.ascontiguousarray(indices, np.int32)
    last_len = np.ascontiguousarray(last_len, np.int32)
    tiles = np.ascontiguousarray(tiles, np.uint32).reshape(-1, 4)
    tsi = np.ascontiguousarray(tile_split_idx, np.uint32)
    batch = indptr.size - 1
    Hq, D, S = params.num_q_heads, params.head_dim, params.max_split_k_tiles
    final = np.zeros(q.shape, np.uint16)
    pout = np.zeros((batch, Hq, S, D), np.float32)
    plse = np.zeros((batch, Hq, S), np.float32)
    lib().ko_decode_stage1(_p(q), _p(_u16(cache_k)), _p(_u16(cache_v)), _p(indptr), _p(indices), _p(last_len),
                           _p(tiles), C.c_uint32(tiles.shape[0]), _p(tsi), _p(final), _p(pout), _p(plse),
                           C.byref(params), dtype)
    return final, pout, plse


def split_k_reduce(partial_out, partial_lse, num_splits_req, final_out, params: GqaParams, dtype: int) -> None:
    ns = np.ascontiguousarray(num_splits_req, np.uint32)
    lib().ko_split_k_reduce(_p(partial_out), _p(partial_lse), _p(ns), _p(final_out), C.c_uint32(ns.size),
                            C.byref(params), dtype)


def decode_partial(q, cache_k, cache_v, indptr, indices, last_len, blk_begin, blk_end, params: GqaParams, dtype: int):
    q = _u16(q)
    indptr = np.ascontiguousarray(indptr, np.int32)
    indices = np.ascontiguousarray(indices, np.int32)
    last_len = np.ascontiguousarray(last_len, np.int32)
    b = np.ascontiguousarray(blk_begin, np.uint32)
    e = np.ascontiguousarray(blk_end, np.uint32)
    batch = indptr.size - 1
    Hq, D = params.num_q_heads, params.head_dim
    m = np.empty((batch, Hq), np.float32)
    l = np.empty((batch, Hq), np.float32)
    o = np.empty((batch, Hq, D), np.float32)
    lib().ko_decode_partial(_p(q), _p(_u16(cache_k)), _p(_u16(cache_v)), _p(indptr), _p(indices), _p(last_len),
                            C.c_uint32(batch), _p(b), _p(e), _p(m), _p(l), _p(o), C.byref(params), dtype)
    return m, l, o


def merge_states(m, l, o) -> np.ndarray:
    """m, l: [parts, rows]; o: [parts, rows, D] -> normalised f32 [rows, D]."""
    m = np.ascontiguousarray(m, np.float32)
    l = np.ascontiguousarray(l, np.float32)
    o = np.ascontiguousarray(o, np.float32)
    parts, rows, D = o.shape
    out = np.empty((rows, D), np.float32)
    lib().ko_merge_states(_p(m), _p(l), _p(o), C.c_uint32(parts), C.c_uint32(rows), C.c_uint32(D), _p(out))
    return out


def prefill_causal(q, cache_k, cache_v, table, prefix_tokens: int, params: GqaParams, dtype: int):
    q = _u16(q)
    table = np.ascontiguousarray(table, np.int32)
    out = np.empty(q.shape, np.uint16)
    outf = np.empty(q.shape, np.float32)
    lib().ko_prefill_causal(_p(q), _p(_u16(cache_k)), _p(_u16(cache_v)), _p(table), C.c_uint32(prefix_tokens),
                            C.c_uint32(q.shape[0]), _p(out), _p(outf), C.byref(params), dtype)
    return out, outf


def tree_verify(tree_q, tree_k, tree_v, cache_k, cache_v, page_indices, tree_mask, params: TreeParams, dtype: int):
    """bsr_paged_gqa_tree_verify: returns (out 16-bit, out fp32), both [nodes, Hq, D]."""
    tree_q = _u16(tree_q)
    idx = np.ascontiguousarray(page_indices, np.int32)
    if idx.size == 0:
        idx = np.zeros(1, np.int32)
    mask = np.ascontiguousarray(tree_mask, np.uint8)
    out = np.empty(tree_q.shape, np.uint16)
    outf = np.empty(tree_q.shape, np.float32)
    lib().ko_tree_verify(_p(tree_q), _p(_u16(tree_k)), _p(_u16(tree_v)), _p(_u16(cache_k)), _p(_u16(cache_v)), _p(idx),
                         _p(mask), _p(out), _p(outf), C.byref(params), dtype)
    return out, outf


def block_copy(cache_k, cache_v, num_layers: int, pairs) -> None:
    """cache_k / cache_v: uint16 [layers, blocks, page, Hkv, D], copied in place."""
    assert cache_k.dtype == np.uint16 and cache_k.flags.c_contiguous and cache_v.flags.c_contiguous
    pairs = np.ascontiguousarray(pairs, np.uint32).reshape(-1, 2)
    layer_stride = int(np.prod(cache_k.shape[1:]))
    block_elems = int(np.prod(cache_k.shape[2:]))
    lib().ko_block_copy(_p(cache_k), _p(cache_v), C.c_size_t(layer_stride), C.c_uint32(num_layers),
                        C.c_size_t(block_elems), _p(pairs), C.c_uint32(pairs.shape[0]))


def slot_write(cache_k, cache_v, stage_k, stage_v, block_size: int, triples) -> None:
    triples = np.ascontiguousarray(triples, np.uint32).reshape(-1, 3)
    kv_dim = int(stage_k.shape[-1]) if stage_k.ndim == 2 else int(np.prod(stage_k.shape[1:]))
    lib().ko_slot_write(_p(cache_k), _p(cache_v), _p(_u16(stage_k)), _p(_u16(stage_v)), C.c_size_t(kv_dim),
                        C.c_uint32(block_size), _p(triples), C.c_uint32(triples.shape[0]))


# ---- the reference's own in-test CPU loops -------------------------------------------------------


def ref_test_rope_softmax_attention(q_raw, k_raw, v_raw) -> np.ndarray:
    q_raw = np.ascontiguousarray(q_raw, np.float32)
    k_raw = np.ascontiguousarray(k_raw, np.float32)
    v_raw = np.ascontiguousarray(v_raw, np.float32)
    tokens, D = q_raw.shape
    out = np.empty(D, np.float32)
    lib().ko_ref_test_rope_softmax_attention(_p(q_raw), _p(k_raw), _p(v_raw), C.c_uint32(tokens), C.c_uint32(D), _p(out))
    return out


def ref_test_causal_prefill(q, k, v, Hq: int, Hkv: int, D: int, sm_scale: float) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    T = q.size // (Hq * D)
    out = np.empty(q.size, np.float32)
    lib().ko_ref_test_causal_prefill(_p(q), _p(k), _p(v), C.c_uint32(T), C.c_uint32(Hq), C.c_uint32(Hkv),
                                     C.c_uint32(D), C.c_float(sm_scale), _p(out))
    return out


def ref_test_online_decode(q, k, v, batch, Hq, Hkv, D, num_blocks, block_sz) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    out = np.empty(batch * Hq * D, np.float32)
    lib().ko_ref_test_online_decode(_p(q), _p(k), _p(v), C.c_uint32(batch), C.c_uint32(Hq), C.c_uint32(Hkv),
                                    C.c_uint32(D), C.c_uint32(num_blocks), C.c_uint32(block_sz), _p(out))
    return out
