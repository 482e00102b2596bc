"""The allocation-free decode entry point (kriya_cuda_paged_gqa_decode_static).

It serves callers that may not call cudaMalloc and so cannot create a context: every buffer here is the caller's
(torch tensors stand in for the host application's arena), the library's scratch is its built-in device array.
The result must equal the context-based entry point's bit for bit on the same inputs (both run the same kernel over
the same work split) and agree with the CPU oracle, on two calls in a row (the second call finds the array as the
first one left it)."""
import ctypes as C

import numpy as np
import pytest
import torch

from kriya_rt_b200 import _native as N
from kriya_rt_b200 import workloads as W
from gpu_util import TOL, dev16, fill_cache, host16, make_executor
from oracle import c_oracle as O

pytestmark = pytest.mark.gpu


def _call_static(lib, shape, batch, q, ck_dev, cv_dev, out, stream=0):
    indptr_h = np.ascontiguousarray(batch.page_indptr, np.int32)
    indptr_d = torch.from_numpy(indptr_h).cuda()
    indices_d = torch.from_numpy(np.ascontiguousarray(batch.page_indices, np.int32)).cuda()
    last_d = torch.from_numpy(np.ascontiguousarray(batch.last_page_len, np.int32)).cuda()
    torch.cuda.synchronize()
    scale = float(np.float32(1.0) / np.sqrt(np.float32(shape.head_dim)))
    p = N.BsrGqaParams(shape.num_q_heads, shape.num_kv_heads, shape.head_dim, 16, 16, 1, scale, 0.0)
    err = C.create_string_buffer(256)
    rc = lib.kriya_cuda_paged_gqa_decode_static(0, stream, shape.dtype, q.data_ptr(), ck_dev.data_ptr(), cv_dev.data_ptr(),
                                                batch.num_blocks, indptr_h.ctypes.data, indptr_d.data_ptr(),
                                                indices_d.data_ptr(), last_d.data_ptr(), batch.batch, out.data_ptr(),
                                                C.byref(p), err, 256)
    torch.cuda.synchronize()
    return rc, err.value.decode()


def _oracle_decode(shape, batch, q16, ck, cv):
    scale = float(np.float32(1.0) / np.sqrt(np.float32(shape.head_dim)))
    p = O.GqaParams(shape.num_q_heads, shape.num_kv_heads, shape.head_dim, 16, 16, 1, scale, 0.0)
    return O.decode(q16, ck, cv, batch.page_indptr, batch.page_indices, batch.last_page_len, p, shape.dtype)[1]


def _context_decode(shape, batch, q, ck, cv, num_blocks):
    """The existing entry point on the CUDA-core kernel (the kernel the static variant launches)."""
    ex = make_executor(shape, num_blocks, max_batch_rows=max(64, batch.batch), max_page_indices=max(16384, num_blocks))
    ex.set_decode_path(1)
    fill_cache(ex, 0, ck, cv)
    out = torch.zeros_like(q)
    torch.cuda.synchronize()
    ex.upload_schedule_plan(batch, batch.positions)
    ex.paged_gqa_decode(0, q, out, ex.gqa_params())
    ex.sync()
    ex.close()
    return out


@pytest.mark.parametrize("Hq,Hkv,D,dtype", [(16, 2, 128, W.BF16), (9, 3, 64, W.FP16)])
def test_static_scratch_decode_matches_context_decode_twice(Hq, Hkv, D, dtype):
    lib = N.cuda_lib()
    shape = W.AttnShape("static", Hq, Hkv, D, dtype)
    rng = np.random.default_rng(71)
    ck = W.normal16(rng, (1024, 16, Hkv, D), dtype)
    cv = W.normal16(rng, (1024, 16, Hkv, D), dtype)
    ck_dev, cv_dev = dev16(ck), dev16(cv)  # the caller's own pool memory
    for call, ctx in enumerate((np.array([5000, 17, 900, 255, 3000]), np.array([64, 4095, 1, 2222]))):
        batch = W.make_decode_batch(shape, ctx, 1024, seed=72 + call)
        q16 = W.normal16(rng, (ctx.size, Hq, D), dtype)
        q = dev16(q16)
        out_static = torch.zeros_like(q)
        rc, msg = _call_static(lib, shape, batch, q, ck_dev, cv_dev, out_static)
        assert rc == 0, msg
        out_ctx = _context_decode(shape, batch, q, ck, cv, 1024)
        assert np.array_equal(host16(out_static), host16(out_ctx))  # same kernel, same split: the same bits
        got = W.from_storage(host16(out_static), dtype)
        assert np.isfinite(got).all()
        assert np.abs(got - _oracle_decode(shape, batch, q16, ck, cv)).max() <= TOL[dtype]


def test_static_scratch_on_a_side_stream_with_the_coarser_split():
    """A batch whose first split would need more than 512 work items takes the coarser second cut; the call is queued
    on a stream of the caller's own and leaves the caller's current device alone."""
    lib = N.cuda_lib()
    shape = W.AttnShape("static", 16, 2, 128, W.BF16)
    ctx = np.concatenate([np.full(200, 10), 3000 + 37 * np.arange(56)])  # 200 one-block rows + 56 long rows
    nb = 14336
    rng = np.random.default_rng(73)
    batch = W.make_decode_batch(shape, ctx, nb, seed=74)
    ck = W.normal16(rng, (nb, 16, 2, 128), W.BF16)
    cv = W.normal16(rng, (nb, 16, 2, 128), W.BF16)
    ck_dev, cv_dev = dev16(ck), dev16(cv)
    q16 = W.normal16(rng, (ctx.size, 16, 128), W.BF16)
    q = dev16(q16)
    ref = _oracle_decode(shape, batch, q16, ck, cv)
    side = torch.cuda.Stream()
    dev_before = torch.cuda.current_device()
    for _ in range(2):
        out = torch.zeros_like(q)
        torch.cuda.synchronize()
        rc, msg = _call_static(lib, shape, batch, q, ck_dev, cv_dev, out, stream=side.cuda_stream)
        assert rc == 0, msg
        assert torch.cuda.current_device() == dev_before
        got = W.from_storage(host16(out), W.BF16)
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= TOL[W.BF16]


def test_static_scratch_limits_are_rejected_with_a_message():
    lib = N.cuda_lib()
    shape = W.AttnShape("static", 16, 2, 128, W.BF16)
    ctx = np.full(300, 20)  # 300 rows > 256
    batch = W.make_decode_batch(shape, ctx, 1024, seed=5)
    q = torch.zeros(300, 16, 128, dtype=torch.int16, device="cuda")
    pool = torch.zeros(1024, 16, 2, 128, dtype=torch.int16, device="cuda")
    rc, msg = _call_static(lib, shape, batch, q, pool, pool, torch.zeros_like(q))
    assert rc == -2 and "256" in msg
    wide = W.AttnShape("wide", 32, 4, 128, W.BF16)  # 32 * 128 = 4096 > 2048
    b2 = W.make_decode_batch(wide, np.array([100]), 1024, seed=6)
    q2 = torch.zeros(1, 32, 128, dtype=torch.int16, device="cuda")
    pool2 = torch.zeros(1024, 16, 4, 128, dtype=torch.int16, device="cuda")
    rc, msg = _call_static(lib, wide, b2, q2, pool2, pool2, torch.zeros_like(q2))
    assert rc == -2 and "2048" in msg
