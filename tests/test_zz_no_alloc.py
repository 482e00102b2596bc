"""The allocation-free decode entry point (kriya_cuda_paged_gqa_decode_static).

It serves callers that may not call cudaMalloc and so cannot create a context: every buffer here is the caller's
(torch tensors stand in for the host application's arena), the library's scratch is its built-in device array.
The result must equal the context-based entry point's on the same inputs, on two calls in a row (the second call
finds the array as the first one left it)."""
import ctypes as C

import numpy as np
import pytest
import torch

from kriya_rt_b200 import _native as N
from kriya_rt_b200 import workloads as W
from gpu_util import TOL, dev16, fill_cache, host16, make_executor

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
        # the existing entry point, CUDA-core kernel (the same kernel the static variant launches)
        ex = make_executor(shape, 1024)
        ex.set_decode_path(1)
        fill_cache(ex, 0, ck, cv)
        out_ctx = torch.zeros_like(q)
        torch.cuda.synchronize()
        ex.upload_schedule_plan(batch, batch.positions)
        ex.paged_gqa_decode(0, q, out_ctx, ex.gqa_params())
        ex.sync()
        ex.close()
        a = W.from_storage(host16(out_static), dtype)
        b = W.from_storage(host16(out_ctx), dtype)
        assert np.isfinite(a).all()
        assert np.abs(a - b).max() <= TOL[dtype]


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
