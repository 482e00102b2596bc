"""The native libraries load and export every symbol the public headers declare (no GPU needed), and the
POD structs have the reference's sizes."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions(header: Path):
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(kriya_(?:kv|cuda)_[a-z0-9_]+)\s*\(", text)))


def test_kv_library_exports_every_declared_symbol():
    from kriya_rt_b200 import _native as N

    lib = N.kv_lib()
    names = declared_functions(ROOT / "include" / "kriya_kv.h")
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), n
    assert set(N.KV_SYMBOLS) == set(names)


def test_cuda_library_exports_every_declared_symbol():
    from kriya_rt_b200 import _native as N

    so = ROOT / "kriya_rt_b200" / "lib" / "libkriya_cuda.so"
    if not so.exists():
        from kriya_rt_b200 import build as B

        B.build_cuda()
    lib = N.cuda_lib()
    names = declared_functions(ROOT / "include" / "kriya_cuda.h")
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert set(N.CUDA_SYMBOLS) == set(names)


def test_pod_struct_sizes_match_reference():
    from kriya_rt_b200 import _native as N

    assert C.sizeof(N.RopeKvWriteParams) == 48  # encoder.rs:159-174, 12 x 4 bytes
    assert C.sizeof(N.BsrGqaParams) == 32  # encoder.rs:176-187
    assert C.sizeof(N.CtaWorkTile) == 16  # bsr_paged.rs:285-297
    assert N.RopeKvWriteParams.rms_eps.offset == 24 and N.RopeKvWriteParams.has_table.offset == 36
    assert N.BsrGqaParams.sm_scale.offset == 24


def test_create_without_gpu_fails_with_device_error_not_a_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from kriya_rt_b200.executor import CudaBackendError, CudaExecutor

    with pytest.raises(CudaBackendError) as e:
        CudaExecutor(num_layers=1, num_kv_blocks=4, block_size_tokens=16, num_q_heads=2, num_kv_heads=1, head_dim=64)
    assert e.value.code == -1  # DeviceInitFailed


def test_product_package_never_imports_the_oracle():
    for py in (ROOT / "kriya_rt_b200").rglob("*.py"):
        src = py.read_text()
        assert "import oracle" not in src and "from oracle" not in src, py
    for cu in (ROOT / "kriya_rt_b200" / "csrc").iterdir():
        assert "oracle" not in cu.read_text().lower() or cu.suffix not in (".cu", ".cpp", ".h", ".cuh"), cu


def test_tree_verify_params_are_32_bytes():
    """TreeVerifyGqaParams, crates/kriya-backend-metal/src/encoder.rs:189-200: 7 x u32 + f32."""
    import ctypes as C
    from kriya_rt_b200._native import TreeVerifyParams
    from oracle.c_oracle import TreeParams
    assert C.sizeof(TreeVerifyParams) == 32 and C.sizeof(TreeParams) == 32
    assert TreeVerifyParams.sm_scale.offset == 28 and TreeVerifyParams.prefix_kv_blocks.offset == 20
