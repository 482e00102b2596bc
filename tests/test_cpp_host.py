"""The C++ host side (include/kriya_executor.hpp over the C ABI): a small host program is compiled with g++, linked against
the two libraries and run.  Without a GPU its executor constructor must fail with DeviceInitFailed (no CPU fallback)."""
import shutil
import subprocess
from pathlib import Path

import pytest

from kriya_rt_b200 import build as B

ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.skipif(shutil.which("g++") is None, reason="g++ not available")
def test_cpp_host_program_builds_links_and_reports_errors(tmp_path):
    B.build_kv()
    B.build_cuda()
    lib = ROOT / "kriya_rt_b200" / "lib"
    exe = tmp_path / "executor_host"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", str(ROOT / "include"),
           str(ROOT / "tests" / "cpp" / "executor_host.cpp"), "-L", str(lib), "-lkriya_cuda", "-lkriya_kv",
           f"-Wl,-rpath,{lib}", "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "DeviceInitFailed" in run.stdout or "executor created" in run.stdout
