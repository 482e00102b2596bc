"""In-tree build of the native libraries (no build system beyond nvcc / g++ / gcc).

    python -m kriya_rt_b200.build            # CUDA library + host bookkeeping library

Outputs (git-ignored, they travel with the tree):
    kriya_rt_b200/lib/libkriya_cuda.so   sm_100a kernels + C ABI (include/kriya_cuda.h)
    kriya_rt_b200/lib/libkriya_kv.so     host bookkeeping C ABI (include/kriya_kv.h)
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "kriya_rt_b200" / "csrc"
LIB = ROOT / "kriya_rt_b200" / "lib"
INCLUDE = ROOT / "include"
OBJ = ROOT / "build" / "obj"

CUDA_SOURCES = ["kriya_ctx.cu", "kriya_append.cu", "kriya_decode.cu", "kriya_decode_tc.cu", "kriya_decode_tc64.cu", "kriya_decode_tcp.cu", "kriya_copy.cu", "kriya_prefill.cu", "kriya_tree.cu", "kriya_static_scratch.cu", "kriya_comm.cu", "kriya_q4.cu"]
INCLUDED_SOURCES = {"kriya_decode_tc64.cu": ["kriya_decode_tc.cu"]}  # sources that #include another source
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def _run(cmd, log: Path | None = None) -> None:
    res = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(" ".join(map(str, cmd)) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("build step failed: " + " ".join(map(str, cmd)))


def build_cuda(force: bool = False) -> Path:
    LIB.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    sources = [s for s in CUDA_SOURCES if (CSRC / s).exists()]
    out = LIB / "libkriya_cuda.so"
    objs = [OBJ / (Path(s).stem + ".o") for s in sources]

    # objects built with other flags are stale even when they are newer than their sources
    extra = os.environ.get("KRIYA_NVCC_EXTRA", "").split()
    flags_file = OBJ / "nvcc_flags.txt"
    flags_now = " ".join([*NVCC_FLAGS, *extra])
    if not flags_file.exists() or flags_file.read_text() != flags_now:
        force = True

    def compile_one(pair):
        src, obj = pair
        if not force and _newer(obj, [CSRC / src] + headers + [CSRC / d for d in INCLUDED_SOURCES.get(src, [])]):
            return
        _run([_nvcc(), *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-I", str(CSRC), "-c", str(CSRC / src), "-o", str(obj)],
             log=OBJ / (Path(src).stem + ".ptxas.log"))

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        list(pool.map(compile_one, zip(sources, objs)))
    if force or not _newer(out, objs):
        _run([_nvcc(), "-shared", "-o", str(out), *map(str, objs)])  # cudart is linked statically (nvcc default)
    flags_file.write_text(flags_now)
    return out


def build_kv(force: bool = False) -> Path:
    LIB.mkdir(parents=True, exist_ok=True)
    out = LIB / "libkriya_kv.so"
    src = CSRC / "kriya_kv.cpp"
    if force or not _newer(out, [src, INCLUDE / "kriya_kv.h"]):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", str(INCLUDE), str(src), "-o", str(out)])
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    print(build_kv(args.force))
    print(build_cuda(args.force))


if __name__ == "__main__":
    main()
