"""Builds the CUDA library in-tree with nvcc for sm_100a (no GPU needed to compile).

`python -m heirloom_b200.build` compiles every `csrc/*.cu` to an object file in parallel and
links `heirloom_b200/lib/libheirloom_b200.so`.  Objects are rebuilt only when their source or a
header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "lib"
LIB = OUT / "libheirloom_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--extended-lambda", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(src: Path, verbose: bool) -> Path:
    obj = OUT / (src.stem + ".o")
    stamp = max(src.stat().st_mtime, _newest_header())
    if obj.exists() and obj.stat().st_mtime >= stamp:
        return obj
    cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(verbose: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources))
    if LIB.exists() and all(LIB.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return LIB
    # linked under another name and renamed, so that a process that opens the library never sees half a file
    tmp = LIB.with_suffix(".so.linking")
    cmd = [NVCC, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart", "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB)
    return LIB


HOST = PKG / "host"
HOST_LIB = OUT / "libheirloom_host.so"
HOST_TESTS = OUT / "host_tests"
CXX = os.environ.get("CXX", "g++")


def build_host() -> Path:
    """The C++ tensor interface above the C ABI (`host/heirloom_host.cpp`) as a shared library, and its
    test driver, both linked against the CUDA library next to them."""
    build()
    newest = max(p.stat().st_mtime for p in list(HOST.glob("*.cpp")) + list(HOST.glob("*.hpp")) +
                 list((PKG.parent / "include").glob("*.h")))
    common = ["-O2", "-std=c++17", "-Wall", "-Wextra", "-fPIC", f"-L{OUT}", "-Wl,-rpath,$ORIGIN"]
    if not HOST_LIB.exists() or HOST_LIB.stat().st_mtime < newest:
        cmd = [CXX, *common, "-shared", "-o", str(HOST_LIB), str(HOST / "heirloom_host.cpp"), "-lheirloom_b200"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"host library failed to build:\n{res.stdout}\n{res.stderr}")
    if not HOST_TESTS.exists() or HOST_TESTS.stat().st_mtime < newest:
        cmd = [CXX, *common, "-o", str(HOST_TESTS), str(HOST / "host_tests.cpp"), "-lheirloom_host", "-lheirloom_b200"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"host test driver failed to build:\n{res.stdout}\n{res.stderr}")
    return HOST_LIB


if __name__ == "__main__" and "--host" in sys.argv:
    print(build_host())
    sys.exit(0)

if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
