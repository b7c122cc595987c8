"""Build the CUDA library in-tree: origindl_b200/libodl_b200.so (sm_100a only).

Every .cu under csrc/ is compiled with nvcc for compute_100a/sm_100a and linked into one shared
library next to this file.  Objects are cached under csrc/build/ and rebuilt when a source or header
is newer.  Run as `python -m origindl_b200.build` or through `__graft_entry__.build()`.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = CSRC / "build"
LIB = HERE / "libodl_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-I", str(HERE.parent / "include"),
]


def _newest_header() -> float:
    hs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((HERE.parent / "include").glob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def build(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    hdr_t = _newest_header()
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.name + ".o")
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_t):
            cmd = [NVCC, *FLAGS, "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stdout + r.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for out in ex.map(run, jobs):
            if verbose and out.strip():
                print(out)
    if jobs or not LIB.exists():
        run([NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *map(str, objs),
             "-cudart", "static"])
    return LIB


def build_host_tests() -> Path:
    """Compile the C++ test program of the host layer (host/origin.hpp) against the library: tests/cpp/build/."""
    root = HERE.parent
    src = root / "tests" / "cpp" / "test_host_api.cpp"
    out_dir = root / "tests" / "cpp" / "build"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / "test_host_api"
    deps = [src, HERE / "host" / "origin.hpp", root / "include" / "odl_b200.h"]
    if exe.exists() and exe.stat().st_mtime >= max(d.stat().st_mtime for d in deps):
        return exe
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O1", "-Wall", "-I", str(root / "include"), "-I", str(HERE / "host"),
           "-I", str(cuda / "include"), str(src), "-o", str(exe), "-L", str(HERE), "-lodl_b200", "-L", str(cuda / "lib64"),
           "-lcudart_static", "-ldl", "-lrt", "-lpthread", f"-Wl,-rpath,{HERE}", "-Wl,-rpath,$ORIGIN/../../../origindl_b200"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the host-layer tests failed:\n" + r.stdout + r.stderr)
    return exe


def build_dp_host() -> Path:
    """Compile the plain C++ host of the data-parallel step (tests/cpp/dp_two_ranks.cpp: C ABI + CUDA runtime only)."""
    root = HERE.parent
    src = root / "tests" / "cpp" / "dp_two_ranks.cpp"
    out_dir = root / "tests" / "cpp" / "build"
    out_dir.mkdir(parents=True, exist_ok=True)
    exe = out_dir / "dp_two_ranks"
    deps = [src, root / "include" / "odl_b200.h"]
    if exe.exists() and exe.stat().st_mtime >= max(d.stat().st_mtime for d in deps):
        return exe
    cuda = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O1", "-Wall", "-I", str(root / "include"), "-I", str(cuda / "include"),
           str(src), "-o", str(exe), "-L", str(HERE), "-lodl_b200", "-L", str(cuda / "lib64"), "-lcudart_static", "-ldl", "-lrt",
           "-lpthread", f"-Wl,-rpath,{HERE}", "-Wl,-rpath,$ORIGIN/../../../origindl_b200"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the data-parallel C++ host failed:\n" + r.stdout + r.stderr)
    return exe


def build_fake_nccl() -> Path:
    """Compile the stand-in NCCL library the CPU tests of the communicator's failure handling load (tests/cpp/fake_nccl.c)."""
    root = HERE.parent
    src = root / "tests" / "cpp" / "fake_nccl.c"
    out_dir = root / "tests" / "cpp" / "build"
    out_dir.mkdir(parents=True, exist_ok=True)
    lib = out_dir / "libfake_nccl.so"
    if lib.exists() and lib.stat().st_mtime >= src.stat().st_mtime:
        return lib
    r = subprocess.run([os.environ.get("CC", "gcc"), "-O1", "-Wall", "-shared", "-fPIC", str(src), "-o", str(lib)],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the fake NCCL library failed:\n" + r.stdout + r.stderr)
    return lib


def build_test_kernels() -> Path:
    """Compile the test-only CUDA sources under tests/cuda/ into tests/cuda/build/libodl_test_kernels.so (they reuse the
    library's device headers; nothing in the product links or loads them)."""
    root = HERE.parent
    srcs = sorted((root / "tests" / "cuda").glob("*.cu"))
    out_dir = root / "tests" / "cuda" / "build"
    out_dir.mkdir(parents=True, exist_ok=True)
    lib = out_dir / "libodl_test_kernels.so"
    newest = max([s.stat().st_mtime for s in srcs] + [_newest_header()])
    if lib.exists() and lib.stat().st_mtime >= newest:
        return lib
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
           "-shared", "-cudart", "static", *map(str, srcs), "-o", str(lib)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the test kernels failed:\n" + r.stdout + r.stderr)
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
