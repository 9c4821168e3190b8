"""Compiles the CUDA engine into pluto_b200/libpluto_b200.so (sm_100a only, in-tree).

Run as `python -m pluto_b200.build` or through `__graft_entry__.build()`.  nvcc cross-compiles
without a GPU; each translation unit is compiled to an object in `pluto_b200/build/` and skipped
when its object is newer than every source and header.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libpluto_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps.append(os.path.join(HERE, "..", "include", "pluto_b200.h"))
    return max(os.path.getmtime(p) for p in deps)


def _compile(name, header_time, verbose):
    src = os.path.join(CSRC, name)
    obj = os.path.join(OBJ, name[:-3] + ".o")
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src), header_time):
        return obj, ""
    proc = subprocess.run([NVCC, *FLAGS, "-c", src, "-o", obj], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {name}:\n{proc.stdout}\n{proc.stderr}")
    return obj, proc.stderr if verbose else ""


def build(verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    header_time = _newest_header()
    with ThreadPoolExecutor(max_workers=8) as pool:
        results = list(pool.map(lambda n: _compile(n, header_time, verbose), sources()))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if (not os.path.exists(LIB)) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        proc = subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-gencode",
                               "arch=compute_100a,code=sm_100a", "-lcudart", "-ldl"],
                              capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    build_host()
    return LIB


HOST_LIB = os.path.join(HERE, "libpluto_b200_host.so")


def build_host() -> str:
    """C++ host adapter (pluto_b200/host): the reference-shaped layer classes over the C ABI."""
    srcs = [os.path.join(HERE, "host", f) for f in ("host.cc", "qwen_layers.cc")]
    deps = srcs + [LIB] + [os.path.join(HERE, "host", f) for f in ("layers.h", "qwen_layers.h", "runtime.h",
                                                                    "status.h")]
    if os.path.exists(HOST_LIB) and os.path.getmtime(HOST_LIB) > max(os.path.getmtime(p) for p in deps):
        return HOST_LIB
    cxx = os.environ.get("CXX", "g++")
    proc = subprocess.run([cxx, "-std=c++17", "-O2", "-fPIC", "-shared", *srcs, "-I/usr/local/cuda/include",
                           "-L" + HERE, "-lpluto_b200", "-L/usr/local/cuda/lib64", "-lcudart",
                           "-Wl,-rpath,$ORIGIN", "-o", HOST_LIB], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"host adapter build failed:\n{proc.stdout}\n{proc.stderr}")
    return HOST_LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
