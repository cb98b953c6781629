"""Ahead-of-time build of libribn_b200.so for sm_100a with nvcc (no JIT, no run-time compile).

`python -m engine_b200.build` compiles every .cu under csrc/ and links the shared library
in-tree, next to this file, where the ctypes loader looks for it.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libribn_b200.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# No --use_fast_math: flush-to-zero or approximate division would break bit-exact dequantisation.
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
              "--expt-relaxed-constexpr"]


def nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc not found; this library has no prebuilt or fallback path")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_input() -> float:
    inputs = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inputs.append(os.path.join(HERE, "..", "include", "ribn_b200.h"))
    inputs.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in inputs)


def build(force: bool = False, verbose: bool = False, extra: list[str] | None = None) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest_input():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    compiler = nvcc()
    flags = ARCH + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + (extra or [])

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        cmd = [compiler, *flags, "-c", src, "-o", obj]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or result.returncode:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objects = list(pool.map(compile_one, sources()))
    link = [compiler, *ARCH, "-shared", "-cudart", "shared", "-o", LIB, *objects,
            "-Xlinker", "-rpath,/usr/local/cuda/lib64"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
