"""Compiles the reference project's own CUDA kernels, from where they lie, into oracle/_ref/.

TEST / BASELINE INFRASTRUCTURE ONLY.  The reference's host side is Rust and cannot be built in
this image (no cargo/rustc), but its device code is plain CUDA C that its Rust wrapper hands to
NVRTC at run time (crates/nvidia/src/quantized.rs:76-88, :169-182 of the reference project).
This script compiles those same sources ahead of time with nvcc for sm_100a:

    oracle/_ref/ref_quantized.cubin   common.cu + q4_k.cu + q8_0.cu + q6_k.cu + q5_k.cu, prefixed with
                                      MAX_BATCH_MEMBERS=8 / MAX_BATCH_ROWS=2 exactly as quantized.rs:171-174 does
    oracle/_ref/ref_model_ops.cubin   the CUDA source string embedded in model_ops.rs (rms_norm, ...)

No reference source is copied into this repository: the translation units are `#include`s of the
files under the mounted reference tree (the model_ops string is extracted into a temporary file
outside the repository), and only the compiled cubins, which are git-ignored, are kept.  The
cubins travel to the GPU box with the snapshot; nothing on the box reads the reference tree.

Used by: tests (our kernels against the reference's kernels on the same inputs) and the benchmark's
"reference CUDA on the same GPU" comparison.  The shipped library never loads them.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
REFERENCE = os.environ.get("RIBN_REFERENCE_ROOT", "")   # root of a checkout of the reference project; unset = build nothing
KERNELS = os.path.join(REFERENCE, "crates", "nvidia", "src", "kernels", "quantized")
QUANTIZED_UNITS = ["common.cu", "q4_k.cu", "q8_0.cu", "q6_k.cu", "q5_k.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-cubin"]


def nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    return "nvcc"


def build() -> list[str]:
    if not REFERENCE or not os.path.isdir(KERNELS):
        print(f"RIBN_REFERENCE_ROOT does not name a checkout of the reference project; keeping whatever is in {OUT}")
        return []
    os.makedirs(OUT, exist_ok=True)
    built = []
    with tempfile.TemporaryDirectory() as tmp:
        # 1. the float GEMV families
        unit = os.path.join(tmp, "ref_quantized.cu")
        with open(unit, "w") as f:
            f.write("#define MAX_BATCH_MEMBERS 8\n#define MAX_BATCH_ROWS 2\n")
            for name in QUANTIZED_UNITS:
                f.write(f'#include "{os.path.join(KERNELS, name)}"\n')
        target = os.path.join(OUT, "ref_quantized.cubin")
        subprocess.run([nvcc(), *NVCC_FLAGS, unit, "-o", target], check=True)
        built.append(target)
        # 2. the CUDA source embedded as a Rust raw string in model_ops.rs
        text = open(os.path.join(REFERENCE, "crates", "nvidia", "src", "model_ops.rs")).read()
        match = re.search(r'r#"(.*?)"#', text, flags=re.S)
        if match and "__global__" in match.group(1):
            unit = os.path.join(tmp, "ref_model_ops.cu")
            with open(unit, "w") as f:
                f.write(match.group(1))
            target = os.path.join(OUT, "ref_model_ops.cubin")
            subprocess.run([nvcc(), *NVCC_FLAGS, unit, "-o", target], check=True)
            built.append(target)
    return built


if __name__ == "__main__":
    for path in build():
        print("built", path)
    sys.exit(0)
