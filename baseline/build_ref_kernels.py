#!/usr/bin/env python
"""Compile the reference's CUDA kernels, unmodified, for sm_100a into
``baseline/_ref/libnangila_ref_kernels.so``.

    python baseline/build_ref_kernels.py [/path/to/nangila_v0.1.0]

The four sources (nangila-cuda/src/kernels/{predict,reconstruct,gamma,crc32}.cu) are plain
``extern "C"`` launchers with no Rust dependency. They are copied to a scratch directory and passed to
nvcc as they are; nothing of them is stored in this repository (``baseline/_ref`` is git-ignored).
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> int:
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NANGILA_REFERENCE_DIR", "")
    src_dir = os.path.join(ref, "nangila-cuda", "src", "kernels")
    if not os.path.isdir(src_dir):
        print(f"reference kernel sources not found under {src_dir!r}", file=sys.stderr)
        return 1
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "libnangila_ref_kernels.so")
    with tempfile.TemporaryDirectory() as tmp:
        srcs = []
        for name in ("predict.cu", "reconstruct.cu", "gamma.cu", "crc32.cu"):
            shutil.copy(os.path.join(src_dir, name), tmp)
            srcs.append(os.path.join(tmp, name))
        nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-shared", "-Xcompiler", "-fPIC", *srcs, "-o", out]
        print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    print("built", out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
