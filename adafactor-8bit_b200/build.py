"""Build libaf8.so (the CUDA kernels and their C ABI) for sm_100a with nvcc.

    python adafactor-8bit_b200/build.py [--force] [--verbose]

The library lands in adafactor-8bit_b200/lib/libaf8.so, next to the Python
package that loads it with ctypes.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libaf8.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    # exact IEEE arithmetic: no contraction, no approximate division / sqrt, no flush to zero
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared", "-cudart", "static",
]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
    out.append(os.path.join(INCLUDE, "af8.h"))
    return out


def build(force=False, verbose=False, extra=(), out=None):
    """extra: additional nvcc arguments (e.g. -D macros for tuning builds);
    out: alternative output path (the default library is left untouched)."""
    os.makedirs(LIB_DIR, exist_ok=True)
    if out is not None:
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        cmd = [nvcc] + NVCC_FLAGS + list(extra) + (["-Xptxas", "-v"] if verbose else []) + [
            "-I", INCLUDE, "-o", out, os.path.join(CSRC, "af8_lib.cu")]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed building " + out)
        return out
    if not force and os.path.exists(LIB):
        newest = max(os.path.getmtime(s) for s in sources())
        if os.path.getmtime(LIB) >= newest:
            return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
        "-I", INCLUDE, "-o", LIB, os.path.join(CSRC, "af8_lib.cu")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libaf8.so")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
