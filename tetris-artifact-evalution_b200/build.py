"""Build recipe of the native library: `nvcc` straight to an in-tree shared object.

    python tetris-artifact-evalution_b200/build.py

compiles csrc/*.cu for sm_100a into libtetris_b200.so beside this file.  The
object is built in-tree (not installed anywhere) so that it travels with the
source tree to the machine that has the GPU.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libtetris_b200.so")
SOURCES = ["api.cu", "compress.cu", "conv_generic.cu", "conv_tiled.cu", "conv_tc.cu", "conv_tc16.cu", "depthwise.cu", "layout.cu",
           "noalloc.cu", "serialize.cu", "chain.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libtetris_b200.so")
    return exe


def needs_build():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "tetris_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not needs_build():
        return LIB
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    cmd += os.environ.get("TETRIS_NVCC_FLAGS", "").split()  # e.g. -DTETRIS_TC16_PROF: the kernel timeline aid
    cmd += ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
