"""Build libsgl_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python starrygl-framework_b200/build.py [--force] [--verbose]

The shared object lands in starrygl-framework_b200/lib/.  nvcc cross-compiles, so no GPU is needed.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
OUT = os.path.join(OUT_DIR, "libsgl_b200.so")
SOURCES = ["api.cu", "sort.cu", "tcsr.cu", "sampler.cu", "relabel.cu", "gather.cu", "comm.cu", "p2p_route.cu", "plan.cu", "mail.cu", "slice.cu"]
FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--expt-relaxed-constexpr",
         "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared"]


def _stale():
    if not os.path.exists(OUT):
        return True
    t = os.path.getmtime(OUT)
    deps = [os.path.join(SRC, f) for f in os.listdir(SRC)] + [os.path.join(HERE, "..", "include", "sgl_b200.h"), __file__]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    if not force and not _stale():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + [os.path.join(SRC, s) for s in SOURCES] + ["-ldl", "-o", OUT]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed building libsgl_b200.so")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
