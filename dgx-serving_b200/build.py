"""Builds libw4a8_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python dgx-serving_b200/build.py [--force]
nvcc cross-compiles without a GPU; the explicit -gencode form is required because the tcgen05 / TMA
instructions exist only for the arch-specific target sm_100a.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "w4a8_b200.cu")
OUT = os.path.join(HERE, "libw4a8_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
]


def sources():
    d = os.path.join(HERE, "csrc")
    files = [os.path.join(d, f) for f in sorted(os.listdir(d))]
    files.append(os.path.join(HERE, "..", "include", "w4a8_b200.h"))
    return files


def up_to_date():
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    return all(os.path.getmtime(f) <= t for f in sources())


def build(force=False, verbose=False):
    """Compile the library unless it is newer than every source.  Returns the path of the .so."""
    if not force and up_to_date():
        return OUT
    if not os.path.exists(NVCC):
        if os.path.exists(OUT):
            return OUT  # no compiler here (a GPU box): use the prebuilt library that travelled with the tree
        raise RuntimeError("nvcc not found at %s and no prebuilt %s" % (NVCC, OUT))
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", OUT, SRC]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
