"""Builds libds41_b200.so in-tree with nvcc for sm_100a (no torch dependency: the library is a plain C-ABI .so)."""
import glob
import hashlib
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libds41_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
STAMP = LIB + ".sha256"   # hash of sources, headers and flags the library was built from (travels with the .so)
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared"]


def sources():
    return sorted(glob.glob(os.path.join(HERE, "csrc", "*.cu")) + glob.glob(os.path.join(HERE, "csrc", "*.cpp")))


def inputs():
    pats = [("csrc", "*.cu"), ("csrc", "*.cpp"), ("csrc", "*.h"), ("csrc", "*.cuh"), ("csrc", "*.inc")]
    files = [p for d, pat in pats for p in glob.glob(os.path.join(HERE, d, pat))]
    return sorted(files + glob.glob(os.path.join(ROOT, "include", "*.h")))


def fingerprint():
    """Content hash (not modification times: a copy or checkout reorders those) of everything the library is built from."""
    h = hashlib.sha256(" ".join(FLAGS).encode())
    for p in inputs():
        h.update(os.path.relpath(p, ROOT).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def stale():
    if not (os.path.exists(LIB) and os.path.exists(STAMP)):
        return True
    with open(STAMP) as f:
        return f.read().strip() != fingerprint()


def build(force=False, verbose=False):
    if not force and not stale():
        return LIB
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          ["-I", os.path.join(ROOT, "include"), "-I", os.path.join(HERE, "csrc"), "-o", LIB] + sources()
    out = subprocess.run(cmd, capture_output=True, text=True)
    if out.returncode:
        raise RuntimeError("nvcc failed:\n" + out.stdout + out.stderr)
    if verbose:
        print(out.stderr)
    with open(STAMP, "w") as f:
        f.write(fingerprint() + "\n")
    return LIB


if __name__ == "__main__":
    build(force=True, verbose=True)
