"""Builds libaether_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m aether_ml_b200.build            # or: from aether_ml_b200.build import build_library
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libaether_b200.so")
DIGEST_PATH = LIB_PATH + ".digest"
SOURCES = ["api.cu", "conv_tc.cu", "conv_halo.cu", "conv_halo_dw.cu", "conv_dw_rows.cu", "conv_generic.cu", "conv_smallc.cu", "conv_first_tc.cu", "layers.cu",
           "block_fused.cu"]
# tcgen05 / TMA PTX only assembles for the arch-specific target, hence compute_100a + sm_100a.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; cannot build libaether_b200.so")
    return nvcc


def _source_digest():
    """sha256 over the CUDA sources, the public header and the compiler flags (what the .so is a function of)."""
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    deps = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)) + [os.path.join(HERE, "..", "include", "aether_b200.h")]
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _stale():
    """True when the library is missing or was built from other sources.  The check compares a digest of the
    sources with the one recorded beside the .so at build time, so it does not depend on file times (a copied
    tree keeps its built library)."""
    if not os.path.exists(LIB_PATH) or not os.path.exists(DIGEST_PATH):
        return True
    with open(DIGEST_PATH) as fh:
        return fh.read().strip() != _source_digest()


def build_library(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources.  Returns the .so path."""
    if not force and not _stale():
        return LIB_PATH
    objs = []
    nvcc = _nvcc()
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, "-c", os.path.join(CSRC, src), "-o", obj] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        if verbose:
            print(r.stderr)
        objs.append(obj)
    cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    with open(DIGEST_PATH, "w") as fh:
        fh.write(_source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
