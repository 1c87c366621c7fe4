"""Builds the REFERENCE's CUDA library for B200 into oracle/_ref/ (test infrastructure).

    python oracle/build_ref.py /path/to/haste      (or HASTE_REFERENCE_ROOT=/path/to/haste)

Compiles the reference's own `lib/*.cu.cc`, untouched and where they lie, with nvcc
for sm_100 (its Makefile targets compute_37/60/70, which CUDA 12.9 no longer
accepts), together with `oracle/ref_shim.cu`, and links cuBLAS.  Nothing from the
reference is copied into this repository; the output directory is git-ignored.
Needs the reference checkout, so it only runs where that exists.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "libhaste_ref.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


def reference_root():
    """The reference checkout: $HASTE_REFERENCE_ROOT, else a `reference` directory beside
    this repository (where the build driver mounts it), else None."""
    env = os.environ.get("HASTE_REFERENCE_ROOT")
    if env:
        return env
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return sibling if os.path.isdir(os.path.join(sibling, "lib")) else None


def build(root=None, force=False):
    root = root or reference_root()
    if not root:
        return LIB if os.path.exists(LIB) else None
    lib_dir = os.path.join(root, "lib")
    if not os.path.isdir(lib_dir):
        return None
    if os.path.exists(LIB) and not force:
        return LIB
    os.makedirs(OUT, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(lib_dir, "*.cu.cc"))) + [os.path.join(HERE, "ref_shim.cu")]
    flags = ["-gencode", "arch=compute_100,code=sm_100", "-O3", "-std=c++17", "-x", "cu",
             "-Xcompiler", "-fPIC", "-I", lib_dir, "-w"]

    def one(src):
        obj = os.path.join(OUT, os.path.basename(src).replace(".cu.cc", "").replace(".cu", "") + ".o")
        r = subprocess.run([NVCC, *flags, "-c", src, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(one, srcs))
    r = subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-lcublas"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr}")
    for o in objs:
        os.remove(o)
    return LIB


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), force=True))
