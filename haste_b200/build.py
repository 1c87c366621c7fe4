"""Builds libhaste_b200.so in-tree with nvcc for sm_100a.

    python -m haste_b200.build            # incremental
    python -m haste_b200.build --force

Only the CUDA toolkit is needed (no torch headers): the library is a plain
C-ABI shared object that the Python layer loads with ctypes.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libhaste_b200.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _newest_header():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    hs.append(os.path.join(HERE, "..", "include", "haste_b200.h"))
    return max(os.path.getmtime(h) for h in hs)


def _compile(src, force):
    obj = os.path.join(OBJ, src[:-3] + ".o")
    spath = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) > max(os.path.getmtime(spath), _newest_header())):
        return obj, ""
    r = subprocess.run([NVCC, *FLAGS, "-c", spath, "-o", obj], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force=False, verbose=False):
    # an existing library that is newer than every source and header needs nothing (the object
    # files may be absent, e.g. on a machine that received only the built library)
    if not force and os.path.exists(LIB):
        newest = max([os.path.getmtime(os.path.join(CSRC, f)) for f in sources()] + [_newest_header()])
        if os.path.getmtime(LIB) > newest:
            return LIB
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=8) as ex:
        results = list(ex.map(lambda s: _compile(s, force), sources()))
    objs = [o for o, _ in results]
    log = "".join(l for _, l in results)
    if log:
        with open(os.path.join(OBJ, "ptxas.log"), "a") as f:
            f.write(log)
        if verbose:
            print(log)
    if (force or not os.path.exists(LIB)
            or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs)):
        r = subprocess.run([NVCC, "-shared", "-o", LIB, *objs],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


TORCH_EXT_SRC = os.path.join(HERE, "torch_ext", "haste_pytorch_lib.cc")
TORCH_EXT = os.path.join(HERE, "torch_ext", "haste_pytorch_lib.so")


def build_torch_ext(force=False):
    """Compiles the pybind11 module `haste_pytorch_lib` (the reference's extension name) against
    the installed torch and links it to libhaste_b200.so, in-tree."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    header = os.path.join(HERE, "..", "include", "haste_b200.h")
    if (not force and os.path.exists(TORCH_EXT) and os.path.exists(LIB)
            and os.path.getmtime(TORCH_EXT) > max(os.path.getmtime(TORCH_EXT_SRC),
                                                  os.path.getmtime(header))):
        return TORCH_EXT
    lib = build()
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incs = ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(HERE, "..", "include"),
                                 os.path.join(cuda_home, "include")]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared",
           "-DTORCH_EXTENSION_NAME=haste_pytorch_lib", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{i}" for i in incs], TORCH_EXT_SRC, "-o", TORCH_EXT,
           f"-L{tlib}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-ltorch_python",
           f"-L{os.path.dirname(lib)}", "-lhaste_b200",
           f"-Wl,-rpath,{tlib}", "-Wl,-rpath,$ORIGIN/.."]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"torch extension build failed:\n{r.stdout}\n{r.stderr}")
    return TORCH_EXT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch-ext" in sys.argv:
        print(build_torch_ext(force="--force" in sys.argv))
