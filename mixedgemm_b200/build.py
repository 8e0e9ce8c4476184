"""In-tree build of the native pieces (no JIT cache: the built files sit beside the sources).

  python -m mixedgemm_b200.build            # libmixedgemm_b200.so (nvcc, sm_100a)
  python -m mixedgemm_b200.build --ext      # + the pybind11/torch module `mixedgemm`

`libmixedgemm_b200.so` is the C-ABI library declared in include/mixedgemm_c.h.
`mixedgemm*.so` (under mixedgemm_b200/ext/) is the drop-in Python module with the
reference's entry points; it links against the C-ABI library.
"""
import argparse
import glob
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INC = os.path.join(ROOT, "include")
LIB = os.path.join(PKG, "libmixedgemm_b200.so")
EXT_DIR = os.path.join(PKG, "ext")

NVCC_FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-Xcompiler", "-fPIC", "-I" + INC, "-I" + CSRC]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_lib(force=False, verbose=False):
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(INC, "*.h"))
    if not force and not _stale(LIB, deps):
        return LIB
    objs = []
    procs = []
    for s in srcs:
        o = os.path.join(CSRC, os.path.basename(s)[:-3] + ".o")
        cmd = ["nvcc"] + NVCC_FLAGS + ["-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd))
        procs.append((subprocess.Popen(cmd), cmd))
        objs.append(o)
    for p, cmd in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    cmd = ["nvcc", "-shared", "-o", LIB] + objs + ["-lcudart", "-ldl"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB


def ext_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    return os.path.join(EXT_DIR, "mixedgemm" + suffix)


def build_ext(force=False, verbose=False):
    """pybind11 + libtorch module `mixedgemm` (the reference's module name)."""
    import torch
    from torch.utils import cpp_extension
    build_lib(force=False, verbose=verbose)
    src = os.path.join(CSRC, "bindings.cpp")
    out = ext_path()
    if not force and not _stale(out, [src, LIB] + glob.glob(os.path.join(INC, "*.h"))):
        return out
    os.makedirs(EXT_DIR, exist_ok=True)
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=mixedgemm",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + INC, "-I" + sysconfig.get_paths()["include"], "-I/usr/local/cuda/include"]
    cmd += ["-I" + p for p in cpp_extension.include_paths()]
    cmd += [src, "-o", out, "-L" + PKG, "-lmixedgemm_b200", "-L" + tlib, "-ltorch", "-ltorch_cpu", "-lc10",
            "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart",
            "-Wl,-rpath,$ORIGIN/..", "-Wl,-rpath," + tlib]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ext", action="store_true")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_lib(force=a.force, verbose=True))
    if a.ext:
        print(build_ext(force=a.force, verbose=True))
