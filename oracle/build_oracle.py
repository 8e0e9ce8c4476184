"""Build recipe for the CPU oracle and, where the reference tree is mounted, for the
compiled reference reorder kernel.  TEST INFRASTRUCTURE ONLY (see mx_oracle.c).

  python oracle/build_oracle.py            # liboracle.so   (gcc, always)
  python oracle/build_oracle.py --ref      # + oracle/_ref/libref_reorder.so (nvcc)

The second target compiles the reference's own `src/reorder.cu` where it lies (it is
never copied) together with `oracle/ref_shim.cu`, for sm_100a.  It needs a CUTLASS header
tree, which the reference does not vendor (README.md:18 clones it); the trees that ship
inside Python packages of this image are searched.  Without the reference sources or a
CUTLASS tree the target is skipped and the tests that use it skip too.
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# where the reference project is checked out: MIXEDGEMM_REFERENCE, else a directory `reference`
# beside this repository
REF_DEFAULT = os.environ.get("MIXEDGEMM_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(verbose=False):
    src = os.path.join(HERE, "mx_oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if _newer(out, [src]):
        cmd = ["gcc", "-O2", "-fopenmp", "-fno-fast-math", "-shared", "-fPIC", "-o", out, src, "-lm"]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
    return out


def find_cutlass():
    import site
    roots = list(site.getsitepackages())
    cands = []
    for r in roots:
        cands += glob.glob(os.path.join(r, "flashinfer/data/cutlass"))
        cands += glob.glob(os.path.join(r, "tilelang/3rdparty/cutlass"))
    for c in cands:
        if os.path.exists(os.path.join(c, "include/cutlass/detail/sm100_blockscaled_layout.hpp")):
            return c
    return None


def build_ref(ref_root=REF_DEFAULT, verbose=False):
    """Compile <reference>/src/reorder.cu + ref_shim.cu -> oracle/_ref/libref_reorder.so."""
    ref_src = os.path.join(ref_root, "src", "reorder.cu")
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libref_reorder.so")
    if not os.path.exists(ref_src):
        return out if os.path.exists(out) else None
    cutlass = find_cutlass()
    if cutlass is None:
        return out if os.path.exists(out) else None
    shim = os.path.join(HERE, "ref_shim.cu")
    if not _newer(out, [ref_src, shim]):
        return out
    os.makedirs(out_dir, exist_ok=True)
    inc = ["-I" + os.path.join(ref_root, "include"), "-I" + os.path.join(HERE, "ref_stub"),
           "-I" + os.path.join(cutlass, "include"), "-I" + os.path.join(cutlass, "tools/util/include")]
    common = ["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-O2",
              "--expt-relaxed-constexpr", "-w", "-Xcompiler", "-fPIC,-fpermissive"] + inc
    objs = []
    for s, o in ((ref_src, "ref_reorder.o"), (shim, "ref_shim.o")):
        obj = os.path.join(out_dir, o)
        cmd = common + ["-c", s, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
        objs.append(obj)
    cmd = ["nvcc", "-shared", "-o", out] + objs + ["-lcudart"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", action="store_true")
    ap.add_argument("--reference-root", default=REF_DEFAULT)
    a = ap.parse_args()
    print(build_oracle(verbose=True))
    if a.ref:
        r = build_ref(a.reference_root, verbose=True)
        print(r if r else "reference reorder kernel: skipped (sources or CUTLASS headers not found)")
        sys.exit(0)
