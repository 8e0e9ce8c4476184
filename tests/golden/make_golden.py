"""Regenerate tests/golden/cutlass_tables.json from CUTLASS's host converters.

  python tests/golden/make_golden.py

Compiles gen_cutlass_tables.cpp with g++ against a CUTLASS header tree found inside the
installed Python packages and writes the JSON beside this script.  Only the
JSON is needed at test time.
"""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle.build_oracle import find_cutlass  # noqa: E402


def main():
    cutlass = find_cutlass()
    if cutlass is None:
        sys.exit("no CUTLASS header tree found")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "gen")
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-w", "-fpermissive", "-I" + os.path.join(cutlass, "include"), "-I/usr/local/cuda/include",
                               os.path.join(HERE, "gen_cutlass_tables.cpp"), "-o", exe])
        out = subprocess.check_output([exe])
    with open(os.path.join(HERE, "cutlass_tables.json"), "wb") as f:
        f.write(out)
    print("wrote cutlass_tables.json (%d bytes) from %s" % (len(out), cutlass))


if __name__ == "__main__":
    main()
