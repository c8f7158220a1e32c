"""Builds the CPU oracle (oracle.cpp -> liboracle.so) with g++. Test infrastructure only."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "oracle.cpp")
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    cmd = ["g++", "-std=c++17", "-O3", "-march=native", "-fopenmp", "-ffp-contract=off", "-shared", "-fPIC", src, "-o", LIB + ".tmp"]
    subprocess.run(cmd, check=True)
    os.replace(LIB + ".tmp", LIB)
    return LIB


def build_reference() -> str | None:
    """The reference's own GPU library for sm_100a (oracle/_ref/libstraydog_ref.so), when its sources are present: the checkout
    STRAYDOG_REFERENCE names, else a `reference` directory beside this repository."""
    out = os.path.join(HERE, "_ref", "libstraydog_ref.so")
    if os.path.exists(out):
        return out
    ref = os.environ.get("STRAYDOG_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    if not os.path.isdir(os.path.join(ref, "gpu")):
        return None
    subprocess.run(["make", "-f", os.path.join(HERE, "Makefile.ref"), f"REF={ref}", "-j5"], check=True, cwd=os.path.dirname(HERE))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    if "--reference" in sys.argv:
        print(build_reference())
