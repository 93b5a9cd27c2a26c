"""Build the CPU oracle (test infrastructure) into oracle/_build/libvx_oracle.so.

-ffp-contract=off keeps a multiply and the add after it as two roundings, as
the reference's CPU loops have them; -fopenmp only splits independent outputs.

The reference's own CPU provider of this path (runtime/host_dispatch_common.h)
includes <ffi.h> through runtime/vx_host_call.h; libffi's headers are not in
this image, so it cannot be compiled here and there is no oracle/_ref build.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libvx_oracle.so")
SRC = os.path.join(HERE, "vx_oracle.cpp")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if (not force and os.path.exists(LIB)
            and os.path.getmtime(LIB) >= os.path.getmtime(SRC)):
        return LIB
    cmd = ["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fopenmp",
           "-shared", "-fPIC", "-Wall", SRC, "-o", LIB + ".tmp"]
    subprocess.run(cmd, check=True)
    os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
