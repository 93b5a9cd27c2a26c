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
TWIN_LIB = os.path.join(OUT_DIR, "libvx_llama_twin.so")
TWIN_SRC = os.path.join(HERE, "llama_twin.c")


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


def build_twin(force: bool = False) -> str:
    """The second, independent restatement of the f32 Llama decode
    (llama_twin.c), a library of its own so that it shares nothing with the
    first."""
    os.makedirs(OUT_DIR, exist_ok=True)
    if (not force and os.path.exists(TWIN_LIB)
            and os.path.getmtime(TWIN_LIB) >= os.path.getmtime(TWIN_SRC)):
        return TWIN_LIB
    cmd = ["gcc", "-std=c99", "-O2", "-ffp-contract=off", "-shared", "-fPIC",
           "-Wall", TWIN_SRC, "-o", TWIN_LIB + ".tmp", "-lm"]
    subprocess.run(cmd, check=True)
    os.replace(TWIN_LIB + ".tmp", TWIN_LIB)
    return TWIN_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    print(build_twin(force="--force" in sys.argv))
