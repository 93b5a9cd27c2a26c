"""Build vx_b200/libvx_cuda_dispatch.so from csrc/*.cu with nvcc for sm_100a.

The library is built in-tree, so that it travels with the source directory; it
links the CUDA runtime statically and opens libcuda.so.1 and libnccl.so.2 at
run time, so it loads (and answers symbol queries) on a machine with no GPU.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libvx_cuda_dispatch.so")

SOURCES = ["dispatch.cu", "gemm_simt.cu", "gemm_umma.cu", "gemm_umma_pair.cu", "nn_kernels.cu",
           "nn_api.cu", "decoder.cu", "flash_attn.cu", "flash_attn_v2.cu", "static_scratch.cu", "rowdot_umma.cu", "prefill.cu", "quantize.cu", "step_kernel.cu", "gemm_f32_split.cu",
           "moe_group.cu", "moe_grouped.cu", "gemm_fp8_rows.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-std=c++17", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
              "-I" + os.path.join(ROOT, "include"),
              "-I" + os.path.join(HERE, "runtime"), "-I" + CSRC]


def _newer_than(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers():
    out = []
    for d in (CSRC, os.path.join(HERE, "runtime"), os.path.join(ROOT, "include")):
        out += [os.path.join(d, f) for f in os.listdir(d)
                if f.endswith((".h", ".cuh"))]
    return out


def _compile(src, verbose):
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    path = os.path.join(CSRC, src)
    if not _newer_than(obj, [path] + _headers()):
        return obj, ""
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
          ["-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on %s:\n%s" % (src, r.stderr))
    return obj, r.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    if force:
        for f in os.listdir(OBJ):
            os.remove(os.path.join(OBJ, f))
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as pool:
        results = list(pool.map(lambda s: _compile(s, verbose), SOURCES))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    if _newer_than(LIB, objs):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", LIB + ".tmp"] + objs + ["-ldl", "-lpthread"]
        subprocess.run(cmd, check=True)
        os.replace(LIB + ".tmp", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
