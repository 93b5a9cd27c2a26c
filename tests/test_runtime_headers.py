"""The reference's own vendor-free runtime tests, compiled against THIS
repository's headers (vx_b200/runtime/*.h, include/vx_hardware_runtime.h).

The test sources stay where they are under the reference tree; a scratch
directory mirrors the reference's layout with links, so their relative includes
(`../../runtime/x.h`) land on our headers. Needs the reference tree (its path
comes from VX_REFERENCE_ROOT), so this runs where that is mounted and skips
elsewhere.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_TESTS = os.path.join(os.environ.get("VX_REFERENCE_ROOT", "/root/reference"),
                         "tests", "runtime")
CASES = ["gemm_plan", "kernel_launch", "payload", "device_pool",
         "arrival_counts", "collective"]

pytestmark = pytest.mark.skipif(not os.path.isdir(REF_TESTS),
                                reason="the reference tree is not mounted")


@pytest.fixture(scope="module")
def shadow(tmp_path_factory):
    top = tmp_path_factory.mktemp("shadow")
    for sub in ("tests/runtime", "runtime", "include"):
        os.makedirs(top / sub)
    ours = os.path.join(ROOT, "vx_b200", "runtime")
    for name in os.listdir(ours):
        os.symlink(os.path.join(ours, name), top / "runtime" / name)
    os.symlink(os.path.join(ROOT, "include", "vx_hardware_runtime.h"),
               top / "include" / "vx_hardware_runtime.h")
    for name in CASES:
        os.symlink(os.path.join(REF_TESTS, name + "_test.cpp"),
                   top / "tests" / "runtime" / (name + "_test.cpp"))
    os.symlink(os.path.join(REF_TESTS, "fake_nccl.cpp"),
               top / "tests" / "runtime" / "fake_nccl.cpp")
    return top


def build(shadow, name):
    exe = shadow / (name + "_test")
    # the flags of tests/integration_test/runtime_test_build.rs:19-49
    subprocess.run(["g++", "-std=c++17", "-O1", "-Wall", "-Werror",
                    "-I" + os.path.join(ROOT, "include"),
                    name + "_test.cpp", "-o", str(exe), "-ldl", "-lpthread"],
                   cwd=shadow / "tests" / "runtime", check=True)
    return exe


@pytest.mark.parametrize("name", CASES[:-1])
def test_reference_runtime_test_passes_on_our_headers(shadow, name):
    exe = build(shadow, name)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]


def test_reference_collective_test_with_its_fake_nccl(shadow, tmp_path):
    exe = build(shadow, "collective")
    fake = shadow / "libfake_nccl.so"
    subprocess.run(["g++", "-std=c++17", "-shared", "-fPIC", "fake_nccl.cpp",
                    "-o", str(fake)], cwd=shadow / "tests" / "runtime",
                   check=True)
    r = subprocess.run([str(exe), str(fake), str(tmp_path)],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
