"""Builds and runs the C++ host-mirror test (tests/cpp/golden_parity.cpp over
include/paged_infer.hpp): the reference's golden-parity test restated in C++."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_exe(tmpdir) -> str:
    from paged_infer_b200 import build
    lib = build.build()
    exe = os.path.join(str(tmpdir), "golden_parity")
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([gxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", "golden_parity.cpp"), "-o", exe,
                           lib, "-Wl,-rpath," + os.path.dirname(lib)])
    return exe


def test_cpp_mirror_compiles(tmp_path):
    assert os.path.exists(build_exe(tmp_path))


@pytest.mark.gpu
def test_cpp_golden_parity(tmp_path):
    exe = build_exe(tmp_path)
    r = subprocess.run([exe, os.path.join(ROOT, "tests", "golden")], capture_output=True, text=True)
    print(r.stdout, r.stderr)
    assert r.returncode == 0 and "PASS" in r.stdout
