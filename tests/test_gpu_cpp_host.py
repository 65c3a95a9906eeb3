"""Builds and runs the C++ host-side tests: tests/cpp/golden_parity.cpp over include/paged_infer.hpp (the
reference's golden-parity test restated in C++) and tests/cpp/engine_tests.cpp over include/paged_infer_engine.hpp
(the engine step loop: admission, prefix reuse, fork + copy-on-write, batched decode)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_exe(tmpdir, name="golden_parity") -> str:
    from paged_infer_b200 import build
    lib = build.build()
    exe = os.path.join(str(tmpdir), name)
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    subprocess.check_call([gxx, "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "cpp", name + ".cpp"), "-o", exe,
                           lib, "-Wl,-rpath," + os.path.dirname(lib)])
    return exe


def test_cpp_mirror_compiles(tmp_path):
    assert os.path.exists(build_exe(tmp_path))
    assert os.path.exists(build_exe(tmp_path, "engine_tests"))


@pytest.mark.gpu
def test_cpp_golden_parity(tmp_path):
    exe = build_exe(tmp_path)
    r = subprocess.run([exe, os.path.join(ROOT, "tests", "golden")], capture_output=True, text=True)
    print(r.stdout, r.stderr)
    assert r.returncode == 0 and "PASS" in r.stdout


@pytest.mark.gpu
def test_cpp_engine_loop(tmp_path):
    """include/paged_infer_engine.hpp: admission with prefix reuse, fork + copy-on-write, batched decode, reclaim."""
    exe = build_exe(tmp_path, "engine_tests")
    r = subprocess.run([exe], capture_output=True, text=True)
    print(r.stdout, r.stderr)
    assert r.returncode == 0 and "PASS" in r.stdout
