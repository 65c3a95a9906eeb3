"""The C++ restatement of the engine's host-side block bookkeeping (include/paged_infer_memory.hpp: BlockAllocator,
BlockTable, PrefixCache, KvCacheManager) against the scenarios of the reference's own unit tests
(src/memory/kv_cache_manager.rs:418-636), plus its chained FNV-1a block hash against an independent Python one.
And the engine step loop (include/paged_infer_engine.hpp) over a host-side fake of the device calls
(tests/cpp/engine_host_tests.cpp): admission gated by memory only, forwards chunked by the scratch capacity.
Pure host logic: runs without a GPU."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def fnv_block_hash(parent: int, tokens) -> int:   # src/memory/prefix_cache.rs:28-40
    prime, mask = 0x00000100000001B3, (1 << 64) - 1
    h = parent ^ 0xCBF29CE484222325
    for t in tokens:
        for byte in int(t).to_bytes(4, "little"):
            h = ((h ^ byte) * prime) & mask
    h ^= len(tokens)
    return (h * prime) & mask


def test_memory_manager_scenarios(tmp_path):
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    if not gxx:
        pytest.skip("no C++ compiler")
    exe = str(tmp_path / "memory_manager_tests")
    subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", os.path.join(ROOT, "tests", "cpp", "memory_manager_tests.cpp"),
                    "-o", exe], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.split("\n")
    assert "all ok" in lines
    for name in ("allocator", "block_table", "lru_preemption", "prefix_reuse", "divergence", "cache_disabled", "cache_survives",
                 "eviction_under_pressure", "rejected_admission", "fork_cow", "unshared", "cow_vs_cache", "release_order", "churn"):
        assert f"ok {name}" in lines, name
    hashes = [int(l.split()[1], 16) for l in lines if l.startswith("hash ")]
    h1 = fnv_block_hash(0, [0, 1, 2, 3])
    assert hashes == [h1, fnv_block_hash(h1, [4, 5, 6, 7]), fnv_block_hash(0, [0xFFFFFFFF, 0x01020304, 7]), fnv_block_hash(0, [])]


def test_engine_loop_over_a_fake_device_library(tmp_path):
    gxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++")
    if not gxx:
        pytest.skip("no C++ compiler")
    exe = str(tmp_path / "engine_host_tests")
    subprocess.run([gxx, "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "engine_host_tests.cpp"), "-o", exe], check=True)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.split("\n")
    for name in ("oversize", "capacity", "passes", "queue"):
        assert f"ok {name}" in lines, name
    assert "all ok" in lines
