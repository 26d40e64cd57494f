"""CPU: the host-side C++ of the KV slab manager under AddressSanitizer and UndefinedBehaviorSanitizer.

`lmdeploy_b200/csrc/cache_manager.cu` is plain host code; it is compiled here with `-fsanitize=address,undefined`
together with a stress program (tests/sanitize/cache_manager_stress.cc) that drives tm_cache_* in host-memory mode
through thousands of seeded operations.  Any out-of-bounds access, use after free or undefined arithmetic aborts the
program.  No GPU is needed (host mode calls no CUDA function; the runtime library is linked but never initialised)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cache_manager_under_asan_and_ubsan(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not found")
    cuda = os.path.dirname(os.path.dirname(nvcc))
    exe, o1, o2 = str(tmp_path / "cache_manager_stress"), str(tmp_path / "cm.o"), str(tmp_path / "stress.o")
    san = ["-fsanitize=address", "-fsanitize=undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g"]
    steps = [
        [nvcc, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), *[a for f in san for a in ("-Xcompiler", f)], "-c",
         os.path.join(ROOT, "lmdeploy_b200", "csrc", "cache_manager.cu"), "-o", o1],
        [gxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(cuda, "include")] + san
        + ["-c", os.path.join(ROOT, "tests", "sanitize", "cache_manager_stress.cc"), "-o", o2],
        [gxx, o1, o2] + san + ["-L", os.path.join(cuda, "lib64"), "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-lcudart", "-o", exe],
    ]
    for cmd in steps:
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 and "cannot find" in r.stderr and ("asan" in r.stderr or "ubsan" in r.stderr):
            pytest.skip("sanitizer runtimes not installed")
        assert r.returncode == 0, " ".join(cmd) + "\n" + r.stdout + r.stderr
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:protect_shadow_gap=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    r = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "cache manager stress ok" in r.stdout
