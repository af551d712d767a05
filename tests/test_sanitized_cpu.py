"""The C++ host (front-end, size binding, range inference, matcher) built with AddressSanitizer and
UndefinedBehaviorSanitizer and driven over the golden corpus, the error corpus and the benchmark / library texts
(tests/cpp/frontend_sanitized.cc).  compute-sanitizer covers nothing here (host code) and is closed on the GPU pool
anyway; this is the host-side half of the memory-safety checks.  No device is touched."""
import glob
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "tensorcomprehensions_b200")


def _nvcc_include():
    for c in ("/usr/local/cuda/include",):
        if os.path.isdir(c):
            return c
    return None


def test_host_front_end_under_asan_and_ubsan():
    cxx = "/usr/bin/g++"
    if not os.path.exists(cxx):
        pytest.skip("g++ not found")
    srcs = [s for s in glob.glob(os.path.join(PKG, "csrc", "host", "**", "*.cc"), recursive=True)
            if os.path.basename(s) != "tclib.cc"]
    exe = os.path.join(PKG, "build", "frontend_sanitized")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    deps = srcs + [os.path.join(ROOT, "tests", "cpp", "frontend_sanitized.cc")] + \
        glob.glob(os.path.join(ROOT, "include", "**", "*.h"), recursive=True)
    if not os.path.exists(exe) or any(os.path.getmtime(d) > os.path.getmtime(exe) for d in deps):
        cmd = [cxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
               "-fno-sanitize-recover=undefined", "-w", "-I" + os.path.join(ROOT, "include")]
        if _nvcc_include():
            cmd.append("-I" + _nvcc_include())
        cmd += [os.path.join(ROOT, "tests", "cpp", "frontend_sanitized.cc")] + srcs + \
               ["-o", exe, "-L" + PKG, "-ltcb200", "-Wl,-rpath," + PKG, "-lpthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    r = subprocess.run([exe, os.path.join(ROOT, "tests", "golden", "lang")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert r.returncode == 0, (r.stdout + r.stderr)[-4000:]
    assert "sanitized front-end ok" in r.stdout and "ERROR: AddressSanitizer" not in r.stderr
    assert "runtime error" not in r.stderr, r.stderr[-2000:]
