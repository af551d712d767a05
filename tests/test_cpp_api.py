"""The C++ API (tc::aten::compile / prepareOutputs / run / profile / ATenAutotuner::tune) used from a
C++ program, the way the reference's example uses it (tc/examples/tensordot.cc).  The program is
compiled once per session against include/tc/**, libtc_core and libtorch."""
import os
import subprocess
import sysconfig

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "tensorcomprehensions_b200")


def _build(name):
    from torch.utils import cpp_extension
    SRC = os.path.join(ROOT, "tests", "cpp", name + ".cc")
    EXE = os.path.join(PKG, "build", name)
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    deps = [SRC, os.path.join(PKG, "libtc_core.so")]
    lib_dir = os.path.join(ROOT, "include", "tc", "library")
    deps += [os.path.join(lib_dir, f) for f in os.listdir(lib_dir)]
    if not os.path.exists(EXE) or any(os.path.getmtime(d) > os.path.getmtime(EXE) for d in deps):
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-w", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
               "-I" + os.path.join(ROOT, "include")] + ["-I" + p for p in cpp_extension.include_paths()] + \
              [SRC, "-o", EXE, "-L" + PKG, "-ltc_core", "-ltcb200", "-L" + tlib, "-ltorch", "-ltorch_cpu", "-lc10",
               "-Wl,-rpath," + PKG, "-Wl,-rpath," + tlib]
        if os.path.exists(os.path.join(tlib, "libtorch_cuda.so")):
            cmd += ["-Wl,--no-as-needed", "-ltorch_cuda", "-lc10_cuda", "-Wl,--as-needed"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-3000:]
    return EXE


@pytest.fixture(scope="session")
def walkthrough_binary():
    return _build("api_walkthrough")


@pytest.fixture(scope="session")
def library_binary():
    return _build("library_cases")


def _run(exe):
    return subprocess.run([exe], capture_output=True, text=True, timeout=600)


def test_cpp_api_compile_time_part(walkthrough_binary):
    if torch.cuda.is_available():
        pytest.skip("covered by the gpu variant")
    r = _run(walkthrough_binary)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "api walkthrough ok (gpu=0)" in r.stdout and "tcb200::tensordot" in r.stdout


@pytest.mark.gpu
def test_cpp_api_full_flow_on_gpu(walkthrough_binary, cuda):
    r = _run(walkthrough_binary)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "api walkthrough ok (gpu=1)" in r.stdout and r.stdout.count("ran in:") == 3


def test_cpp_library_texts_compile(library_binary):
    """Every text of the operator library (include/tc/library/*.h) and the benchmarks' other cases match a
    kernel family and infer the reference's output shapes (no device needed)."""
    if torch.cuda.is_available():
        pytest.skip("covered by the gpu variant")
    r = _run(library_binary)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "library cases ok: 22 (gpu=0)" in r.stdout


@pytest.mark.gpu
def test_cpp_library_cases_on_gpu(library_binary, cuda):
    r = _run(library_binary)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "library cases ok: 22 (gpu=1)" in r.stdout


@pytest.mark.gpu
def test_one_executor_on_several_devices(cuda):
    """Compiled once, run from one host thread per device (needs two GPUs)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    r = _run(_build("multi_device"))
    assert r.returncode == 0, r.stdout + r.stderr
    assert "multi device ok" in r.stdout
