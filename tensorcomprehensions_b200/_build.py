"""In-tree build of the native parts (no JIT cache: the built files sit next to the sources).

    python -m tensorcomprehensions_b200._build            # everything that is stale
    python -m tensorcomprehensions_b200._build --force

Products:
    libtcb200.so   CUDA kernels + C ABI (include/tcb200.h), nvcc, sm_100a only
    libtc_core.so  C++ host: TC front-end, range inference, matcher, executor, tile sweep
    tclib*.so      pybind11 module over the ATen-facing API (needs libtorch)
"""
import glob
import os
import shutil
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")

NVCC_FLAGS = ["-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
              "-Xcompiler", "-fPIC"]


def _nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found: the CUDA kernel library cannot be built")


def _cxx():
    for c in (os.environ.get("TC_CXX"), "/usr/bin/g++", shutil.which("g++")):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("g++ not found")


def _stale(out, deps):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n%s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return r


def kernel_sources():
    return sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")))


def build_kernels(force=False, verbose=False, ptxas_v=False):
    out = os.path.join(PKG, "libtcb200.so")
    srcs = kernel_sources()
    deps = srcs + glob.glob(os.path.join(CSRC, "kernels", "*.cuh")) + [os.path.join(INCLUDE, "tcb200.h")]
    if not force and not _stale(out, deps):
        return out
    objs = []
    objdir = os.path.join(PKG, "build", "kernels")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    for s in srcs:
        o = os.path.join(objdir, os.path.basename(s) + ".o")
        objs.append(o)
        if not force and not _stale(o, [s] + deps[len(srcs):]):
            continue
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + \
              ["-I" + INCLUDE, "-I" + os.path.join(CSRC, "kernels"), "-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        txt, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed:\n%s\n%s" % (" ".join(cmd), txt))
        if ptxas_v:
            print(txt)
    _run([_nvcc(), "-shared", "-o", out] + objs + ["-lcudart"], verbose)
    return out


def host_sources():
    return sorted(glob.glob(os.path.join(CSRC, "host", "**", "*.cc"), recursive=True))


def build_host(force=False, verbose=False):
    """libtc_core.so: the torch-free C++ host (front-end, inference, matcher, executor, sweep)."""
    srcs = [s for s in host_sources() if os.path.basename(s) != "tclib.cc"]
    if not srcs:
        return None
    out = os.path.join(PKG, "libtc_core.so")
    hdrs = glob.glob(os.path.join(INCLUDE, "**", "*.h"), recursive=True)
    if not force and not _stale(out, srcs + hdrs):
        return out
    build_kernels(force=False, verbose=verbose)
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    objdir = os.path.join(PKG, "build", "host")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(objdir, os.path.relpath(s, CSRC).replace(os.sep, "_") + ".o")
        objs.append(o)
        if not force and not _stale(o, [s] + hdrs):
            continue
        cmd = [_cxx(), "-std=c++17", "-O2", "-fPIC", "-Wall", "-Wno-unused-function", "-I" + INCLUDE,
               "-I" + cuda_inc, "-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        txt, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("g++ failed:\n%s\n%s" % (" ".join(cmd), txt))
    cuda_lib = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "lib64")
    _run([_cxx(), "-shared", "-o", out] + objs +
         ["-L" + PKG, "-ltcb200", "-L" + cuda_lib, "-lcudart", "-Wl,-rpath,$ORIGIN", "-lpthread"], verbose)
    return out


def build_tclib(force=False, verbose=False):
    """pybind11 module over tc::aten (compile / run / profile / tune on torch tensors)."""
    src = os.path.join(CSRC, "host", "python", "tclib.cc")
    if not os.path.exists(src):
        return None
    import torch  # noqa: F401  (headers + libs)
    from torch.utils import cpp_extension
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(PKG, "tclib" + ext)
    hdrs = glob.glob(os.path.join(INCLUDE, "**", "*.h"), recursive=True)
    core = build_host(force=False, verbose=verbose)
    if not force and not _stale(out, [src, core] + hdrs):
        return out
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    incs = ["-I" + INCLUDE, "-I" + os.path.join(cuda_home, "include"), "-I" + sysconfig.get_paths()["include"]]
    incs += ["-I" + p for p in cpp_extension.include_paths()]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [_cxx(), "-std=c++17", "-O2", "-fPIC", "-shared", "-w", "-DTORCH_EXTENSION_NAME=tclib",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + incs + [src, "-o", out,
           "-L" + PKG, "-ltc_core", "-ltcb200", "-L" + tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
           "-L" + os.path.join(cuda_home, "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
    if os.path.exists(os.path.join(tlib, "libc10_cuda.so")):
        cmd += ["-lc10_cuda", "-ltorch_cuda"]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False):
    outs = [build_kernels(force, verbose), build_host(force, verbose), build_tclib(force, verbose)]
    return [o for o in outs if o]


if __name__ == "__main__":
    force = "--force" in sys.argv
    for o in build_all(force=force, verbose=True):
        print("ok", o)
