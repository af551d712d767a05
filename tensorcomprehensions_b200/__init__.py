"""tensorcomprehensions_b200 — Tensor Comprehensions on hand-written sm_100a kernels.

The user-facing API mirrors the reference's Python package
(tensor_comprehensions/__init__.py): define / compile / autotune / MappingOptions /
assert_almost_equal.  It is imported lazily so that `import tensorcomprehensions_b200.cabi`
(the raw C ABI) works without libtorch being loaded.
"""
__all__ = ["cabi", "workloads"]


def __getattr__(name):
    # Python API (needs the tclib extension) is resolved on first use.
    if name in ("define", "compile", "autotune", "autotune_and_compile", "MappingOptions", "TC", "HostStagedExecutor",
                "Tuner", "TunerConfig", "Executor", "assert_almost_equal", "make_naive_options_factory",
                "make_load_from_cache_options_factory", "make_autotuned_options_factory",
                "MappingOptionsCache", "tclib", "sharding", "make_autograd", "logtostderr", "debug_lang",
                "debug_halide", "debug_tc_mapper", "debug_tuner", "dump_cuda", "dump_ptx", "cuda_compiler",
                "llvm_flags", "nvcc_flags"):
        import importlib
        api = importlib.import_module(".api", __name__)
        return getattr(api, name)
    raise AttributeError(name)
