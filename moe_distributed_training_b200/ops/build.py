"""In-tree build of the sm_100a extension.

`build()` compiles `csrc/*.cu` with `-gencode arch=compute_100a,code=sm_100a` and the
pybind bindings into `moe_distributed_training_b200/_ext/mdt_ext.so`; `load()` imports
that file without rebuilding and raises if it is missing.
"""
from __future__ import annotations

import importlib.util
import os
import sys

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_ROOT = os.path.dirname(_PKG)
CSRC = os.path.join(_ROOT, "csrc")
EXT_DIR = os.path.join(_PKG, "_ext")
EXT_NAME = "mdt_ext"

SOURCES = ["bindings.cpp", "gemm_sm100.cu", "skinny.cu", "elementwise.cu", "router.cu", "attention.cu", "comm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources():
    return [os.path.join(CSRC, s) for s in SOURCES]


def build(verbose: bool = False):
    from torch.utils import cpp_extension
    os.makedirs(EXT_DIR, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    defines = []
    return cpp_extension.load(
        name=EXT_NAME, sources=sources(), extra_include_paths=[CSRC],
        extra_cflags=["-O2", "-std=c++17"] + defines, extra_cuda_cflags=NVCC_FLAGS + defines,
        build_directory=EXT_DIR, with_cuda=True, verbose=verbose)


_loaded = None


def load():
    """Import the built extension (no compilation); raises if it has not been built."""
    global _loaded
    if _loaded is not None:
        return _loaded
    path = os.path.join(EXT_DIR, EXT_NAME + ".so")
    if not os.path.exists(path):
        raise RuntimeError(
            f"the sm_100a extension is not built ({path} is missing); run "
            "`python -c 'import __graft_entry__ as g; g.build()'` from the repository root")
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location(EXT_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[EXT_NAME] = mod
    _loaded = mod
    return mod
