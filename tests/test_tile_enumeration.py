"""Index arithmetic of the GEMM kernels, checked on the host: the persistent kernels' tile enumeration
(`get_tile`, `get_pair_tile` in csrc/gemm_sm100.cu) is compiled for the CPU and run over random dense, row-grouped
and depth-grouped problems (tests/host/tile_enumeration.cu)."""
import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def test_every_output_block_is_covered_exactly_once(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("needs nvcc")
    exe = str(tmp_path / "tile_enumeration")
    build = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17", "--expt-relaxed-constexpr",
                            "-I", os.path.join(HERE, "..", "csrc"), "-o", exe, os.path.join(HERE, "host", "tile_enumeration.cu")], capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stdout[-3000:]
    assert "0 failures" in run.stdout
