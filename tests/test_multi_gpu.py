"""Multi-GPU tests (skipped with fewer than two GPUs): the peer-memory exchange and the peer-memory
parameter collectives reproduce the library (NCCL) path.  Ranks are child processes; NVLS is off in NCCL
(NCCL_NVLS_ENABLE=0) and symmetric memory is mapped without an NVLink multicast object
(TORCH_SYMM_MEM_DISABLE_MULTICAST=1), so a rank that ends leaves nothing bound in the switch."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(n, mode, tmp_path, port):
    out = str(tmp_path / f"res_{mode}.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "multi_gpu_worker.py"), out, mode]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    return json.load(open(out))


MODES = ["full", "lora", "fsdp", "fsdp-lora", "full-pool", "fsdp-lora-pool"]


@pytest.mark.parametrize("mode", MODES)
def test_fused_exchange_matches_nccl_exchange(tmp_path, mode):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    # two ranks by default; MDT_TEST_RANKS=4 (with at least four GPUs) runs the same comparison on four
    n = 4 if (n >= 4 and os.environ.get("MDT_TEST_RANKS") == "4") else 2
    res = _run(n, mode, tmp_path, 29610 + MODES.index(mode))
    for rank_res in res:
        a, b = rank_res["nccl"], rank_res["fused"]
        for la, lb in zip(a["losses"], b["losses"]):
            assert abs(la - lb) < 2e-2 * abs(la), (a, b)
        assert abs(a["checksum"] - b["checksum"]) < 1e-3 * abs(a["checksum"]), (a, b)


def test_tensor_parallel_experts_peer_all_reduce_matches_nccl(tmp_path):
    """Tensor-parallel experts need a 2-D (dp, tp) mesh, i.e. four GPUs."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs at least four GPUs")
    res = _run(4, "tp", tmp_path, 29630)
    for rank_res in res:
        a, b = rank_res["nccl"], rank_res["fused"]
        for la, lb in zip(a["losses"], b["losses"]):
            assert abs(la - lb) < 2e-2 * abs(la), (a, b)
        assert abs(a["checksum"] - b["checksum"]) < 1e-3 * abs(a["checksum"]), (a, b)


def test_rank_that_leaves_between_steps_is_detected_on_the_host(tmp_path):
    """A rank exits between two steps (nothing of its in flight); the others see it in the store before their next
    launch, raise RankFailure on the host, and their CUDA contexts stay usable (status word clean)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    n = 2
    out = str(tmp_path / "res_exit.json")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29640", os.path.join(HERE, "multi_gpu_worker.py"), out, "rank-exit"]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    res = [json.load(open(f"{out}.rank{r}")) for r in range(n)]
    assert res[n - 1].get("left") is True
    for r in range(n - 1):
        assert res[r]["detected"] == [n - 1], res[r]
        assert res[r]["step_count"] == 1          # the second step never started
