"""Host-side helpers of bench.py: the time-limit decision of a two-arm child job and how its ranks share it."""
import os
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402


def test_second_arm_runs_only_when_it_fits_the_time_limit():
    now = 1000.0
    assert bench.second_arm_fits(30.0, now, now + 100.0)          # 30 s first arm: 76 s needed
    assert not bench.second_arm_fits(30.0, now, now + 70.0)
    assert not bench.second_arm_fits(5.0, now, now + 15.0)


def test_ranks_share_the_decision_of_rank_zero(tmp_path):
    for decision in (True, False):
        path = str(tmp_path / f"d_{decision}")
        got = {}

        def other(rank):
            got[rank] = bench.share_decision(path, rank, None, wait_s=5.0)
        threads = [threading.Thread(target=other, args=(r,)) for r in (1, 2, 3)]
        for t in threads:
            t.start()
        time.sleep(0.2)                                             # the others are already polling
        got[0] = bench.share_decision(path, 0, decision)
        for t in threads:
            t.join()
        assert got == {0: decision, 1: decision, 2: decision, 3: decision}


def test_a_decision_that_never_arrives_means_no(tmp_path):
    assert bench.share_decision(str(tmp_path / "never"), 1, None, wait_s=0.2) is False


def test_reference_arm_reports_unavailable_and_exits_zero():
    """`bench.py --impl reference` must print one JSON line with `impl` and `unavailable` and exit 0 when the
    reference's entry points cannot run (their third-party imports are missing in this environment)."""
    import json
    import subprocess
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(here, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    if "unavailable" in line:
        assert isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]
    else:                                   # an environment that has the reference's dependencies
        assert "value" in line
