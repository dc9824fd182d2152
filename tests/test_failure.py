"""Failure detection, exercised on the host only (gloo ranks on CPU; nothing here touches a GPU)."""
import datetime
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_distributed
from moe_distributed_training_b200.utils.failure import Heartbeat, RankFailure


def test_heartbeat_reports_a_silent_rank_with_a_fake_clock():
    store = dist.HashStore()
    now = [1000.0]
    hb0 = Heartbeat(store, 0, 3, limit_s=30, clock=lambda: now[0])
    hb1 = Heartbeat(store, 1, 3, limit_s=30, clock=lambda: now[0])
    hb2 = Heartbeat(store, 2, 3, limit_s=30, clock=lambda: now[0])
    for hb in (hb0, hb1, hb2):
        hb.beat(1)
    hb0.check()
    now[0] += 20
    hb0.beat(2); hb2.beat(2)             # rank 1 goes silent
    now[0] += 20
    assert hb0.stale_ranks() == [1]
    with pytest.raises(RankFailure) as e:
        hb0.check()
    assert e.value.ranks == [1]
    hb2.mark_failed("ValueError")        # a rank that raised marks itself
    assert sorted(hb0.stale_ranks()) == [1, 2]


def _rank_that_raises(rank, world):
    store = dist.TCPStore("127.0.0.1", int(__import__("os").environ["MASTER_PORT"]) + 1, world, rank == 0,
                          timeout=datetime.timedelta(seconds=20))
    hb = Heartbeat(store, rank, world, limit_s=1.0)
    hb.beat(0)
    if rank == 1:
        hb.mark_failed("RuntimeError")   # this rank "raises" before the next step and leaves
        return "left"
    deadline = time.time() + 10
    while time.time() < deadline:
        try:
            hb.check()
        except RankFailure as exc:
            return exc.ranks
        time.sleep(0.05)
    return "not detected"


def test_rank_that_raises_is_detected_before_the_next_launch():
    res = run_distributed(_rank_that_raises, 2, timeout=60)
    assert res[0] == [1] and res[1] == "left"


def _collective_with_missing_rank(rank, world):
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t)                   # everyone joins the first collective
    if rank == 1:
        time.sleep(8)                    # never joins the second one in time
        return "late"
    try:
        dist.all_reduce(t)
        return "no error"
    except Exception as exc:  # noqa: BLE001
        return "timeout:" + type(exc).__name__


def test_collective_times_out_when_a_rank_never_joins():
    res = run_distributed(_collective_with_missing_rank, 2, timeout=60)
    assert res[0].startswith("timeout:")


def test_wrong_counts_are_caught_by_the_capacity_check():
    """Host-side statement of the device check: a receive layout larger than the buffer is an error."""
    from moe_distributed_training_b200.parallel.symm import ep_capacities
    rows, slots = ep_capacities(ws=8, num_experts=8, max_tokens=1024, top_k=2)
    assert rows >= 8 * 2048 and slots == 2048
    small, _ = ep_capacities(ws=8, num_experts=8, max_tokens=1024, top_k=2, capacity_factor=2.0)
    assert small < rows
