"""Failure detection on the host.

The reference relies on torchrun's default behaviour (a failed rank eventually takes the job down) and
has no detection of its own.  Here:

  * every device-side wait is bounded and reports through a status word; `check_device_status` turns
    a non-zero word into a Python exception between steps, with the context still usable;
  * `Heartbeat` lets ranks learn on the host that a peer stopped making progress (each rank stamps a
    key in a c10d store once per step; a rank whose stamp is older than the limit is reported)
    before they launch kernels that would wait for it;
  * `collective_timeout` builds process groups whose collectives raise instead of blocking forever.

No rank is recovered or replaced: the job stops with a message naming the failed ranks.
"""
from __future__ import annotations

import datetime
import time
from typing import List, Optional

import torch


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], detail: str = ""):
        super().__init__(f"ranks {ranks} stopped responding {detail}".strip())
        self.ranks = ranks


class Heartbeat:
    """Per-step liveness stamps in a c10d key-value store (TCPStore / FileStore / HashStore)."""

    def __init__(self, store, rank: int, world_size: int, limit_s: float = 60.0, clock=time.time):
        self.store, self.rank, self.world, self.limit, self.clock = store, rank, world_size, limit_s, clock

    def beat(self, step: int) -> None:
        self.store.set(f"hb/{self.rank}", f"{step}:{self.clock():.3f}")

    def mark_failed(self, reason: str) -> None:
        self.store.set(f"failed/{self.rank}", reason)

    def stale_ranks(self) -> List[int]:
        now, bad = self.clock(), []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if self.store.check([f"failed/{r}"]):
                    bad.append(r)
                    continue
                if not self.store.check([f"hb/{r}"]):
                    continue  # has not started yet
                _, stamp = self.store.get(f"hb/{r}").decode().split(":")
                if now - float(stamp) > self.limit:
                    bad.append(r)
            except Exception:  # noqa: BLE001  (store unreachable counts as a failure of the store host)
                bad.append(r)
        return bad

    def check(self) -> None:
        bad = self.stale_ranks()
        if bad:
            raise RankFailure(bad, f"(no heartbeat for more than {self.limit:.0f} s, or marked failed)")


def check_device_status(device) -> None:
    """Raise if a kernel reported a wait that ran out of time since the last check."""
    if torch.device(device).type != "cuda":
        return
    from ..ops import cuda_ops
    cuda_ops.check_status(device)


def collective_timeout(seconds: float) -> datetime.timedelta:
    return datetime.timedelta(seconds=seconds)


def guarded_step(engine, microbatches, heartbeat: Optional[Heartbeat] = None):
    """`engine.train_step` with liveness checks around it."""
    if heartbeat is not None:
        heartbeat.check()
    try:
        out = engine.train_step(microbatches)
        check_device_status(engine.device)
    except Exception as exc:  # noqa: BLE001
        if heartbeat is not None:
            heartbeat.mark_failed(type(exc).__name__)
        raise
    if heartbeat is not None:
        heartbeat.beat(engine.step_count)
    return out
