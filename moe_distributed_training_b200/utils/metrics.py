"""Metric lines, device timers and launch accounting.

The reference prints one JSON object per optimizer step with the keys `epoch,
loss, learning_rate, gpu_mem_used_now, gpu_mem_used_peak, grad_norm`, and at the
end `train_runtime, train_steps_per_second` from a pair of CUDA events
(train_accelerate_fsdp2.py:395-471).  The same keys are produced here, plus
tokens/s timed on the device and reduced as the maximum time over ranks.
"""
from __future__ import annotations

import json
import time
from contextlib import contextmanager

import torch
import torch.distributed as dist


class DeviceTimer:
    """CUDA-event stopwatch (falls back to the host clock on CPU)."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.t0 = None
        self.start_ev = self.end_ev = None

    def start(self):
        if self.cuda:
            torch.cuda.synchronize()
            self.start_ev = torch.cuda.Event(enable_timing=True)
            self.end_ev = torch.cuda.Event(enable_timing=True)
            self.start_ev.record()
        else:
            self.t0 = time.perf_counter()

    def stop(self) -> float:
        """Seconds since start()."""
        if self.cuda:
            self.end_ev.record()
            torch.cuda.synchronize()
            return self.start_ev.elapsed_time(self.end_ev) / 1e3
        return time.perf_counter() - self.t0


def max_over_ranks(value: float, device) -> float:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return value


def sum_over_ranks(value: float, device) -> float:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t)
        return float(t.item())
    return value


def memory_stats(device) -> dict:
    if torch.device(device).type != "cuda":
        return {"gpu_mem_used_now": 0.0, "gpu_mem_used_peak": 0.0}
    gib = 1024 ** 3
    return {"gpu_mem_used_now": round(torch.cuda.memory_allocated(device) / gib, 3),
            "gpu_mem_used_peak": round(torch.cuda.max_memory_allocated(device) / gib, 3)}


def log_json(rank: int, **kv):
    if rank == 0:
        print(json.dumps(kv), flush=True)


@contextmanager
def nvtx_range(name: str, enabled: bool = True):
    """NVTX range around a phase (router / dispatch / experts / combine / attention / optimizer)."""
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
