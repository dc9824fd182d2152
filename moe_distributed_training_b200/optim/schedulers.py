"""Learning-rate schedules by name, as `transformers.get_scheduler` offers them.

The reference requests `get_scheduler(lr_scheduler_type, optimizer, num_warmup_steps,
num_training_steps)` (train_accelerate_fsdp2.py:323-328); the names accepted here
are the ones that call understands: linear, cosine, constant, constant_with_warmup.
One `step()` per optimizer step.
"""
from __future__ import annotations

import math

from torch.optim.lr_scheduler import LambdaLR


def get_scheduler(name: str, optimizer, num_warmup_steps: int = 0, num_training_steps: int = 1):
    W, N = num_warmup_steps, max(1, num_training_steps)

    def warm(s):
        return s / max(1, W)

    if name == "linear":
        fn = lambda s: warm(s) if s < W else max(0.0, (N - s) / max(1, N - W))
    elif name == "cosine":
        fn = lambda s: warm(s) if s < W else max(0.0, 0.5 * (1 + math.cos(math.pi * (s - W) / max(1, N - W))))
    elif name == "constant":
        fn = lambda s: 1.0
    elif name == "constant_with_warmup":
        fn = lambda s: warm(s) if s < W else 1.0
    else:
        raise ValueError(f"unknown lr_scheduler_type '{name}'")
    return LambdaLR(optimizer, fn)
