"""Grouped-linear primitives under the reference's names (`scattermoe_utils/kernels/ops.py`).

The reference implements `scatter2scatter_lora` and `group_bwd_AB` as Triton kernels over
un-padded expert groups (ops.py:13-255).  Here they are thin adapters onto the framework's
block-padded grouped GEMM family (tcgen05 kernels on CUDA, PyTorch on CPU):

    Y = X W_e + (alpha/r) (X A_e) B_e      per expert group e
    dA_e = s X_e^T (DY_e B_e^T),  dB_e = s (X_e A_e)^T DY_e     (full reductions)
"""
from __future__ import annotations

import torch

from moe_distributed_training_b200 import ops
from moe_distributed_training_b200.ops.reference import BLOCK_ROWS

BLOCK_M = BLOCK_ROWS


def padded_block_indices(sorted_experts_idxs: torch.Tensor, k: int, N_BLOCK_SIZE: int = BLOCK_M):
    """(start row of every work block, inclusive cumsum of per-expert counts) — scattermoe's helper.

    Expert groups are not padded in memory: counts (300, 200) give blocks starting at
    [0, 128, 256, 300, 428].
    """
    counts = torch.bincount(sorted_experts_idxs.long(), minlength=k)
    expert_offsets = counts.cumsum(-1)
    starts = expert_offsets - counts
    blocks = []
    for s, c in zip(starts.tolist(), counts.tolist()):
        blocks += list(range(s, s + c, N_BLOCK_SIZE))
    return torch.tensor(blocks, dtype=torch.long, device=sorted_experts_idxs.device), expert_offsets


def _plan_from_sorted(sorted_expert_idxs: torch.Tensor, E: int):
    return ops.make_plan(sorted_expert_idxs.int()[:, None].contiguous(), E)


def scatter2scatter_lora(X, W, A, B, lora_alp, sorted_expert_idxs, sorted_scattered_idxs, k,
                         padded_block_idxs=None, x_grouped=False, y_grouped=False, out=None):
    """Y = X W + lora_alp (X A) B over expert groups.

    W [E,K,N], A [E,K,r], B [E,r,N].  Rows of X are read through
    `sorted_scattered_idxs // k` unless `x_grouped`; the result is written in sorted order
    when `y_grouped`, otherwise scattered back to slot order.
    """
    E = W.shape[0]
    plan = _plan_from_sorted(sorted_expert_idxs, E)
    xs = X if x_grouped else X.index_select(0, torch.div(sorted_scattered_idxs, k, rounding_mode="floor"))
    xg = ops.gather_rows(xs, plan)
    lora = (A, B, float(lora_alp)) if A is not None else None
    yg = ops.grouped_linear(xg, W, plan, trans_b=False, lora=lora)
    ys = ops.combine_rows(yg, plan, None)
    if not y_grouped:
        res = torch.empty_like(ys)
        res = res.index_copy(0, sorted_scattered_idxs.long(), ys)
        ys = res
    if out is not None:
        out.copy_(ys)
        return out
    return ys


def group_bwd_AB(DY, X, A, B, scaling, expert_offsets, E):
    """LoRA factor gradients on expert-grouped X [M,K], DY [M,N]; returns (dA [E,K,r], dB [E,r,N])."""
    counts = torch.diff(expert_offsets, prepend=expert_offsets.new_zeros(1))
    sorted_ids = torch.repeat_interleave(torch.arange(E, device=X.device), counts.long(), output_size=X.shape[0])
    plan = _plan_from_sorted(sorted_ids, E)
    Al, Bl = A.detach().requires_grad_(True), B.detach().requires_grad_(True)
    xg = ops.gather_rows(X.detach(), plan)
    W0 = torch.zeros(E, X.shape[1], DY.shape[1], dtype=X.dtype, device=X.device)
    with torch.enable_grad():
        yg = ops.grouped_linear(xg, W0, plan, trans_b=False, lora=(Al, Bl, float(scaling)))
    dyg = ops.gather_rows(DY, plan)
    dA, dB = torch.autograd.grad(yg, [Al, Bl], dyg)
    return dA, dB
