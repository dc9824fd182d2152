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
    [0, 128, 256, 300, 428].  Computed with tensor operations on the input's device (the number of blocks
    depends on the data, so sizing the result costs one read of a scalar).
    """
    counts = torch.bincount(sorted_experts_idxs.long(), minlength=k)
    expert_offsets = counts.cumsum(-1)
    starts = expert_offsets - counts
    blocks_per = (counts + (N_BLOCK_SIZE - 1)) // N_BLOCK_SIZE
    first_block = blocks_per.cumsum(-1) - blocks_per
    expert_of_block = torch.repeat_interleave(torch.arange(k, device=counts.device), blocks_per)
    j = torch.arange(expert_of_block.numel(), device=counts.device) - first_block[expert_of_block]
    return starts[expert_of_block] + j * N_BLOCK_SIZE, expert_offsets


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
    """LoRA factor gradients on expert-grouped X [M,K], DY [M,N]; returns (dA [E,K,r], dB [E,r,N]).

    On CUDA: four launches of the grouped GEMM family, nothing else (no base-weight product):
    `s DY B^T` and `s X A` as row-grouped products, then the two depth-grouped reductions
    `dA_e = X_e^T (s DY_e B_e^T)` and `dB_e = (s X_e A_e)^T DY_e`, each over all rows of the expert.
    """
    counts = torch.diff(expert_offsets, prepend=expert_offsets.new_zeros(1))
    sorted_ids = torch.repeat_interleave(torch.arange(E, device=X.device), counts.long(), output_size=X.shape[0])
    plan = _plan_from_sorted(sorted_ids, E)
    xg = ops.gather_rows(X.detach(), plan)
    dyg = ops.gather_rows(DY.detach(), plan)
    if X.is_cuda and ops.get_backend() == "native":
        from moe_distributed_training_b200.ops import cuda_ops as C
        Ad, Bd = A.detach().contiguous(), B.detach().contiguous()
        r, K, N, R = Ad.shape[2], X.shape[1], DY.shape[1], xg.shape[0]
        dt = torch.empty(R, r, dtype=X.dtype, device=X.device)
        C._g(1, dyg, False, Bd, False, dt, r, N, plan, alpha=float(scaling))
        t = torch.empty(R, r, dtype=X.dtype, device=X.device)
        C._g(1, xg, False, Ad, True, t, r, K, plan, alpha=float(scaling))
        dA, dB = torch.empty_like(Ad), torch.empty_like(Bd)
        C._g(2, xg, True, dt, True, dA, r, 0, plan)
        C._g(2, t, True, dyg, True, dB, N, 0, plan)
        return dA, dB
    # CPU / library path: the same two reductions, stated per expert
    dA, dB = torch.zeros_like(A), torch.zeros_like(B)
    offs = plan.padded_offsets.tolist()
    cnt = plan.tokens_per_expert.tolist()
    for e in range(E):
        xe, dye = xg[offs[e]:offs[e] + cnt[e]].float(), dyg[offs[e]:offs[e] + cnt[e]].float()
        dA[e] = (float(scaling) * xe.t() @ (dye @ B[e].float().t())).to(A.dtype)
        dB[e] = (float(scaling) * (xe @ A[e].float()).t() @ dye).to(B.dtype)
    return dA, dB
