"""`parallel_linear_lora` under the reference's name and signature.

Reference: scattermoe_utils/parallel_linear_lora.py:151-187 (an autograd op over Triton
kernels, with an optional `khd` implementation).  Here the op is composed from the
framework's differentiable gather / grouped GEMM / combine ops, so gradients flow to the
inputs, the gates, the LoRA factors and — unlike the reference, which returns no gradient
for it (parallel_linear_lora.py:136-138) — to the base expert weight when it requires one.
"""
from __future__ import annotations

import torch

from moe_distributed_training_b200 import ops


def parallel_linear_lora(inputs, expert_weights, expert_lora_A, expert_lora_B, lora_r, lora_alp, k,
                         sorted_expert_idxs, sorted_scattered_idxs, padded_block_idxs=None, expert_offsets=None,
                         gates=None, grouped_in=False, grouped_out=False, use_khd=False):
    """inputs [T,K] (or [T*k,K] when grouped_in); weights [E,K,N]; A [E,K,r]; B [E,r,N].

    Returns [T*k, N] in slot order (or sorted order when grouped_out), or [T, N] when `gates`
    [T,k] is given (gate-weighted sum over the k choices of a token).
    """
    E = expert_weights.shape[0]
    plan = ops.make_plan(sorted_expert_idxs.int()[:, None].contiguous(), E)
    idx = sorted_scattered_idxs.long()
    xs = inputs if grouped_in else inputs.index_select(0, torch.div(idx, k, rounding_mode="floor"))
    xg = ops.gather_rows(xs, plan)
    lora = None
    if expert_lora_A is not None:
        lora = (expert_lora_A, expert_lora_B, float(lora_alp) / float(lora_r) if lora_r else float(lora_alp))
    yg = ops.grouped_linear(xg, expert_weights, plan, trans_b=False, lora=lora)
    ys = ops.combine_rows(yg, plan, None)                      # sorted order, un-padded
    if grouped_out:
        assert gates is None, "gates need slot order"
        return ys
    out = torch.zeros_like(ys).index_copy(0, idx, ys)          # slot order [T*k, N]
    if gates is not None:
        out = (out.view(gates.shape[0], gates.shape[1], -1) * gates[..., None].to(out.dtype)).sum(1)
    return out


class ParallelLinearLora:
    """Name kept for users of the reference; `apply` forwards to `parallel_linear_lora`."""

    @staticmethod
    def apply(x, expert_weights, lora_A, lora_B, lora_r, lora_alp, k, sorted_expert_idxs, sorted_scattered_idxs,
              padded_block_idxs=None, expert_offsets=None, gates=None, grouped_in=False, grouped_out=False):
        return parallel_linear_lora(x, expert_weights, lora_A, lora_B, lora_r, lora_alp, k, sorted_expert_idxs,
                                    sorted_scattered_idxs, padded_block_idxs, expert_offsets, gates, grouped_in, grouped_out)
