"""Operator front end.

Every op has exactly two implementations: the hand-written sm_100a kernels in
the in-tree extension (`ops.cuda_ops`, taken for CUDA tensors; it raises if the
extension is not built) and the plain PyTorch statement in `ops.reference`
(taken for CPU tensors; also the numerical oracle in the tests).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import reference
from .reference import BLOCK_ROWS, RoutingPlan, plan_capacity


_BACKEND = "native"


def set_backend(name: str) -> None:
    """"native": sm_100a kernels for CUDA tensors.  "library": the PyTorch statements (cuBLAS, SDPA,
    ATen) also on CUDA tensors; this is the baseline the kernels are measured against, never a fallback."""
    global _BACKEND
    if name not in ("native", "library"):
        raise ValueError(name)
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def _native(t) -> bool:
    return t.is_cuda and _BACKEND == "native"


def _cuda():
    from . import cuda_ops  # raises a clear error if the extension is missing
    return cuda_ops


def cuda_ops_ext():
    """The built extension module (raises if it is missing)."""
    return _cuda().ext


def router(x, w_router, top_k, normalize=True, jitter_eps=None, training=False, with_stats=False):
    """with_stats: a fourth result, fp32 [2E] = per-expert (token, choice) counts followed by per-expert sums of the
    scores (from the router kernel's own pass on CUDA; restated with tensor ops elsewhere)."""
    if _native(x) and jitter_eps is None:
        return _cuda().router(x, w_router, top_k, normalize, with_stats)
    scores, weights, idx = reference.router(x, w_router, top_k, normalize, jitter_eps, training)
    if not with_stats:
        return scores, weights, idx
    E = w_router.shape[0]
    with torch.no_grad():
        counts = torch.bincount(idx.reshape(-1).long(), minlength=E).float()
        stats = torch.cat([counts, scores.float().sum(0)])
    return scores, weights, idx, stats


def make_plan(top_experts, num_experts, block=BLOCK_ROWS, capacity=None) -> RoutingPlan:
    if _native(top_experts):
        return _cuda().make_plan(top_experts, num_experts, block, capacity)
    return reference.make_plan(top_experts, num_experts, block, capacity)


def gather_rows(x, plan: RoutingPlan):
    if _native(x):
        return _cuda().gather_rows(x, plan)
    return reference.gather_rows(x, plan.src_slot, plan.top_k)


def combine_rows(y, plan: RoutingPlan, weights: Optional[torch.Tensor]):
    if _native(y):
        return _cuda().combine_rows(y, plan, weights)
    return reference.combine_rows(y, plan.dest_row, weights, plan.top_k)


def grouped_swiglu_mlp(xg, w1, w2, w3, plan: RoutingPlan, lora=None, wgrad_scale: float = 1.0, wgrad_out=None):
    """Expert MLP over block-padded groups; w1, w2, w3 are [E_local, F, H].

    wgrad_out: optional (dw1, dw2, dw3) buffers the CUDA weight-gradient kernels accumulate into
    directly (no gradient tensor is returned for the weights then)."""
    if _native(xg):
        return _cuda().grouped_swiglu_mlp(xg, w1, w2, w3, plan, lora, wgrad_scale, wgrad_out)
    return reference.grouped_swiglu_mlp(xg, w1, w2, w3, plan.padded_offsets, plan.tokens_per_expert, lora, wgrad_scale)


def grouped_linear(x, w, plan: RoutingPlan, trans_b: bool, lora=None, wgrad_scale: float = 1.0):
    if _native(x):
        return _cuda().grouped_linear(x, w, plan, trans_b, lora, wgrad_scale)
    if wgrad_scale != 1.0:
        w = reference.scale_gradient(w, wgrad_scale)
        if lora is not None:
            lora = (reference.scale_gradient(lora[0], wgrad_scale), reference.scale_gradient(lora[1], wgrad_scale), lora[2])
    return reference.grouped_linear(x, w, plan.padded_offsets, trans_b, plan.tokens_per_expert, lora)


def linear(x, w, lora=None):
    if _native(x):
        return _cuda().linear(x, w, lora)
    return reference.linear(x, w, lora)


def rmsnorm(x, weight, eps):
    if _native(x):
        return _cuda().rmsnorm(x, weight, eps)
    return reference.rmsnorm(x, weight, eps)


def rope(x, positions, theta):
    if _native(x):
        return _cuda().rope(x, positions, theta)
    return reference.rope(x, positions, theta)


def attention(q, k, v, cu_seqlens, max_seqlen=None):
    if _native(q):
        return _cuda().attention(q, k, v, cu_seqlens, max_seqlen)
    if q.is_cuda:
        from . import attention_cuda
        return attention_cuda.sdpa_attention(q, k, v, cu_seqlens, max_seqlen)
    return reference.attention(q, k, v, cu_seqlens)


def cross_entropy_sum(hidden, w_head, labels, ignore_index=-100):
    if _native(hidden):
        return _cuda().cross_entropy_sum(hidden, w_head, labels, ignore_index)
    return reference.cross_entropy_sum(hidden, w_head, labels, ignore_index)


def embedding(ids, weight):
    if _native(weight):
        return _cuda().embedding(ids, weight)
    return torch.nn.functional.embedding(ids, weight)


def swiglu(g, u):
    if _native(g):
        return _cuda().swiglu(g, u)
    return reference.swiglu(g, u)
