"""Dropless mixture-of-experts layer: local, expert-parallel and tensor-parallel forms.

What the reference obtains by patching megablocks' `dMoE`/`MoE`
(megablocks_utils/config_utils.py:71-284) is written here as one self-contained
module:

  dMoE.forward(x[B,S,H]) -> (out[B,S,H], None)        (config_utils.py:75-95)
    router -> (scores, weights, top_experts)           (config_utils.py:255-284)
    experts(x, scores, weights, top_experts)
       local:  sort slots by expert, gather, grouped SwiGLU MLP, weighted combine
       EP:     exchange counts, send every (token, choice) row to the rank that
               owns its expert, compute, send back, weighted combine
               (megablocks `parallel_forward_once`, selected by
               megablocks_utils/shard_moe_utils.py:39)
       TP:     every rank holds a slice of each expert's FFN dim; partial
               outputs are summed over the group (config_utils.py:168-184)

The EP token exchange has two implementations: "nccl" issues
`all_to_all_single` with split sizes read on the host (this also runs on gloo),
"fused" pushes rows into peer GPUs' buffers from inside a kernel.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..config import MoEArguments
from .experts import SparseMLPv2
from .router import LearnedRouter


# ----------------------------------------------------------------------------
# differentiable collectives
# ----------------------------------------------------------------------------
class _AllToAll(torch.autograd.Function):
    """Uneven all-to-all of rows; the backward is the same exchange with splits swapped."""

    @staticmethod
    def forward(ctx, x, recv_splits, send_splits, group):
        ctx.splits = (recv_splits, send_splits)
        ctx.group = group
        out = x.new_empty((sum(recv_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_splits,
                               input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        recv_splits, send_splits = ctx.splits
        out = grad.new_empty((sum(send_splits),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(out, grad.contiguous(), output_split_sizes=send_splits,
                               input_split_sizes=recv_splits, group=ctx.group)
        return out, None, None, None


def _tp_all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    """Sum over the tensor-parallel group: the peer-memory kernel on CUDA (native backend), else the library call."""
    x = x.contiguous()
    if x.is_cuda and ops.get_backend() == "native" and x.dtype in (torch.bfloat16, torch.float32) \
            and os.environ.get("MDT_PEER_COLLECTIVES", "1") != "0":
        from ..parallel import fused_ep, symm
        if fused_ep.available():
            nbytes = x.numel() * x.element_size()
            ar = symm.PeerAllReduce.for_group(group, max(nbytes, 64 << 20), x.device)
            if nbytes <= ar.half:
                return ar(x)
    x = x.clone()
    dist.all_reduce(x, group=group)
    return x


class _ReduceFromTP(torch.autograd.Function):
    """Forward: sum over the tensor-parallel group.  Backward: identity."""

    @staticmethod
    def forward(ctx, x, group):
        return _tp_all_reduce(x, group)

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _CopyToTP(torch.autograd.Function):
    """Forward: identity.  Backward: sum the input gradient over the tensor-parallel group."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, grad):
        return _tp_all_reduce(grad, ctx.group), None


# ----------------------------------------------------------------------------
# experts
# ----------------------------------------------------------------------------
class ParallelDroplessMLP(nn.Module):
    """The `experts` sub-module of the MoE layer (parameter path `experts.mlp.w{1,2,3}`)."""

    def __init__(self, args: MoEArguments):
        super().__init__()
        self.args = args
        self.mlp = SparseMLPv2(args)
        self.num_experts = args.moe_num_experts
        self.top_k = args.moe_top_k
        self.ep_group = args.expert_parallel_group if args.moe_expert_model_parallelism else None
        self.tp_group = args.tensor_parallel_group if args.tensor_parallel_size > 1 else None
        self._fused = None  # lazily created in-kernel dispatch/combine engine
        self.last_tokens_per_expert: Optional[torch.Tensor] = None

    # -- helpers -----------------------------------------------------------
    @property
    def ep_size(self) -> int:
        return self.ep_group.size() if self.ep_group is not None else 1

    def _dispatch_impl(self, x: torch.Tensor) -> str:
        impl = self.args.dispatch_impl
        if impl == "auto":
            from ..parallel import fused_ep
            impl = "fused" if (x.is_cuda and fused_ep.available()) else "nccl"
        return impl

    # -- single-rank path --------------------------------------------------
    def forward_once(self, x, expert_weights, top_experts):
        plan = ops.make_plan(top_experts, self.num_experts)
        self.last_tokens_per_expert = plan.tokens_per_expert
        xg = ops.gather_rows(x, plan)
        if self.tp_group is not None:
            xg = _CopyToTP.apply(xg, self.tp_group)
        yg = self.mlp(xg, plan)
        if self.tp_group is not None:
            yg = _ReduceFromTP.apply(yg, self.tp_group)
        return ops.combine_rows(yg, plan, expert_weights)

    # -- expert-parallel path, library collectives --------------------------
    def parallel_forward_once(self, x, expert_weights, top_experts):
        ep, E, k = self.ep_size, self.num_experts, self.top_k
        E_l = E // ep
        # 1. sort slots by (global) expert id: destination-rank-major, no padding
        send_plan = ops.make_plan(top_experts, E, block=1, capacity=top_experts.numel())
        counts = send_plan.tokens_per_expert
        self.last_tokens_per_expert = counts
        # 2. exchange per-expert counts
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.ep_group)
        # 3. host-side split sizes (one device->host read, as the reference does)
        both = torch.stack([counts.view(ep, E_l).sum(1), recv_counts.view(ep, E_l).sum(1)]).tolist()
        send_splits, recv_splits = both[0], both[1]
        # 4. rows in destination order, then the exchange
        xs = ops.gather_rows(x, send_plan)
        xr = _AllToAll.apply(xs, recv_splits, send_splits, self.ep_group)
        # 5. received rows are source-major, expert-sorted inside each chunk
        n_recv = sum(recv_splits)
        local_ids = torch.arange(E_l, device=x.device, dtype=torch.int32).repeat(ep)
        row_expert = torch.repeat_interleave(local_ids, recv_counts.long(), output_size=n_recv)
        plan = ops.make_plan(row_expert[:, None], E_l)
        xg = ops.gather_rows(xr, plan)
        yg = self.mlp(xg, plan)
        yr = ops.combine_rows(yg, plan, None)
        # 6. back to the source ranks, un-sort, gate-weight, sum over top-k
        ys = _AllToAll.apply(yr, send_splits, recv_splits, self.ep_group)
        return ops.combine_rows(ys, send_plan, expert_weights)

    # -- expert-parallel path, in-kernel peer stores -------------------------
    def fused_parallel_forward_once(self, x, expert_weights, top_experts):
        if self._fused is None:
            from ..parallel.fused_ep import FusedExpertParallel
            self._fused = FusedExpertParallel.for_group(self.ep_group, self.args, x.device)
        return self._fused.forward(self, x, expert_weights, top_experts)

    def forward(self, x, scores, expert_weights, top_experts):
        shape = x.shape
        x2d = x.reshape(-1, shape[-1])
        if self.ep_group is not None and self.ep_size > 1:
            if self._dispatch_impl(x2d) == "fused":
                out = self.fused_parallel_forward_once(x2d, expert_weights, top_experts)
            else:
                out = self.parallel_forward_once(x2d, expert_weights, top_experts)
        else:
            out = self.forward_once(x2d, expert_weights, top_experts)
        return out.view(shape)


class dMoE(nn.Module):
    """Router + dropless experts; returns `(hidden, None)` like HF's sparse MoE block."""

    def __init__(self, args: MoEArguments):
        super().__init__()
        self.args = args
        self.router = LearnedRouter(args)
        self.experts = ParallelDroplessMLP(args)
        self.last_scores: Optional[torch.Tensor] = None

    def forward(self, x: torch.Tensor):
        scores, expert_weights, top_experts = self.router(x)
        if self.args.moe_loss_weight > 0:
            self.last_scores = (scores, top_experts)
        out = self.experts(x, scores, expert_weights, top_experts)
        return out, None

    def as_dtensors(self) -> dict:
        """The layer's parameters as `DTensor`s over the mesh `shard_moe` built, under the reference's names:
        `router.layer.weight` replicated, `experts.mlp.w{1,2,3}` `[E*F, H]` with `Shard(0)` on the expert-parallel
        mesh dim and `Replicate` on the data-parallel one (megablocks_utils/shard_moe_utils.py:172-201, 240-248).
        The kernels work on the local tensors (`to_local()` of these); this view is for code that inspects or
        gathers the sharded model the way it would the reference's.  Without a mesh the plain parameters are returned.
        """
        names = {"router.layer.weight": self.router.layer.weight, "experts.mlp.w1": self.experts.mlp.w1,
                 "experts.mlp.w2": self.experts.mlp.w2, "experts.mlp.w3": self.experts.mlp.w3}
        mesh, placements = getattr(self, "_ep_mesh", None), getattr(self, "_ep_placements", None)
        if mesh is None:
            return names
        from torch.distributed.tensor import DTensor, Replicate
        out = {}
        for name, p in names.items():
            pl = [Replicate()] * mesh.ndim if name.startswith("router") else list(placements)
            out[name] = DTensor.from_local(p.detach(), mesh, pl, run_check=False)
        return out

    def aux_loss(self):
        if self.last_scores is None:
            return None
        scores, top = self.last_scores
        E, k = self.args.moe_num_experts, self.args.moe_top_k
        stats = getattr(self.router, "last_stats", None)
        if stats is not None and stats.numel() == 2 * E and not self.args.uniform_expert_assignment:
            # f_e from the histogram the router kernel made while routing; P_e through `scores`, which carries the gradient
            f = (stats[:E] / max(scores.shape[0] * k, 1)).to(scores.dtype)
            return self.args.moe_loss_weight * E * torch.sum(f * scores.mean(dim=0))
        from ..ops.reference import load_balancing_loss
        return self.args.moe_loss_weight * load_balancing_loss(scores, top, E, k)


# The tensor-parallel variant uses the same module; the name is kept for users of the reference,
# which instantiates megablocks `MoE` for that mode (megablocks_utils/shard_moe_utils.py:297-306).
MoE = dMoE
