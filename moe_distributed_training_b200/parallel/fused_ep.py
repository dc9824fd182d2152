"""Expert-parallel token exchange with in-kernel peer stores (no NCCL, no host synchronisation).

The reference's exchange (megablocks `parallel_forward_once`, selected by
megablocks_utils/shard_moe_utils.py:39) is: all-to-all of counts, a device->host read of the split
sizes, `all_to_all_single` of the rows, local re-sort, expert compute, `all_to_all_single` back.
Here every step runs on the device: counts are written into the peers' symmetric workspaces, each
rank derives all offsets itself, rows are stored straight into their final expert-grouped, block-padded
position in the owner's buffer (so the grouped GEMM reads them in place, with no local permute), and
expert outputs are stored straight back into the source rank's buffer in its sorted slot order.
The backward pass runs the same two movements in the opposite roles with the saved offsets.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..ops.reference import RoutingPlan
from . import symm


def available() -> bool:
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
        from ..ops import build
        import os
        return os.path.exists(os.path.join(build.EXT_DIR, build.EXT_NAME + ".so"))
    except Exception:  # noqa: BLE001
        return False


class _Phase:
    """Parity bookkeeping shared by the two halves (dispatch, combine) of one exchange."""

    def __init__(self, engine):
        self.engine = engine
        self.parity = None

    def begin(self):
        self.parity = self.engine.next_phase()
        return self.parity


class _Dispatch(torch.autograd.Function):
    """Rows of x (indexed through the send plan) -> owner ranks' receive buffers.  Returns this rank's buffer."""

    @staticmethod
    def forward(ctx, x, eng, send_plan, expert_of_slot, meta, fwd_phase, bwd_phase, keep):
        parity = fwd_phase.begin()
        eng.dispatch(x, send_plan.src_slot, expert_of_slot, None, meta, send_plan.top_k, parity)
        ctx.eng, ctx.send_plan, ctx.meta, ctx.bwd_phase = eng, send_plan, meta, bwd_phase
        out = eng.wspace.recv_x()
        return out.clone() if keep else out

    @staticmethod
    def backward(ctx, d_rows):
        eng, plan = ctx.eng, ctx.send_plan
        # gradient rows travel back to the ranks the rows came from, in their sorted slot order
        d_sorted = eng.combine(d_rows.contiguous(), ctx.meta, ctx.bwd_phase.parity, plan.dest_row.numel(), clone=False)
        from ..ops import cuda_ops
        dx = cuda_ops.ext.combine_rows(d_sorted, plan.dest_row, None, plan.top_k)
        return dx, None, None, None, None, None, None, None


class _CombineBack(torch.autograd.Function):
    """Expert-output rows -> source ranks (sorted slot order).  Returns [slots, hidden]."""

    @staticmethod
    def forward(ctx, y, eng, meta, n_slots, expert_sorted, fwd_phase, bwd_phase):
        ctx.eng, ctx.meta, ctx.expert_sorted, ctx.bwd_phase = eng, meta, expert_sorted, bwd_phase
        return eng.combine(y, meta, fwd_phase.parity, n_slots, clone=True)

    @staticmethod
    def backward(ctx, d_sorted):
        eng = ctx.eng
        parity = ctx.bwd_phase.begin()
        eng.dispatch(d_sorted.contiguous(), eng.identity(d_sorted.shape[0]), ctx.expert_sorted, None, ctx.meta, 1, parity)
        return eng.wspace.recv_x(), None, None, None, None, None, None


class FusedExpertParallel:
    """One per expert-parallel group and device; owns the symmetric workspace."""

    _instances = {}

    def __init__(self, wspace: symm.EpWorkspace, top_k: int, device):
        from ..ops import cuda_ops
        self.ext, self.cuda_ops = cuda_ops.ext, cuda_ops
        self.wspace, self.top_k, self.device = wspace, top_k, device
        self.count_epoch = 0
        self.phase = 0
        self.meta_size = int(self.ext.ep_meta_offsets(wspace.ws, wspace.num_experts)[8])
        self.meta_off = [int(v) for v in self.ext.ep_meta_offsets(wspace.ws, wspace.num_experts)]
        self._identity = None

    @classmethod
    def for_group(cls, group, args, device, max_tokens: Optional[int] = None):
        key = (group.group_name, torch.device(device).index)
        if key not in cls._instances:
            max_tokens = max_tokens or args.ep_max_tokens
            ws = symm.create_ep_workspace(group, args.moe_num_experts, args.hidden_size, max_tokens, args.moe_top_k, device)
            cls._instances[key] = cls(ws, args.moe_top_k, device)
        return cls._instances[key]

    # ------------------------------------------------------------------ primitives
    def next_phase(self) -> int:
        self.phase += 1
        return self.phase & 1

    def identity(self, n: int) -> torch.Tensor:
        if self._identity is None or self._identity.numel() < n:
            self._identity = torch.arange(max(n, self.wspace.capacity_slots), dtype=torch.int32, device=self.device)
        return self._identity[:n]

    def status(self):
        return self.cuda_ops.status_tensor(self.device)

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        w = self.wspace
        self.count_epoch += 1
        parity = self.count_epoch & 1
        # (the wait kernel writes every entry: real offsets, or all zeros = "no rows" when a peer's counts never came)
        meta = torch.empty(self.meta_size, dtype=torch.int32, device=self.device)
        self.ext.ep_counts_send(counts, w.peer_base, w.layout, w.rank, parity, self.count_epoch)
        self.ext.ep_counts_wait_meta(w.my_base, w.layout, w.rank, parity, self.count_epoch, meta, self.status())
        return meta

    def dispatch(self, x, src_slot, expert_of_slot, slot_scale, meta, top_k, parity, wait: bool = True):
        """Send my rows; `wait=False` leaves the waiting to a GEMM that checks the per-tile arrival counters."""
        w = self.wspace
        assert expert_of_slot.numel() <= w.capacity_slots, "more (token, choice) slots than the workspace was sized for"
        self.ext.ep_dispatch(x, src_slot, expert_of_slot, slot_scale, meta, w.peer_base, w.layout, w.rank, top_k, parity, self.status())
        self.ext.ep_recv_prepare(w.my_base, w.layout, meta, w.cols, parity, self.status(), wait)

    def combine(self, y, meta, parity, n_slots, clone: bool):
        w = self.wspace
        self.ext.ep_combine_send(y, meta, w.peer_base, w.layout, w.rank, w.capacity_rows, parity, self.status())
        return self.wait_rows(meta, parity, n_slots, 1, clone)

    def wait_rows(self, meta, parity, n_slots, mult: int, clone: bool):
        w = self.wspace
        self.ext.ep_wait_rows(w.my_base, w.layout, meta, parity, self.status(), mult)
        out = w.recv_y()[:n_slots]
        return out.clone() if clone else out

    # -- pieces for GEMMs that take part in the exchange themselves
    def fused_meta(self, meta):
        """(row -> source rank, row -> position at the source, rows expected per 128-row tile) of my receive layout."""
        w = self.wspace
        return self.ext.ep_fused_meta(meta, w.layout, w.rank)

    def gemm_wait(self, parity, tile_expected):
        return (self.wspace.tile_counters(parity), tile_expected)

    def gemm_scatter(self, parity, row_rank, row_pos):
        w = self.wspace
        if not hasattr(self, "_peer_out"):
            self._peer_out = torch.tensor([b + w.layout[9] for b in w.bases], dtype=torch.int64, device=self.device)
            self._peer_arrive = [torch.tensor([b + w.layout[7] + 4 * par for b in w.bases], dtype=torch.int64, device=self.device)
                                 for par in (0, 1)]
        return (row_rank, row_pos, self._peer_out, self._peer_arrive[parity])


    def recv_plan(self, meta) -> RoutingPlan:
        w = self.wspace
        El = w.num_experts // w.ws
        o = self.meta_off
        return RoutingPlan(meta[o[1]:o[1] + El], meta[o[2]:o[2] + El + 1], None, None, 1, El, capacity_rows=w.capacity_rows)

    # ------------------------------------------------------------------ layer forward
    def forward(self, layer, x, expert_weights, top_experts):
        E, k = layer.num_experts, layer.top_k
        n_slots = top_experts.numel()
        send_plan = ops.make_plan(top_experts, E, block=1, capacity=n_slots)
        layer.last_tokens_per_expert = send_plan.tokens_per_expert
        meta = self.exchange_counts(send_plan.tokens_per_expert)
        expert_of_slot = top_experts.reshape(-1).int().contiguous()
        expert_sorted = expert_of_slot.index_select(0, send_plan.src_slot.long()) if torch.is_grad_enabled() else None
        fwd_phase, bwd_phase = _Phase(self), _Phase(self)
        keep = torch.is_grad_enabled()
        xr = _Dispatch.apply(x.contiguous(), self, send_plan, expert_of_slot, meta, fwd_phase, bwd_phase, keep)
        yg = layer.mlp(xr, self.recv_plan(meta))
        ys = _CombineBack.apply(yg, self, meta, n_slots, expert_sorted, fwd_phase, bwd_phase)
        return ops.combine_rows(ys, send_plan, expert_weights)
