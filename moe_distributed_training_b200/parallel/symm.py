"""Symmetric workspaces: buffers of identical layout on every GPU of a group, mapped into all peers.

The mapping itself comes from `torch.distributed._symmetric_memory` (CUDA virtual-memory handles
exchanged over the process group); everything that happens in the buffers is done by this
framework's kernels (`csrc/comm.cu`), which receive the peers' base addresses as a device table.
`emulate` builds the same structure for several pretend ranks inside one GPU, so that the kernels of
all ranks can be run one after another on a single device in tests.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


# The kernels of this framework address peers with plain loads and stores only.  torch's rendezvous would otherwise
# also bind every symmetric buffer to an NVLink multicast object on NVSwitch machines, which nothing here uses and
# which makes the other ranks' GPUs raise NVLink errors when one rank's process ends while its memory is still
# bound.  The variable is read by torch when the first buffer is allocated; a value set by the user wins.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


@dataclass
class EpWorkspace:
    ws: int
    rank: int
    num_experts: int
    cols: int
    capacity_rows: int
    capacity_slots: int
    layout: List[int]
    nbytes: int
    buffer: torch.Tensor            # this rank's workspace (uint8)
    bases: List[int]                # base address of every rank's workspace, as seen from this GPU
    peer_base: torch.Tensor         # the same, int64 on the device
    handle: object = None

    @property
    def my_base(self) -> int:
        return self.bases[self.rank]

    def recv_x(self) -> torch.Tensor:
        off = self.layout[8]
        return self.buffer[off:off + self.capacity_rows * self.cols * 2].view(torch.bfloat16).view(self.capacity_rows, self.cols)

    def tile_counters(self, parity: int) -> torch.Tensor:
        n = self.capacity_rows // 128
        off = self.layout[10] + parity * n * 4
        return self.buffer[off:off + n * 4].view(torch.int32)

    def recv_y(self) -> torch.Tensor:
        off = self.layout[9]
        return self.buffer[off:off + self.capacity_slots * self.cols * 2].view(torch.bfloat16).view(self.capacity_slots, self.cols)


def ep_layout(ws: int, num_experts: int, cols: int, capacity_rows: int, capacity_slots: int):
    off = 0
    off_counts = off; off = _align(off + 2 * ws * num_experts * 4)
    off_flags = off; off = _align(off + 2 * ws * 4)
    off_ax = off; off = _align(off + 8)
    off_ay = off; off = _align(off + 8)
    off_rx = off; off = _align(off + capacity_rows * cols * 2)
    off_ry = off; off = _align(off + capacity_slots * cols * 2)
    off_tc = off; off = _align(off + 2 * (capacity_rows // 128) * 4)
    return [ws, num_experts, capacity_rows, capacity_slots, off_counts, off_flags, off_ax, off_ay, off_rx, off_ry, off_tc], off


def ep_capacities(ws: int, num_experts: int, max_tokens: int, top_k: int, capacity_factor: Optional[float] = None):
    """Rows of the receive buffer.  Dropless worst case: every slot of every rank lands here."""
    slots = max_tokens * top_k
    e_local = num_experts // ws
    worst = ws * slots + e_local * 127
    rows = worst if capacity_factor is None else int(slots * capacity_factor) + e_local * 127
    return ((rows + 127) // 128) * 128, slots


def create_ep_workspace(group, num_experts: int, cols: int, max_tokens: int, top_k: int, device,
                        capacity_factor: Optional[float] = None) -> EpWorkspace:
    import torch.distributed._symmetric_memory as symm_mem
    ws, rank = dist.get_world_size(group), dist.get_rank(group)
    cap_rows, cap_slots = ep_capacities(ws, num_experts, max_tokens, top_k, capacity_factor)
    layout, nbytes = ep_layout(ws, num_experts, cols, cap_rows, cap_slots)
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    handle = symm_mem.rendezvous(buf, group.group_name)
    bases = [int(p) for p in handle.buffer_ptrs]
    torch.cuda.synchronize(device)
    dist.barrier(group)
    peer_base = torch.tensor(bases, dtype=torch.int64, device=device)
    return EpWorkspace(ws, rank, num_experts, cols, cap_rows, cap_slots, layout, nbytes, buf, bases, peer_base, handle)


def emulate_ep_workspaces(ws: int, num_experts: int, cols: int, max_tokens: int, top_k: int, device) -> List[EpWorkspace]:
    cap_rows, cap_slots = ep_capacities(ws, num_experts, max_tokens, top_k)
    layout, nbytes = ep_layout(ws, num_experts, cols, cap_rows, cap_slots)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(ws)]
    bases = [b.data_ptr() for b in bufs]
    peer_base = torch.tensor(bases, dtype=torch.int64, device=device)
    return [EpWorkspace(ws, r, num_experts, cols, cap_rows, cap_slots, layout, nbytes, bufs[r], bases, peer_base) for r in range(ws)]


class FlatPeers:
    """Peer address tables for the flat all-gather / reduce-scatter kernels over one symmetric buffer."""

    def __init__(self, group, nbytes: int, device, flag_slots: int = 64):
        import torch.distributed._symmetric_memory as symm_mem
        self.ws, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.flag_bytes = _align(flag_slots * self.ws * 4)
        self.nbytes = _align(nbytes) + self.flag_bytes
        self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group.group_name)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self.device = device
        self.epoch = 0

    def table(self, byte_offset: int) -> torch.Tensor:
        return torch.tensor([b + byte_offset for b in self.bases], dtype=torch.int64, device=self.device)


class PeerAllReduce:
    """Sum of bf16 / fp32 tensors over a group through peer memory: one kernel per call.

    Every rank copies its contribution into its half-buffer of the current parity, and one kernel announces that to
    the peers, waits for their announcements and adds up all ranks' buffers (`csrc/comm.cu::rs_block_kernel` with
    `all_reduce`).  Two parities make a second barrier unnecessary: a rank reaches call c + 2, which overwrites the
    buffer of call c, only after its kernel of call c + 1 has seen every peer announce call c + 1, and a peer
    announces call c + 1 after its own kernel of call c (which did all its reads) has finished, in stream order.
    Used for the partial sums of tensor-parallel experts (the reference's `dist.all_reduce`,
    megablocks_utils/config_utils.py:168-184).
    """

    _instances = {}

    def __init__(self, group, max_bytes: int, device):
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops import cuda_ops
        self.ext, self.cuda_ops = cuda_ops.ext, cuda_ops
        self.ws, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.half = _align(max_bytes)
        self.flag_bytes = _align(2 * self.ws * 4)
        self.nbytes = 2 * self.half + self.flag_bytes
        self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group.group_name)
        self.bases = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self.device = device
        self.calls = 0
        self.tables = [torch.tensor([b + par * self.half for b in self.bases], dtype=torch.int64, device=device) for par in (0, 1)]
        self.flag_table = torch.tensor([b + 2 * self.half for b in self.bases], dtype=torch.int64, device=device)

    @classmethod
    def for_group(cls, group, max_bytes: int, device):
        key = (group.group_name, torch.device(device).index)
        inst = cls._instances.get(key)
        if inst is None or inst.half < max_bytes:
            inst = cls._instances[key] = cls(group, max_bytes, device)
        return inst

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        nbytes = x.numel() * x.element_size()
        assert nbytes <= self.half and x.dtype in (torch.bfloat16, torch.float32)
        self.calls += 1
        par = self.calls & 1
        mine = self.buffer[par * self.half: par * self.half + nbytes].view(x.dtype).view(x.shape)
        mine.copy_(x)
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
        self.ext.rs_block(out.view(-1), self.tables[par], self.flag_table, self.bases[self.rank] + 2 * self.half, par, self.ws, self.rank,
                          x.dtype == torch.float32, 1.0, False, self.calls, self.cuda_ops.status_tensor(self.device), 0, True)
        return out
