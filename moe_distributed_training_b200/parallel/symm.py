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
