"""Parameter sharding (ZeRO-3 / FSDP2 semantics) with block-wise recomputation.

The reference applies torch's `fully_shard` to every decoder block and to the
root module, wraps each block in an activation-checkpoint wrapper, and excludes
the MoE modules from sharding when they are expert-parallel
(train_accelerate_fsdp2.py:163-238).  This module provides the same behaviour
with explicit control over buffers and streams:

  * each unit (one decoder block; the root = embeddings + final norm + lm_head)
    keeps its dense parameters as one flat buffer, split evenly over the shard
    group; the flat shard is the `nn.Parameter` the optimizer sees
  * before a block runs, its full flat buffer is gathered (prefetched one block
    ahead on a side stream) and the modules' weights become views into it
  * a block's forward runs without a graph; its backward gathers again,
    recomputes the block, back-propagates, and reduce-scatters the flat gradient
    (scaled by 1/shard-group size, reduced over the replicate group for HSDP)
  * MoE parameters that are expert-parallel stay ordinary local parameters;
    their gradients get the data-parallel reductions the reference omits
    (router: mean over all ranks; experts: mean over expert replicas)

On a 2-D `(data_parallel, expert_parallel)` mesh the dense parameters are
sharded over the expert_parallel dim and replicated over data_parallel, which is
what passing that mesh to `fully_shard` does in the reference
(train_accelerate_fsdp2.py:141-160,187).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..models.mixtral import CausalLMOutput, MixtralForCausalLM, PackedBatch
from ..utils.metrics import nvtx_range
from . import collectives as coll

NVTX = os.environ.get("MDT_NVTX") == "1"


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _gemm_only_weight(qualname: str, p) -> bool:
    """Projection and expert weight matrices: read by nothing but the GEMM kernels' weight-operand loads."""
    if p.dim() != 2 or p.numel() < int(os.environ.get("MDT_GEMM_ONLY_MIN_NUMEL", 1 << 20)) or "lora_" in qualname:
        return False
    leaf = qualname.rsplit(".", 2)
    return qualname.endswith("_proj.weight") or (len(leaf) >= 2 and leaf[-1] in ("w1", "w2", "w3") and ".experts." in qualname)


class FlatParamGroup:
    """Parameters of one unit flattened into a single buffer sharded over `group`."""

    ALIGN = 128  # elements; keeps every rank's shard 256-byte aligned for bf16

    def __init__(self, entries, group, trainable: bool):
        # entries: list of (module, attribute name, parameter)
        self.group = group
        self.ws, self.rank = coll.group_size(group), coll.group_rank(group)
        self.trainable = trainable
        self.specs = []
        off = 0
        p0 = entries[0][2]
        self.dtype, self.device = p0.dtype, p0.device
        self.qualnames = []
        # Large matrices that are only ever read as the weight operand of a GEMM go to the back of the buffer;
        # everything else (norm weights, the router, adapters) comes first.  A gather with progress flags then
        # delivers the small front part first, and the GEMMs wait for their own part of the rest themselves.
        entries = sorted(entries, key=lambda e: 1 if _gemm_only_weight(e[3], e[2]) else 0)
        self.small_numel = 0
        for mod, name, p, qual in entries:
            if not _gemm_only_weight(qual, p):
                self.small_numel = off + _round_up(p.numel(), 8)
            self.specs.append((mod, name, tuple(p.shape), p.numel(), off))
            self.qualnames.append(qual)
            off += _round_up(p.numel(), 8)  # 16-byte aligned starts (bulk-copy friendly)
        self.numel = off
        self.padded = _round_up(off, self.ws * self.ALIGN)
        self.shard_numel = self.padded // self.ws
        lo, hi = self.rank * self.shard_numel, (self.rank + 1) * self.shard_numel
        shard = torch.zeros(self.shard_numel, dtype=self.dtype, device=self.device)
        with torch.no_grad():
            for (mod, name, shape, n, o), (_, _, p, _q) in zip(self.specs, entries):
                a, b = max(o, lo), min(o + n, hi)
                if a < b:
                    shard[a - lo:b - lo].copy_(p.detach().reshape(-1)[a - o:b - o])
                del mod._parameters[name]
                setattr(mod, name, None)
        self.shard = nn.Parameter(shard, requires_grad=trainable)
        self.full: Optional[torch.Tensor] = None
        self.acc: Optional[torch.Tensor] = None  # fp32 full-size local accumulation (sync_each_batch=False)

    def install(self, full: torch.Tensor, as_leaves: bool) -> List[torch.Tensor]:
        """Point the modules' weights at views of `full`.

        Trainable groups always get autograd-leaf views (harmless in graph-free forwards, needed by the
        recomputing backward); the views of every distinct buffer are built once and re-used, and
        nothing is done at all when the same buffer is already installed.
        """
        self.full = full
        key = full.data_ptr()
        cache = self.__dict__.setdefault("_view_cache", {})
        entry = cache.get(key)
        if entry is None:
            views, leaves = [], []
            for mod, name, shape, n, o in self.specs:
                v = full[o:o + n].view(shape)
                if self.trainable:
                    v = v.detach().requires_grad_(True)
                    leaves.append(v)
                views.append(v)
            entry = cache[key] = (views, leaves)
        if self.__dict__.get("_installed_key") != key:
            for (mod, name, shape, n, o), v in zip(self.specs, entry[0]):
                setattr(mod, name, v)
            self._installed_key = key
        return entry[1]

    def installed_leaves(self) -> List[torch.Tensor]:
        """Autograd-leaf views of the buffer that is currently installed (empty for frozen groups)."""
        if self.full is None:
            return []
        entry = self.__dict__.get("_view_cache", {}).get(self.full.data_ptr())
        return entry[1] if entry is not None else []

    def flat_grad(self, grads: List[Optional[torch.Tensor]], out: torch.Tensor) -> torch.Tensor:
        """Write per-parameter grads into the flat layout (zeros where a grad is missing)."""
        for (mod, name, shape, n, o), g in zip(self.specs, grads):
            if g is None:
                out[o:o + n].zero_()
            else:
                out[o:o + n].copy_(g.reshape(-1))
        return out


class FsdpUnit:
    def __init__(self, name: str, roots, group, exclude=()):
        # roots: list of (qualified prefix, module) whose parameters belong to this unit
        self.name = name
        excluded = set()
        for m in exclude:
            excluded.update(id(p) for p in m.parameters())
        train, frozen = [], []
        for prefix, root in roots:
            for mname, mod in root.named_modules():
                for pname, p in list(mod._parameters.items()):
                    if p is None or id(p) in excluded:
                        continue
                    qual = ".".join(x for x in (prefix, mname, pname) if x)
                    (train if p.requires_grad else frozen).append((mod, pname, p, qual))
        self.groups: List[FlatParamGroup] = []
        if train:
            self.groups.append(FlatParamGroup(train, group, True))
        if frozen:
            self.groups.append(FlatParamGroup(frozen, group, False))
        self.local_params = [p for m in exclude for p in m.parameters()]
        self.buffers: Optional[List[torch.Tensor]] = None   # gathered flat buffers currently held
        self.ready_event = None

    @property
    def trainable_group(self) -> Optional[FlatParamGroup]:
        for g in self.groups:
            if g.trainable:
                return g
        return None


class _BufferPool:
    """Round-robin pool of full-size flat buffers shared by the decoder-block units."""

    def __init__(self, sizes, dtype, device, slots: int):
        self.slots = [[torch.empty(s, dtype=dtype, device=device) for s in sizes] for _ in range(slots)]
        self.free_events = [None] * slots
        self.owner = [None] * slots
        self.next = 0

    def acquire(self, owner):
        for _ in range(len(self.slots)):
            i = self.next
            self.next = (self.next + 1) % len(self.slots)
            if self.owner[i] is None:
                self.owner[i] = owner
                return i
        raise RuntimeError("parameter buffer pool exhausted (a unit was not released)")

    def release(self, i, event):
        self.owner[i] = None
        self.free_events[i] = event

    def flags(self, slot, groups, ext):
        """Progress-flag tensors of the buffers of `slot` (one per group; created on first use).  A flag tensor belongs
        to a buffer, not to a unit: its epoch grows with every gather into that buffer."""
        store = self.__dict__.setdefault("_flags", {})
        out = []
        for j, g in enumerate(groups):
            key = (slot, j)
            if key not in store:
                # sized for the largest unit that can use the buffer: flags of a chunk layout never exceed one per 16 bytes
                n = max(int(ext.ag_chunks(g.ws, 16 * ((self.slots[slot][j].numel() * self.slots[slot][j].element_size() // g.ws + 15) // 16))[0]), 1)
                store[key] = {"ready": torch.zeros(n + g.ws, dtype=torch.int32, device=self.slots[slot][j].device), "epoch": 0}
            out.append(store[key])
        return out


class _LayerFn(torch.autograd.Function):
    """One decoder block: graph-free forward, recompute + backward + gradient reduction."""

    @staticmethod
    def forward(ctx, runner, idx, batch, x, *shards):
        ctx.runner, ctx.idx, ctx.batch = runner, idx, batch
        ctx.save_for_backward(x)
        layer = runner.model.model.layers[idx]
        layer._ckpt_mode = 1 if runner.stash_exchange else 0     # the MoE sub-block may keep its exchange results
        try:
            with torch.no_grad():
                return layer(x, batch)
        finally:
            layer._ckpt_mode = 0

    @staticmethod
    def backward(ctx, gout):
        runner: "ShardedMixtral" = ctx.runner
        idx, batch = ctx.idx, ctx.batch
        (x,) = ctx.saved_tensors
        unit = runner.units[idx]
        runner._acquire(idx, backward=True)
        runner._prefetch(idx - 1, backward=True)
        leaves = []
        for g, buf in zip(unit.groups, unit.buffers):
            leaves += g.install(buf, as_leaves=True)
        local = [p for p in unit.local_params if p.requires_grad]
        xin = x.detach().requires_grad_(True)
        layer = runner.model.model.layers[idx]
        layer._ckpt_mode = 2 if runner.stash_exchange else 0
        try:
            with torch.enable_grad():
                y = layer(xin, batch)
        finally:
            layer._ckpt_mode = 0
            layer._moe_stash = None
        grads = torch.autograd.grad(y, [xin] + leaves + local, gout, allow_unused=True)
        dx = grads[0]
        runner._reduce_unit_grads(unit, list(grads[1:1 + len(leaves)]))
        for p, g in zip(local, grads[1 + len(leaves):]):
            if g is not None:
                p.grad = g if p.grad is None else p.grad.add_(g)
        runner._release(idx)
        return (None, None, None, dx) + (None,) * (len(ctx.needs_input_grad) - 4)


class ShardedMixtral:
    """Runs a `MixtralForCausalLM` with sharded dense parameters and block recomputation.

    Installed as `model.layer_runner`; `model(input_ids, labels=...)` then goes
    through `embed` / `run_layer` / `head` below.
    """

    def __init__(self, model: MixtralForCausalLM, shard_group=None, replicate_group=None,
                 expert_dp_group=None, world_group=None, shard_experts: bool = False,
                 sync_each_batch: bool = False, pool_slots: int = 3, resident_params: Optional[bool] = None,
                 resident_limit_bytes: int = 16 << 30, recompute: bool = True, lazy_init=None):
        self.model = model
        self.shard_group, self.replicate_group = shard_group, replicate_group
        self.expert_dp_group, self.world_group = expert_dp_group, world_group
        self.sync_each_batch = sync_each_batch
        self.ws = coll.group_size(shard_group)
        self.rep = coll.group_size(replicate_group)
        layers = model.model.layers
        self.units: List[FsdpUnit] = []
        for i, layer in enumerate(layers):
            exclude = () if shard_experts else (layer.block_sparse_moe,)
            if lazy_init is not None:
                # blocks still on the meta device: create this block's tensors now; FlatParamGroup keeps the shard
                # and drops the rest before the next block is created
                from ..models.init import materialize_module
                materialize_module(layer, lazy_init[0], lazy_init[1], f"model.layers.{i}", std=lazy_init[2])
            self.units.append(FsdpUnit(f"layers.{i}", [(f"model.layers.{i}", layer)], shard_group, exclude))
        self.root = FsdpUnit("root", [("model.embed_tokens", model.model.embed_tokens),
                                      ("model.norm", model.model.norm), ("lm_head", model.lm_head)], shard_group)
        # register the flat shards so that model.parameters() / the optimizer see them
        shards = nn.ParameterList()
        for u in self.units + [self.root]:
            for g in u.groups:
                shards.append(g.shard)
        model._flat_shards = shards
        dev = next(p for p in model.parameters() if p.device.type != "meta").device
        self.device = dev
        self.is_cuda = dev.type == "cuda"
        # side streams get a high priority: their kernels are small and others wait for what they deliver
        self.comm_stream = torch.cuda.Stream(device=dev, priority=-1) if (self.is_cuda and self.ws > 1) else None
        self.rs_stream = torch.cuda.Stream(device=dev, priority=-1) if (self.is_cuda and self.ws > 1) else None
        self.pool = None
        self._last_microbatch = False
        self._rs_epoch = 0
        self._rs_events = []
        # MDT_FLAGGED_GATHER=0: the compute stream waits for a whole gather instead of the GEMMs waiting per chunk
        self.flagged_gather = os.environ.get("MDT_FLAGGED_GATHER", "1") != "0"
        # MDT_OVERLAP_RS=0: all gradient reduce-scatters after the last backward instead of block by block during it
        self.overlap_rs = os.environ.get("MDT_OVERLAP_RS", "1") != "0"
        # With 180 GB per GPU the gathered dense parameters of a Mixtral-8x7B (3.2 GB in bf16) can simply stay
        # resident: every rank keeps a full copy next to its shard and re-reads from its peers only the groups an
        # optimizer step has changed (ZeRO-2 style).  Frozen groups are gathered once per run instead of twice per
        # block per micro-batch.  Default: on when the full copies fit in `resident_limit_bytes`.
        full_bytes = sum(g.padded * g.shard.element_size() for u in self.units + [self.root] for g in u.groups)
        if os.environ.get("MDT_RESIDENT_LIMIT_GIB"):
            # e.g. 100 keeps even the experts of a no-EP run resident (93 GB in bf16 for Mixtral-8x7B): no per-block
            # gathers at all, at the price of a full parameter copy per GPU
            resident_limit_bytes = int(float(os.environ["MDT_RESIDENT_LIMIT_GIB"]) * (1 << 30))
        self.full_param_bytes = full_bytes
        if resident_params is None:
            resident_params = os.environ.get("MDT_RESIDENT_PARAMS", "1") != "0" and full_bytes <= resident_limit_bytes
        self.resident = bool(resident_params) and self.ws > 1
        self._param_version = 1
        self._frozen_version = 1
        # Block recomputation (the reference wraps every decoder block in an activation-checkpoint wrapper,
        # train_accelerate_fsdp2.py:206-224) is the default.  With `recompute=False` the blocks run under autograd
        # directly and keep their activations (a few GB per micro-batch for Mixtral-8x7B); that needs parameter
        # buffers that stay valid until the backward pass, i.e. resident copies or a single rank.
        self.recompute = bool(recompute) or not (self.resident or self.ws == 1)
        self._direct_units = set()
        # Recomputed blocks keep what their MoE sub-block received and got back in the first pass (~20 MB per block
        # and micro-batch, plus one receive-buffer copy under expert parallelism), so that the recomputation repeats
        # neither the token exchange nor the down projection.  MDT_STASH_EXCHANGE=0 recomputes everything.
        self.stash_exchange = os.environ.get("MDT_STASH_EXCHANGE", "1") != "0"
        if self.ws > 1 and self.resident:
            self.root_buffers = None
        elif self.ws > 1:
            n_groups = max(len(u.groups) for u in self.units)
            sizes = [max((u.groups[j].padded for u in self.units if len(u.groups) > j), default=0) for j in range(n_groups)]
            dts = self.units[0].groups[0].dtype
            self.pool = _BufferPool(sizes, dts, dev, pool_slots)
            self.root_buffers = [torch.empty(g.padded, dtype=g.dtype, device=dev) for g in self.root.groups]
        self._slot = {}
        self._root_leaves: List[torch.Tensor] = []
        self._grad_tmp = {}
        self.peers = None
        if self.is_cuda and self.ws > 1 and not sync_each_batch and os.environ.get("MDT_PEER_COLLECTIVES", "1") != "0":
            self._setup_peer_arena()
        model.layer_runner = self

    # ------------------------------------------------------------------ peer-memory arena
    def _setup_peer_arena(self):
        """Move every flat shard (and the fp32 gradient accumulators) into one symmetric buffer, so that the
        all-gather / reduce-scatter kernels of `csrc/comm.cu` can read the peers' copies directly."""
        from ..ops import cuda_ops
        from . import symm
        groups = [g for u in self.all_units() for g in u.groups]
        off = 0
        for g in groups:
            g.arena_shard_off = off
            off = symm._align(off + g.shard_numel * g.shard.element_size())
            if g.trainable:
                g.arena_acc_off = off
                off = symm._align(off + g.padded * 4)
        self.peers = symm.FlatPeers(self.shard_group, off, self.device, flag_slots=max(64, len(self.units) + 8))
        self._ext = cuda_ops.ext
        self._status = cuda_ops.status_tensor(self.device)
        buf = self.peers.buffer
        for g in groups:
            nb = g.shard_numel * g.shard.element_size()
            view = buf[g.arena_shard_off:g.arena_shard_off + nb].view(g.dtype)
            view.copy_(g.shard.data)
            g.shard.data = view
            g.shard_table = self.peers.table(g.arena_shard_off)
            if g.trainable:
                g.acc = buf[g.arena_acc_off:g.arena_acc_off + g.padded * 4].view(torch.float32)
                g.acc.zero_()
                g._acc_dirty = False
                g.acc_table = self.peers.table(g.arena_acc_off)
        self._flag_off = self.peers.nbytes - self.peers.flag_bytes
        self._flag_table = self.peers.table(self._flag_off)
        for i, u in enumerate(self.all_units()):
            u.flag_index = 1 + i                     # slot 0 belongs to the barrier
        self.peer_barrier()

    def peer_barrier(self):
        """Device-side barrier over the shard group (arrive on every peer's flag row, wait for all)."""
        if self.peers is None:
            return
        p = self.peers
        p.epoch += 1
        self._ext.barrier_arrive(self._flag_table, p.ws, p.rank, p.epoch)
        self._ext.barrier_wait(p.bases[p.rank] + self._flag_off, p.ws, p.epoch, self._status, 0)

    def invalidate_gathered(self):
        """Call after writing parameter shards by hand (checkpoint load): every resident copy is re-read."""
        self._param_version += 1
        self._frozen_version += 1
        if self.peers is not None:
            self.peer_barrier()

    def after_optimizer_step(self):
        """Peers must not gather a shard that its owner is still updating; resident copies of trainable groups
        are stale from here on."""
        self._param_version += 1
        self.peer_barrier()

    # ------------------------------------------------------------------ buffers
    def _gather_into(self, unit: FsdpUnit, buffers, flags=None):
        with nvtx_range("all_gather." + unit.name, NVTX):
            return self._gather_into_impl(unit, buffers, flags)

    def _gather_into_impl(self, unit: FsdpUnit, buffers, flags=None):
        """`flags` (one entry per group, None or a dict with the progress-flag tensor of the destination buffer): the
        gather publishes its progress there and returns what a consumer needs to wait on the small front part."""
        waits = []
        for j, (g, buf) in enumerate(zip(unit.groups, buffers)):
            if self.peers is not None:
                nbytes = g.shard_numel * g.shard.element_size()
                fl = flags[j] if flags is not None else None
                if fl is not None and g.small_numel < g.numel:
                    fl["epoch"] += 1
                    nflags, chunk_bytes = self._ext.ag_chunks(g.ws, nbytes)
                    cpr = nflags // g.ws
                    small = g.small_numel * g.shard.element_size()
                    last = ((small - 1) // nbytes) * cpr + ((small - 1) % nbytes) // chunk_bytes if small > 0 else -1
                    self._ext.ag_pull_flagged(buf[:g.padded], g.shard_table, g.ws, g.rank, nbytes, fl["ready"], fl["epoch"], last + 1)
                    waits.append((fl["ready"], last + 1, fl["epoch"]))
                else:
                    self._ext.ag_pull(buf[:g.padded], g.shard_table, g.ws, g.rank, nbytes)
                    waits.append(None)
            else:
                coll.all_gather_flat(buf[:g.padded], g.shard.data, g.group)
                waits.append(None)
        return waits

    def _start_gather(self, idx: int):
        """Issue the all-gather of unit idx (on the side stream when there is one)."""
        unit = self.units[idx]
        if unit.buffers is not None or idx in self._slot:
            return
        if self.ws == 1:
            unit.buffers = [g.shard.data for g in unit.groups]
            return
        if self.resident:
            self._refresh_resident(unit, side_stream=True)
            unit.buffers = unit.resident
            return
        slot = self.pool.acquire(idx)
        self._slot[idx] = slot
        bufs = self.pool.slots[slot][:len(unit.groups)]
        flags = None
        if self.peers is not None and self.flagged_gather and ops.get_backend() == "native":
            flags = self.pool.flags(slot, [g for g in unit.groups], self._ext)
        unit.flag_waits = None
        if self.comm_stream is not None:
            ev = self.pool.free_events[slot]
            # the shards may have just been written by the optimizer on the compute stream
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                if ev is not None:
                    self.comm_stream.wait_event(ev)
                waits = self._gather_into(unit, bufs, flags)
                unit.ready_event = torch.cuda.Event()
                unit.ready_event.record(self.comm_stream)
            if any(w is not None for w in waits):
                unit.flag_waits = waits
        else:
            self._gather_into(unit, bufs)
        unit.buffers = bufs

    def _refresh_resident(self, unit: FsdpUnit, side_stream: bool):
        """Bring the unit's resident full copies up to date: groups changed since their last gather are re-read."""
        if getattr(unit, "resident", None) is None:
            unit.resident = [torch.empty(g.padded, dtype=g.dtype, device=self.device) for g in unit.groups]
            unit.resident_version = [0] * len(unit.groups)
        want = [self._param_version if g.trainable else self._frozen_version for g in unit.groups]
        stale = [j for j in range(len(unit.groups)) if unit.resident_version[j] != want[j]]
        if not stale:
            return

        def gather():
            for j in stale:
                g, buf = unit.groups[j], unit.resident[j]
                if self.peers is not None:
                    self._ext.ag_pull(buf[:g.padded], g.shard_table, g.ws, g.rank, g.shard_numel * g.shard.element_size())
                else:
                    coll.all_gather_flat(buf[:g.padded], g.shard.data, g.group)
                unit.resident_version[j] = want[j]
        if side_stream and self.comm_stream is not None:
            # the shards may have just been written by the optimizer on the compute stream, and earlier work on
            # the compute stream may still read the copies that are about to be replaced
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.comm_stream):
                gather()
                unit.ready_event = torch.cuda.Event()
                unit.ready_event.record(self.comm_stream)
        else:
            gather()

    def _acquire(self, idx: int, backward: bool = False):
        unit = self.units[idx]
        self._start_gather(idx)
        if unit.ready_event is not None:
            waits = getattr(unit, "flag_waits", None)
            if waits is None:
                torch.cuda.current_stream().wait_event(unit.ready_event)
            else:
                # The compute stream does not wait for the gather: it waits (one small kernel) for the front part of
                # each flagged buffer, which every kernel may read, and the GEMMs wait for the chunks of their weight
                # operands themselves (csrc/gemm_sm100.cu: wait_b_tile), starting on what has arrived.
                for w in waits:
                    if w is not None and w[1] > 0:
                        self._ext.ag_wait_chunks(w[0], 0, w[1], w[2], self._status)
                # (a group gathered without flags, e.g. the adapters, is copied by an earlier kernel on the same side
                # stream than a flagged group that follows it, so a published chunk of the latter implies that the
                # former is complete; if no flagged group has a front part to wait for, or the flagged group comes
                # first, fall back to the event)
                last_plain = max((j for j, w in enumerate(waits) if w is None), default=-1)
                first_waited = min((j for j, w in enumerate(waits) if w is not None and w[1] > 0), default=None)
                if first_waited is None or last_plain > first_waited:
                    torch.cuda.current_stream().wait_event(unit.ready_event)
                unit.flag_waits = None
            unit.ready_event = None
        if not backward:
            for g, buf in zip(unit.groups, unit.buffers):
                g.install(buf, as_leaves=False)

    def _prefetch(self, idx: int, backward: bool = False):
        if 0 <= idx < len(self.units):
            self._start_gather(idx)

    def _release(self, idx: int):
        unit = self.units[idx]
        if self.ws == 1 or unit.buffers is None:
            unit.buffers = None if self.ws > 1 else unit.buffers
            return
        if self.resident:
            unit.buffers = None
            return
        ev = None
        if self.is_cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
        self.pool.release(self._slot.pop(idx), ev)
        unit.buffers = None

    # ------------------------------------------------------------------ gradients
    def begin_microbatch(self, is_last: bool):
        """Tell the runner whether the micro-batch about to run is the last one of its optimizer step.  In the last one
        every block's gradient reduce-scatter starts, on a side stream, as soon as that block's backward has finished
        (the reference's FSDP2 reduces inside backward too, train_accelerate_fsdp2.py:334-339), instead of all of them
        after the last backward."""
        self._last_microbatch = bool(is_last)
        if is_last:
            self._rs_epoch += 1

    def _reduce_unit_grads(self, unit: FsdpUnit, grads):
        g = unit.trainable_group
        if g is None:
            return
        scale = 1.0 / (self.ws * self.rep)
        if self.sync_each_batch or self.ws == 1:
            # double-buffered flat gradient: the reduction of one block runs on the side stream while the next block's
            # backward fills the other buffer
            key = (g.padded, g.dtype)
            ring = self._grad_tmp.get(key)
            if ring is None:
                n_buf = 2 if (self.rs_stream is not None and self.overlap_rs) else 1
                ring = self._grad_tmp[key] = {"bufs": [torch.zeros(g.padded, dtype=g.dtype, device=self.device) for _ in range(n_buf)],
                                              "events": [None] * n_buf, "next": 0}
            i = ring["next"]
            ring["next"] = (i + 1) % len(ring["bufs"])
            tmp = ring["bufs"][i]
            if ring["events"][i] is not None:
                torch.cuda.current_stream().wait_event(ring["events"][i])     # its previous reduction has read it
            g.flat_grad(grads, tmp)
            if g.shard.grad is None:
                g.shard.grad = torch.zeros_like(g.shard.data)
            if len(ring["bufs"]) > 1 and self.ws > 1:
                ready = torch.cuda.Event()
                ready.record(torch.cuda.current_stream())
                with torch.cuda.stream(self.rs_stream):
                    self.rs_stream.wait_event(ready)
                    coll.reduce_scatter_flat(g.shard.grad, tmp, g.group, scale=scale, accumulate=True)
                    done = torch.cuda.Event()
                    done.record(self.rs_stream)
                ring["events"][i] = done
                self._rs_events.append(done)
            else:
                coll.reduce_scatter_flat(g.shard.grad, tmp, g.group, scale=scale, accumulate=True)
        else:
            if g.acc is None:
                g.acc = torch.zeros(g.padded, dtype=torch.float32, device=self.device)
                g._acc_dirty = False
            views = g.__dict__.get("_acc_views")
            if views is None or g.__dict__.get("_acc_views_ptr") != g.acc.data_ptr():
                views = g._acc_views = [g.acc[o:o + n].view(shape) for (mod, name, shape, n, o) in g.specs]
                g._acc_views_ptr = g.acc.data_ptr()
            dst = [v for v, gr in zip(views, grads) if gr is not None]
            src = [gr for gr in grads if gr is not None]
            if dst:
                if self.is_cuda and ops.get_backend() == "native":
                    ops.cuda_ops_ext().multi_add(dst, src)      # one launch for the unit's gradients (fp32 += bf16)
                else:
                    torch._foreach_add_(dst, src)
            g._acc_dirty = True
            if self.peers is not None and self.overlap_rs and self._last_microbatch:
                self._reduce_block_now(unit, g, scale)

    def _reduce_block_now(self, unit: FsdpUnit, g: FlatParamGroup, scale: float):
        """Last micro-batch: this block's accumulator is final.  One kernel on the side stream announces that to the
        peers, waits for their announcements, reads their slices and writes the scaled, cast shard gradient, while the
        compute stream goes on with the next block's backward."""
        fresh = g.shard.grad is None
        if fresh:
            g.shard.grad = torch.empty_like(g.shard.data)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream())
        p = self.peers
        with torch.cuda.stream(self.rs_stream):
            self.rs_stream.wait_event(ready)
            self._ext.rs_block(g.shard.grad, g.acc_table, self._flag_table, p.bases[p.rank] + self._flag_off, unit.flag_index, g.ws, g.rank,
                               True, scale, not fresh, self._rs_epoch, self._status)
            done = torch.cuda.Event()
            done.record(self.rs_stream)
        self._rs_events.append(done)
        g._rs_done = True

    def reduce_gradients(self):
        """Finish the gradient reductions of one optimizer step (call after the last backward)."""
        scale = 1.0 / (self.ws * self.rep)
        for ev in self._rs_events:                       # reductions that ran beside the backward pass
            torch.cuda.current_stream().wait_event(ev)
        self._rs_events = []
        pending = [u.trainable_group for u in self.units + [self.root]
                   if u.trainable_group is not None and u.trainable_group.acc is not None
                   and getattr(u.trainable_group, "_acc_dirty", False) and not getattr(u.trainable_group, "_rs_done", False)]
        if self.peers is not None and pending:
            self.peer_barrier()          # every rank has finished adding into its accumulators
        for g in pending:
            if self.peers is not None:
                # read the peers' accumulators; scale, cast and write the shard gradient in one pass
                fresh = g.shard.grad is None
                if fresh:
                    g.shard.grad = torch.empty_like(g.shard.data)
                self._ext.rs_pull(g.shard.grad, g.acc_table, g.ws, g.rank, True, scale, not fresh)
            else:
                if g.shard.grad is None:
                    g.shard.grad = torch.zeros_like(g.shard.data)
                coll.reduce_scatter_flat(g.shard.grad, g.acc, g.group, scale=scale, accumulate=True)
        dirty = [u.trainable_group for u in self.units + [self.root]
                 if u.trainable_group is not None and u.trainable_group.acc is not None and getattr(u.trainable_group, "_acc_dirty", False)]
        if self.peers is not None and dirty:
            self.peer_barrier()          # every rank has finished reading before the accumulators are cleared
        for g in dirty:
            g.acc.zero_()
            g._acc_dirty = False
            g._rs_done = False
        self._last_microbatch = False
        for u in self.units + [self.root]:
            g = u.trainable_group
            if g is None:
                continue
            if self.rep > 1 and g.shard.grad is not None:
                coll.all_reduce_flat(g.shard.grad, self.replicate_group)
        # router: mean over all ranks; experts (and their LoRA factors): mean over expert replicas; adapter factors that
        # are whole on every tensor-parallel rank: first the sum of the ranks' partial gradients
        router_grads, expert_grads, tp_partial = [], [], {}
        for u in self.units:
            for p in u.local_params:
                if p.grad is None:
                    continue
                (expert_grads if getattr(p, "_is_expert_param", False) else router_grads).append(p.grad)
                tpg = getattr(p, "_tp_partial_grad_group", None)
                if tpg is not None:
                    tp_partial.setdefault(id(tpg), (tpg, []))[1].append(p.grad)
        for tpg, grads in tp_partial.values():
            _all_reduce_list(grads, tpg, 1.0)
        wg = self.world_group
        if router_grads and coll.group_size(wg) > 1:
            _all_reduce_list(router_grads, wg, 1.0 / coll.group_size(wg))
        if expert_grads and coll.group_size(self.expert_dp_group) > 1:
            _all_reduce_list(expert_grads, self.expert_dp_group, 1.0 / coll.group_size(self.expert_dp_group))

    # ------------------------------------------------------------------ model hooks
    def _install_root(self):
        root = self.root
        if self.ws == 1:
            bufs = [g.shard.data for g in root.groups]
        elif self.resident:
            self._refresh_resident(root, side_stream=False)
            bufs = root.resident
        else:
            bufs = self.root_buffers
            self._gather_into(root, bufs)
        need_grad = torch.is_grad_enabled()
        self._root_leaves = []
        for g, buf in zip(root.groups, bufs):
            self._root_leaves += g.install(buf, as_leaves=need_grad)

    def embed(self, ids):
        self._install_root()
        self._prefetch(0)
        return ops.embedding(ids, self.model.model.embed_tokens.weight)

    def run_layer(self, idx, layer, x, batch: PackedBatch):
        self._acquire(idx)
        self._prefetch(idx + 1)
        if torch.is_grad_enabled() and not self.recompute:
            # activations are kept: the block is part of the autograd graph; the gradients of its flat-parameter
            # views are collected in finish_microbatch()
            self._direct_units.add(idx)
            y = layer(x, batch)
            self._release(idx)
            return y
        if torch.is_grad_enabled():
            shards = [g.shard for g in self.units[idx].groups if g.trainable]
            local = [p for p in self.units[idx].local_params if p.requires_grad]
            y = _LayerFn.apply(self, idx, batch, x, *shards, *local)
        else:
            y = layer(x, batch)
        last = idx == len(self.units) - 1
        if not (last and torch.is_grad_enabled()):
            self._release(idx)
        return y

    def head(self, x, lab, batch, return_logits=False) -> CausalLMOutput:
        return self.model.head(x, lab, batch, return_logits)

    def finish_microbatch(self):
        """Collect the root unit's gradients after `loss.backward()`."""
        g = self.root.trainable_group
        if g is not None and self._root_leaves:
            grads = [leaf.grad for leaf in self._root_leaves]
            self._reduce_unit_grads(self.root, grads)
            for leaf in self._root_leaves:
                leaf.grad = None
        self._root_leaves = []
        for idx in sorted(self._direct_units, reverse=True):
            unit = self.units[idx]
            tg = unit.trainable_group
            if tg is not None:
                leaves = tg.installed_leaves()
                grads = [leaf.grad for leaf in leaves]
                if any(gr is not None for gr in grads):
                    self._reduce_unit_grads(unit, grads)
                for leaf in leaves:
                    leaf.grad = None
        self._direct_units.clear()
        for idx in list(self._slot):
            self._release(idx)

    def zero_grad(self):
        for p in self.model.parameters():
            p.grad = None

    # ------------------------------------------------------------------ unsharded views (checkpoint export)
    def full_state(self, unit: FsdpUnit, grads: bool = False):
        """Gathered {qualified name: tensor} of one unit's dense parameters (or their grads), on every rank."""
        out = {}
        for g in unit.groups:
            src = g.shard.data
            if grads:
                if not g.trainable:
                    continue
                src = g.shard.grad if g.shard.grad is not None else torch.zeros_like(g.shard.data)
            full = torch.empty(g.padded, dtype=src.dtype, device=g.device)
            coll.all_gather_flat(full, src.contiguous(), g.group)
            for (mod, name, shape, n, o), qual in zip(g.specs, g.qualnames):
                out[qual] = full[o:o + n].view(shape).clone()
        return out

    def all_units(self):
        return self.units + [self.root]


def _all_reduce_list(tensors, group, scale: float, bucket_bytes: int = 256 << 20):
    """Mean-reduce a list of gradients over `group`, in place and in their own dtype.

    Large tensors (expert weight gradients: 2.8 GB per layer in bf16) are reduced where they are; small ones are
    packed into buckets of at most `bucket_bytes` so that a model's few hundred router / adapter gradients cost a
    handful of collectives.  No full-size temporary exists at any time.
    """
    small = {}
    for t in tensors:
        nbytes = t.numel() * t.element_size()
        if nbytes >= bucket_bytes // 4 and t.is_contiguous():
            dist.all_reduce(t, group=group)
            if scale != 1.0:
                t.mul_(scale)
        else:
            small.setdefault(t.dtype, []).append(t)
    for dtype, items in small.items():
        bucket, size = [], 0
        def flush():
            if not bucket:
                return
            flat = torch.cat([b.reshape(-1) for b in bucket])
            dist.all_reduce(flat, group=group)
            if scale != 1.0:
                flat.mul_(scale)
            off = 0
            for b in bucket:
                n = b.numel()
                b.copy_(flat[off:off + n].view_as(b))
                off += n
        for t in items:
            nbytes = t.numel() * t.element_size()
            if bucket and size + nbytes > bucket_bytes:
                flush()
                bucket, size = [], 0
            bucket.append(t)
            size += nbytes
        flush()
