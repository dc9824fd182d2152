"""Training engine: builds the sharded model and runs optimizer steps.

This is the public API both entry scripts, the benchmark and the tests use:

    engine = build_engine(cfg, ep_size=8, use_lora="none", ...)
    stats = engine.train_step(list_of_microbatches)

The construction order follows the reference's `main`
(train_accelerate_fsdp2.py:48-345): model -> shard_moe (mesh) -> LoRA ->
parameter sharding with block recomputation -> AdamW -> scheduler.  One
`train_step` is one optimizer step: `gradient_accumulation_steps` micro-batches
of forward/backward (loss divided by the number of micro-batches, as
accelerate's `backward` does), gradient reductions, optional clipping, AdamW,
scheduler tick.  Unlike the reference (see its `zero_grad` placement,
train_accelerate_fsdp2.py:416-422, and clipping after the step, :426-436) the
gradients of all micro-batches are kept and clipping acts before the update.
"""
from __future__ import annotations

import gc

import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh

from ..config import LoraConfig, MixtralConfig
from ..models.init import materialize_module
from ..models.mixtral import MixtralForCausalLM, moe_args_from_config
from ..moe.layer import dMoE
from ..optim.adamw import FusedAdamW
from ..optim.clip import clip_grad_norm_
from ..optim.schedulers import get_scheduler
from ..parallel.fsdp import ShardedMixtral
from ..parallel.shard_moe import (KEY_DATA_PARALLEL, KEY_EXPERT_PARALLEL, get_moe_kwargs, shard_moe)
from ..peft.lora import ATTENTION_TARGETS, get_peft_model
from ..utils.metrics import nvtx_range


NVTX = os.environ.get("MDT_NVTX") == "1"     # NVTX ranges per phase (also inside the C++-issued blocks)


def init_distributed(device_type: str = "cuda"):
    """Initialise torch.distributed from the torchrun environment; returns (rank, world, device)."""
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if device_type == "cuda":
        device = torch.device(f"cuda:{local}")
        torch.cuda.set_device(device)
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if device_type == "cuda":
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world)
    return rank, world, device


@dataclass
class Engine:
    model: MixtralForCausalLM
    runner: ShardedMixtral
    optimizer: FusedAdamW
    scheduler: object
    mesh: object
    device: torch.device
    rank: int
    world_size: int
    ep_size: int
    shard_group: object = None
    ep_group: object = None
    max_grad_norm: Optional[float] = None
    sort_microbatches: bool = True
    balance_microbatches: bool = True
    manage_gc: bool = True
    gc_every: int = 50
    step_count: int = 0
    last: dict = field(default_factory=dict)

    def to_device(self, mb: dict) -> dict:
        out = {}
        for k, v in mb.items():
            out[k] = v.to(self.device, non_blocking=True) if torch.is_tensor(v) else v
        return out

    def forward_backward(self, mb: dict, scale: float):
        mb = self.to_device(mb)
        out = self.model(mb["input_ids"], labels=mb["labels"], cu_seqlens=mb.get("cu_seqlens"),
                         max_seqlen=mb.get("max_seqlen"))
        (out.loss * scale).backward()
        self.runner.finish_microbatch()
        return out.loss.detach()

    def train_step(self, microbatches: List[dict]) -> dict:
        # A cyclic-garbage collection that starts in the middle of a step on one rank stalls every expert-parallel
        # peer at the next MoE layer.  Collection is therefore switched off while a step runs and done between
        # steps (generation 0 every step, a full collection every `gc_every` steps).
        gc_was_on = gc.isenabled()
        if self.manage_gc and gc_was_on:
            gc.disable()
        try:
            return self._train_step(microbatches)
        finally:
            if self.manage_gc and gc_was_on:
                gc.enable()
                gc.collect(2 if self.step_count % self.gc_every == 0 else 0)

    def _balance_across_ranks(self, microbatches: List[dict]) -> Optional[List[dict]]:
        """Re-deal the step's sequences over the ranks so that micro-batch i has nearly the same length on every rank.

        Expert-parallel ranks meet at every MoE layer, so micro-batch i costs all of them the time of the longest
        sequence any of them holds at position i; sorting each rank's own micro-batches leaves a spread of the order
        of +-20 % between the ranks' i-th longest.  Here the lengths of all ranks are gathered, the world x GA
        sequences are ranked by length, and position i of every rank is filled from ranks i*world ... (i+1)*world - 1
        of that list (in alternating rank order, which also evens out the ranks' token totals).  The sequences then
        change owners with one small all-to-all.  The set of sequences in the global batch, and therefore the
        averaged gradient, is unchanged.  Only for micro-batches of one sequence each (the reference's
        per_device_train_batch_size=1); returns None when that does not hold.
        """
        world, rank, ga = self.world_size, self.rank, len(microbatches)
        single = all(mb["input_ids"].dim() == 1 and mb.get("cu_seqlens") is not None and mb["cu_seqlens"].numel() == 2
                     and mb.get("labels") is not None for mb in microbatches)
        lens = torch.tensor([int(mb["input_ids"].numel()) for mb in microbatches], dtype=torch.int64, device=self.device)
        # every rank must take the same decision: it is taken on what all of them report
        mine = torch.tensor([ga, 1 if single else 0], dtype=torch.int64, device=self.device)
        everyone = torch.empty(2 * world, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(everyone, mine)
        everyone = everyone.view(world, 2).tolist()
        if any(g != ga or ok != 1 for g, ok in everyone):
            return None
        gathered = torch.empty(world * ga, dtype=torch.int64, device=self.device)
        dist.all_gather_into_tensor(gathered, lens)
        all_lens = gathered.view(world, ga).tolist()
        order = sorted(((all_lens[r][i], r, i) for r in range(world) for i in range(ga)), key=lambda t: (-t[0], t[1], t[2]))
        # owner[(src rank, src index)] = (dst rank, slot)
        plan = {}
        for slot in range(ga):
            chunk = order[slot * world:(slot + 1) * world]
            ranks = range(world) if slot % 2 == 0 else range(world - 1, -1, -1)
            for (n, r, i), dst in zip(chunk, ranks):
                plan[(r, i)] = (dst, slot, n)
        send = [[] for _ in range(world)]              # my sequences by destination, in slot order
        for i in range(ga):
            dst, slot, n = plan[(rank, i)]
            send[dst].append((slot, i))
        recv = [[] for _ in range(world)]              # (slot, length) of what each source sends me, in its send order
        for (r, i), (dst, slot, n) in plan.items():
            if dst == rank:
                recv[r].append((slot, n))
        for lst in send + recv:
            lst.sort()
        parts, in_splits = [], []
        for dst in range(world):
            n_dst = 0
            for slot, i in send[dst]:
                mb = microbatches[i]
                ids = mb["input_ids"].to(self.device, non_blocking=True).reshape(-1).long()
                lab = mb["labels"].to(self.device, non_blocking=True).reshape(-1).long()
                parts += [ids, lab]
                n_dst += 2 * ids.numel()
            in_splits.append(n_dst)
        out_splits = [2 * sum(n for _, n in recv[r]) for r in range(world)]
        flat_in = torch.cat(parts) if parts else torch.empty(0, dtype=torch.int64, device=self.device)
        flat_out = torch.empty(sum(out_splits), dtype=torch.int64, device=self.device)
        dist.all_to_all_single(flat_out, flat_in, output_split_sizes=out_splits, input_split_sizes=in_splits)
        result = [None] * ga
        off = 0
        for r in range(world):
            for slot, n in recv[r]:
                ids, lab = flat_out[off:off + n], flat_out[off + n:off + 2 * n]
                off += 2 * n
                result[slot] = {"input_ids": ids, "labels": lab,
                                "cu_seqlens": torch.tensor([0, n], dtype=torch.int32, device=self.device), "max_seqlen": n}
        return result if all(mb is not None for mb in result) else None

    def _train_step(self, microbatches: List[dict]) -> dict:
        ga = len(microbatches)
        balanced = None
        if self.world_size > 1 and self.sort_microbatches and self.balance_microbatches:
            balanced = self._balance_across_ranks(microbatches)
        if balanced is not None:
            microbatches = balanced              # position i: nearly the same length on every rank, longest first
        elif self.world_size > 1 and self.sort_microbatches:
            # Gradient accumulation does not depend on the order, so each rank at least runs its own micro-batches
            # longest first: ranks then work on sequences of similar length at the same time.
            microbatches = sorted(microbatches, key=lambda mb: -int(mb["input_ids"].numel()))
        loss_sum = None
        for i, mb in enumerate(microbatches):
            if hasattr(self.runner, "begin_microbatch"):
                self.runner.begin_microbatch(i == ga - 1)
            with nvtx_range(f"microbatch.{i}", NVTX):
                l = self.forward_backward(mb, 1.0 / ga)
            loss_sum = l if loss_sum is None else loss_sum + l
        with nvtx_range("reduce_gradients", NVTX):
            self.runner.reduce_gradients()
        grad_norm = None
        if self.max_grad_norm is not None and self.max_grad_norm > 0:
            with nvtx_range("grad_norm", NVTX):
                grad_norm = clip_grad_norm_(self.model, self.max_grad_norm, self.shard_group, self.ep_group, self.optimizer)
        with nvtx_range("optimizer", NVTX):
            self.optimizer.step()
        if hasattr(self.runner, "after_optimizer_step"):
            self.runner.after_optimizer_step()
        self.scheduler.step()
        self.optimizer.zero_grad(set_to_none=True)
        self.step_count += 1
        self.last = {"loss": loss_sum / ga, "grad_norm": grad_norm}
        return self.last

    @torch.no_grad()
    def eval_loss(self, mb: dict) -> torch.Tensor:
        mb = self.to_device(mb)
        return self.model(mb["input_ids"], labels=mb["labels"], cu_seqlens=mb.get("cu_seqlens"),
                          max_seqlen=mb.get("max_seqlen")).loss


def lora_targets(use_lora: str, expert_lora_ok: bool) -> Optional[List[str]]:
    """Target modules per `use_lora` (train_accelerate_fsdp2.py:242-289)."""
    if use_lora in (None, "none", False):
        return None
    if use_lora == "attn-only":
        return list(ATTENTION_TARGETS)
    if use_lora == "all":
        return list(ATTENTION_TARGETS) + ["experts"]
    if use_lora == "mlp-only":
        return ["experts"]
    raise ValueError(f"use_lora must be one of none, attn-only, all, mlp-only; got '{use_lora}'")


def build_engine(cfg: MixtralConfig, *, dtype: torch.dtype = torch.bfloat16, device_type: str = "cuda",
                 ep_size: Optional[int] = None, use_tp_sharding: bool = False, use_lora: str = "none",
                 lora_r: int = 16, lora_alpha: int = 16, learning_rate: float = 1e-5,
                 lr_scheduler_type: str = "linear", num_warmup_steps: int = 0, num_training_steps: int = 1000,
                 max_grad_norm: Optional[float] = 1.0, weight_decay: float = 0.01,
                 checkpoint: Optional[str] = None, seed: int = 0, mlp_impl: str = "sparse",
                 dispatch_impl: str = "auto", sync_each_batch: bool = False,
                 optimizer_state_dtype: Optional[torch.dtype] = None, ep_max_tokens: int = 4096,
                 activation_checkpointing: bool = True, resident_params: Optional[bool] = None) -> Engine:
    rank, world, device = init_distributed(device_type)
    ep_size = ep_size or 1
    if ep_size > 1 and world % ep_size != 0:
        raise ValueError("world_size must be a multiple of expert_degree")

    moe_args = moe_args_from_config(cfg, dtype, "meta")
    moe_args.mlp_impl, moe_args.dispatch_impl, moe_args.ep_max_tokens = mlp_impl, dispatch_impl, ep_max_tokens
    model = MixtralForCausalLM(cfg, moe_args, dtype=dtype, device="meta")

    mesh = None
    if world > 1 and ep_size > 1:
        kw = get_moe_kwargs(cfg, bf16=dtype == torch.bfloat16, fp16=dtype == torch.float16, mlp_impl=mlp_impl,
                            use_tensor_parallelism=use_tp_sharding)
        kw["dispatch_impl"], kw["ep_max_tokens"] = dispatch_impl, ep_max_tokens
        mesh = shard_moe(model, dMoE, checkpoint, rank, world, ep_size, kw, device_type=device_type,
                         parallize_tensor=use_tp_sharding, seed=seed)
    elif world > 1:
        mesh = init_device_mesh(device_type, (world,), mesh_dim_names=(KEY_DATA_PARALLEL,))
    targets = lora_targets(use_lora, True)
    # Without expert parallelism every rank would first hold the whole model (93 GB of bf16 for Mixtral-8x7B) only
    # to keep an eighth of it.  The decoder blocks then stay on the meta device here and the sharding layer creates
    # each block's tensors just before it cuts out its shard (same seeds per tensor name, so the same values).
    lazy_blocks = (world > 1 and ep_size <= 1 and checkpoint is None
                   and (targets is None or "experts" not in targets))
    if lazy_blocks:
        for prefix, mod in (("model.embed_tokens", model.model.embed_tokens), ("model.norm", model.model.norm), ("lm_head", model.lm_head)):
            materialize_module(mod, device, seed, prefix, std=cfg.initializer_range)
    else:
        materialize_module(model, device, seed, "", std=cfg.initializer_range)
    if checkpoint is not None:
        from ..checkpoint import hf_safetensors as hfst
        from ..parallel.shard_moe import get_resolved_checkpoint_location
        ckpt_dir = get_resolved_checkpoint_location(checkpoint)
        wm = hfst.read_weight_map(ckpt_dir)
        hfst.load_dense(model, ckpt_dir, wm)
        if not (world > 1 and ep_size > 1):
            for i, layer in enumerate(model.model.layers):
                hfst.load_moe_layer(layer.block_sparse_moe, ckpt_dir, wm, f"model.layers.{i}", "block_sparse_moe",
                                    range(cfg.num_local_experts))

    if targets is not None:
        get_peft_model(model, LoraConfig(r=lora_r, lora_alpha=lora_alpha, target_modules=targets),
                       adapter_dtype=dtype, seed=seed)

    shard_group = replicate_group = expert_dp_group = ep_group = None
    world_group = dist.group.WORLD if world > 1 else None
    shard_experts = False
    if mesh is not None:
        if mesh.ndim == 2:
            shard_group = mesh[KEY_EXPERT_PARALLEL].get_group()
            replicate_group = expert_dp_group = mesh[KEY_DATA_PARALLEL].get_group()
            ep_group = shard_group
        else:
            shard_group = mesh[KEY_DATA_PARALLEL].get_group()
            if ep_size > 1:
                ep_group = shard_group
            else:
                shard_experts = True  # no expert parallelism: experts are sharded like everything else
    if shard_experts and targets is None and not sync_each_batch:
        # full fine-tuning with the experts sharded like everything else: a full-size local gradient
        # accumulator would be 4 bytes x 46.7 G parameters, so gradients are reduce-scattered every micro-batch
        sync_each_batch = True
    runner = ShardedMixtral(model, shard_group, replicate_group, expert_dp_group, world_group,
                            shard_experts=shard_experts, sync_each_batch=sync_each_batch,
                            recompute=activation_checkpointing, resident_params=resident_params,
                            lazy_init=(device, seed, cfg.initializer_range) if lazy_blocks else None)
    params = [p for p in model.parameters() if p.requires_grad]
    opt = FusedAdamW(params, lr=learning_rate, weight_decay=weight_decay, state_dtype=optimizer_state_dtype)
    sched = get_scheduler(lr_scheduler_type, opt, num_warmup_steps, num_training_steps)
    eng = Engine(model, runner, opt, sched, mesh, device, rank, world, ep_size, shard_group, ep_group, max_grad_norm)
    # tensor-parallel peers share their batches, so sequences cannot change owners there
    eng.balance_microbatches = not use_tp_sharding and os.environ.get("MDT_BALANCE_MICROBATCHES", "1") != "0"
    return eng
