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

    def _train_step(self, microbatches: List[dict]) -> dict:
        ga = len(microbatches)
        if self.world_size > 1 and self.sort_microbatches:
            # Expert-parallel ranks meet at every MoE layer, so a micro-batch costs every rank the time of the
            # longest sequence among them.  Gradient accumulation does not depend on the order, so each rank runs
            # its micro-batches longest first: ranks then work on sequences of similar length at the same time.
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
                 activation_checkpointing: bool = True) -> Engine:
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
                            recompute=activation_checkpointing,
                            lazy_init=(device, seed, cfg.initializer_range) if lazy_blocks else None)
    params = [p for p in model.parameters() if p.requires_grad]
    opt = FusedAdamW(params, lr=learning_rate, weight_decay=weight_decay, state_dtype=optimizer_state_dtype)
    sched = get_scheduler(lr_scheduler_type, opt, num_warmup_steps, num_training_steps)
    return Engine(model, runner, opt, sched, mesh, device, rank, world, ep_size, shard_group, ep_group, max_grad_norm)
