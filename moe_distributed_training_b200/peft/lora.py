"""LoRA adapters for attention projections and for expert-parallel expert weights.

Attention: the reference hands `q_proj,k_proj,v_proj,o_proj` to peft
(train_accelerate_fsdp2.py:245-266); here `Linear.add_lora` creates parameters
with peft's names (`...q_proj.lora_A.default.weight [r, in]`,
`...lora_B.default.weight [out, r]`) so adapter files interchange.

Experts: the reference wraps megablocks' expert container in a peft `LoraLayer`
and publishes `_lora_pointers[name] = (A, B, r, alpha, hidden, ffn)` on it
(megablocks_utils/peft_utils.py:13-142); the grouped kernels then consume
`A:[E_l, in, r]`, `B:[E_l, r, out]` views (megablocks_utils/config_utils.py:37-61).
Here the adapters are stored directly in those compute shapes.  They work on the
1-D mesh (ep_size == world) as well as on the 2-D mesh.
"""
from __future__ import annotations

import math
from typing import Iterable, List

import torch
import torch.distributed as dist
import torch.nn as nn

from ..config import LoraConfig
from ..models.init import _seed_of
from ..models.mixtral import Linear
from ..moe.experts import SparseMLPv2
from ..moe.layer import ParallelDroplessMLP as _BaseParallelDroplessMLP

ARTIFACTS: dict = {}  # {'device_mesh': mesh}; kept for users of the reference's injection point

ATTENTION_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj")
EXPERT_TARGETS = ("w1", "w2", "w3")


class ExpertLoraAdapters(nn.Module):
    """Per-expert LoRA factors for w1, w2, w3 of one `SparseMLPv2`."""

    def __init__(self, mlp: SparseMLPv2, r: int, alpha: float, names: Iterable[str] = EXPERT_TARGETS, dtype=None,
                 seed: int = 0, tag: str = ""):
        super().__init__()
        E, F, H = mlp.experts_per_rank, mlp.features_per_rank, mlp.args.hidden_size
        F_full = mlp.args.ffn_hidden_size
        dev, dt = mlp.w1.device, dtype or mlp.w1.dtype
        self.r, self.alpha = r, alpha
        self.lora_A = nn.ParameterDict()
        self.lora_B = nn.ParameterDict()
        args = mlp.args
        ep_rank = 0
        if args.moe_expert_model_parallelism and args.expert_parallel_group is not None:
            ep_rank = dist.get_rank(args.expert_parallel_group)
        tp_rank = dist.get_rank(args.tensor_parallel_group) if args.tensor_parallel_size > 1 else 0
        for name in names:
            fin, fout = (F, H) if name == "w2" else (H, F)
            A = torch.empty(E, fin, r, dtype=dt, device=dev)
            if dev.type != "meta":
                # kaiming_uniform(a=sqrt(5)) on the [r, in] matrix of the unsharded expert, seeded per
                # global expert so that the values do not depend on the sharding
                fin_full = F_full if name == "w2" else H
                bound = 1.0 / math.sqrt(fin_full)
                for i in range(E):
                    full = seeded_uniform_(torch.empty(fin_full, r, dtype=dt, device=dev), bound, seed,
                                           f"{tag}.{ep_rank * E + i}.{name}.lora_A")
                    A[i].copy_(full[tp_rank * F:(tp_rank + 1) * F] if (name == "w2" and F != F_full) else full)
            self.lora_A[name] = nn.Parameter(A)
            self.lora_B[name] = nn.Parameter(torch.zeros(E, r, fout, dtype=dt, device=dev))
            self.lora_A[name]._is_expert_param = True
            self.lora_B[name]._is_expert_param = True
            if args.tensor_parallel_size > 1:
                # With tensor-parallel experts the factor on the hidden side (A of w1/w3, B of w2) is whole on every
                # rank and sees only that rank's slice of the FFN dim: its gradient is a partial sum over the group.
                whole = self.lora_B[name] if name == "w2" else self.lora_A[name]
                whole._tp_partial_grad_group = args.tensor_parallel_group
            mlp._lora_pointers[name] = (self.lora_A[name], self.lora_B[name], r, alpha, H, F)


class ParallelDroplessMLP(_BaseParallelDroplessMLP):
    """Name under which the reference exposes its expert LoRA wrapper (peft_utils.py:13)."""

    @staticmethod
    def wrap(experts: _BaseParallelDroplessMLP, r: int, alpha: float, names=EXPERT_TARGETS):
        return add_expert_lora(experts, r, alpha, names)


ParallelMLP = ParallelDroplessMLP  # tensor-parallel experts use the same adapter container


def seeded_uniform_(t: torch.Tensor, bound: float, seed: int, tag: str) -> torch.Tensor:
    gen = torch.Generator(device=t.device)
    gen.manual_seed(_seed_of(seed, tag))
    return t.uniform_(-bound, bound, generator=gen)


def add_expert_lora(experts: _BaseParallelDroplessMLP, r: int, alpha: float, names=EXPERT_TARGETS, dtype=None,
                    seed: int = 0, tag: str = ""):
    experts.lora = ExpertLoraAdapters(experts.mlp, r, alpha, names, dtype, seed, tag)
    for w in (experts.mlp.w1, experts.mlp.w2, experts.mlp.w3):
        w.requires_grad_(False)
    return experts


def get_peft_model(model: nn.Module, cfg: LoraConfig, adapter_dtype=None, seed: int = 0) -> nn.Module:
    """Freeze the base model and add LoRA to the modules named in `cfg.target_modules`.

    "experts" (or any of w1/w2/w3) in the target list adds per-expert adapters.
    """
    if cfg.lora_dropout != 0.0:
        raise ValueError("LoRA dropout is not supported by the fused kernels (reference: tests/test_scattermoe.py:110-113)")
    if cfg.bias != "none":
        raise ValueError("LoRA bias is not supported")
    for p in model.parameters():
        p.requires_grad_(False)
    targets = set(cfg.target_modules)
    expert_names = [n for n in EXPERT_TARGETS if n in targets] or (list(EXPERT_TARGETS) if "experts" in targets else [])
    for name, mod in model.named_modules():
        leaf = name.rsplit(".", 1)[-1]
        if isinstance(mod, Linear) and leaf in targets:
            mod.add_lora(cfg.r, cfg.lora_alpha, adapter_dtype)
            a = mod.lora_A["default"].weight
            if a.device.type != "meta":
                with torch.no_grad():
                    seeded_uniform_(a, 1.0 / math.sqrt(mod.in_features), seed, f"{name}.lora_A")
        elif isinstance(mod, _BaseParallelDroplessMLP) and expert_names:
            add_expert_lora(mod, cfg.r, cfg.lora_alpha, expert_names, adapter_dtype, seed, name)
    model.peft_config = {"default": cfg}
    return model


def lora_parameters(model: nn.Module) -> List[nn.Parameter]:
    return [p for n, p in model.named_parameters() if "lora_" in n]


def prepare_peft(model, peft_config: LoraConfig, bf16: bool = True, gradient_checkpointing: bool = True,
                 gradient_checkpointing_kwargs=None, autocast_adapter_dtype: bool = False):
    """Counterpart of the reference's `prepare_peft` (utils.py:14-89).

    The k-bit and input-require-grads handling there exists for HF/peft internals;
    block recomputation here does not need inputs that require grad.  Adapters are
    created in bf16 when `bf16` (the reference casts them afterwards, utils.py:76-87).
    """
    dt = torch.bfloat16 if (bf16 and not autocast_adapter_dtype) else None
    return get_peft_model(model, peft_config, adapter_dtype=dt)
