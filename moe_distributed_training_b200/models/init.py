"""Deterministic materialisation of meta-device modules.

A 47 B-parameter model is first built on the meta device; each rank then
creates only the tensors it owns.  Every tensor (and every expert inside the
expert-major MoE weights) gets its own generator seed derived from its name, so
the values do not depend on the sharding: an expert has the same weights whether
one rank owns all experts or eight ranks own one each.  That property is what the
EP-vs-unsharded equivalence tests rely on.
"""
from __future__ import annotations

import zlib
from typing import Optional

import torch
import torch.nn as nn


def _seed_of(seed: int, tag: str) -> int:
    return (seed * 1000003 + zlib.crc32(tag.encode())) % (2 ** 31 - 1)


def seeded_normal_(t: torch.Tensor, std: float, seed: int, tag: str) -> torch.Tensor:
    gen = torch.Generator(device=t.device)
    gen.manual_seed(_seed_of(seed, tag))
    if t.dtype in (torch.float32, torch.bfloat16, torch.float16):
        t.normal_(0.0, std, generator=gen)
    else:
        t.copy_(torch.empty(t.shape, dtype=torch.float32, device=t.device).normal_(0.0, std, generator=gen))
    return t


@torch.no_grad()
def init_moe_(moe, seed: int, layer_name: str, expert_ids, ffn_slice: Optional[slice], F_full: int):
    """Fill a (possibly sharded) dMoE: router + the listed experts' (sliced) weights."""
    args = moe.args
    H = args.hidden_size
    seeded_normal_(moe.router.layer.weight, args.init_std, seed, f"{layer_name}.router")
    mlp = moe.experts.mlp
    Fl = mlp.features_per_rank
    for wname in ("w1", "w2", "w3"):
        p = getattr(mlp, wname)
        for i, e in enumerate(expert_ids):
            dst = p[i * Fl:(i + 1) * Fl]
            if ffn_slice is None:
                seeded_normal_(dst, args.init_std, seed, f"{layer_name}.experts.{e}.{wname}")
            else:
                full = torch.empty(F_full, H, device=p.device, dtype=p.dtype)
                seeded_normal_(full, args.init_std, seed, f"{layer_name}.experts.{e}.{wname}")
                dst.copy_(full[ffn_slice])


@torch.no_grad()
def materialize_module(module: nn.Module, device, seed: int, prefix: str, std: float = 0.02):
    """Replace meta parameters of `module` (recursively) by initialised tensors on `device`."""
    from ..moe.layer import dMoE
    for name, sub in module.named_modules():
        full_name = ".".join(x for x in (prefix, name) if x)
        if isinstance(sub, dMoE):
            if sub.router.layer.weight.device.type == "meta":
                args = sub.args
                args.device = device
                old_r = sub.router.layer.weight
                sub.router.layer.weight = nn.Parameter(torch.empty_like(old_r, device=device), requires_grad=old_r.requires_grad)
                for wname in ("w1", "w2", "w3"):
                    old = getattr(sub.experts.mlp, wname)
                    setattr(sub.experts.mlp, wname, nn.Parameter(torch.empty_like(old, device=device), requires_grad=old.requires_grad))
                init_moe_(sub, seed, full_name, range(args.moe_num_experts), None, args.ffn_hidden_size)
            continue
        for pname, p in list(sub._parameters.items()):
            if p is None or p.device.type != "meta":
                continue
            if ".block_sparse_moe" in full_name:
                continue
            t = torch.empty_like(p, device=device)
            tag = f"{full_name}.{pname}"
            if tag.endswith("layernorm.weight") or tag.endswith("model.norm.weight") or tag.endswith(".norm.weight"):
                t.fill_(1.0)
            elif "lora_B" in tag:
                t.zero_()
            elif ".lora_A." in tag:
                # adapter created on the meta device: the same seeded kaiming-uniform values that
                # `peft.lora.get_peft_model` gives an adapter created on a real device
                gen = torch.Generator(device=t.device)
                gen.manual_seed(_seed_of(seed, tag.split(".lora_A.")[0] + ".lora_A"))
                bound = 1.0 / (t.shape[-1] ** 0.5)
                t.uniform_(-bound, bound, generator=gen)
            else:
                seeded_normal_(t, std, seed, tag)
            sub._parameters[pname] = nn.Parameter(t, requires_grad=p.requires_grad)
    return module
