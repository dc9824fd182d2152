"""Expert-parallel / tensor-parallel sharding of the MoE layers of a model.

Same entry point and return value as the reference's `shard_moe`
(megablocks_utils/shard_moe_utils.py:203-323): build the `ep x dp` DeviceMesh,
replace every MoE module by one that owns only this rank's experts (EP) or this
rank's slice of every expert's FFN dimension (TP), fill it from the HF
safetensors checkpoint, and return the mesh.

Mesh rules (shard_moe_utils.py:224-248):
  dp_size = world_size // ep_size
  dp_size == 1 -> 1-D mesh ("data_parallel",) of size ep; the EP group is that dim
  otherwise    -> 2-D mesh ("data_parallel", "expert_parallel") of shape (dp, ep)

Rank r of the EP group owns experts [r*E_l, (r+1)*E_l) because the expert-major
`[E*F, H]` tensor is split on dim 0.
"""
from __future__ import annotations

import os
from typing import Optional, Type

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from ..checkpoint import hf_safetensors as hfst
from ..config import MoEArguments
from ..models.init import init_moe_
from ..moe.layer import dMoE

KEY_DATA_PARALLEL = "data_parallel"
KEY_EXPERT_PARALLEL = "expert_parallel"
DIM_EXPERT = 0
KEY_ROUTER = hfst.KEY_ROUTER
KEY_EXPERTS = hfst.KEY_EXPERTS
FILE_SAFETENSOR_INDEX = hfst.FILE_SAFETENSOR_INDEX


def get_moe_kwargs(config, has_bias: bool = False, fp16: bool = False, bf16: bool = False,
                   mlp_impl: str = "sparse", use_tensor_parallelism: bool = False) -> dict:
    """Model config -> MoE layer kwargs (megablocks_utils/shard_moe_utils.py:26-46)."""
    return {
        "hidden_size": config.hidden_size,
        "ffn_hidden_size": config.intermediate_size,
        "moe_num_experts": config.num_local_experts,
        "moe_top_k": config.num_experts_per_tok,
        "moe_expert_model_parallelism": not use_tensor_parallelism,
        "memory_optimized_mlp": False,
        "bias": has_bias,
        "moe_normalize_expert_weights": True,
        "fp16": fp16,
        "bf16": bf16,
        "mlp_impl": mlp_impl,
    }


def get_resolved_checkpoint_location(name_or_path: str, revision: str = "main") -> str:
    """Directory holding the checkpoint files.

    A local directory is returned as is; a hub id is looked up in the local HF
    cache (no download: there may be no network).  The snapshot is the one that
    `refs/<revision>` names (what `from_pretrained` resolves, and so what the
    reference obtains by hooking config loading, megablocks_utils/shard_moe_utils.py:50-63);
    `revision` may also be a commit hash.  Without a matching ref the only
    snapshot present is taken; several snapshots and no ref is an error.
    """
    if os.path.isdir(name_or_path):
        return name_or_path
    cache = os.environ.get("HF_HUB_CACHE") or os.path.join(
        os.environ.get("HF_HOME", os.path.expanduser("~/.cache/huggingface")), "hub")
    root = os.path.join(cache, "models--" + name_or_path.replace("/", "--"))
    repo = os.path.join(root, "snapshots")
    if os.path.isdir(repo):
        ref = os.path.join(root, "refs", revision)
        if os.path.isfile(ref):
            with open(ref) as f:
                commit = f.read().strip()
            if os.path.isdir(os.path.join(repo, commit)):
                return os.path.join(repo, commit)
        if os.path.isdir(os.path.join(repo, revision)):
            return os.path.join(repo, revision)
        snaps = sorted(os.listdir(repo))
        if len(snaps) == 1:
            return os.path.join(repo, snaps[0])
        if snaps:
            raise ValueError(f"checkpoint '{name_or_path}': {len(snaps)} cached snapshots and no refs/{revision}; pass a directory")
    raise ValueError(f"checkpoint '{name_or_path}' is neither a directory nor in the local HF cache")


def build_mesh(world_size: int, ep_size: int, device_type: str,
               key_dp: str = KEY_DATA_PARALLEL, key_ep: str = KEY_EXPERT_PARALLEL):
    """Returns (mesh, name of the EP dim, placements of the expert tensors)."""
    from torch.distributed.tensor import Replicate, Shard
    assert world_size % ep_size == 0, "world_size must be divisible by ep_size"
    dp_size = world_size // ep_size
    if dp_size == 1:
        mesh = init_device_mesh(device_type, (ep_size,), mesh_dim_names=(key_dp,))
        return mesh, key_dp, [Shard(DIM_EXPERT)]
    mesh = init_device_mesh(device_type, (dp_size, ep_size), mesh_dim_names=(key_dp, key_ep))
    return mesh, key_ep, [Replicate(), Shard(DIM_EXPERT)]


def _find_moe_modules(model: nn.Module, moe_cls):
    found = []
    for name, mod in model.named_modules():
        if isinstance(mod, moe_cls):
            parent_name, _, child = name.rpartition(".")
            found.append((parent_name, child, mod))
    return found


def _slice_from_module(old: dMoE, new: dMoE, expert_ids, ffn_slice, F_full: int):
    """Initialise `new` from an already materialised unsharded MoE module."""
    with torch.no_grad():
        new.router.layer.weight.copy_(old.router.layer.weight)
        H = old.args.hidden_size
        for wname in ("w1", "w2", "w3"):
            w = getattr(old.experts.mlp, wname).view(-1, F_full, H)[list(expert_ids)]
            if ffn_slice is not None:
                w = w[:, ffn_slice]
            getattr(new.experts.mlp, wname).copy_(w.reshape(-1, H))


def shard_moe(model: nn.Module, moe_cls: Type = dMoE, checkpoint_name_or_path: Optional[str] = None,
              rank: int = 0, world_size: int = 1, ep_size: Optional[int] = None, moe_kwargs: Optional[dict] = None,
              device_type: str = "cuda", key_dp: str = KEY_DATA_PARALLEL, key_ep: str = KEY_EXPERT_PARALLEL,
              parallize_tensor: bool = False, seed: int = 0) -> DeviceMesh:
    """Shard the experts of every `moe_cls` module of `model` over `ep_size` ranks.

    parallize_tensor=False: expert parallelism, rank owns E/ep whole experts.
    parallize_tensor=True : tensor parallelism, rank owns F/ep columns of every expert.
    """
    ep_size = ep_size or world_size
    assert ep_size > 1, "expert/tensor sharding needs ep_size > 1"
    moe_kwargs = dict(moe_kwargs or {})
    if device_type == "cuda":
        local = int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
        device = torch.device(f"cuda:{local}")
    else:
        device = torch.device(device_type)

    mesh, ep_dim, placements = build_mesh(world_size, ep_size, device_type, key_dp, key_ep)
    if parallize_tensor and mesh.ndim != 2:
        raise ValueError("tensor-parallel experts need ep_size < world_size (a 2-D mesh)")
    group = mesh[ep_dim].get_group()
    ep_rank = dist.get_rank(group)

    found = _find_moe_modules(model, moe_cls)
    if not found:
        raise ValueError(f"no modules of type {moe_cls.__name__} in the model")
    E = moe_kwargs.get("moe_num_experts", found[0][2].args.moe_num_experts)
    F_full = moe_kwargs.get("ffn_hidden_size", found[0][2].args.ffn_hidden_size)
    if not parallize_tensor and E % ep_size != 0:
        raise ValueError(f"{E} experts cannot be split over ep_size={ep_size}")

    weight_map, ckpt_dir, files = None, None, None
    if checkpoint_name_or_path is not None:
        ckpt_dir = get_resolved_checkpoint_location(checkpoint_name_or_path)
        weight_map = hfst.read_weight_map(ckpt_dir)
        files = hfst._Files(ckpt_dir)

    for parent_name, child, old in found:
        base = dict(vars(old.args)) if isinstance(getattr(old, "args", None), MoEArguments) else {}
        base.update({k: v for k, v in moe_kwargs.items() if k in MoEArguments.__dataclass_fields__})
        base["device"] = device
        if parallize_tensor:
            base.update(moe_expert_model_parallelism=False, expert_parallel_group=None,
                        tensor_parallel_group=group, tensor_parallel_size=ep_size)
            expert_ids = range(E)
            Fl = F_full // ep_size
            ffn_slice = slice(ep_rank * Fl, (ep_rank + 1) * Fl)
        else:
            base.update(moe_expert_model_parallelism=True, expert_parallel_group=group,
                        tensor_parallel_group=None, tensor_parallel_size=1)
            E_l = E // ep_size
            expert_ids = range(ep_rank * E_l, (ep_rank + 1) * E_l)
            ffn_slice = None
        args = MoEArguments(**base)
        new = dMoE(args)
        try:
            if weight_map is not None:
                hfst.load_moe_layer(new, ckpt_dir, weight_map, parent_name, child, expert_ids, ffn_slice, files)
            elif old.router.layer.weight.device.type != "meta":
                _slice_from_module(old, new, expert_ids, ffn_slice, F_full)
            else:
                init_moe_(new, seed, f"{parent_name}.{child}", expert_ids, ffn_slice, F_full)
        except Exception as exc:  # noqa: BLE001
            raise ValueError(f"failed to shard MoE module '{parent_name}.{child}': {exc}") from exc
        new._ep_mesh, new._ep_placements = mesh, placements
        for p in new.experts.parameters():
            p._is_expert_param = True
        new.train(old.training)
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, child, new)
    if files is not None:
        files.close()
    return mesh
