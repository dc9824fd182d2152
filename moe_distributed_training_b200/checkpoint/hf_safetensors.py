"""Hugging Face Mixtral safetensors <-> this framework's parameter layout.

On disk (unchanged from HF):
    model.layers.{L}.block_sparse_moe.gate.weight              [E, H]
    model.layers.{L}.block_sparse_moe.experts.{e}.w1.weight    [F, H]
    model.layers.{L}.block_sparse_moe.experts.{e}.w2.weight    [H, F]
    model.layers.{L}.block_sparse_moe.experts.{e}.w3.weight    [F, H]
In memory (same as the reference, megablocks_utils/shard_moe_utils.py:131-201):
    ...block_sparse_moe.router.layer.weight                     [E, H]      replicated
    ...block_sparse_moe.experts.mlp.w{1,2,3}                    [E_l*F_l, H] expert-major, w2 transposed

Differences from the reference's loader: a rank reads only the byte ranges of
the experts (and FFN slices) it owns instead of assembling the full `[E*F, H]`
tensor and scattering it, and the inverse mapping (save) exists.
"""
from __future__ import annotations

import json
import os
import re
from collections import defaultdict
from typing import Dict, Iterable, List, Optional, Tuple

import torch
from safetensors import safe_open
from safetensors.torch import save_file

FILE_SAFETENSOR_INDEX = "model.safetensors.index.json"
KEY_ROUTER = "router.layer.weight"
KEY_EXPERTS = "experts.mlp"
_EXPERT_RE = re.compile(r"(gate|experts)\.?(\d+)?\.?(\w+)?\.weight")


def read_weight_map(checkpoint_dir: str) -> Dict[str, str]:
    index = os.path.join(checkpoint_dir, FILE_SAFETENSOR_INDEX)
    if os.path.exists(index):
        with open(index) as f:
            return json.load(f)["weight_map"]
    single = os.path.join(checkpoint_dir, "model.safetensors")
    if os.path.exists(single):
        with safe_open(single, framework="pt") as f:
            return {k: "model.safetensors" for k in f.keys()}
    raise ValueError(f"no safetensors checkpoint found in {checkpoint_dir}")


def get_router_experts_sharded_safetensor(weight_map: Dict[str, str], prefix: str, instance_name: str,
                                          router_name: str = "gate", expert_name: str = "experts"):
    """Group the checkpoint keys of one MoE layer by destination parameter.

    Returns {KEY_ROUTER: [(key, file)], 'experts.mlp.w1': [(key, file) ordered by expert], ...}.
    Same contract as megablocks_utils/shard_moe_utils.py:70-125.
    """
    out: Dict[str, list] = defaultdict(list)
    pre = f"{prefix}.{instance_name}."
    for key, fname in weight_map.items():
        if not key.startswith(pre):
            continue
        rel = key[len(pre):]
        m = _EXPERT_RE.fullmatch(rel)
        if m is None:
            raise ValueError(f"unexpected key '{key}' under MoE module '{pre}'")
        kind, idx, wname = m.groups()
        if kind == router_name and idx is None:
            out[KEY_ROUTER].append((key, fname))
        elif kind == expert_name and idx is not None and wname in ("w1", "w2", "w3"):
            dest = out[f"{KEY_EXPERTS}.{wname}"]
            e = int(idx)
            while len(dest) <= e:
                dest.append(None)
            dest[e] = (key, fname)
        else:
            raise ValueError(f"unexpected key '{key}' under MoE module '{pre}'")
    if not out:
        raise ValueError(f"no checkpoint keys found for '{pre}'")
    for name, entries in out.items():
        if any(e is None for e in entries):
            raise ValueError(f"missing expert tensors for {pre}{name}")
    return dict(out)


class _Files:
    """Lazy cache of open safetensors handles."""

    def __init__(self, root: str):
        self.root, self.handles = root, {}

    def get(self, fname: str):
        if fname not in self.handles:
            self.handles[fname] = safe_open(os.path.join(self.root, fname), framework="pt", device="cpu").__enter__()
        return self.handles[fname]

    def close(self):
        for h in self.handles.values():
            h.__exit__(None, None, None)
        self.handles.clear()


def load_expert_shard(files: _Files, entries: List[Tuple[str, str]], wname: str, expert_ids: Iterable[int],
                      ffn_slice: Optional[slice], dtype: torch.dtype) -> torch.Tensor:
    """Read `[len(expert_ids) * F_l, H]` for one of w1/w2/w3 touching only the needed bytes."""
    parts = []
    for e in expert_ids:
        key, fname = entries[e]
        sl = files.get(fname).get_slice(key)
        if wname == "w2":  # stored [H, F] -> want [F, H]
            t = sl[:, ffn_slice] if ffn_slice is not None else sl[:, :]
            t = t.t()
        else:
            t = sl[ffn_slice, :] if ffn_slice is not None else sl[:, :]
        parts.append(t.to(dtype))
    return torch.cat(parts, dim=0).contiguous()


def load_moe_layer(moe_module, checkpoint_dir: str, weight_map: Dict[str, str], prefix: str, instance_name: str,
                   expert_ids: Iterable[int], ffn_slice: Optional[slice] = None, files: Optional[_Files] = None):
    """Fill one MoE layer (router + this rank's expert shard) from a checkpoint."""
    own = files is None
    files = files or _Files(checkpoint_dir)
    groups = get_router_experts_sharded_safetensor(weight_map, prefix, instance_name)
    with torch.no_grad():
        (key, fname), = groups[KEY_ROUTER]
        rw = moe_module.router.layer.weight
        rw.copy_(files.get(fname).get_tensor(key).to(rw.dtype))
        for wname in ("w1", "w2", "w3"):
            p = getattr(moe_module.experts.mlp, wname)
            t = load_expert_shard(files, groups[f"{KEY_EXPERTS}.{wname}"], wname, list(expert_ids), ffn_slice, p.dtype)
            assert t.shape == p.shape, f"{prefix}.{wname}: checkpoint {tuple(t.shape)} vs parameter {tuple(p.shape)}"
            p.copy_(t)
    if own:
        files.close()


def assign_mlp_v2_weights(dmoe, directory: str, settings: Dict[str, List[Tuple[str, str]]], device_mesh=None,
                          placements=None, parallize_tensor: bool = False):
    """Fill one MoE module from `settings`, the mapping `get_router_experts_sharded_safetensor` returns.

    Same call as the reference's function of this name (megablocks_utils/shard_moe_utils.py:131-201), which reads
    whole expert tensors on every rank, concatenates them and lets `distribute_tensor` scatter the shards.  Here a
    rank reads only its own byte ranges: with `parallize_tensor` the slice `[rank * F/n, (rank+1) * F/n)` of every
    expert's FFN dimension, otherwise the experts `[rank * E/n, (rank+1) * E/n)`, where rank and n come from the last
    dimension of `device_mesh` (or, without a mesh, from the module's expert-parallel / tensor-parallel group).
    `placements` is accepted for signature compatibility; the layout is implied by the module.
    """
    args = dmoe.args
    E = args.moe_num_experts
    group = None
    if device_mesh is not None:
        group = device_mesh.get_group(device_mesh.ndim - 1) if hasattr(device_mesh, "ndim") else device_mesh.get_group()
    elif parallize_tensor:
        group = args.tensor_parallel_group
    elif args.moe_expert_model_parallelism:
        group = args.expert_parallel_group
    import torch.distributed as dist
    n = dist.get_world_size(group) if group is not None else 1
    r = dist.get_rank(group) if group is not None else 0
    mlp = dmoe.experts.mlp
    if parallize_tensor:
        Fl = args.ffn_hidden_size // n
        expert_ids, ffn_slice = range(E), slice(r * Fl, (r + 1) * Fl)
    else:
        El = E // n
        expert_ids, ffn_slice = range(r * El, (r + 1) * El), None
    files = _Files(directory)
    with torch.no_grad():
        (key, fname), = settings[KEY_ROUTER]
        rw = dmoe.router.layer.weight
        rw.copy_(files.get(fname).get_tensor(key).to(rw.dtype))
        for wname in ("w1", "w2", "w3"):
            p = getattr(mlp, wname)
            t = load_expert_shard(files, settings[f"{KEY_EXPERTS}.{wname}"], wname, list(expert_ids), ffn_slice, p.dtype)
            assert t.shape == p.shape, f"{wname}: checkpoint shard {tuple(t.shape)} vs parameter {tuple(p.shape)}"
            p.copy_(t)
    files.close()


def load_dense(model, checkpoint_dir: str, weight_map: Optional[Dict[str, str]] = None, strict: bool = True):
    """Load every non-MoE parameter (names are identical to HF's)."""
    weight_map = weight_map or read_weight_map(checkpoint_dir)
    files = _Files(checkpoint_dir)
    missing = []
    with torch.no_grad():
        for name, p in model.named_parameters():
            if ".block_sparse_moe." in name or "lora_" in name:
                continue
            if name not in weight_map:
                missing.append(name)
                continue
            p.copy_(files.get(weight_map[name]).get_tensor(name).to(p.dtype))
    files.close()
    if strict and missing:
        raise ValueError(f"checkpoint is missing {missing[:5]}{'...' if len(missing) > 5 else ''}")
    return missing


def export_moe_layer(moe_module, prefix: str, instance_name: str, expert_ids: List[int],
                     ffn_slice: Optional[slice] = None) -> Dict[str, torch.Tensor]:
    """Inverse of `load_moe_layer` for the experts this rank owns (full FFN dim only)."""
    assert ffn_slice is None, "export gathers FFN slices before calling this"
    out = {}
    mlp = moe_module.experts.mlp
    F = mlp.features_per_rank
    base = f"{prefix}.{instance_name}"
    out[f"{base}.gate.weight"] = moe_module.router.layer.weight.detach().cpu().contiguous()
    for wname in ("w1", "w2", "w3"):
        w = getattr(mlp, wname).detach()
        for i, e in enumerate(expert_ids):
            t = w[i * F:(i + 1) * F]
            if wname == "w2":
                t = t.t()
            out[f"{base}.experts.{e}.{wname}.weight"] = t.cpu().contiguous()
    return out


def save_sharded(tensors_by_file: Dict[str, Dict[str, torch.Tensor]], out_dir: str, write_index: bool = True):
    """Write several safetensors files and the HF index json that points into them."""
    os.makedirs(out_dir, exist_ok=True)
    weight_map, total = {}, 0
    for fname, tensors in tensors_by_file.items():
        save_file(tensors, os.path.join(out_dir, fname), metadata={"format": "pt"})
        for k, t in tensors.items():
            weight_map[k] = fname
            total += t.numel() * t.element_size()
    if write_index:
        with open(os.path.join(out_dir, FILE_SAFETENSOR_INDEX), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": dict(sorted(weight_map.items()))}, f, indent=2)
    return weight_map


def merge_index(out_dir: str, partial_maps: List[Dict[str, str]]):
    """Combine the per-rank weight maps into one index json (rank 0 calls this after a gather)."""
    weight_map = {}
    for m in partial_maps:
        weight_map.update(m)
    total = 0
    for fname in set(weight_map.values()):
        total += os.path.getsize(os.path.join(out_dir, fname))
    with open(os.path.join(out_dir, FILE_SAFETENSOR_INDEX), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": dict(sorted(weight_map.items()))}, f, indent=2)
