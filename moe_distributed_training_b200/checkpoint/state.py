"""Saving models (HF Mixtral safetensors, peft adapter files) and resumable training state.

The reference never writes a checkpoint from its FSDP2 script and has no mapping
from its expert layout back to HF keys (train_accelerate_fsdp2.py has no save;
accelerate.yaml:30 only configures FSDP1's FULL_STATE_DICT).  This module adds:

  save_model            HF-format export.  Every rank writes the experts it owns to
                        its own `model-rank{r}.safetensors`; rank 0 also writes the
                        gathered dense parameters and the merged index json.
  save_adapter          LoRA factors under peft's key names in `adapter_model.safetensors`
                        plus `adapter_config.json`.
  save/load_training_state   per-rank optimizer moments, scheduler and step counter.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch
import torch.distributed as dist
from safetensors.torch import load_file, save_file

from . import hf_safetensors as hfst


def _world():
    return (dist.get_rank(), dist.get_world_size()) if dist.is_initialized() else (0, 1)


def _gather_dense(engine) -> Dict[str, torch.Tensor]:
    out = {}
    for u in engine.runner.all_units():
        for name, t in engine.runner.full_state(u).items():
            out[name] = t
    return out


def _expert_ids(engine, moe):
    args = moe.args
    E = args.moe_num_experts
    if args.moe_expert_model_parallelism and args.expert_parallel_group is not None:
        r, n = dist.get_rank(args.expert_parallel_group), dist.get_world_size(args.expert_parallel_group)
        return list(range(r * (E // n), (r + 1) * (E // n)))
    return list(range(E))


def save_model(engine, out_dir: str):
    """Write the model in HF Mixtral safetensors layout (base weights; adapters go to save_adapter)."""
    rank, world = _world()
    os.makedirs(out_dir, exist_ok=True)
    dense = _gather_dense(engine)  # collective: every rank participates
    mine: Dict[str, torch.Tensor] = {}
    layers = engine.model.model.layers
    for i, layer in enumerate(layers):
        moe = layer.block_sparse_moe
        prefix = f"model.layers.{i}"
        if moe.router.layer.weight is None:
            # experts were sharded like dense parameters: rebuild the HF tensors from the gathered flat state
            E, F, H = moe.args.moe_num_experts, moe.args.ffn_hidden_size, moe.args.hidden_size
            if rank == 0:
                mine[f"{prefix}.block_sparse_moe.gate.weight"] = dense.pop(f"{prefix}.block_sparse_moe.router.layer.weight").cpu().contiguous()
                for w in ("w1", "w2", "w3"):
                    full = dense.pop(f"{prefix}.block_sparse_moe.experts.mlp.{w}").view(E, F, H)
                    for e in range(E):
                        t = full[e].t() if w == "w2" else full[e]
                        mine[f"{prefix}.block_sparse_moe.experts.{e}.{w}.weight"] = t.cpu().contiguous()
            continue
        if moe.args.tensor_parallel_size > 1:
            mine.update(_export_tp_layer(moe, prefix))
            continue
        ids = _expert_ids(engine, moe)
        dp_rank = dist.get_rank(engine.runner.expert_dp_group) if (engine.runner.expert_dp_group is not None) else 0
        if dp_rank == 0:  # one replica writes
            exp = hfst.export_moe_layer(moe, prefix, "block_sparse_moe", ids)
            if rank != 0:
                exp.pop(f"{prefix}.block_sparse_moe.gate.weight")
            mine.update(exp)
    files = {}
    if rank == 0:
        for name, t in dense.items():
            if "lora_" in name:
                continue
            mine[name] = t.cpu().contiguous()
    if mine:
        files[f"model-rank{rank:05d}.safetensors"] = mine
    wm = hfst.save_sharded(files, out_dir, write_index=False) if files else {}
    if world > 1:
        maps = [None] * world
        dist.all_gather_object(maps, wm)
        dist.barrier()
    else:
        maps = [wm]
    if rank == 0:
        hfst.merge_index(out_dir, maps)
        engine.model.config.save_pretrained(out_dir)
    if any("lora_" in n for n, _ in engine.model.named_parameters()) or any("lora_" in n for n in dense):
        save_adapter(engine, out_dir, dense)
    if world > 1:
        dist.barrier()


def _export_tp_layer(moe, prefix):
    """Tensor-parallel experts: gather the FFN slices over the group, group rank 0 writes."""
    args = moe.args
    group = args.tensor_parallel_group
    n, r = dist.get_world_size(group), dist.get_rank(group)
    E, Fl, H = args.moe_num_experts, moe.experts.mlp.features_per_rank, args.hidden_size
    out = {}
    for w in ("w1", "w2", "w3"):
        local = getattr(moe.experts.mlp, w).detach().view(E, Fl, H).contiguous()
        parts = [torch.empty_like(local) for _ in range(n)]
        dist.all_gather(parts, local, group=group)
        if r == 0 and dist.get_rank() == 0:
            full = torch.cat(parts, dim=1)
            for e in range(E):
                t = full[e].t() if w == "w2" else full[e]
                out[f"{prefix}.block_sparse_moe.experts.{e}.{w}.weight"] = t.cpu().contiguous()
    if r == 0 and dist.get_rank() == 0:
        out[f"{prefix}.block_sparse_moe.gate.weight"] = moe.router.layer.weight.detach().cpu().contiguous()
    return out


def _adapter_key(qualname: str) -> str:
    """peft's key for a parameter of this model (`...lora_A.default.weight` -> `base_model.model....lora_A.weight`)."""
    return "base_model.model." + qualname.replace(".default", "")


def save_adapter(engine, out_dir: str, dense: Dict[str, torch.Tensor] = None):
    """peft-style adapter files: one `adapter_model.safetensors` (written by rank 0) plus `adapter_config.json`.

    Expert adapters are stored per global expert: `...block_sparse_moe.experts.{e}.{w}.lora_A.weight` is `[r, in]`,
    `lora_B.weight` is `[out, r]`.  With expert parallelism every rank contributes the experts it owns (one replica
    of each); the pieces are collected on rank 0, so that the file does not depend on the sharding it was saved from.
    """
    rank, world = _world()
    os.makedirs(out_dir, exist_ok=True)
    dense = dense if dense is not None else _gather_dense(engine)
    tensors = {}
    if rank == 0:
        for name, t in dense.items():
            if "lora_" in name:
                tensors[_adapter_key(name)] = t.cpu().contiguous()
    mine = {}
    for i, layer in enumerate(engine.model.model.layers):
        moe = layer.block_sparse_moe
        lora = getattr(moe.experts, "lora", None)
        if lora is None:
            continue
        if moe.args.tensor_parallel_size > 1:
            raise NotImplementedError("saving expert adapters of tensor-parallel experts is not supported")
        dp_rank = dist.get_rank(engine.runner.expert_dp_group) if engine.runner.expert_dp_group is not None else 0
        if dp_rank != 0:
            continue
        ids = _expert_ids(engine, moe)
        for w in lora.lora_A:
            if lora.lora_A[w] is None:      # sharded like a dense parameter: saved with the flat state above
                continue
            A, B = lora.lora_A[w].detach(), lora.lora_B[w].detach()
            for j, e in enumerate(ids):
                base = f"base_model.model.model.layers.{i}.block_sparse_moe.experts.{e}.{w}"
                mine[f"{base}.lora_A.weight"] = A[j].t().cpu().contiguous()
                mine[f"{base}.lora_B.weight"] = B[j].t().cpu().contiguous()
    if world > 1:
        pieces = [None] * world if rank == 0 else None
        dist.gather_object(mine, pieces, dst=0)
        if rank == 0:
            for piece in pieces:
                tensors.update(piece)
    else:
        tensors.update(mine)
    if rank == 0:
        if tensors:
            save_file(tensors, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
        cfg = engine.model.peft_config["default"].to_dict() if hasattr(engine.model, "peft_config") else {}
        with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
            json.dump(cfg, f, indent=2)


def save_training_state(engine, out_dir: str, step: int):
    rank, _ = _world()
    os.makedirs(out_dir, exist_ok=True)
    params = [p for g in engine.optimizer.param_groups for p in g["params"]]
    state = {"step": step, "scheduler": engine.scheduler.state_dict(), "moments": [],
             "lrs": [g["lr"] for g in engine.optimizer.param_groups]}
    for p in params:
        st = engine.optimizer.state.get(p, {})
        state["moments"].append({k: (v.cpu() if torch.is_tensor(v) else v) for k, v in st.items()})
    state["params"] = [p.detach().cpu() for p in params]
    torch.save(state, os.path.join(out_dir, f"training_state-rank{rank:05d}.pt"))


def load_training_state(engine, in_dir: str) -> int:
    rank, _ = _world()
    state = torch.load(os.path.join(in_dir, f"training_state-rank{rank:05d}.pt"), map_location="cpu", weights_only=False)
    params = [p for g in engine.optimizer.param_groups for p in g["params"]]
    assert len(params) == len(state["params"]), "training state does not match this model / sharding"
    with torch.no_grad():
        for p, saved, st in zip(params, state["params"], state["moments"]):
            p.copy_(saved.to(p.device))
            if st:
                engine.optimizer.state[p] = {k: (v.to(p.device) if torch.is_tensor(v) else v) for k, v in st.items()}
    if hasattr(engine.runner, "invalidate_gathered"):
        engine.runner.invalidate_gathered()
    engine.scheduler.load_state_dict(state["scheduler"])
    for g, lr in zip(engine.optimizer.param_groups, state.get("lrs", [])):
        g["lr"] = lr
    engine.step_count = state["step"]
    return int(state["step"])


def load_adapter(engine, in_dir: str):
    """Load `adapter_model.safetensors` (as written by save_adapter or by peft) into the sharded model.

    Attention adapters live inside the flat parameter shards: each rank copies the slice it owns.  Expert adapters
    are re-stacked from the per-expert matrices into this rank's `[E_local, in, r]` / `[E_local, r, out]` tensors.
    Raises if an adapter parameter of the model has no tensor in the file, or a tensor in the file matches nothing
    (tensors of experts that other ranks own are expected and skipped).
    """
    path = os.path.join(in_dir, "adapter_model.safetensors")
    tensors = load_file(path)
    used, missing = set(), []
    with torch.no_grad():
        for u in engine.runner.all_units():
            for g in u.groups:
                lo, hi = g.rank * g.shard_numel, (g.rank + 1) * g.shard_numel
                for (mod, name, shape, n, o), qual in zip(g.specs, g.qualnames):
                    if "lora_" not in qual:
                        continue
                    key = _adapter_key(qual)
                    if key not in tensors:
                        missing.append(key)
                        continue
                    t = tensors[key]
                    if tuple(t.shape) != tuple(shape):
                        raise ValueError(f"{key}: file has shape {tuple(t.shape)}, the model needs {tuple(shape)}")
                    used.add(key)
                    a, b = max(o, lo), min(o + n, hi)
                    if a < b:
                        g.shard.data[a - lo:b - lo].copy_(t.reshape(-1)[a - o:b - o].to(g.shard.dtype))
        expert_keys_elsewhere = set()
        for i, layer in enumerate(engine.model.model.layers):
            moe = layer.block_sparse_moe
            lora = getattr(moe.experts, "lora", None)
            prefix = f"base_model.model.model.layers.{i}.block_sparse_moe.experts."
            if lora is None:
                continue
            if moe.args.tensor_parallel_size > 1:
                raise NotImplementedError("loading expert adapters into tensor-parallel experts is not supported")
            ids = _expert_ids(engine, moe)
            expert_keys_elsewhere.update(k for k in tensors if k.startswith(prefix))
            for w in lora.lora_A:
                A, B = lora.lora_A[w], lora.lora_B[w]
                if A is None:               # sharded like a dense parameter: loaded with the flat state above
                    continue
                for j, e in enumerate(ids):
                    for mat, suffix in ((A, "lora_A"), (B, "lora_B")):
                        key = f"{prefix}{e}.{w}.{suffix}.weight"
                        if key not in tensors:
                            missing.append(key)
                            continue
                        t = tensors[key].t()
                        if tuple(t.shape) != tuple(mat[j].shape):
                            raise ValueError(f"{key}: file has shape {tuple(tensors[key].shape)}, the model needs {tuple(mat[j].t().shape)}")
                        mat[j].copy_(t.to(mat.dtype))
                        used.add(key)
    unmatched = sorted(set(tensors) - used - expert_keys_elsewhere)
    if missing or unmatched:
        raise KeyError(f"adapter file {path} does not fit the model: missing {missing[:5]} ({len(missing)} in all), "
                       f"unmatched {unmatched[:5]} ({len(unmatched)} in all)")
    if hasattr(engine.runner, "invalidate_gathered"):
        engine.runner.invalidate_gathered()
    return []
