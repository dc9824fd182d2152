"""The training program behind both entry scripts.

Flag names, defaults and validation follow the reference's `main`
(train_accelerate_fsdp2.py:48-65,117-138,268-272); the metric lines keep its keys
(`epoch, loss, learning_rate, gpu_mem_used_now, gpu_mem_used_peak, grad_norm`,
then `train_runtime, train_steps_per_second`, :439-471) and add tokens/s timed
on the device (maximum over ranks).  Data: a JSON/JSONL file whose records have an
`output` field holding the formatted prompt + response (:87-96) when a tokenizer
is available locally, otherwise synthetic instruction-shaped sequences.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from ..config import MixtralConfig
from ..data.collator import DataCollatorForCompletionOnlyLM
from ..data.synthetic import SyntheticInstructionDataset, collate_packed
from ..utils.metrics import DeviceTimer, log_json, max_over_ranks, memory_stats, sum_over_ranks
from .engine import build_engine

MODEL_NAME = "mistralai/Mixtral-8x7B-Instruct-v0.1"


def validate_flags(use_megablocks_sharding, use_scattermoe, use_tp_sharding, use_lora, world_size, expert_degree):
    """Flag rules of the reference (train_accelerate_fsdp2.py:117-138,268-272)."""
    if use_scattermoe and not (use_megablocks_sharding or use_tp_sharding):
        raise ValueError("use_scattermoe=True only works with use_megablocks_sharding or use_tp_sharding")
    if use_megablocks_sharding and use_tp_sharding:
        raise ValueError("choose one of use_megablocks_sharding and use_tp_sharding")
    if use_lora not in ("none", "attn-only", "all", "mlp-only"):
        raise ValueError("use_lora must be one of none, attn-only, all, mlp-only")
    if use_megablocks_sharding or use_tp_sharding:
        if expert_degree is None:
            expert_degree = world_size
        if world_size % expert_degree != 0:
            raise ValueError("expert_degree must divide the number of processes")
        if use_tp_sharding and expert_degree == world_size and world_size > 1:
            raise ValueError("use_tp_sharding needs expert_degree < number of processes (a 2-D mesh)")
    else:
        expert_degree = 1
    return expert_degree


def _resolve_config(model_name_or_path: Optional[str], preset: str) -> (MixtralConfig, Optional[str]):
    if model_name_or_path:
        from ..parallel.shard_moe import get_resolved_checkpoint_location
        try:
            path = get_resolved_checkpoint_location(model_name_or_path)
            if os.path.exists(os.path.join(path, "config.json")):
                return MixtralConfig.from_pretrained(path), path
        except ValueError:
            pass   # neither a directory nor a cached hub id: random init of the preset (a tokenizer-only directory too)
    return (MixtralConfig.tiny() if preset == "tiny" else MixtralConfig.mixtral_8x7b()), None


def _load_text_dataset(path: str, tokenizer_path: str, max_seq_length: int) -> Optional[List[dict]]:
    """Tokenise `output` fields; returns None when no tokenizer can be loaded offline."""
    if not os.path.exists(path):
        return None
    try:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(tokenizer_path, model_max_length=max_seq_length, local_files_only=True)
    except Exception:  # noqa: BLE001
        return None
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    with open(path) as f:
        text = f.read().strip()
    records = json.loads(text) if text.startswith("[") else [json.loads(l) for l in text.splitlines() if l.strip()]
    # Two record layouts: {"output": full text with " ### Response"} (train_accelerate_fsdp2.py:85-101) and alpaca
    # records {"instruction", "output"}, which the FSDP1 script formats itself and masks up to " ### Answer:"
    # (train_fsdp1.py:49-61).
    alpaca = bool(records) and "instruction" in records[0]
    template = tok.encode(" ### Answer:" if alpaca else " ### Response", add_special_tokens=False)
    # The reference drops the first two ids of the encoded template (train_fsdp1.py:59-61) because a sentencepiece
    # tokenizer encodes a leading space and "###" differently at the start of a text than inside one.  How many
    # leading ids differ depends on the tokenizer, so the longest of template, template[1:], template[2:] that
    # occurs in the example is used.
    collators = [DataCollatorForCompletionOnlyLM(template[d:], tok.pad_token_id) for d in range(min(3, len(template)))]

    def occurs(ids, sub):
        n = len(sub)
        return n > 0 and any(ids[i:i + n] == sub for i in range(len(ids) - n + 1))
    out = []
    for rec in records:
        body = f"### Question: {rec['instruction']}\n ### Answer: {rec['output']}" if alpaca else rec["output"]
        ids = tok(body)["input_ids"][:max_seq_length]
        collator = next((c for d, c in enumerate(collators) if occurs(list(ids), template[d:])), collators[-1])
        b = collator([{"input_ids": ids}])
        out.append({"input_ids": b["input_ids"][0], "labels": b["labels"][0]})
    return out


def _sync_each_batch(flag: bool) -> bool:
    """The launcher passes `gradient_accumulation_kwargs.sync_each_batch` of an accelerator config
    (accelerator_config.json:1-4) through MDT_SYNC_EACH_BATCH; it overrides the script's default."""
    env = os.environ.get("MDT_SYNC_EACH_BATCH")
    return flag if env is None else env == "1"


def run_training(
    max_seq_length: int = 4096,
    load_model_dtype: str = "bfloat16",
    attn_implementation: str = "sdpa",
    per_device_train_batch_size: int = 1,
    gradient_accumulation_steps: int = 1,
    use_megablocks_sharding: bool = False,
    use_scattermoe: bool = False,
    use_tp_sharding: bool = False,
    lr_scheduler_type: str = "linear",
    num_epochs: int = 1,
    num_warmup_steps: int = 0,
    max_grad_norm: float = 1.0,
    learning_rate: float = 1e-5,
    truncate_model_for_debug: bool = False,
    expert_degree: Optional[int] = None,
    use_lora: str = "none",
    # extensions
    model_name_or_path: str = MODEL_NAME,
    model_preset: str = "mixtral-8x7b",
    data_path: str = "data.json",
    num_synthetic_examples: int = 64,
    synthetic_min_len: int = 128,
    synthetic_max_len: int = 1024,
    device_type: str = "cuda",
    dispatch_impl: str = "auto",
    sync_each_batch: bool = False,
    activation_checkpointing: bool = True,
    seed: int = 0,
    save_path: Optional[str] = None,
    resume_from: Optional[str] = None,
    max_steps: int = 0,
    profile_trace: Optional[str] = None,
    profile_steps: int = 2,
    sharding_strategy: str = "fsdp2",
):
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    ep = validate_flags(use_megablocks_sharding, use_scattermoe, use_tp_sharding, use_lora, world, expert_degree)
    if not torch.cuda.is_available():
        device_type = "cpu"
    dtype = getattr(torch, load_model_dtype)
    cfg, ckpt = _resolve_config(model_name_or_path, model_preset)
    if truncate_model_for_debug:
        cfg.num_hidden_layers = 2  # same shortcut as the reference (train_accelerate_fsdp2.py:74-76)

    examples = _load_text_dataset(data_path, ckpt or model_name_or_path, max_seq_length)
    if examples is None:
        ds = SyntheticInstructionDataset(cfg.vocab_size, num_synthetic_examples, synthetic_min_len,
                                         min(synthetic_max_len, max_seq_length), seed=seed, rank=rank)
        examples = ds.examples
    else:
        # every rank tokenised the whole file; keep this rank's share (TP peers share a batch, :346-382)
        dp_rank, dp_size = (rank // ep, world // ep) if use_tp_sharding else (rank, world)
        examples = examples[dp_rank::dp_size]
    bs, ga = per_device_train_batch_size, gradient_accumulation_steps
    micro = [collate_packed(examples[i:i + bs]) for i in range(0, len(examples) - bs + 1, bs)]
    steps_per_epoch = len(micro) // ga
    total_steps = steps_per_epoch * num_epochs
    if max_steps:
        total_steps = min(total_steps, max_steps)

    engine = build_engine(
        cfg, dtype=dtype, device_type=device_type, ep_size=ep, use_tp_sharding=use_tp_sharding, use_lora=use_lora,
        learning_rate=learning_rate, lr_scheduler_type=lr_scheduler_type, num_warmup_steps=num_warmup_steps,
        num_training_steps=max(total_steps, 1), max_grad_norm=max_grad_norm, checkpoint=ckpt, seed=seed,
        mlp_impl="scattermoe" if use_scattermoe else "sparse", dispatch_impl=dispatch_impl,
        sync_each_batch=_sync_each_batch(sync_each_batch), activation_checkpointing=activation_checkpointing,
        # the FSDP1 entry re-gathers every unit's flat parameters per use (accelerate.yaml: FULL_SHARD, re-shard after
        # forward); the FSDP2 entry may keep the gathered dense parameters resident when they fit
        resident_params=False if sharding_strategy == "fsdp1" else None)
    start_step = 0
    if resume_from:
        from ..checkpoint.state import load_training_state
        start_step = load_training_state(engine, resume_from)

    dev = engine.device
    if dev.type == "cuda":
        torch.cuda.reset_peak_memory_stats(dev)
    timer = DeviceTimer(dev)
    timer.start()
    tokens_local = 0
    step = start_step
    # optional torch.profiler trace of `profile_steps` optimizer steps after the first one (one file per rank,
    # chrome://tracing format); the steps under the profiler are slower, so use it on short runs
    prof, prof_until, prof_done = None, 0, False
    while step < total_steps:
        epoch, k = divmod(step, max(steps_per_epoch, 1))
        mbs = micro[k * ga:(k + 1) * ga]
        tokens_local += sum(int(m["input_ids"].numel()) for m in mbs)
        if profile_trace and prof is None and not prof_done and step == start_step + min(1, total_steps - start_step - 1):
            from torch.profiler import ProfilerActivity, profile
            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if dev.type == "cuda" else [])
            prof = profile(activities=acts)
            prof.__enter__()
            prof_until = step + max(1, profile_steps)
        out = engine.train_step(mbs)
        step += 1
        if prof is not None and (step >= prof_until or step >= total_steps):
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            prof.__exit__(None, None, None)
            os.makedirs(profile_trace, exist_ok=True)
            prof.export_chrome_trace(os.path.join(profile_trace, f"trace_rank{rank:05d}.json"))
            prof, prof_done = None, True
        gn = out["grad_norm"]
        log_json(rank, epoch=round(step / max(steps_per_epoch, 1), 2), loss=float(out["loss"]),
                 learning_rate=engine.scheduler.get_last_lr()[0], grad_norm=float(gn) if gn is not None else 0.0,
                 **memory_stats(dev))
    runtime = max_over_ranks(timer.stop(), dev)
    tokens = sum_over_ranks(tokens_local, dev)
    done = step - start_step
    log_json(rank, train_runtime=round(runtime, 3), train_steps_per_second=round(done / max(runtime, 1e-9), 4),
             train_tokens_per_second=round(tokens / max(runtime, 1e-9), 1))
    if save_path:
        from ..checkpoint.state import save_model, save_training_state
        save_model(engine, save_path)
        save_training_state(engine, save_path, step)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return engine
