"""Config-file launcher: the `accelerate launch --config_file accelerate.yaml script.py ...` workflow.

    python -m moe_distributed_training_b200.launch --config_file accelerate.yaml [--num_processes 8] \
        train_fsdp1.py --use_megablocks_sharding ...

The reference starts its FSDP1 script through accelerate with a YAML of FSDP-plugin settings
(accelerate.yaml:1-51) and reads gradient-accumulation behaviour from a JSON
(accelerator_config.json:1-4).  Here the same files are understood directly: process counts and
rendezvous settings become a `torch.distributed.run` command line, and the few settings that change
this framework's behaviour are handed to the training script through environment variables.  Settings
that describe things this framework always does (transformer-block wrapping, full state dict on save,
per-rank loading of only the bytes a rank owns) are accepted and ignored; settings it cannot honour
(CPU offload, no sharding) are rejected with a message instead of being silently dropped.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional

SHARDING = {"1": "FULL_SHARD", "2": "SHARD_GRAD_OP", "3": "NO_SHARD", "4": "HYBRID_SHARD", "5": "HYBRID_SHARD_ZERO2"}
ACCEPTED_AND_IMPLIED = ("fsdp_auto_wrap_policy", "fsdp_backward_prefetch_policy", "fsdp_backward_prefetch",
                        "fsdp_forward_prefetch", "fsdp_state_dict_type", "fsdp_cpu_ram_efficient_loading",
                        "fsdp_sync_module_states", "fsdp_transformer_layer_cls_to_wrap", "fsdp_use_orig_params")


@dataclass
class LaunchPlan:
    command: List[str]
    env: Dict[str, str] = field(default_factory=dict)
    notes: List[str] = field(default_factory=list)


def _load_yaml(path: str) -> dict:
    import yaml
    with open(path) as f:
        return yaml.safe_load(f) or {}


def plan_launch(config: dict, script_and_args: List[str], num_processes: Optional[int] = None,
                accelerator_config: Optional[dict] = None, main_process_port: Optional[int] = None) -> LaunchPlan:
    """Translate an accelerate-style config into a torchrun command line and environment."""
    notes: List[str] = []
    env: Dict[str, str] = {}
    dist_type = str(config.get("distributed_type", "FSDP")).upper()
    if dist_type not in ("FSDP", "MULTI_GPU", "NO"):
        raise ValueError(f"distributed_type {dist_type} is not supported (FSDP, MULTI_GPU or NO)")
    nproc = int(num_processes if num_processes is not None else config.get("num_processes", 1))
    machines = int(config.get("num_machines", 1))
    if nproc % machines != 0:
        raise ValueError("num_processes must be a multiple of num_machines")
    fsdp = dict(config.get("fsdp_config") or {})
    strategy = str(fsdp.pop("fsdp_sharding_strategy", "1"))
    strategy = SHARDING.get(strategy, strategy).upper()
    if strategy == "NO_SHARD":
        raise ValueError("fsdp_sharding_strategy NO_SHARD: parameters are always sharded here; use SHARD_GRAD_OP "
                         "to keep full parameter copies resident between optimizer steps")
    if strategy in ("SHARD_GRAD_OP", "HYBRID_SHARD_ZERO2"):
        env["MDT_RESIDENT_PARAMS"] = "1"      # gathered parameters stay resident; gradients and optimizer state sharded
    elif strategy in ("FULL_SHARD", "HYBRID_SHARD"):
        env["MDT_RESIDENT_PARAMS"] = "0"      # re-gather per use, as FULL_SHARD does
    else:
        raise ValueError(f"unknown fsdp_sharding_strategy {strategy}")
    if bool(fsdp.pop("fsdp_offload_params", False)):
        raise ValueError("fsdp_offload_params: CPU offload is not implemented (parameters fit in 180 GB per GPU)")
    for key in list(fsdp):
        if key in ACCEPTED_AND_IMPLIED:
            notes.append(f"{key}={fsdp.pop(key)!r}: built in, no switch needed")
    for key in fsdp:
        notes.append(f"{key}: unknown FSDP setting, ignored")
    mp = str(config.get("mixed_precision", "no")).lower()
    if mp not in ("no", "bf16"):
        raise ValueError(f"mixed_precision {mp}: parameters and math are bf16 with fp32 accumulation; 'no' or 'bf16'")
    if accelerator_config:
        ga = accelerator_config.get("gradient_accumulation_kwargs") or {}
        if "sync_each_batch" in ga:
            env["MDT_SYNC_EACH_BATCH"] = "1" if ga["sync_each_batch"] else "0"
    addr = str(config.get("main_process_ip", "127.0.0.1"))
    port = int(main_process_port if main_process_port is not None else config.get("main_process_port", 29500))
    cmd = [sys.executable, "-m", "torch.distributed.run", f"--nnodes={machines}", f"--nproc-per-node={nproc // machines}"]
    if str(config.get("rdzv_backend", "static")).lower() == "c10d":
        cmd += ["--rdzv-backend=c10d", f"--rdzv-endpoint={addr}:{port}"]
    else:
        cmd += [f"--node-rank={int(config.get('machine_rank', 0))}", "--master-addr", addr, "--master-port", str(port)]
    return LaunchPlan(cmd + list(script_and_args), env, notes)


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    config_file, accel_json, nproc, port, dry = None, None, None, None, False
    while argv and argv[0].startswith("--"):
        flag = argv.pop(0)
        if flag == "--dry_run":
            dry = True
            continue
        if "=" in flag:
            flag, value = flag.split("=", 1)
        else:
            value = argv.pop(0)
        if flag == "--config_file":
            config_file = value
        elif flag == "--accelerator_config":
            accel_json = value
        elif flag == "--num_processes":
            nproc = int(value)
        elif flag == "--main_process_port":
            port = int(value)
        else:
            raise SystemExit(f"unknown launcher flag {flag}")
    if not argv:
        raise SystemExit("usage: python -m moe_distributed_training_b200.launch --config_file cfg.yaml script.py [args]")
    config = _load_yaml(config_file) if config_file else {}
    accel = json.load(open(accel_json)) if accel_json else None
    plan = plan_launch(config, argv, nproc, accel, port)
    for n in plan.notes:
        print(f"[launch] {n}", file=sys.stderr)
    if dry:
        print(json.dumps({"command": plan.command, "env": plan.env}))
        return 0
    return subprocess.call(plan.command, env={**os.environ, **plan.env})


if __name__ == "__main__":
    sys.exit(main())
