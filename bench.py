"""Flagship benchmark: Mixtral-8x7B expert-parallel fine-tuning throughput (tokens/s).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 3 --warmup 3

One step = one optimizer step = 16 micro-batches of one synthetic instruction sequence per GPU
(length uniform in [128, 1024], first 40 % label-masked), bf16, block recomputation, AdamW,
linear schedule.  Weak scaling: the per-GPU work is fixed.  Two timed regions, both bracketed
by a barrier + synchronize and timed with CUDA events (maximum over ranks):

  value      inputs already on the device, no host read inside the region
  e2e.value  through `Engine.train_step` with pinned host inputs: includes every micro-batch's
             host->device copy and one device->host read of the step's loss

Modes: `lora-attn` (default; LoRA r=16 on q/k/v/o, frozen bf16 base: the one Mixtral-8x7B
fine-tuning configuration that fits 1, 2, 4 and 8 GPUs, so the scaling series is one workload),
`lora-all` (adapters on the experts too) and `full` (full fine-tuning; needs >= 4 GPUs for memory).
"""
import argparse
import json
import os
import subprocess
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"])
    ap.add_argument("--mode", default="lora-attn", choices=["lora-attn", "lora-all", "full"])
    ap.add_argument("--ep", type=int, default=0, help="expert-parallel size (default: number of GPUs)")
    ap.add_argument("--grad-accum", type=int, default=16)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the result invalid)")
    ap.add_argument("--min-len", type=int, default=128)
    ap.add_argument("--max-len", type=int, default=1024)
    ap.add_argument("--dispatch", default="auto")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-recompute", action="store_true",
                    help="keep activations instead of recomputing each block in backward (not the named configuration: "
                         "the result is labelled gradient_checkpointing=false)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx = max(mx, float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_step_batches(vocab, ga, min_len, max_len, seed, rank, pin):
    import torch
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, collate_packed
    ds = SyntheticInstructionDataset(vocab, ga, min_len, max_len, seed=seed, rank=rank)
    out = []
    for ex in ds.examples:
        mb = collate_packed([ex])
        if pin:
            mb = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in mb.items()}
        out.append(mb)
    return out


def main():
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is not installable offline: no setup.py/pyproject.toml, and its imports "
                          "(megablocks, stk, scattermoe, khd, peft, trl, accelerate, fire, torch==2.3.1) are absent "
                          "from the image and the wheelhouse"}))
        return 0
    import torch
    import torch.distributed as dist
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.train.engine import build_engine

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    cfg = MixtralConfig.mixtral_8x7b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    ep = args.ep or world
    if args.impl == "library":
        from moe_distributed_training_b200 import ops
        ops.set_backend("library")
    use_lora = {"lora-attn": "attn-only", "lora-all": "all", "full": "none"}[args.mode]
    total_steps = args.steps * 2 + args.warmup + 4
    eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=ep if world > 1 else 1,
                       use_lora=use_lora, lora_r=16, lora_alpha=32 if use_lora != "none" else 16, learning_rate=5e-5,
                       lr_scheduler_type="linear", num_training_steps=total_steps, max_grad_norm=1.0, seed=0,
                       dispatch_impl=args.dispatch, ep_max_tokens=args.max_len,
                       activation_checkpointing=not args.no_recompute)
    dev = eng.device
    ga = args.grad_accum

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run_region(n_steps, seed0, on_device):
        """Returns (seconds on the device, tokens of this rank, h2d bytes/step, d2h bytes/step, losses)."""
        steps = [make_step_batches(cfg.vocab_size, ga, args.min_len, args.max_len, seed0 + s, rank, pin=not on_device)
                 for s in range(n_steps)]
        tokens = sum(int(mb["input_ids"].numel()) for st in steps for mb in st)
        h2d = sum(int(v.numel() * v.element_size()) for st in steps for mb in st for v in mb.values()
                  if torch.is_tensor(v)) // max(n_steps, 1)
        if on_device:
            steps = [[eng.to_device(mb) for mb in st] for st in steps]
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        losses = []
        for st in steps:
            out = eng.train_step(st)
            if not on_device:
                losses.append(float(out["loss"]))      # device->host read of the step's result
        e1.record()
        sync()
        sec = e0.elapsed_time(e1) / 1e3
        if world > 1:
            t = torch.tensor([sec], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
            tk = torch.tensor([tokens], device=dev, dtype=torch.float64)
            dist.all_reduce(tk)
            tokens_all = float(tk.item())
        else:
            tokens_all = float(tokens)
        return sec, tokens_all, h2d, 4 if not on_device else 0, losses

    from moe_distributed_training_b200.ops import cuda_ops
    run_region(args.warmup, 1000, on_device=True)                      # warm-up (untimed)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = cuda_ops.launch_count()
    sec, tokens, _, _, _ = run_region(args.steps, 2000, on_device=True)
    launches = cuda_ops.launch_count() - l0
    e2e = None
    if not args.no_e2e:
        run_region(1, 2500, on_device=False)                           # warm the pinned-input path
        sec_e, tok_e, h2d, d2h, losses = run_region(args.steps, 3000, on_device=False)
        e2e = {"value": round(tok_e / sec_e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": round(sec_e / args.steps * 1e3, 2), "last_loss": losses[-1]}
    clocks = sampler.stop() if rank == 0 else None
    cuda_ops.check_status(dev)
    mem = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    if rank == 0:
        dp = world // ep if world > 1 else 1
        par = f"ep{ep}" + (f"xdp{dp}" if dp > 1 else "") if world > 1 else "single-gpu"
        line = {
            "metric": "Mixtral-8x7B EP finetune tokens/s", "value": round(tokens / sec, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec / args.steps * 1e3, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform token ids, lengths uniform in [128,1024], first 40% label-masked), random-init N(0,0.02) weights",
            "impl": args.impl,
            "config": {"model": "Mixtral-8x7B" + (f" (TRUNCATED to {args.layers} layers: debug, invalid)" if args.layers else ""),
                       "mode": args.mode, "global_batch": world * ga, "micro_batch": 1, "grad_accum": ga,
                       "seq_len": f"uniform[{args.min_len},{args.max_len}]", "parallelism": par,
                       "gradient_checkpointing": not args.no_recompute, "optimizer": "AdamW lr 5e-5 linear", "lora_r": 16 if use_lora != "none" else None,
                       "l2": "working set (>= 11 GB of weights per GPU) is larger than the 126 MB L2; no explicit flush",
                       "peak_mem_gib": round(mem, 1)},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
