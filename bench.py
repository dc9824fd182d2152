"""Flagship benchmark: Mixtral-8x7B expert-parallel fine-tuning throughput (tokens/s).

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 3 --warmup 3

One step = one optimizer step = 16 micro-batches of one synthetic instruction sequence per GPU
(length uniform in [128, 1024], first 40 % label-masked), bf16, block recomputation, AdamW,
linear schedule.  Weak scaling: the per-GPU work is fixed.  Two timed regions over the SAME
batches, both bracketed by a barrier + synchronize and timed with CUDA events (maximum over ranks):

  value      inputs already on the device, no host read inside the region
  e2e.value  through `Engine.train_step` with pinned host inputs: includes every micro-batch's
             host->device copy and one device->host read of the step's loss

The line's `value` is the series workload, the one Mixtral-8x7B fine-tuning configuration that fits
1, 2, 4 and 8 GPUs: `lora-attn` (LoRA r=16 on q/k/v/o, frozen bf16 base), expert-parallel over all GPUs.
After that measurement the process group is closed, the other ranks leave, and rank 0 runs further
configurations as child jobs of their own (fresh processes on the same GPUs, a time limit each), whose
results go into the line's `configs` object:

  series workload on the library arm (torch kernels, NCCL all-to-all with host-read split sizes):
      `vs_baseline` = value / that number, measured in the same run on the same box
  at 2+ GPUs: two optimizer steps with the fused exchange and two with the NCCL exchange from the same
      initial state on the same batch: losses and a parameter checksum of both (`fused_vs_nccl`)
  at 8 GPUs: full fine-tune ep8, LoRA-attn ep4 x dp2, LoRA-all ep4 x dp2, and no expert parallelism
      (everything sharded over 8 GPUs; LoRA-attn and full), each on both arms (native, then library)

`--mode`, `--ep`, `--impl library` select one of those configurations directly (that is what the child
jobs do); `--configs none` skips the child jobs.
"""
import argparse
import json
import os
import signal
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
T_START = time.time()
sys.path.insert(0, HERE)

DATA = "synthetic (uniform token ids, lengths uniform in [128,1024], first 40% label-masked), random-init N(0,0.02) weights"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"])
    ap.add_argument("--mode", default="lora-attn", choices=["lora-attn", "lora-all", "full"])
    ap.add_argument("--ep", type=int, default=0, help="expert-parallel size (default: number of GPUs; 1 = no expert "
                                                      "parallelism, experts sharded like every other parameter)")
    ap.add_argument("--grad-accum", type=int, default=16)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (marks the result invalid)")
    ap.add_argument("--min-len", type=int, default=128)
    ap.add_argument("--max-len", type=int, default=1024)
    ap.add_argument("--dispatch", default="auto")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-recompute", action="store_true",
                    help="keep activations instead of recomputing each block in backward (not the named configuration: "
                         "the result is labelled gradient_checkpointing=false)")
    ap.add_argument("--configs", default="auto", choices=["auto", "none"],
                    help="auto: after the series measurement run the other named configurations as child jobs")
    ap.add_argument("--extras-budget-s", type=float, default=700.0, help="time limit for all child jobs together")
    ap.add_argument("--total-budget-s", type=float, default=790.0,
                    help="the child jobs also end this long after this process started, whatever the series measurement took")
    ap.add_argument("--extra-steps", type=int, default=2)
    ap.add_argument("--extra-warmup", type=int, default=3)
    ap.add_argument("--sub", default="", help="internal: this process is a child job (run | pair | check)")
    ap.add_argument("--sub-out", default="")
    ap.add_argument("--abs-deadline", type=float, default=0.0,
                    help="internal: wall-clock time (epoch seconds) by which a child job should have ended by itself")
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


def make_step_batches(vocab, ga, min_len, max_len, seed, rank):
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, collate_packed
    ds = SyntheticInstructionDataset(vocab, ga, min_len, max_len, seed=seed, rank=rank)
    return [collate_packed([ex]) for ex in ds.examples]


def reference_arm():
    """The reference itself: installed (code only) under baseline/_ref, but its entry point cannot be imported."""
    ref = os.path.join(HERE, "baseline", "_ref")
    why = "baseline/_ref is missing"
    if os.path.isdir(ref):
        probe = ("import sys; sys.path.insert(0, sys.argv[1]); import importlib\n"
                 "missing = []\n"
                 "for m in ('megablocks', 'stk', 'scattermoe', 'khd', 'peft', 'trl', 'accelerate', 'fire'):\n"
                 "    try:\n        importlib.import_module(m)\n    except Exception:\n        missing.append(m)\n"
                 "print(','.join(missing))\n")
        try:
            out = subprocess.run([sys.executable, "-c", probe, ref], capture_output=True, text=True, timeout=120)
            missing = out.stdout.strip().splitlines()[-1] if out.stdout.strip() else ""
        except Exception as exc:  # noqa: BLE001
            missing = f"probe failed: {exc}"
        why = ("the reference's files are installed under baseline/_ref (pip --no-deps from a copy with a minimal pyproject), but its "
               f"training entry point needs packages that are in neither the image nor the wheelhouse: {missing or 'none missing?'}; "
               "its two Triton kernels, the only part that runs here, are timed by benchmarks/ref_triton_kernels.py")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def parallelism_name(world, ep):
    if world == 1:
        return "single-gpu"
    if ep <= 1:
        return f"fsdp{world} (no expert parallelism)"
    dp = world // ep
    return f"ep{ep}" + (f"xdp{dp}" if dp > 1 else "")


def release_engine():
    """Drop what a finished engine left behind in this process (cached exchange workspaces, allocator blocks)."""
    import gc
    import torch
    try:
        from moe_distributed_training_b200.parallel.fused_ep import FusedExpertParallel
        FusedExpertParallel._instances.clear()
    except Exception:  # noqa: BLE001
        pass
    gc.collect()
    torch.cuda.empty_cache()


def run_measurement(args):
    """Builds the engine for (mode, ep, impl), measures `value` and `e2e`; returns (result dict on rank 0 or None)."""
    import torch
    import torch.distributed as dist
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.train.engine import build_engine

    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus and args.gpus > 1 and world == 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    cfg = MixtralConfig.mixtral_8x7b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    ep = args.ep or world
    if world == 1:
        ep = 1
    from moe_distributed_training_b200 import ops
    dispatch = args.dispatch
    if args.impl == "library":
        ops.set_backend("library")
        os.environ["MDT_PEER_COLLECTIVES"] = "0"        # NCCL all-gather / reduce-scatter
        if dispatch == "auto":
            dispatch = "nccl"
    else:
        ops.set_backend("native")
        os.environ.pop("MDT_PEER_COLLECTIVES", None)
    use_lora = {"lora-attn": "attn-only", "lora-all": "all", "full": "none"}[args.mode]
    total_steps = args.steps * 2 + args.warmup + 4
    eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=ep,
                       use_lora=use_lora, lora_r=16, lora_alpha=32 if use_lora != "none" else 16, learning_rate=5e-5,
                       lr_scheduler_type="linear", num_training_steps=total_steps, max_grad_norm=1.0, seed=0,
                       dispatch_impl=dispatch, ep_max_tokens=args.max_len,
                       activation_checkpointing=not args.no_recompute)
    dev = eng.device
    ga = args.grad_accum

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def host_batches(n_steps, seed0):
        return [make_step_batches(cfg.vocab_size, ga, args.min_len, args.max_len, seed0 + s, rank) for s in range(n_steps)]

    def run_region(steps, on_device):
        """Returns (seconds on the device, tokens of all ranks, h2d bytes/step, d2h bytes/step, losses)."""
        n_steps = len(steps)
        tokens = sum(int(mb["input_ids"].numel()) for st in steps for mb in st)
        h2d = sum(int(v.numel() * v.element_size()) for st in steps for mb in st for v in mb.values()
                  if torch.is_tensor(v)) // max(n_steps, 1)
        if on_device:
            steps = [[eng.to_device(mb) for mb in st] for st in steps]
        else:
            steps = [[{k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in mb.items()} for mb in st] for st in steps]
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
    run_region(host_batches(args.warmup, 1000), on_device=True)            # warm-up (untimed)
    timed = host_batches(args.steps, 2000)                                 # both timed regions use these batches
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = cuda_ops.launch_count()
    sec, tokens, _, _, _ = run_region(timed, on_device=True)
    launches = cuda_ops.launch_count() - l0
    e2e = None
    if not args.no_e2e:
        run_region(host_batches(1, 2500), on_device=False)                 # warm the pinned-input path
        sec_e, tok_e, h2d, d2h, losses = run_region(timed, on_device=False)
        e2e = {"value": round(tok_e / sec_e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": round(sec_e / args.steps * 1e3, 2), "last_loss": losses[-1],
               "batches": "the same as in the device-input region"}
    clocks = sampler.stop() if rank == 0 else None
    cuda_ops.check_status(dev)
    mem = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    line = None
    if rank == 0:
        line = {
            "metric": "Mixtral-8x7B EP finetune tokens/s", "value": round(tokens / sec, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec / args.steps * 1e3, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": DATA,
            "impl": args.impl,
            "config": {"model": "Mixtral-8x7B" + (f" (TRUNCATED to {args.layers} layers: debug, invalid)" if args.layers else ""),
                       "mode": args.mode, "global_batch": world * ga, "micro_batch": 1, "grad_accum": ga,
                       "seq_len": f"uniform[{args.min_len},{args.max_len}]", "parallelism": parallelism_name(world, ep),
                       "gradient_checkpointing": not args.no_recompute, "optimizer": "AdamW lr 5e-5 linear",
                       "lora_r": 16 if use_lora != "none" else None,
                       "l2": "working set (>= 11 GB of weights per GPU) is larger than the 126 MB L2; no explicit flush",
                       "peak_mem_gib": round(mem, 1)},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
    del eng
    release_engine()
    return line


def second_arm_fits(first_arm_s, now, abs_deadline):
    """Whether the library arm of a pair job can still finish by `abs_deadline`: it builds the same model and runs the
    same steps 1.5-2x as slowly as the native arm, which took `first_arm_s`."""
    return now + 2.2 * first_arm_s + 10.0 < abs_deadline


def share_decision(path, rank, decision=None, wait_s=60.0):
    """Rank 0 publishes a yes/no decision in `path`; every rank returns it (no: also when nothing appears in time)."""
    if rank == 0:
        with open(path + ".tmp", "w") as f:
            f.write("go" if decision else "skip")
        os.replace(path + ".tmp", path)
    t0 = time.time()
    while not os.path.exists(path) and time.time() - t0 < wait_s:
        time.sleep(0.05)
    try:
        with open(path) as f:
            return f.read().strip() == "go"
    except OSError:
        return False


def run_pair(args):
    """One configuration on both arms in one job: native first, then library.  The result file is rewritten after
    each arm, so that the first arm's numbers survive if the second one fails or runs out of time."""
    rank = int(os.environ.get("RANK", 0))
    out = {}
    t_arm = time.time()
    for impl in ("native", "library"):
        args.impl = impl
        if impl == "library" and args.abs_deadline > 0:
            # Rather end here than be stopped in the middle of a collective: rank 0 decides from the first arm's duration
            # and tells the other ranks through a file.
            go = share_decision(args.sub_out + ".decision", rank,
                                second_arm_fits(time.time() - t_arm, time.time(), args.abs_deadline) if rank == 0 else None)
            if not go:
                out[impl] = {"skipped": "not enough of the run's time limit left for this arm"}
                if rank == 0:
                    with open(args.sub_out, "w") as f:
                        json.dump(out, f)
                break
        try:
            out[impl] = brief(run_measurement(args)) if rank == 0 else run_measurement(args)
        except Exception as exc:  # noqa: BLE001
            out[impl] = {"error": repr(exc)[:400]}
            if rank == 0:
                with open(args.sub_out, "w") as f:
                    json.dump(out, f)
            raise
        if rank == 0:
            with open(args.sub_out, "w") as f:
                json.dump(out, f)
    return out if rank == 0 else None


def run_check(args):
    """One optimizer step with the fused exchange and one with the NCCL exchange, same initial state, same batch."""
    import torch
    import torch.distributed as dist
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.ops import cuda_ops
    from moe_distributed_training_b200.train.engine import build_engine
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    cfg = MixtralConfig.mixtral_8x7b()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    step = make_step_batches(cfg.vocab_size, 4, args.min_len, args.max_len, 4000, rank)
    out = {}
    for impl in ("fused", "nccl"):
        eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=world, use_lora="attn-only", lora_r=16,
                           lora_alpha=32, learning_rate=1e-3, lr_scheduler_type="constant", num_training_steps=4,
                           max_grad_norm=1.0, seed=0, dispatch_impl=impl, ep_max_tokens=args.max_len)
        losses = [float(eng.train_step(step)["loss"]) for _ in range(2)]      # the second step sees the first one's update
        cuda_ops.check_status(eng.device)
        chk = torch.zeros(1, dtype=torch.float64, device=eng.device)
        for p in eng.model.parameters():
            if p.requires_grad:
                chk += p.detach().double().abs().sum()
        if world > 1:
            dist.all_reduce(chk)
            lt = torch.tensor(losses, dtype=torch.float64, device=eng.device)
            dist.all_reduce(lt)
            losses = (lt / world).tolist()
        out[impl] = {"losses_mean_over_ranks": [round(x, 6) for x in losses], "trainable_abs_sum": float(chk.item())}
        del eng
        release_engine()
    a, b = out["fused"], out["nccl"]
    out["max_rel_loss_diff"] = max(abs(x - y) / max(abs(y), 1e-9) for x, y in zip(a["losses_mean_over_ranks"], b["losses_mean_over_ranks"]))
    out["rel_checksum_diff"] = abs(a["trainable_abs_sum"] - b["trainable_abs_sum"]) / max(abs(b["trainable_abs_sum"]), 1e-9)
    out["what"] = "LoRA-attn, ep = all GPUs, 2 optimizer steps of 4 micro-batches at lr 1e-3 from seed 0, per exchange implementation"
    return out if rank == 0 else None


# ----------------------------------------------------------------------------------------------- child jobs
def _clean_env():
    env = dict(os.environ)
    for k in list(env):
        if k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_NAME", "ROLE_WORLD_SIZE",
                 "GROUP_WORLD_SIZE", "MASTER_PORT", "MASTER_ADDR", "OMP_NUM_THREADS") or k.startswith("TORCHELASTIC") or k.startswith("TORCH_NCCL_ASYNC"):
            env.pop(k)
    return env


def run_child(n, extra_args, timeout_s, port):
    """Runs `bench.py --sub ...` on n GPUs as a job of its own; returns its result dict or {"error": ...}."""
    out_path = os.path.join("/tmp", f"mdt_bench_child_{os.getpid()}_{port}.json")
    for stale in (out_path, out_path + ".decision"):
        if os.path.exists(stale):
            os.remove(stale)
    base = [os.path.join(HERE, "bench.py"), "--gpus", str(n), "--sub-out", out_path, "--abs-deadline", f"{time.time() + timeout_s - 8.0:.1f}"] + extra_args
    if n > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
               "--master-port", str(port)] + base
    else:
        cmd = [sys.executable] + base
    t0 = time.time()
    try:
        proc = subprocess.Popen(cmd, env=_clean_env(), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)
        try:
            log, _ = proc.communicate(timeout=timeout_s)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)       # the session this function started, nothing else
            proc.communicate()
            res = _read_partial(out_path)
            res["error"] = f"child job exceeded its {int(timeout_s)} s limit"
            res["wall_s"] = round(time.time() - t0, 1)
            return res
        if proc.returncode != 0 or not os.path.exists(out_path):
            tail = [ln[-300:] for ln in (log or "").strip().splitlines() if ln.strip()][-6:]
            res = _read_partial(out_path)
            res.update({"error": f"child job exited with {proc.returncode}", "log_tail": tail, "wall_s": round(time.time() - t0, 1)})
            return res
        res = _read_partial(out_path)
        res["wall_s"] = round(time.time() - t0, 1)
        return res
    except Exception as exc:  # noqa: BLE001
        return {"error": repr(exc), "wall_s": round(time.time() - t0, 1)}


def _read_partial(path):
    try:
        if os.path.exists(path + ".decision"):
            os.remove(path + ".decision")
        with open(path) as f:
            res = json.load(f)
        os.remove(path)
        return res if isinstance(res, dict) else {}
    except Exception:  # noqa: BLE001
        return {}


def brief(res):
    """The few fields of a child's result line that the configs table keeps."""
    if res is None or "error" in res:
        return res
    keep = {"tokens_per_s": res["value"], "ms_per_step": res["ms_per_step"], "steps": res["steps"], "warmup": res["warmup"],
            "peak_mem_gib": res["config"]["peak_mem_gib"], "parallelism": res["config"]["parallelism"]}
    if res.get("e2e"):
        keep["e2e_tokens_per_s"] = res["e2e"]["value"]
        keep["last_loss"] = res["e2e"]["last_loss"]
    return keep


def run_extras(args, world, line):
    """Child jobs after the series measurement (rank 0 only, the process group is closed, the other ranks are gone)."""
    deadline = min(time.time() + args.extras_budget_s, T_START + args.total_budget_s)
    port0 = int(os.environ.get("MASTER_PORT", "29500")) + 101
    common = ["--steps", str(args.extra_steps), "--warmup", str(args.extra_warmup), "--configs", "none", "--no-e2e",
              "--min-len", str(args.min_len), "--max-len", str(args.max_len), "--grad-accum", str(args.grad_accum)]
    if args.layers:
        common += ["--layers", str(args.layers)]
    # in order of importance: what does not fit the time limit is reported as skipped
    jobs = [("series_library", ["--sub", "run", "--mode", "lora-attn", "--impl", "library"])]
    # the named configurations belong to 8 GPUs; MDT_BENCH_ALL_CONFIGS=1 runs their counterparts on fewer (to try the
    # machinery on a small box; the names then carry the actual sizes)
    all_configs = world == 8 or (world >= 2 and os.environ.get("MDT_BENCH_ALL_CONFIGS") == "1")
    half = world // 2
    if all_configs:
        jobs.append((f"full_ep{world}", ["--sub", "pair", "--mode", "full", "--ep", str(world)]))
        if half >= 2:
            jobs += [(f"lora_attn_ep{half}xdp2", ["--sub", "pair", "--mode", "lora-attn", "--ep", str(half)]),
                     (f"lora_all_ep{half}xdp2", ["--sub", "pair", "--mode", "lora-all", "--ep", str(half)])]
        jobs.append(("lora_attn_no_ep", ["--sub", "pair", "--mode", "lora-attn", "--ep", "1"]))
    if world >= 2:
        jobs.append(("fused_vs_nccl", None))
    if all_configs:
        jobs.append(("full_no_ep", ["--sub", "pair", "--mode", "full", "--ep", "1"]))
    configs = {}
    for i, (name, extra) in enumerate(jobs):
        left = deadline - time.time()
        if left < 45:
            configs[name] = {"skipped": "time limit for the additional configurations reached"}
            continue
        limit = min(left, 330.0)
        if extra is None:
            sub = ["--sub", "check", "--configs", "none", "--min-len", str(args.min_len), "--max-len", str(args.max_len)]
            if args.layers:
                sub += ["--layers", str(args.layers)]
            configs[name] = run_child(world, sub, limit, port0 + i)
        elif "pair" in extra:
            configs[name] = run_child(world, common + extra, limit, port0 + i)
        else:
            res = run_child(world, common + extra, limit, port0 + i)
            configs[name] = brief(res) if "value" in res else res
    lib = configs.get("series_library") or {}
    if lib.get("tokens_per_s"):
        line["vs_baseline"] = round(line["value"] / lib["tokens_per_s"], 3)
        line["vs_baseline_is"] = ("value / tokens_per_s of the same workload on this repo's library arm (torch kernels, NCCL all-to-all with "
                                  "host-read split sizes) measured by a child job of this run; the reference publishes no tokens/s and "
                                  "cannot be run here")
    for name, pair in configs.items():
        a, b = (pair.get("native") or {}), (pair.get("library") or {})
        if a.get("tokens_per_s") and b.get("tokens_per_s"):
            pair["native_over_library"] = round(a["tokens_per_s"] / b["tokens_per_s"], 3)

    def tps(c, impl="native"):
        return ((configs.get(c) or {}).get(impl) or {}).get("tokens_per_s")
    # the reference's README reports run-time ratios of expert parallelism over plain FSDP2: 3.49x (full), 2.43x (LoRA)
    ratios = {}
    if tps(f"full_ep{world}") and tps("full_no_ep"):
        ratios[f"full_ep{world}_over_no_ep"] = round(tps(f"full_ep{world}") / tps("full_no_ep"), 2)
    if tps("lora_attn_no_ep"):
        ratios[f"lora_attn_ep{world}_over_no_ep"] = round(line["value"] / tps("lora_attn_no_ep"), 2)
    if ratios:
        ratios["reference_readme_other_hardware_8_gpus"] = {"full_ep8_over_no_ep": 3.49, "lora_attn_ep8_over_no_ep": 2.43}
        configs["ep_over_no_ep"] = ratios
    line["configs"] = configs
    line["configs_note"] = (f"child jobs on the same GPUs after the series measurement, {args.extra_warmup} warm-up + {args.extra_steps} timed "
                            f"optimizer steps per arm, same data recipe, device-input timing; together limited to {int(args.extras_budget_s)} s and to {int(args.total_budget_s)} s "
                            f"after the start of the whole run")


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm()
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    if args.sub == "check":
        res = run_check(args)
    elif args.sub == "pair":
        res = run_pair(args)
    else:
        res = run_measurement(args)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if args.sub:
        if rank == 0:
            with open(args.sub_out, "w") as f:
                json.dump(res, f)
        return 0
    if rank != 0:
        return 0
    # rank 0 of the top-level job: everything of the series run is released; child jobs get the GPUs
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    if args.configs == "auto" and args.impl == "native" and args.mode == "lora-attn" and not args.ep and not args.no_recompute:
        try:
            run_extras(args, world, res)
        except Exception as exc:  # noqa: BLE001
            res["configs_error"] = repr(exc)
    print(json.dumps(res), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
