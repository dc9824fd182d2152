"""Per-kernel shares of a training step, from torch's profiler (no ncu needed; works with several ranks).

    python benchmarks/step_profile.py [--layers 8] [--mode attn-only|all|none]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/step_profile.py

Builds a Mixtral-8x7B-shaped model truncated to `--layers` decoder blocks (profiles are per block; the full
model only repeats them), runs a few untimed optimizer steps, then profiles one whole optimizer step through
`Engine.train_step` (16 micro-batches, sorted by length as in training).  Every rank prints one line with the time
its GPU spent waiting for peers and in the GEMM kernels; rank 0 prints the kernel table and the same table divided
by layers x micro-batches.  Durations under the profiler are for shares, not benchmark values.
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--mode", default="attn-only", choices=["attn-only", "all", "none"])
    ap.add_argument("--ep", type=int, default=0)
    ap.add_argument("--per-unit-rows", type=int, default=28)
    ap.add_argument("--rows", type=int, default=40)
    args = ap.parse_args()
    from bench import make_step_batches
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.train.engine import build_engine
    from torch.profiler import ProfilerActivity, profile
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    cfg = MixtralConfig.mixtral_8x7b()
    cfg.num_hidden_layers = args.layers
    eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", ep_size=(args.ep or world) if world > 1 else 1, use_lora=args.mode,
                       lora_alpha=32, learning_rate=5e-5, num_training_steps=100, ep_max_tokens=1024)
    for s in range(3):
        st = [eng.to_device(mb) for mb in make_step_batches(cfg.vocab_size, 16, 128, 1024, s, rank)]
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        eng.train_step(st)
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        if rank == 0:
            print(f"layers {args.layers} step {s}: host {1e3 * (t1 - t0):.1f} ms, host+device {1e3 * (t2 - t0):.1f} ms", flush=True)
    st = [eng.to_device(mb) for mb in make_step_batches(cfg.vocab_size, 16, 128, 1024, 99, rank)]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
        eng.train_step(st)
        torch.cuda.synchronize()
    ka = prof.key_averages()

    def total(sub):
        return sum(getattr(e, "self_device_time_total", 0) for e in ka if sub in e.key) / 1e3
    tokens = sum(int(mb["input_ids"].numel()) for mb in st)
    print(f"rank {rank}: tokens {tokens}, waiting for peers' counts {total('ep_counts_wait_meta'):.1f} ms, for returned rows "
          f"{total('ep_wait_rows'):.1f} ms, GEMM kernels {total('gemm_sm100'):.1f} ms", flush=True)
    if rank == 0:
        print(ka.table(sort_by="cuda_time_total", row_limit=args.rows, max_name_column_width=60))
        units = args.layers * len(st)
        rows = sorted(((getattr(e, "self_device_time_total", 0), e.count, e.key) for e in ka if getattr(e, "self_device_time_total", 0) > 0), reverse=True)
        all_us = sum(r[0] for r in rows)
        print(f"per layer and micro-batch ({units} of them): device time {all_us / units / 1e3:.3f} ms in all")
        for us, cnt, key in rows[:args.per_unit_rows]:
            print(f"  {us / units / 1e3:8.4f} ms  {cnt / units:6.2f} launches  {key[:90]}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
