"""Timed CPU run of the plumbing configuration: tiny Mixtral-style MoE, fp32, gloo, expert parallel.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/cpu_config1.py [--steps 5]

2 decoder layers, hidden 256, 4 heads / 2 KV heads, 4 SwiGLU experts of FFN 512, top-2, vocabulary 1024; per rank two
sequences of 128 tokens with the first 40 % label-masked; one forward/backward/AdamW step per iteration on the
PyTorch statement of every op (`ops/reference.py`), tokens exchanged with gloo all-to-all.  Prints one JSON line
(maximum over ranks).  This is the oracle the CUDA kernels are tested against, timed for the record.
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, collate_packed
    from moe_distributed_training_b200.train.engine import build_engine
    torch.manual_seed(0)
    cfg = MixtralConfig.tiny()
    world = int(os.environ.get("WORLD_SIZE", 1))
    eng = build_engine(cfg, dtype=torch.float32, device_type="cpu", ep_size=world if world > 1 else 1, learning_rate=1e-3,
                       max_grad_norm=None, seed=0, lr_scheduler_type="constant")
    ds = SyntheticInstructionDataset(cfg.vocab_size, 2, fixed_len=128, seed=0, rank=eng.rank)
    mb = collate_packed([ds[0], ds[1]])
    tokens = int(mb["input_ids"].numel())
    times, loss = [], None
    for s in range(args.warmup + args.steps):
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        loss = float(eng.train_step([mb])["loss"])
        if world > 1:
            dist.barrier()
        if s >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = 1e3 * sum(times) / len(times)
    t = torch.tensor([ms], dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if eng.rank == 0:
        print(json.dumps({"config": "tiny MoE, fp32, gloo, ep%d" % world, "ms_per_step": round(float(t), 2),
                          "tokens_per_s": round(world * tokens / (float(t) / 1e3), 1), "tokens_per_rank": tokens,
                          "last_loss": round(loss, 4), "threads": torch.get_num_threads()}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
