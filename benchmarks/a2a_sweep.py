"""Isolated expert-parallel dispatch + combine sweep.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/a2a_sweep.py [--out file.json]

Per GPU: T tokens (1024 ... 65536), hidden 4096, 8 experts, top-2, bf16 rows; router logits N(0,1) plus a
per-expert bias drawn from N(0,0.5) (load imbalance).  Two implementations of the same movement:

  fused   counts written into peers' symmetric buffers, rows stored straight into the owner's
          expert-grouped buffer and straight back (csrc/comm.cu), no host involvement
  nccl    all_to_all of counts, device->host read of the split sizes, all_to_all_single of the rows,
          local re-sort, and the way back (what the reference's exchange does)

Timed with CUDA events after warm-up, maximum over ranks.  GB/s = bytes this rank sends to other GPUs in
both phases / time; the roofline is the slower phase at the measured 770 GB/s per direction.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LINK_GBS = 770.0


def timed(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(); dist.barrier()
    best = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best.append(float(t))
    best.sort()
    return best[len(best) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--tokens", default="1024,4096,16384,65536")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--capacity-factor", type=float, default=2.5,
                    help="receive buffers hold this many times the balanced load (smaller = denser buffers)")
    ap.add_argument("--phases", action="store_true", help="also time dispatch alone (plan + counts + dispatch + wait)")
    args = ap.parse_args()
    from moe_distributed_training_b200.train.engine import init_distributed
    rank, ws, dev = init_distributed("cuda")
    from moe_distributed_training_b200.ops import cuda_ops as C
    from moe_distributed_training_b200.parallel import fused_ep, symm
    ext = C.ext
    E, k, H = 8, 2, args.hidden
    group = dist.group.WORLD
    g = torch.Generator(device=dev).manual_seed(1234)
    bias = torch.randn(E, device=dev, generator=g) * 0.5          # same on every rank
    results = []
    for T in [int(t) for t in args.tokens.split(",")]:
        gl = torch.Generator(device=dev).manual_seed(100 + rank)
        x = torch.randn(T, H, device=dev, generator=gl).to(torch.bfloat16)
        top = (torch.randn(T, E, device=dev, generator=gl) + bias).topk(k, -1).indices.int()
        wsp = symm.create_ep_workspace(group, E, H, T, k, dev, capacity_factor=args.capacity_factor * ws if ws > 1 else None)
        eng = fused_ep.FusedExpertParallel(wsp, k, dev)
        eos = top.reshape(-1).contiguous()
        El = E // ws
        remote = int(((eos // El) != rank).sum())
        bytes_remote = remote * H * 2

        def fused():
            plan = C.make_plan(top, E, 1, top.numel())
            meta = eng.exchange_counts(plan.tokens_per_expert)
            par = eng.next_phase()
            eng.dispatch(x, plan.src_slot, eos, None, meta, k, par)
            eng.combine(wsp.recv_x(), meta, par, top.numel(), clone=False)

        def nccl():
            plan = C.make_plan(top, E, 1, top.numel())
            counts = plan.tokens_per_expert
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts)
            both = torch.stack([counts.view(ws, El).sum(1), recv_counts.view(ws, El).sum(1)]).tolist()
            xs = ext.gather_rows(x, plan.src_slot, plan.padded_offsets, E, None, k)
            xr = xs.new_empty(sum(both[1]), H)
            dist.all_to_all_single(xr, xs, both[1], both[0])
            ids = torch.repeat_interleave(torch.arange(El, device=dev, dtype=torch.int32).repeat(ws), recv_counts.long(), output_size=xr.shape[0])
            p2 = C.make_plan(ids[:, None], El)
            xg = ext.gather_rows(xr, p2.src_slot, p2.padded_offsets, El, None, 1)
            yr = ext.combine_rows(xg, p2.dest_row, None, 1)
            ys = xs.new_empty(sum(both[0]), H)
            dist.all_to_all_single(ys, yr, both[0], both[1])

        def fused_dispatch_only():
            plan = C.make_plan(top, E, 1, top.numel())
            meta = eng.exchange_counts(plan.tokens_per_expert)
            par = eng.next_phase()
            eng.dispatch(x, plan.src_slot, eos, None, meta, k, par)

        t_f = timed(fused)
        C.check_status(dev)
        t_d = timed(fused_dispatch_only) if args.phases else None
        C.check_status(dev)
        t_n = timed(nccl)
        tot = torch.tensor([bytes_remote], device=dev, dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.MAX)
        mx = float(tot)
        row = {"tokens_per_gpu": T, "n_gpus": ws, "remote_bytes_per_phase_max_rank": mx,
               "fused_ms": round(t_f, 4), "nccl_ms": round(t_n, 4),
               "fused_gbs_per_direction": round(2 * mx / t_f / 1e6, 1), "nccl_gbs_per_direction": round(2 * mx / t_n / 1e6, 1),
               "fused_fraction_of_measured_link": round(2 * mx / t_f / 1e6 / LINK_GBS, 3),
               "speedup_vs_nccl": round(t_n / t_f, 2)}
        if t_d is not None:
            row["fused_dispatch_only_ms"] = round(t_d, 4)
            row["fused_dispatch_gbs"] = round(mx / t_d / 1e6, 1)
        results.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
        del wsp, eng
        torch.cuda.empty_cache()
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        json.dump(results, open(args.out, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
