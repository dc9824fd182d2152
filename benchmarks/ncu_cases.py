"""Small single-GPU cases for profiler captures: one kernel family per case, a handful of launches.

    python benchmarks/ncu_cases.py gemm|gemm_pair|gemm_split|gather_gemm|rs_block|expert_mlp|attention|dispatch|gemm_exchange

Sizes keep the working set above the 126 MB L2 where DRAM figures matter, but far below a GB of launches.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    case = sys.argv[1]
    from moe_distributed_training_b200.ops import cuda_ops as C
    dev, bf = "cuda", torch.bfloat16
    torch.manual_seed(0)
    if case in ("gemm", "gemm_pair"):
        x = torch.randn(8192, 4096, device=dev, dtype=bf)
        w = torch.randn(8192, 4096, device=dev, dtype=bf)
        out = torch.empty(8192, 8192, device=dev, dtype=bf)
        C.ext.gemm_set_pair_policy(2 if case == "gemm_pair" else 0)   # CTA-pair kernel or single-CTA kernel
        for _ in range(4):
            C.mm_nt(x, w, out=out)
    elif case == "gemm_split":
        # down-projection shape of one micro-batch: 10 x 16 = 160 tiles on 148 SMs, the last round shared along the depth
        x = torch.randn(1280, 14336, device=dev, dtype=bf)
        w = torch.randn(4096, 14336, device=dev, dtype=bf) * 0.02
        out = torch.empty(1280, 4096, device=dev, dtype=bf)
        C.ext.gemm_set_pair_policy(0)
        for _ in range(4):
            C.mm_nt(x, w, out=out)
    elif case == "gather_gemm":
        # The all-gather of one decoder block's attention weights (8 emulated shards, 84 MB) runs on a side stream and
        # publishes its progress; the q projection on the main stream finds its weight in the registry of gathered
        # buffers and waits, tile by tile, for the chunks it needs.
        ws_, H, T = 8, 4096, 1152
        C.ext.set_peer_wait_limit_ms(500)       # a wait that could not be satisfied would end quickly, also under a profiler
        n_el = (4096 + 1024 + 1024 + 4096) * H
        shard = n_el // ws_
        full = torch.randn(n_el, device=dev, dtype=bf) * 0.02
        shards = [full[r * shard:(r + 1) * shard].clone() for r in range(ws_)]
        table = torch.tensor([t.data_ptr() for t in shards], dtype=torch.int64, device=dev)
        nflags, _ = C.ext.ag_chunks(ws_, shard * 2)
        ready = torch.zeros(nflags, dtype=torch.int32, device=dev)
        out = torch.zeros(n_el, device=dev, dtype=bf)
        x = torch.randn(T, H, device=dev, dtype=bf)
        side = torch.cuda.Stream()
        for epoch in range(1, 4):
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                C.ext.ag_pull_flagged(out, table, ws_, 0, shard * 2, ready, epoch, 1)
            C.mm_nt(x, out[:H * H].view(H, H))
        C.ext.gather_registry_clear()
    elif case == "expert_mlp":
        E, F, H, rows = 1, 14336, 4096, 1152
        top = torch.zeros(rows, 1, dtype=torch.int32, device=dev)
        plan = C.make_plan(top, E)
        xg = C.ext.gather_rows(torch.randn(rows, H, device=dev, dtype=bf), plan.src_slot, plan.padded_offsets, E, None, 1)
        w1, w2, w3 = (torch.randn(E, F, H, device=dev, dtype=bf) * 0.02 for _ in range(3))
        with torch.no_grad():
            for _ in range(3):
                C.grouped_swiglu_mlp(xg, w1, w2, w3, plan)
    elif case == "attention":
        T, Hq, Hkv, d = 1024, 32, 8, 128
        q = torch.randn(T, Hq, d, device=dev, dtype=bf, requires_grad=True)
        k = torch.randn(T, Hkv, d, device=dev, dtype=bf, requires_grad=True)
        v = torch.randn(T, Hkv, d, device=dev, dtype=bf, requires_grad=True)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        for _ in range(3):
            o = C.attention(q, k, v, cu, T)
            o.backward(o)
    elif case == "dispatch":
        from moe_distributed_training_b200.parallel import symm
        ws, E, k, H, T = 2, 8, 2, 4096, 8192
        spaces = symm.emulate_ep_workspaces(ws, E, H, T, k, dev)
        status = C.status_tensor(dev)
        xs = [torch.randn(T, H, device=dev, dtype=bf) for _ in range(ws)]
        tops = [torch.randn(T, E, device=dev).topk(k, -1).indices.int() for _ in range(ws)]
        plans = [C.make_plan(tp, E, 1, tp.numel()) for tp in tops]
        off = [int(v) for v in C.ext.ep_meta_offsets(ws, E)]
        metas = [torch.zeros(off[8], dtype=torch.int32, device=dev) for _ in range(ws)]
        for epoch in (1, 2, 3):
            par = epoch & 1
            for r, w in enumerate(spaces):
                C.ext.ep_counts_send(plans[r].tokens_per_expert, w.peer_base, w.layout, r, par, epoch)
            for r, w in enumerate(spaces):
                C.ext.ep_counts_wait_meta(w.my_base, w.layout, r, par, epoch, metas[r], status)
            for r, w in enumerate(spaces):
                C.ext.ep_dispatch(xs[r], plans[r].src_slot, tops[r].reshape(-1).contiguous(), None, metas[r], w.peer_base, w.layout, r, k, par, status)
            for r, w in enumerate(spaces):
                C.ext.ep_recv_prepare(w.my_base, w.layout, metas[r], H, par, status, True)
            for r, w in enumerate(spaces):
                C.ext.ep_combine_send(w.recv_x(), metas[r], w.peer_base, w.layout, r, w.capacity_rows, par, status)
            for r, w in enumerate(spaces):
                C.ext.ep_wait_rows(w.my_base, w.layout, metas[r], par, status, 1)
    elif case == "gemm_exchange":
        # The down-projection-shaped grouped GEMM as it runs inside the expert-parallel exchange: its producer waits
        # per 128-row tile on counters the dispatch kernel raised, and its epilogue stores every result row into the
        # buffer of the rank that sent the token and raises that rank's arrival counter.  Two ranks emulated on one
        # GPU: both ranks' sends are issued before any GEMM, so no launch waits for a later one.
        from moe_distributed_training_b200.ops.reference import RoutingPlan
        from moe_distributed_training_b200.parallel import symm
        ws, E, k, H, N, T = 2, 2, 2, 4096, 4096, 4096
        El = E // ws
        spaces_out = symm.emulate_ep_workspaces(ws, E, N, T, k, dev)
        spaces_in = symm.emulate_ep_workspaces(ws, E, H, T, k, dev)
        status = C.status_tensor(dev)
        W = torch.randn(E, N, H, device=dev, dtype=bf) * 0.02
        xs = [torch.randn(T, H, device=dev, dtype=bf) for _ in range(ws)]
        tops = [torch.randn(T, E, device=dev).topk(k, -1).indices.int() for _ in range(ws)]
        plans = [C.make_plan(tp, E, 1, tp.numel()) for tp in tops]
        off = [int(v) for v in C.ext.ep_meta_offsets(ws, E)]
        metas = [torch.zeros(off[8], dtype=torch.int32, device=dev) for _ in range(ws)]
        for epoch in (1, 2, 3):
            par = epoch & 1
            for r, w in enumerate(spaces_in):
                C.ext.ep_counts_send(plans[r].tokens_per_expert, w.peer_base, w.layout, r, par, epoch)
            for r, w in enumerate(spaces_in):
                C.ext.ep_counts_wait_meta(w.my_base, w.layout, r, par, epoch, metas[r], status)
            for r, w in enumerate(spaces_in):
                C.ext.ep_dispatch(xs[r], plans[r].src_slot, tops[r].reshape(-1).contiguous(), None, metas[r], w.peer_base, w.layout, r, k, par, status)
            for r, w in enumerate(spaces_in):
                C.ext.ep_recv_prepare(w.my_base, w.layout, metas[r], H, par, status, False)
            for r, (wi, wo) in enumerate(zip(spaces_in, spaces_out)):
                rr, rp, te = C.ext.ep_fused_meta(metas[r], wi.layout, r)
                m = metas[r]
                rplan = RoutingPlan(m[off[1]:off[1] + El], m[off[2]:off[2] + El + 1], None, None, 1, El, capacity_rows=wi.capacity_rows)
                peer_out = torch.tensor([b + wo.layout[9] for b in wo.bases], dtype=torch.int64, device=dev)
                peer_arr = torch.tensor([b + wo.layout[7] + 4 * par for b in wo.bases], dtype=torch.int64, device=dev)
                dummy = torch.empty(wi.capacity_rows, N, dtype=bf, device=dev)
                C._g(1, wi.recv_x(), False, W[r * El:(r + 1) * El], False, dummy, N, H, rplan,
                     wait=(wi.tile_counters(par), te), scatter=(rr, rp, peer_out, peer_arr))
            for r, wo in enumerate(spaces_out):
                C.ext.ep_wait_rows(wo.my_base, wo.layout, metas[r], par, status, (N + 255) // 256)
    elif case == "rs_block":
        # Gradient reduce-scatter of one decoder block's attention parameters (full fine-tune: 42 M fp32 accumulator
        # elements per rank) as one kernel: announce, wait for the peers' announcements, read this rank's slice of
        # every rank's accumulator with 16-byte loads, scale, cast to bf16, add to the shard gradient.  Eight ranks
        # emulated on one GPU: their kernels run one after another, so all announcements are written beforehand and
        # no launch waits for a later one.
        ws_ = 8
        n = (4096 + 1024 + 1024 + 4096) * 4096 // ws_
        C.ext.set_peer_wait_limit_ms(500)
        fulls = [torch.randn(ws_ * n, device=dev) for _ in range(ws_)]
        ftable = torch.tensor([f.data_ptr() for f in fulls], dtype=torch.int64, device=dev)
        flags = [torch.zeros(8 * ws_, dtype=torch.int32, device=dev) for _ in range(ws_)]
        flag_table = torch.tensor([f.data_ptr() for f in flags], dtype=torch.int64, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        shard = torch.zeros(n, dtype=bf, device=dev)
        flush = torch.zeros(96 * 1024 * 1024, device=dev)
        times = []
        for epoch in range(1, 6):
            for f in flags:
                f.view(8, ws_)[3].fill_(epoch)
            flush.add_(1.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            C.ext.rs_block(shard, ftable, flag_table, flags[0].data_ptr(), 3, ws_, 0, True, 1.0 / ws_, True, epoch, status)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = sorted(times)[len(times) // 2]
        print(f"rs_block: {ws_} x {n * 4 / 1e6:.1f} MB read, {n * 2 / 1e6:.1f} MB written in {ms:.4f} ms = {(ws_ * n * 4 + 2 * n * 2) / ms / 1e6:.0f} GB/s")
        assert int(status.item()) == 0
    else:
        raise SystemExit("unknown case")
    torch.cuda.synchronize()
    C.check_status(dev)
    print("ok", case)


if __name__ == "__main__":
    main()
