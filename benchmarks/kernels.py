"""Isolated timings of the sm_100a kernels at Mixtral-8x7B shapes.

    python benchmarks/kernels.py [--tokens 1152] [--experts 1] [--out file.json]

Each kernel is timed with CUDA events after warm-up; between timed launches a
buffer larger than L2 is overwritten so that inputs come from HBM.  Fractions
are relative to the measured copy / cuBLAS peaks in MEASURED_PEAKS.json when
that file exists.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timeit(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.add_(1.0)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1152)
    ap.add_argument("--experts", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--out", default="")
    ap.add_argument("--split", action="store_true",
                    help="only compare products with and without sharing the last round of tiles along the depth")
    ap.add_argument("--tilings", action="store_true",
                    help="only compare the three GEMM tilings (128-row, CTA pair, tall) on a few shapes")
    args = ap.parse_args()
    from moe_distributed_training_b200.ops import cuda_ops as ops
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak_tf = peaks.get("bf16_tflops", 1590.0)
    peak_bw = peaks.get("hbm_gbs", 6650.0)
    dev = "cuda"
    flush = torch.zeros(96 * 1024 * 1024, device=dev)  # 384 MB > 126 MB L2
    T, E, H, F = args.tokens, args.experts, args.hidden, args.ffn
    res = {"tokens": T, "experts": E, "peaks": {"bf16_tflops": peak_tf, "hbm_gbs": peak_bw, "source": "measured" if peaks else "fallback"}}
    bf = torch.bfloat16

    def report(name, ms, flops=0, bytes_=0):
        r = {"ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1); r["frac_of_gemm_peak"] = round(flops / ms / 1e9 / peak_tf, 3)
        if bytes_:
            r["gbs"] = round(bytes_ / ms / 1e6, 1); r["frac_of_copy_peak"] = round(bytes_ / ms / 1e6 / peak_bw, 3)
        res[name] = r
        print(name, r, flush=True)

    if args.split:
        for (M, N, K) in [(576, 4096, 4096), (576, 1024, 4096), (1152, 4096, 4096), (1152, 4096, 14336), (1280, 4096, 14336),
                          (1408, 4096, 14336), (1280, 4096, 28672), (1152, 14336, 4096), (576, 4096, 1024)]:
            x, w = torch.randn(M, K, device=dev, dtype=bf) * 0.1, torch.randn(N, K, device=dev, dtype=bf) * 0.1
            out = torch.empty(M, N, device=dev, dtype=bf)
            prev_policy = ops.ext.gemm_set_pair_policy(0)
            for name, on in (("shared_last_round", 1), ("whole_tiles_only", 0)):
                old = ops.ext.gemm_set_split(on)
                report(f"gemm_nt_{M}x{N}x{K}_{name}", timeit(lambda: ops.mm_nt(x, w, out=out), flush=flush), flops=2.0 * M * N * K)
                ops.ext.gemm_set_split(old)
            ops.ext.gemm_set_pair_policy(prev_policy)
            report(f"gemm_nt_{M}x{N}x{K}_default_choice", timeit(lambda: ops.mm_nt(x, w, out=out), flush=flush), flops=2.0 * M * N * K)
            report(f"cublas_nt_{M}x{N}x{K}", timeit(lambda: torch.matmul(x, w.t(), out=out), flush=flush), flops=2.0 * M * N * K)
            del x, w, out
        ops.check_status(dev)
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            json.dump(res, open(args.out, "w"), indent=1)
        return

    if args.tilings:
        for (M, N, K) in [(8192, 8192, 8192), (8192, 8192, 512), (1152, 4096, 4096), (1280, 14336, 4096), (1280, 4096, 14336),
                          (4096, 4096, 4096)]:
            x, w = torch.randn(M, K, device=dev, dtype=bf) * 0.1, torch.randn(N, K, device=dev, dtype=bf) * 0.1
            out = torch.empty(M, N, device=dev, dtype=bf)
            for name, policy in (("tile128", 0), ("pair", 2), ("tall", 4)):
                prev = ops.ext.gemm_set_pair_policy(policy)
                report(f"gemm_nt_{M}x{N}x{K}_{name}", timeit(lambda: ops.mm_nt(x, w, out=out), flush=flush), flops=2.0 * M * N * K)
                ops.ext.gemm_set_pair_policy(prev)
            del x, w, out
        ops.check_status(dev)
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            json.dump(res, open(args.out, "w"), indent=1)
        return

    # dense GEMMs (attention projections at T tokens) and a square reference point
    for (M, N, K) in [(8192, 8192, 8192), (T, 4096, 4096), (T, 32000, 4096)]:
        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)
        report(f"gemm_nt_{M}x{N}x{K}", timeit(lambda: ops.mm_nt(x, w, out=out), flush=flush), flops=2.0 * M * N * K)
        report(f"cublas_nt_{M}x{N}x{K}", timeit(lambda: torch.matmul(x, w.t(), out=out), flush=flush), flops=2.0 * M * N * K)
        del x, w, out

    # grouped expert MLP: rows spread evenly over E experts
    rows = T
    top = (torch.arange(rows, device=dev) % E).int()[:, None]
    plan = ops.make_plan(top, E)
    x = torch.randn(rows, H, device=dev, dtype=bf)
    xg = ops.gather_rows(x, plan)
    w1 = torch.randn(E, F, H, device=dev, dtype=bf) * 0.02
    w2 = torch.randn(E, F, H, device=dev, dtype=bf) * 0.02
    w3 = torch.randn(E, F, H, device=dev, dtype=bf) * 0.02
    padded = int(plan.padded_offsets[-1])
    with torch.no_grad():
        ms = timeit(lambda: ops.grouped_swiglu_mlp(xg, w1, w2, w3, plan), flush=flush)
    report("expert_mlp_fwd", ms, flops=6.0 * padded * H * F, bytes_=3 * E * F * H * 2)
    xg2 = xg.clone().requires_grad_(True)
    for w in (w1, w2, w3):
        w.requires_grad_(True)

    def fwd_bwd():
        y = ops.grouped_swiglu_mlp(xg2, w1, w2, w3, plan)
        y.backward(y)
        w1.grad = w2.grad = w3.grad = None
    report("expert_mlp_fwd_bwd_full", timeit(fwd_bwd, iters=5, flush=flush), flops=18.0 * padded * H * F)

    # causal GQA attention, one sequence of T tokens and one of 1024 (32 query heads, 8 key/value heads, head_dim 128);
    # FLOPs = the causal half of 4 * T^2 * 128 per head (forward), 2.5x that for the backward pass
    for Ta in sorted({T, 1024}):
        q = torch.randn(Ta, 32, 128, device=dev, dtype=bf)
        k = torch.randn(Ta, 8, 128, device=dev, dtype=bf)
        v = torch.randn(Ta, 8, 128, device=dev, dtype=bf)
        cu = torch.tensor([0, Ta], device=dev, dtype=torch.int32)
        fl = 4.0 * Ta * Ta * 128 * 32 / 2
        o, lse = ops.ext.attention_fwd(q, k, v, cu, Ta, 128 ** -0.5)
        report(f"attention_fwd_T{Ta}", timeit(lambda: ops.ext.attention_fwd(q, k, v, cu, Ta, 128 ** -0.5), flush=flush), flops=fl)
        do = torch.randn_like(o)
        report(f"attention_bwd_T{Ta}", timeit(lambda: ops.ext.attention_bwd(q, k, v, o, do, lse, cu, Ta, 128 ** -0.5), flush=flush), flops=2.5 * fl)

    # memory-bound kernels
    xx = torch.randn(T, H, device=dev, dtype=bf)
    g = torch.ones(H, device=dev, dtype=bf)
    report("rmsnorm_fwd", timeit(lambda: ops.ext.rmsnorm_fwd(xx, g, 1e-5), flush=flush), bytes_=2 * T * H * 2)
    n = 250 * 1000 * 1000   # not a power of two: four power-of-two sized arrays would start on the same memory channel
    p, gr, m, v = (torch.zeros(n, device=dev, dtype=bf) for _ in range(4))
    report("adamw_250M", timeit(lambda: ops.adamw_multi([p], [gr], [m], [v], 1e-3, 0.9, 0.999, 1e-8, 0.01, 1), iters=5), bytes_=7 * n * 2)
    ops.check_status(dev)
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        json.dump(res, open(args.out, "w"), indent=1)


if __name__ == "__main__":
    main()
