"""Numerics of every sm_100a kernel against a plain PyTorch fp32 statement of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp(min=1e-12)).item()


def _close(a, b, tol=2e-2, name=""):
    """Norm-wise relative error of the whole tensor, and of every row and every column on its own, so that a
    single wrong row, or one wrong column block, fails although it barely moves the overall norm.  Rows and columns
    are measured against their own norm, floored at a tenth of the typical one (near-zero rows of a reference
    carry no relative information)."""
    err = _rel_err(a, b)
    assert err < tol, f"{name}: relative error {err:.4g} (tolerance {tol})"
    a2, b2 = a.float(), b.float()
    if a2.dim() < 2 or a2.numel() == 0:
        return
    a2, b2 = a2.reshape(-1, a2.shape[-1]), b2.reshape(-1, b2.shape[-1])
    for dim, what in ((1, "row"), (0, "column")):
        ref_norm = b2.norm(dim=dim)
        floor = 0.1 * ref_norm.mean().clamp(min=1e-12)
        rel = (a2 - b2).norm(dim=dim) / ref_norm.clamp(min=floor)
        worst = int(rel.argmax())
        assert float(rel[worst]) < 4 * tol, f"{name}: {what} {worst} relative error {float(rel[worst]):.4g} (tolerance {4 * tol})"


@pytest.fixture(scope="module")
def ops():
    from moe_distributed_training_b200.ops import cuda_ops
    return cuda_ops


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


# ------------------------------------------------------------------------------------------ GEMM family
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (300, 520, 200), (1024, 4096, 4096), (77, 136, 4096)])
def test_gemm_nt(ops, M, N, K):
    torch.manual_seed(0)
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    y = ops.mm_nt(x, w)
    _close(y, x.float() @ w.float().t(), name=f"nt {M}x{N}x{K}")
    ops.check_status(DEV)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (300, 520, 200), (1024, 4096, 1024)])
def test_gemm_nn(ops, M, N, K):
    torch.manual_seed(1)
    x, w = _rand(M, K), _rand(K, N, scale=0.05)
    _close(ops.mm_nn(x, w), x.float() @ w.float(), name=f"nn {M}x{N}x{K}")
    ops.check_status(DEV)


@pytest.mark.parametrize("R,M,N", [(128, 128, 128), (200, 136, 264), (1000, 1024, 4096), (64, 16, 512), (512, 4096, 16)])
def test_gemm_tn(ops, R, M, N):
    torch.manual_seed(2)
    a, b = _rand(R, M), _rand(R, N, scale=0.05)
    _close(ops.mm_tn(a, b), a.float().t() @ b.float(), name=f"tn {R}x{M}x{N}")
    out32 = torch.ones(M, N, device=DEV)
    ops.mm_tn(a, b, out=out32, alpha=0.5, accumulate=True)
    _close(out32, 1.0 + 0.5 * (a.float().t() @ b.float()), name="tn accumulate fp32")
    ops.check_status(DEV)


def test_gemm_lora_segment(ops):
    torch.manual_seed(3)
    M, N, K, r = 300, 512, 1024, 16
    x, w = _rand(M, K), _rand(N, K, scale=0.03)
    t, b = _rand(M, r), _rand(N, r, scale=0.1)
    y = ops.mm_nt(x, w, lora=(t, b))
    _close(y, x.float() @ w.float().t() + t.float() @ b.float().t(), name="nt + lora")
    w2, b2 = _rand(K, N, scale=0.03), _rand(r, N, scale=0.1)
    y2 = ops.mm_nn(x, w2, lora=(t, b2))
    _close(y2, x.float() @ w2.float() + t.float() @ b2.float(), name="nn + lora")
    ops.check_status(DEV)


def _plan(ops, T, k, E, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    logits = torch.randn(T, E, device=DEV, generator=g)
    top = logits.topk(k, dim=-1).indices.int()
    return top, ops.make_plan(top, E)


@pytest.mark.parametrize("T,k,E", [(64, 2, 4), (1000, 2, 8), (5000, 2, 8), (300, 1, 2)])
def test_make_plan(ops, T, k, E):
    from moe_distributed_training_b200.ops import reference
    top, plan = _plan(ops, T, k, E)
    ref = reference.make_plan(top.cpu(), E)
    assert torch.equal(plan.tokens_per_expert.cpu(), ref.tokens_per_expert)
    assert torch.equal(plan.padded_offsets.cpu(), ref.padded_offsets)
    assert torch.equal(plan.dest_row.cpu(), ref.dest_row)
    assert torch.equal(plan.src_slot.cpu(), ref.src_slot)


def test_gather_combine(ops):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(4)
    T, k, E, H = 700, 2, 8, 512
    top, plan = _plan(ops, T, k, E)
    x = _rand(T, H).requires_grad_(True)
    w = torch.rand(T, k, device=DEV).to(torch.bfloat16).requires_grad_(True)
    xg = ops.gather_rows(x, plan)
    n_used = int(plan.padded_offsets[-1])
    ref_xg = reference.gather_rows(x.detach().float(), plan.src_slot, k)
    _close(xg[:n_used], ref_xg[:n_used], 1e-6, "gather")
    y = ops.combine_rows(xg * 1.0, plan, w)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = reference.combine_rows(reference.gather_rows(xr, plan.src_slot, k), plan.dest_row, wr, k)
    _close(y, yr, 1e-2, "combine")
    go = _rand(T, H)
    y.backward(go)
    yr.backward(go.float())
    _close(x.grad, xr.grad, 1e-2, "combine->gather dx")
    _close(w.grad, wr.grad, 2e-2, "combine dweights")


@pytest.mark.parametrize("T,E,H,F,lora", [(600, 4, 256, 512, False), (1500, 8, 1024, 2048, False), (600, 4, 256, 512, True)])
def test_grouped_swiglu_mlp(ops, T, E, H, F, lora):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(5)
    k, r = 2, 16
    top, plan = _plan(ops, T, k, E)
    x = _rand(T, H)
    ws = [(_rand(E, F, H, scale=0.05)).requires_grad_(True) for _ in range(3)]
    lo, lo_ref, lparams = None, None, []
    if lora:
        lo, lo_ref = {}, {}
        for name in ("w1", "w2", "w3"):
            fin, fout = (F, H) if name == "w2" else (H, F)
            A = _rand(E, fin, r, scale=0.05).requires_grad_(True)
            B = _rand(E, r, fout, scale=0.05).requires_grad_(True)
            lparams += [A, B]
            lo[name] = (A, B, 2.0)
    xg = ops.gather_rows(x, plan).detach().requires_grad_(True)
    y = ops.grouped_swiglu_mlp(xg, ws[0], ws[1], ws[2], plan, lo, 0.5)
    # fp32 reference on the same rows
    xr = xg.detach().float().requires_grad_(True)
    wr = [w.detach().float().requires_grad_(True) for w in ws]
    lr_params = []
    if lora:
        lo_ref = {}
        for i, name in enumerate(("w1", "w2", "w3")):
            A, B = lparams[2 * i].detach().float().requires_grad_(True), lparams[2 * i + 1].detach().float().requires_grad_(True)
            lr_params += [A, B]
            lo_ref[name] = (A, B, 2.0)
    yr = reference.grouped_swiglu_mlp(xr, wr[0], wr[1], wr[2], plan.padded_offsets, plan.tokens_per_expert, lo_ref, 0.5)
    n_used = int(plan.padded_offsets[-1])
    valid = (plan.src_slot[:n_used] >= 0)
    _close(y[:n_used][valid], yr[:n_used][valid], 2e-2, "mlp forward")
    go = torch.zeros_like(y)
    go[:n_used][valid] = _rand(int(valid.sum()), H)
    y.backward(go)
    yr.backward(go.float())
    _close(xg.grad[:n_used][valid], xr.grad[:n_used][valid], 3e-2, "mlp dx")
    for i in range(3):
        _close(ws[i].grad, wr[i].grad, 3e-2, f"mlp dw{i + 1}")
    for i, (p, q) in enumerate(zip(lparams, lr_params)):
        _close(p.grad, q.grad, 4e-2, f"mlp lora grad {i}")
    ops.check_status(DEV)


def _under_pair_policy(ops, policy, fn):
    prev = ops.ext.gemm_set_pair_policy(policy)
    try:
        return fn()
    finally:
        ops.ext.gemm_set_pair_policy(prev)


@pytest.mark.parametrize("policy", [2, 4], ids=["pair", "tall"])
def test_gemm_pair_kernel_matches_single_cta_kernel(ops, policy):
    """The CTA-pair (cta_group::2) kernel and the tall 256 x 256 kernel, forced for every 256-wide tile, against
    the 128-row kernel."""
    torch.manual_seed(21)
    cases = []
    for M, N, K in [(300, 520, 200), (1024, 4096, 4096), (77, 264, 4096), (512, 256, 64)]:
        x, w = _rand(M, K), _rand(N, K, scale=0.05)
        cases.append((f"nt {M}x{N}x{K}", lambda x=x, w=w: ops.mm_nt(x, w), x.float() @ w.float().t()))
    x, w = _rand(300, 200), _rand(200, 520, scale=0.05)
    cases.append(("nn", lambda x=x, w=w: ops.mm_nn(x, w), x.float() @ w.float()))
    for R, M, N in [(1000, 1024, 4096), (200, 136, 264)]:
        a, b = _rand(R, M), _rand(R, N, scale=0.05)
        cases.append((f"tn {R}x{M}x{N}", lambda a=a, b=b: ops.mm_tn(a, b), a.float().t() @ b.float()))

        def acc(a=a, b=b):
            out = torch.ones(a.shape[1], b.shape[1], device=DEV)
            ops.mm_tn(a, b, out=out, alpha=0.5, accumulate=True)
            return out
        cases.append((f"tn accumulate {R}x{M}x{N}", acc, 1.0 + 0.5 * (a.float().t() @ b.float())))
    for name, fn, want in cases:
        single = _under_pair_policy(ops, 0, fn)
        pair = _under_pair_policy(ops, policy, fn)
        ops.check_status(DEV)
        _close(pair, want, 2e-2, f"pair kernel {name} vs fp32")
        _close(pair, single, 1e-3, f"pair kernel {name} vs single-CTA kernel")


@pytest.mark.parametrize("policy", [2, 4], ids=["pair", "tall"])
@pytest.mark.parametrize("T,E,H,F,lora", [(600, 4, 256, 512, True), (1500, 8, 1024, 2048, False), (333, 3, 512, 1024, False)])
def test_grouped_mlp_pair_kernel_matches_single_cta_kernel(ops, T, E, H, F, lora, policy):
    """Row groups with odd and even numbers of 128-row blocks (idle second halves), forward and backward."""
    torch.manual_seed(22)
    k, r = 2, 16
    top, plan = _plan(ops, T, k, E)
    x = _rand(T, H)
    ws = [_rand(E, F, H, scale=0.05) for _ in range(3)]
    lo_t = None
    if lora:
        lo_t = {}
        for name in ("w1", "w2", "w3"):
            fin, fout = (F, H) if name == "w2" else (H, F)
            lo_t[name] = (_rand(E, fin, r, scale=0.05), _rand(E, r, fout, scale=0.05), 2.0)
    n_used = int(plan.padded_offsets[-1])
    valid = (plan.src_slot[:n_used] >= 0)
    go = torch.zeros(plan.capacity, H, device=DEV, dtype=torch.bfloat16)
    go[:n_used][valid] = _rand(int(valid.sum()), H)

    def run():
        w = [t.clone().requires_grad_(True) for t in ws]
        lo = None if lo_t is None else {n: (A.clone().requires_grad_(True), B.clone().requires_grad_(True), sc) for n, (A, B, sc) in lo_t.items()}
        xg = ops.gather_rows(x, plan).detach().requires_grad_(True)
        y = ops.grouped_swiglu_mlp(xg, w[0], w[1], w[2], plan, lo, 0.5)
        y.backward(go[:y.shape[0]])
        outs = [y.detach()[:n_used][valid], xg.grad[:n_used][valid]] + [t.grad for t in w]
        if lo is not None:
            for n in ("w1", "w2", "w3"):
                outs += [lo[n][0].grad, lo[n][1].grad]
        return outs
    single = _under_pair_policy(ops, 0, run)
    pair = _under_pair_policy(ops, policy, run)
    ops.check_status(DEV)
    for i, (a, b) in enumerate(zip(pair, single)):
        _close(a, b, 2e-3, f"grouped mlp output {i}: pair vs single-CTA kernel")


# ------------------------------------------------------------------------------------------ small ops
@pytest.mark.parametrize("M,K,r", [(576, 4096, 16), (77, 1024, 8), (1000, 4096, 32), (5, 264, 12)])
def test_skinny_mm(ops, M, K, r):
    torch.manual_seed(30)
    x, A, B = _rand(M, K), _rand(r, K, scale=0.05), _rand(K, r, scale=0.05)
    _close(ops.ext.skinny_mm(x, A, False, 0.5), 0.5 * (x.float() @ A.float().t()), 1e-2, "skinny x A^T")
    _close(ops.ext.skinny_mm(x, B, True, 2.0), 2.0 * (x.float() @ B.float()), 1e-2, "skinny x B")
    xs = _rand(M, K + 64)[:, :K]          # row stride larger than K
    _close(ops.ext.skinny_mm(xs, A, False, 1.0), xs.float() @ A.float().t(), 1e-2, "skinny strided x")


def test_linear_lora_backward(ops):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(6)
    M, K, N, r = 200, 512, 1024, 16
    x = _rand(M, K).requires_grad_(True)
    w = _rand(N, K, scale=0.05).requires_grad_(True)
    A = _rand(r, K, scale=0.05).requires_grad_(True)
    B = _rand(N, r, scale=0.05).requires_grad_(True)
    y = ops.linear(x, w, (A, B, 2.0))
    ref_in = [t.detach().float().requires_grad_(True) for t in (x, w, A, B)]
    yr = reference.linear(ref_in[0], ref_in[1], (ref_in[2], ref_in[3], 2.0))
    _close(y, yr, 2e-2, "linear+lora fwd")
    go = _rand(M, N)
    y.backward(go); yr.backward(go.float())
    for t, rt, name in zip((x, w, A, B), ref_in, "x w A B".split()):
        _close(t.grad, rt.grad, 3e-2, f"linear+lora d{name}")


def test_rmsnorm(ops):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(7)
    x = _rand(333, 4096).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(4096, device=DEV)).to(torch.bfloat16).requires_grad_(True)
    y = ops.rmsnorm(x, w, 1e-5)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = reference.rmsnorm(xr, wr, 1e-5)
    _close(y, yr, 1e-2, "rmsnorm fwd")
    go = _rand(333, 4096)
    y.backward(go); yr.backward(go.float())
    _close(x.grad, xr.grad, 1e-2, "rmsnorm dx")
    _close(w.grad, wr.grad, 2e-2, "rmsnorm dw")


def test_rope(ops):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(8)
    x = _rand(500, 8, 128).requires_grad_(True)
    pos = torch.arange(500, device=DEV, dtype=torch.int32)
    y = ops.rope(x, pos, 1e6)
    xr = x.detach().float().requires_grad_(True)
    yr = reference.rope(xr, pos, 1e6)
    _close(y, yr, 1e-2, "rope fwd")
    go = _rand(500, 8, 128)
    y.backward(go); yr.backward(go.float())
    _close(x.grad, xr.grad, 1e-2, "rope bwd")


def test_router(ops):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(9)
    T, H, E, k = 777, 1024, 8, 2
    x = _rand(T, H).requires_grad_(True)
    w = _rand(E, H, scale=0.05).requires_grad_(True)
    s, wt, idx = ops.router(x, w, k, True)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    sr, wtr, idxr = reference.router(xr, wr, k, True)
    assert (idx == idxr).float().mean() > 0.995
    _close(s, sr, 1e-2, "router scores")
    same = (idx == idxr).all(dim=1)
    _close(wt[same], wtr[same], 1e-2, "router weights")
    go = torch.rand(T, k, device=DEV).to(torch.bfloat16)
    go = go * same[:, None]
    wt.backward(go)
    wtr.backward(go.float())
    _close(x.grad, xr.grad, 3e-2, "router dx")
    _close(w.grad, wr.grad, 3e-2, "router dw")


def test_embedding_and_cross_entropy(ops):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(10)
    T, H, V = 300, 256, 2048
    table = _rand(V, H).requires_grad_(True)
    ids = torch.randint(0, V, (T,), device=DEV)
    e = ops.embedding(ids, table)
    assert torch.equal(e, table.detach()[ids])
    e.backward(torch.ones_like(e))
    ref = torch.zeros(V, H, device=DEV)
    ref.index_add_(0, ids, torch.ones(T, H, device=DEV))
    _close(table.grad, ref, 1e-3, "embedding bwd")
    hidden = _rand(T, H).requires_grad_(True)
    head = _rand(V, H, scale=0.05).requires_grad_(True)
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[: T // 3] = -100
    ls, n = ops.cross_entropy_sum(hidden, head, labels)
    loss = ls / n
    hr, wr = hidden.detach().float().requires_grad_(True), head.detach().float().requires_grad_(True)
    lsr, nr = reference.cross_entropy_sum(hr, wr, labels)
    lossr = lsr / nr
    assert abs(loss.item() - lossr.item()) < 2e-2 * abs(lossr.item())
    assert int(n.item()) == int(nr.item())
    (loss * 3.0).backward(); (lossr * 3.0).backward()
    _close(hidden.grad, hr.grad, 3e-2, "ce dhidden")
    _close(head.grad, wr.grad, 3e-2, "ce dhead")


def test_adamw(ops):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(11)
    shapes = [(1000,), (257, 33), (4096, 512)]
    ps = [_rand(*s) for s in shapes]
    gs = [_rand(*s, scale=0.1) for s in shapes]
    ms = [torch.zeros_like(p) for p in ps]
    vs = [torch.zeros_like(p) for p in ps]
    ref = [[t.clone().float() for t in group] for group in (ps, gs, ms, vs)]
    for step in (1, 2, 3):
        ops.adamw_multi(ps, gs, ms, vs, 1e-2, 0.9, 0.999, 1e-8, 0.01, step, 0.5)
        for p, g, m, v in zip(*ref):
            reference.adamw_step(p, g, m, v, 1e-2, 0.9, 0.999, 1e-8, 0.01, step, 0.5)
    for p, pr in zip(ps, ref[0]):
        _close(p, pr, 1e-2, "adamw param")


def test_adamw_tails_and_fp32_states(ops):
    """Sizes that are not multiples of 8, misaligned views and fp32 moments take the element-wise path."""
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(12)
    base = _rand(8 * 1024 + 13)
    edge = base.clone()
    ps = [base[3:8 * 1024 + 5], _rand(100003), _rand(77)]
    gs = [_rand(p.numel(), scale=0.1) for p in ps]
    ms = [torch.zeros(p.numel(), device=DEV, dtype=torch.float32 if i == 1 else torch.bfloat16) for i, p in enumerate(ps)]
    vs = [torch.zeros_like(m) for m in ms]
    ref = [[t.clone().float() for t in group] for group in (ps, gs, ms, vs)]
    for step in (1, 2):
        ops.adamw_multi(ps, gs, ms, vs, 1e-2, 0.9, 0.999, 1e-8, 0.01, step, 1.0)
        for p, g, m, v in zip(*ref):
            reference.adamw_step(p, g, m, v, 1e-2, 0.9, 0.999, 1e-8, 0.01, step, 1.0)
    for p, pr in zip(ps, ref[0]):
        _close(p, pr, 1e-2, "adamw param (tail)")
    assert torch.equal(base[:3], edge[:3]) and torch.equal(base[8 * 1024 + 5:], edge[8 * 1024 + 5:])  # neighbours untouched


def test_sumsq_and_axpby(ops):
    torch.manual_seed(13)
    for n, dt in ((100003, torch.bfloat16), (8 * 4096, torch.bfloat16), (50001, torch.float32)):
        x = torch.randn(n, device=DEV, dtype=dt)
        out = torch.zeros(1, device=DEV, dtype=torch.float32)
        ops.ext.sumsq(x, out)
        ref = x.double().pow(2).sum().item()
        assert abs(out.item() - ref) <= 1e-3 * ref, (n, dt, out.item(), ref)
    y, x = _rand(100003), _rand(100003)
    want = (0.5 * y.float() + 2.0 * x.float())
    ops.ext.axpby(y, x, 0.5, 2.0)
    _close(y, want, 1e-2, "axpby")


def test_end_to_end_matches_reference_path(ops):
    """One training step of a small bf16 model: CUDA kernels vs the PyTorch statement of every op."""
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.data.synthetic import SyntheticInstructionDataset, batches
    from moe_distributed_training_b200.train.engine import build_engine
    cfg = MixtralConfig(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                        num_attention_heads=2, num_key_value_heads=1, head_dim=128, num_local_experts=4, num_experts_per_tok=2)
    ds = SyntheticInstructionDataset(cfg.vocab_size, 2, 100, 200)
    mbs = list(batches(ds, 1))
    eng = build_engine(cfg, dtype=torch.bfloat16, device_type="cuda", learning_rate=1e-3, seed=0)
    l_gpu = [float(eng.train_step(mbs)["loss"]) for _ in range(3)]
    ref = build_engine(cfg, dtype=torch.float32, device_type="cpu", learning_rate=1e-3, seed=0)
    l_ref = [float(ref.train_step(mbs)["loss"]) for _ in range(3)]
    ops.check_status(DEV)
    for a, b in zip(l_gpu, l_ref):
        assert abs(a - b) < 0.05 * abs(b), (l_gpu, l_ref)
    assert l_gpu[-1] < l_gpu[0]


@pytest.mark.parametrize("lens", [[128], [200], [577], [1024], [100, 300, 77], [256, 256]])
def test_attention(ops, lens):
    from moe_distributed_training_b200.ops import reference
    torch.manual_seed(12)
    T, Hq, Hkv, d = sum(lens), 8, 2, 128
    q, k, v = (_rand(T, h, d).requires_grad_(True) for h in (Hq, Hkv, Hkv))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    o = ops.attention(q, k, v, cu, max(lens))
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf = reference.attention(qr, kr, vr, cu)
    _close(o, orf, 2e-2, f"attention fwd {lens}")
    go = _rand(T, Hq, d)
    o.backward(go); orf.backward(go.float())
    _close(q.grad, qr.grad, 3e-2, "attention dq")
    _close(k.grad, kr.grad, 3e-2, "attention dk")
    _close(v.grad, vr.grad, 3e-2, "attention dv")
    ops.check_status(DEV)


@pytest.mark.parametrize("lora", [False, True])
def test_fused_attention_block_matches_composed_ops(ops, lora):
    """The single-node attention sub-block against the same layer evaluated op by op."""
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.models.mixtral import MixtralDecoderLayer, PackedBatch, moe_args_from_config
    from moe_distributed_training_b200.ops import fused_blocks
    torch.manual_seed(13)
    cfg = MixtralConfig(vocab_size=512, hidden_size=512, intermediate_size=512, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=128, num_local_experts=2, num_experts_per_tok=1)
    layer = MixtralDecoderLayer(cfg, moe_args_from_config(cfg, torch.bfloat16, DEV), torch.bfloat16, DEV)
    with torch.no_grad():
        for n, p in layer.named_parameters():
            if "layernorm" in n:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            else:
                p.normal_(0, 0.05)
    if lora:
        for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.o_proj):
            lin.add_lora(16, 32)
            with torch.no_grad():
                lin.lora_B["default"].weight.normal_(0, 0.05)
    lens = [150, 300]
    T = sum(lens)
    cu = torch.tensor([0, 150, 450], dtype=torch.int32, device=DEV)
    pos = torch.cat([torch.arange(n, device=DEV) for n in lens]).int()
    batch = PackedBatch(cu, pos, max(lens))
    x1 = _rand(T, 512).requires_grad_(True)
    x2 = x1.detach().clone().requires_grad_(True)
    params = [p for n, p in layer.named_parameters() if "block_sparse_moe" not in n and "post_attention" not in n and p.requires_grad]
    y1 = fused_blocks.attention_block(layer, x1, batch)
    y2 = x2 + layer.self_attn(layer.input_layernorm(x2), batch)
    _close(y1, y2, 1e-2, "fused attention block fwd")
    go = _rand(T, 512)
    g1 = torch.autograd.grad(y1, [x1] + params, go)
    g2 = torch.autograd.grad(y2, [x2] + params, go)
    for a, b, n in zip(g1, g2, ["x"] + [str(i) for i in range(len(params))]):
        _close(a, b, 2e-2, f"fused attention block grad {n}")
    ops.check_status(DEV)


@pytest.mark.parametrize("lora", [False, True])
def test_fused_moe_block_matches_composed_ops(ops, lora):
    """The single-node MoE sub-block (local experts) against the same layer evaluated op by op."""
    from moe_distributed_training_b200 import MixtralConfig
    from moe_distributed_training_b200.models.mixtral import MixtralDecoderLayer, moe_args_from_config
    from moe_distributed_training_b200.ops import fused_blocks
    from moe_distributed_training_b200.peft.lora import add_expert_lora
    torch.manual_seed(14)
    cfg = MixtralConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, head_dim=128, num_local_experts=4, num_experts_per_tok=2)
    layer = MixtralDecoderLayer(cfg, moe_args_from_config(cfg, torch.bfloat16, DEV), torch.bfloat16, DEV)
    with torch.no_grad():
        for n, p in layer.named_parameters():
            if "layernorm" in n:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            else:
                p.normal_(0, 0.05)
    if lora:
        add_expert_lora(layer.block_sparse_moe.experts, 16, 32)
        with torch.no_grad():
            for p in layer.block_sparse_moe.experts.lora.lora_B.values():
                p.normal_(0, 0.05)
    T = 700
    x1 = _rand(T, 512).requires_grad_(True)
    x2 = x1.detach().clone().requires_grad_(True)
    params = [p for n, p in layer.named_parameters() if ("block_sparse_moe" in n or "post_attention" in n) and p.requires_grad]
    assert fused_blocks.moe_block_supported(layer, x1)
    y1 = fused_blocks.moe_block(layer, x1)
    g1 = torch.autograd.grad(y1, [x1] + params, torch.ones_like(y1) * 0.01, allow_unused=True)
    direct = {id(p): p.grad.clone() for p in params if p.grad is not None}     # expert weights accumulate straight into .grad
    for p in params:
        p.grad = None
    moe_out, _ = layer.block_sparse_moe(layer.post_attention_layernorm(x2))
    y2 = x2 + moe_out
    _close(y1, y2, 1e-2, "fused moe block fwd")
    g2 = torch.autograd.grad(y2, [x2] + params, torch.ones_like(y2) * 0.01, allow_unused=True)
    for i, (a, b, p) in enumerate(zip(g1, g2, [None] + params)):
        if a is None and p is not None:
            a = direct.get(id(p))
        if b is None and p is not None and p.grad is not None:
            b = p.grad
        assert (a is None) == (b is None), i
        if a is not None:
            _close(a, b, 3e-2, f"fused moe block grad {i}")
    ops.check_status(DEV)


def test_group_bwd_ab_direct_products_match_fp32():
    """The reference-named LoRA gradient entry point: four grouped-GEMM launches, full reductions over K and N."""
    from scattermoe_utils.kernels.ops import group_bwd_AB, padded_block_indices
    torch.manual_seed(21)
    E, K, N, r, s = 3, 384, 640, 16, 2.0
    counts = [300, 0, 212]
    M = sum(counts)
    X = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    DY = torch.randn(M, N, device=DEV).to(torch.bfloat16)
    A = (torch.randn(E, K, r, device=DEV) * 0.1).to(torch.bfloat16)
    B = (torch.randn(E, r, N, device=DEV) * 0.1).to(torch.bfloat16)
    offs = torch.tensor(counts, device=DEV).cumsum(0)
    dA, dB = group_bwd_AB(DY, X, A, B, s, offs, E)
    lo = 0
    for e, c in enumerate(counts):
        xe, dye = X[lo:lo + c].float(), DY[lo:lo + c].float()
        wantA = s * xe.t() @ (dye @ B[e].float().t()).to(torch.bfloat16).float()
        wantB = s * (xe @ A[e].float()).to(torch.bfloat16).float().t() @ dye
        if c == 0:
            assert float(dA[e].float().abs().max()) == 0 and float(dB[e].float().abs().max()) == 0
        else:
            _close(dA[e], wantA, 3e-2, f"dA[{e}]")
            _close(dB[e], wantB, 3e-2, f"dB[{e}]")
        lo += c
    ids = torch.repeat_interleave(torch.arange(E, device=DEV), torch.tensor(counts, device=DEV))
    pbi, eo = padded_block_indices(ids, E)
    assert pbi.tolist() == [0, 128, 256, 300, 428] and eo.tolist() == [300, 300, 512]


def test_residual_connections_fused_into_their_producers(ops):
    """x + f(x) without a separate add: the GEMM epilogue, the gate-weighted combine and the RMSNorm backward take the
    residual (or its gradient) as an extra input; the router backward adds into an existing gradient."""
    torch.manual_seed(31)
    ext = ops.ext
    M, K, N = 333, 512, 768
    x, w, res = _rand(M, K), _rand(N, K, scale=0.05), _rand(M, N)
    for policy in (0, 4):                                   # 128-row tiles and the tall kernel (coalescing epilogue off)
        prev = ext.gemm_set_pair_policy(policy)
        try:
            got = ops.mm_nt(x, w, residual=res)
        finally:
            ext.gemm_set_pair_policy(prev)
        _close(got, x.float() @ w.float().t() + res.float(), name=f"gemm + residual (policy {policy})")
    # combine
    T, k, H = 200, 2, 256
    y = _rand(T * k + 56, H)
    dest = torch.randperm(T * k + 56, device=DEV)[:T * k].int()
    wts = torch.rand(T, k, device=DEV).to(torch.bfloat16)
    r2 = _rand(T, H)
    got = ext.combine_rows(y, dest, wts, k, r2)
    want = (y.float()[dest.long()].view(T, k, H) * wts.float()[:, :, None]).sum(1) + r2.float()
    _close(got, want, name="combine + residual")
    # rmsnorm backward + residual gradient, and the weight gradient finished in one launch
    R, C = 300, 512
    xx, ww, dy, dres = _rand(R, C), (1 + 0.1 * torch.randn(C, device=DEV)).to(torch.bfloat16), _rand(R, C), _rand(R, C)
    _, rstd = ext.rmsnorm_fwd(xx, ww, 1e-5)
    dx, dwp = ext.rmsnorm_bwd(xx, ww, dy, rstd, dres)
    xf = xx.float().requires_grad_(True)
    wf = ww.float().requires_grad_(True)
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    yf.backward(dy.float())
    _close(dx, xf.grad + dres.float(), name="rmsnorm dx + residual gradient")
    _close(ext.rmsnorm_dw(dwp, ww)[None], wf.grad[None], 3e-2, name="rmsnorm dw")
    # router backward accumulating into an existing gradient
    Tk, Hh, E = 150, 256, 8
    xr, wr = _rand(Tk, Hh), _rand(E, Hh, scale=0.1)
    _, _, idx = ext.router_fwd(xr, wr, 2, True)
    dwts = _rand(Tk, 2)
    dx_plain, _ = ext.router_bwd(xr, wr, idx, dwts, None, True)
    base = _rand(Tk, Hh)
    acc = base.clone()
    ext.router_bwd(xr, wr, idx, dwts, None, True, acc)
    _close(acc, base.float() + dx_plain.float(), name="router dx accumulate")


def test_deterministic_kernels_are_bitwise_reproducible(ops):
    """Routing plan, row gather, the GEMM family (dense, row-grouped with fused SwiGLU, depth-grouped), RMSNorm and
    the gate-weighted combine use no atomics on their results: two runs on the same inputs agree bit for bit."""
    torch.manual_seed(41)
    ext = ops.ext
    T, k, E, H, F = 900, 2, 4, 512, 1024
    x = _rand(T, H)
    top = torch.randn(T, E, device=DEV).topk(k, -1).indices.int()
    w1, w2, w3 = (_rand(E, F, H, scale=0.05) for _ in range(3))
    wts = torch.rand(T, k, device=DEV).to(torch.bfloat16)

    def run():
        plan = ops.make_plan(top, E)
        xg = ext.gather_rows(x, plan.src_slot, plan.padded_offsets, E, None, k)
        y = ops.grouped_swiglu_mlp(xg, w1, w2, w3, plan)
        out = ext.combine_rows(y, plan.dest_row, wts, k, x)
        dw = torch.empty(E, F, H, dtype=torch.bfloat16, device=DEV)
        ops._g(2, y.new_zeros(xg.shape[0], F) + 1, True, xg, True, dw, H, 0, plan)
        dense = ops.mm_nt(x, w1[0])
        xn, rstd = ext.rmsnorm_fwd(x, torch.ones(H, dtype=torch.bfloat16, device=DEV), 1e-5)
        used = int(plan.padded_offsets[-1])      # rows past the padded groups are never written
        return [plan.tokens_per_expert, plan.padded_offsets, plan.dest_row, plan.src_slot, xg[:used], y[:used], out, dw, dense, xn, rstd]

    a, b = run(), run()
    torch.cuda.synchronize()
    for i, (p, q) in enumerate(zip(a, b)):
        assert torch.equal(p, q), f"output {i} differs between two runs"
    ops.check_status(DEV)


def test_router_kernel_histogram_and_score_sums(ops):
    """The router kernel's optional statistics (per-expert slot counts and score sums, the f_e and P_e of the
    load-balancing loss) against a count and a sum over its own outputs; the loss built from them equals the plain one."""
    from moe_distributed_training_b200.ops.reference import load_balancing_loss
    torch.manual_seed(51)
    for (T, H, E, k) in [(700, 512, 8, 2), (37, 256, 16, 4)]:
        x, w = _rand(T, H), _rand(E, H, scale=0.2)
        scores, weights, idx, stats = ops.ext.router_fwd(x, w, k, True, True)
        counts = torch.bincount(idx.reshape(-1).long(), minlength=E).float()
        assert torch.equal(stats[:E], counts)
        assert torch.allclose(stats[E:], scores.float().sum(0), rtol=1e-4, atol=1e-3)
        s2, w2, i2 = ops.ext.router_fwd(x, w, k, True)
        assert torch.equal(s2, scores) and torch.equal(i2, idx) and torch.equal(w2, weights)
        f = stats[:E] / (T * k)
        loss = E * torch.sum(f * scores.float().mean(0))
        assert torch.allclose(loss, load_balancing_loss(scores.float(), idx, E, k), rtol=1e-5)


def test_gemm_last_round_shared_along_the_depth(ops):
    """Products whose last round of 128-row tiles would leave most SMs idle: the k blocks of that round are cut into one
    piece per SM, partial sums meet in an fp32 workspace, the last contributor of each tile quarter finishes it.  Checked
    against fp32 and against the same product with the sharing switched off, for the epilogue variants that can meet it
    (plain, LoRA segment, residual, fp32 accumulation, MN-major weights, row groups), twice in a row (the workspace
    must come back clean)."""
    ext = ops.ext
    torch.manual_seed(61)
    prev_policy = ext.gemm_set_pair_policy(0)          # the 128-row kernel
    try:
        for (M, N, K) in [(1280, 4096, 2048), (576, 4096, 1024), (576, 1024, 4096), (200, 2048, 8192)]:
            x, w = _rand(M, K), _rand(N, K, scale=0.05)
            want = x.float() @ w.float().t()
            for rep in range(2):
                _close(ops.mm_nt(x, w), want, name=f"split nt {M}x{N}x{K} run {rep}")
            old = ext.gemm_set_split(0)
            try:
                unsplit = ops.mm_nt(x, w)
            finally:
                ext.gemm_set_split(old)
            _close(ops.mm_nt(x, w), unsplit.float(), 1e-2, name=f"split vs unsplit {M}x{N}x{K}")
        M, N, K, r = 576, 4096, 1024, 16
        x, w, res = _rand(M, K), _rand(N, K, scale=0.05), _rand(M, N)
        t, b = _rand(M, r), _rand(N, r, scale=0.1)
        _close(ops.mm_nt(x, w, lora=(t, b), residual=res), x.float() @ w.float().t() + t.float() @ b.float().t() + res.float(),
               name="split + lora + residual")
        w2 = _rand(K, N, scale=0.05)
        out32 = torch.ones(M, N, device=DEV)
        ops._gemm(0, x, False, w2, True, out32, M, N, K, accumulate=True, alpha=0.5)
        _close(out32, 1.0 + 0.5 * (x.float() @ w2.float()), name="split + fp32 accumulate, MN-major weights")
        # row groups (expert down projection): 3 experts
        E, F, H = 3, 2048, 4096
        top = (torch.arange(700, device=DEV) % E).int()[:, None]
        plan = ops.make_plan(top, E)
        hg = _rand(int(plan.src_slot.numel()), F)
        w2g = _rand(E, F, H, scale=0.03)
        y = torch.empty(hg.shape[0], H, dtype=torch.bfloat16, device=DEV)
        ops._g(1, hg, False, w2g, True, y, H, F, plan)
        offs = plan.padded_offsets.tolist()
        for e in range(E):
            a, bnd = offs[e], offs[e + 1]
            _close(y[a:bnd], hg[a:bnd].float() @ w2g[e].float(), name=f"split grouped rows, expert {e}")
    finally:
        ext.gemm_set_pair_policy(prev_policy)
    ops.check_status(DEV)


def test_multi_tensor_gradient_accumulate(ops):
    """fp32 accumulators += bf16 / fp32 gradients of many tensors in one launch per 16."""
    torch.manual_seed(71)
    shapes = [(16, 4096), (4096, 16), (1024, 16), (16, 1024), (7,), (3, 5, 11)] * 4      # 24 tensors: two launches
    dst = [torch.randn(*s_, device=DEV) for s_ in shapes]
    src = [(torch.randn(*s_, device=DEV).to(torch.bfloat16) if i % 3 else torch.randn(*s_, device=DEV)) for i, s_ in enumerate(shapes)]
    want = [d + s_.float() for d, s_ in zip(dst, src)]
    ops.ext.multi_add(dst, src)
    for got, w in zip(dst, want):
        assert torch.equal(got, w)
