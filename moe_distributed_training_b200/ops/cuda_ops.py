"""CUDA implementations of the ops: autograd wrappers over the in-tree sm_100a extension.

Every matrix product here is one launch of the tcgen05 GEMM family in
`csrc/gemm_sm100.cu` (dense, row-grouped, depth-grouped; K-major or MN-major
operands; optional LoRA depth segment; optional fused SwiGLU), so forward,
input-gradient and weight-gradient products all run on the same kernel without
materialised transposes.  Importing this module fails if the extension has not
been built: there is no silent PyTorch fallback for CUDA tensors.
"""
from __future__ import annotations


import torch

from . import build as _build
from .reference import BLOCK_ROWS, RoutingPlan, plan_capacity

ext = _build.load()

# Limit of every device-side wait for a peer (counts, rows, chunks of a gather, announcements of a reduction): 10 s by
# default, which covers start-up skew; MDT_PEER_WAIT_MS sets another one for the process.  After the limit a kernel sets
# the status word and returns, and every later kernel of that exchange does nothing (see check_status).
import os as _os
if _os.environ.get("MDT_PEER_WAIT_MS"):
    ext.set_peer_wait_limit_ms(int(_os.environ["MDT_PEER_WAIT_MS"]))

_status = {}


def status_tensor(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when one of their bounded waits gives up."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device) -> None:
    code = int(status_tensor(device).item())
    if code != 0:
        status_tensor(device).zero_()
        raise RuntimeError(f"a kernel reported a wait that ran out of time (status code {code})")


def launch_count() -> int:
    return int(ext.launch_count())


def _gemm(mode, A, a_mn, B, b_mn, C, M, N, K, G=1, offsets=None, capacity=0, B2=None, A_l=None, a_mn_l=False,
          B_l=None, B2_l=None, b_mn_l=False, K_l=0, C2=None, C3=None, accumulate=False, alpha=1.0, wait=None, scatter=None,
          residual=None):
    """wait = (tile_ready, tile_expected): A rows arrive from peers, tile by tile.  scatter = (row_rank, row_pos,
    peer_out table, peer_arrive table): result rows are stored into peers' buffers instead of C."""
    w0, w1 = wait if wait is not None else (None, None)
    s0, s1, s2, s3 = scatter if scatter is not None else (None, None, None, None)
    ext.gemm(mode, A, a_mn, B, b_mn, C, M, N, K, G, offsets, capacity, B2, A_l, a_mn_l, B_l, B2_l, b_mn_l, K_l,
             C2, C3, accumulate, alpha, status_tensor(A.device), w0, w1, s0, s1, s2, s3, residual)
    return C


def mm_nt(x, w, out=None, alpha=1.0, lora=None, residual=None):
    """x [M,K] @ w[N,K]^T (+ LoRA segment: (A_l [M,r], B_l [N,r])) (+ residual [M,N], added in the epilogue)."""
    M, K = x.shape
    N = w.shape[0]
    out = out if out is not None else torch.empty(M, N, dtype=x.dtype, device=x.device)
    if lora is None:
        return _gemm(0, x, False, w, False, out, M, N, K, alpha=alpha, residual=residual)
    t, b = lora
    return _gemm(0, x, False, w, False, out, M, N, K, A_l=t, B_l=b, b_mn_l=False, K_l=t.shape[1], alpha=alpha, residual=residual)


def mm_nn(x, w, out=None, alpha=1.0, accumulate=False, lora=None):
    """x [M,K] @ w[K,N] (w row-major, N contiguous)."""
    M, K = x.shape
    N = w.shape[1]
    out = out if out is not None else torch.empty(M, N, dtype=x.dtype, device=x.device)
    if lora is None:
        return _gemm(0, x, False, w, True, out, M, N, K, alpha=alpha, accumulate=accumulate)
    t, b = lora  # t [M,r], b [r,N]
    return _gemm(0, x, False, w, True, out, M, N, K, A_l=t, B_l=b, b_mn_l=True, K_l=t.shape[1], alpha=alpha,
                 accumulate=accumulate)


def mm_tn(a, b, out=None, alpha=1.0, accumulate=False, out_dtype=None):
    """a[R,M]^T @ b[R,N] -> [M,N] (reduction over rows)."""
    R, M = a.shape
    N = b.shape[1]
    out = out if out is not None else torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    return _gemm(2, a, True, b, True, out, M, N, R, alpha=alpha, accumulate=accumulate)


# ----------------------------------------------------------------------------------------------- dense linear
def _skinny(x, A, a_is_kr, alpha):
    """x A^T (A [r, K]) or x A (A [K, r]) for a LoRA rank r: CUDA-core kernel for r <= 32, else the GEMM."""
    r = A.shape[1] if a_is_kr else A.shape[0]
    if r <= 32 and x.shape[1] % 8 == 0 and A.is_contiguous() and x.dtype == torch.bfloat16 and A.dtype == torch.bfloat16:
        return ext.skinny_mm(x, A, a_is_kr, float(alpha))
    return mm_nn(x, A, alpha=alpha) if a_is_kr else mm_nt(x, A, alpha=alpha)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, A, B, scaling):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        t = None
        if A is not None:
            t = _skinny(x2, A, False, scaling)        # [M, r] = s * x A^T
            y = mm_nt(x2, w, lora=(t, B))
        else:
            y = mm_nt(x2, w)
        ctx.save_for_backward(x2, w, A, B, t)
        ctx.scaling, ctx.shape = scaling, shape
        return y.view(*shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, A, B, t = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = dA = dB = None
        dt = None
        if A is not None:
            dt = _skinny(dy2, B, True, ctx.scaling)    # [M, r] = s * dy B
        if ctx.needs_input_grad[0]:
            dx = mm_nn(dy2, w, lora=(dt, A) if A is not None else None).view(ctx.shape)
        if ctx.needs_input_grad[1]:
            dw = mm_tn(dy2, x2)
        if A is not None and ctx.needs_input_grad[2]:
            dA = mm_tn(dt, x2)                         # [r, K]
        if B is not None and ctx.needs_input_grad[3]:
            dB = mm_tn(dy2, t)                         # [N, r]
        return dx, dw, dA, dB, None


def linear(x, w, lora=None):
    if lora is None:
        return _Linear.apply(x, w, None, None, 0.0)
    A, B, s = lora
    return _Linear.apply(x, w, A, B, float(s))


# ----------------------------------------------------------------------------------------------- router / plan
class _Router(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, top_k, normalize, with_stats=False):
        res = ext.router_fwd(x.contiguous(), w.contiguous(), top_k, bool(normalize), bool(with_stats))
        scores, weights, idx = res[:3]
        stats = res[3] if with_stats else torch.empty(0, dtype=torch.float32, device=x.device)
        ctx.save_for_backward(x, w, idx)
        ctx.normalize = bool(normalize)
        ctx.mark_non_differentiable(idx, stats)
        return scores, weights, idx, stats

    @staticmethod
    def backward(ctx, dscores, dweights, _didx, _dstats=None):
        x, w, idx = ctx.saved_tensors
        if dweights is None:
            dweights = torch.zeros(idx.shape, dtype=x.dtype, device=x.device)
        dx, dw = ext.router_bwd(x.contiguous(), w.contiguous(), idx, dweights.to(x.dtype), dscores, ctx.normalize)
        return dx, dw.to(w.dtype), None, None, None


def router(x, w_router, top_k, normalize=True, with_stats=False):
    """(scores, weights, indices), plus with `with_stats` the kernel's per-expert statistics (fp32 [2E]: slot counts,
    then score sums) as a fourth, non-differentiable result."""
    if normalize is not True and normalize not in (None, False, 1):
        raise ValueError("the fused router kernel normalises with the L1 norm only")
    out = _Router.apply(x, w_router, top_k, normalize is True or normalize == 1, with_stats)
    return out if with_stats else out[:3]


def make_plan(top_experts, num_experts, block=BLOCK_ROWS, capacity=None) -> RoutingPlan:
    if top_experts.dim() == 1:
        top_experts = top_experts[:, None]
    T, k = top_experts.shape
    n = T * k
    cap = capacity if capacity is not None else plan_capacity(n, num_experts, block)
    counts, offs, dest, src = ext.make_plan(top_experts.reshape(-1).int().contiguous(), num_experts, block, cap)
    return RoutingPlan(counts, offs, dest, src, k, num_experts)


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan: RoutingPlan):
        ctx.plan = plan
        return ext.gather_rows(x.contiguous(), plan.src_slot, plan.padded_offsets, plan.num_experts, None, plan.top_k)

    @staticmethod
    def backward(ctx, dxg):
        plan = ctx.plan
        return ext.combine_rows(dxg.contiguous(), plan.dest_row, None, plan.top_k), None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, weights, plan: RoutingPlan):
        ctx.plan = plan
        y = y.contiguous()
        w = weights.contiguous() if weights is not None else None
        ctx.save_for_backward(y, w)
        return ext.combine_rows(y, plan.dest_row, w, plan.top_k)

    @staticmethod
    def backward(ctx, dout):
        plan = ctx.plan
        y, w = ctx.saved_tensors
        dout = dout.contiguous()
        dy = ext.gather_rows(dout, plan.src_slot, plan.padded_offsets, plan.num_experts,
                             w.reshape(-1) if w is not None else None, plan.top_k)
        dw = ext.combine_wgrad(y, plan.dest_row, dout, plan.top_k) if (w is not None and ctx.needs_input_grad[1]) else None
        return dy, dw, None


def gather_rows(x, plan):
    return _Gather.apply(x, plan)


def combine_rows(y, plan, weights):
    return _Combine.apply(y, weights, plan)


# ----------------------------------------------------------------------------------------------- expert MLP
def _g(mode, A, a_mn, B, b_mn, C, N, K, plan, **kw):
    G = C.shape[0] if mode == 2 else (B.shape[0] if B.dim() == 3 else 1)
    return _gemm(mode, A, a_mn, B, b_mn, C, C.shape[-2] if mode == 2 else A.shape[0], N, K, G=G,
                 offsets=plan.padded_offsets, capacity=plan.capacity, **kw)


class _GroupedSwiGLUMLP(torch.autograd.Function):
    """(silu(x W1^T) * (x W3^T)) W2 over block-padded row groups, with optional per-expert LoRA."""

    @staticmethod
    def forward(ctx, xg, w1, w2, w3, plan, lora, wgrad_scale, wgrad_out, lora_ids, *lora_tensors):
        E, F, H = w1.shape
        R = xg.shape[0]
        dev, dt = xg.device, xg.dtype
        need_grad = any(ctx.needs_input_grad)
        l1 = lora.get("w1") if lora else None
        l2 = lora.get("w2") if lora else None
        l3 = lora.get("w3") if lora else None
        kw = {}
        t13 = A13 = B1p = B3p = None
        # rows still arriving from peer GPUs: the first GEMM that reads xg waits tile by tile
        wait = getattr(plan, "ep_wait", None)
        if l1 is not None or l3 is not None:
            assert l1 is not None and l3 is not None, "expert LoRA must cover w1 and w3 together"
            (A1, B1, s1), (A3, B3, s3) = l1, l3
            r = A1.shape[2]
            A13 = torch.cat([A1 * s1 if s1 != 1.0 else A1, A3 * s3 if s3 != 1.0 else A3], dim=2).contiguous()  # [E,H,2r], scale folded
            t13 = torch.empty(R, 2 * r, dtype=dt, device=dev)
            _g(1, xg, False, A13, True, t13, 2 * r, H, plan, wait=wait)
            wait = None
            z = torch.zeros_like(B1)
            B1p, B3p = torch.cat([B1, z], dim=1).contiguous(), torch.cat([z, B3], dim=1).contiguous()  # [E,2r,F]
            kw = dict(A_l=t13, B_l=B1p, B2_l=B3p, b_mn_l=True, K_l=2 * r)
        h = torch.empty(R, F, dtype=dt, device=dev)
        g = u = None
        if need_grad:
            g, u = torch.empty_like(h), torch.empty_like(h)
        _g(1, xg, False, w1, False, h, F, H, plan, B2=w3, C2=g, C3=u, wait=wait, **kw)
        if getattr(plan, "ep_clone_input", False):
            xg = xg.clone()          # all rows have arrived now; the receive buffer is re-used by later exchanges
        t2 = None
        kw2 = {}
        if l2 is not None:
            A2, B2, s2 = l2
            t2 = torch.empty(R, A2.shape[2], dtype=dt, device=dev)
            _g(1, h, False, A2, True, t2, A2.shape[2], F, plan, alpha=s2)
            kw2 = dict(A_l=t2, B_l=B2, b_mn_l=True, K_l=A2.shape[2])
        y = torch.empty(R, H, dtype=dt, device=dev)
        # with ep_scatter the result rows go straight into the source ranks' buffers (y itself stays unwritten)
        _g(1, h, False, w2, True, y, H, F, plan, scatter=getattr(plan, "ep_scatter", None), **kw2)
        if need_grad:
            ctx.plan, ctx.lora, ctx.wgrad_scale, ctx.wgrad_out = plan, lora, wgrad_scale, wgrad_out
            ctx.n_lora, ctx.lora_ids = len(lora_tensors), lora_ids
            ctx.save_for_backward(xg, w1, w2, w3, g, u, h, t13, t2)
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, w1, w2, w3, g, u, h, t13, t2 = ctx.saved_tensors
        plan, lora, ws = ctx.plan, ctx.lora, ctx.wgrad_scale
        E, F, H = w1.shape
        R = xg.shape[0]
        dev, dt = xg.device, xg.dtype
        dy = dy.contiguous()
        l1 = lora.get("w1") if lora else None
        l2 = lora.get("w2") if lora else None
        l3 = lora.get("w3") if lora else None
        grads = {}
        wait = getattr(plan, "ep_wait", None)        # dy rows still arriving from peers (fused exchange)
        scatter = getattr(plan, "ep_scatter", None) if l1 is None else None
        plan.ep_scattered = scatter is not None
        # ---- down projection
        kw = {}
        dt2 = None
        if l2 is not None:
            A2, B2, s2 = l2
            r = A2.shape[2]
            dt2 = torch.empty(R, r, dtype=dt, device=dev)
            _g(1, dy, False, B2, False, dt2, r, H, plan, alpha=s2, wait=wait)  # s * dy B2^T
            wait = None
            kw = dict(A_l=dt2, B_l=A2, b_mn_l=False, K_l=r)
        dh = torch.empty(R, F, dtype=dt, device=dev)
        _g(1, dy, False, w2, False, dh, F, H, plan, wait=wait, **kw)            # dy W2^T (W2 stored [F,H])
        wg = ctx.wgrad_out
        dw1 = dw2 = dw3 = None
        need_w = ctx.needs_input_grad[1] or ctx.needs_input_grad[2] or ctx.needs_input_grad[3]
        if need_w:
            if wg is not None:
                _g(2, h, True, dy, True, wg[1], H, 0, plan, alpha=ws, accumulate=True)
            else:
                dw2 = torch.empty_like(w2)
                _g(2, h, True, dy, True, dw2, H, 0, plan, alpha=ws)
        if l2 is not None:
            A2, B2, s2 = l2
            dA2 = torch.empty_like(A2); _g(2, h, True, dt2, True, dA2, A2.shape[2], 0, plan, alpha=ws)
            dB2 = torch.empty_like(B2); _g(2, t2, True, dy, True, dB2, H, 0, plan, alpha=ws)
            grads[id(A2)], grads[id(B2)] = dA2, dB2
        # ---- SwiGLU
        dg, du = ext.swiglu_bwd(g, u, dh, plan.padded_offsets)
        # ---- up projections
        dx = torch.empty(R, H, dtype=dt, device=dev)
        _g(1, dg, False, w1, True, dx, H, F, plan, A_l=du, B_l=w3, b_mn_l=True, K_l=F, scatter=scatter)   # dg W1 + du W3
        if need_w:
            if wg is not None:
                _g(2, dg, True, xg, True, wg[0], H, 0, plan, alpha=ws, accumulate=True)
                _g(2, du, True, xg, True, wg[2], H, 0, plan, alpha=ws, accumulate=True)
            else:
                dw1 = torch.empty_like(w1); _g(2, dg, True, xg, True, dw1, H, 0, plan, alpha=ws)
                dw3 = torch.empty_like(w3); _g(2, du, True, xg, True, dw3, H, 0, plan, alpha=ws)
        if l1 is not None:
            (A1, B1, s1), (A3, B3, s3) = l1, l3
            r = A1.shape[2]
            dt1 = torch.empty(R, r, dtype=dt, device=dev); _g(1, dg, False, B1, False, dt1, r, F, plan, alpha=s1)
            dt3 = torch.empty(R, r, dtype=dt, device=dev); _g(1, du, False, B3, False, dt3, r, F, plan, alpha=s3)
            _g(1, dt1, False, A1, False, dx, H, r, plan, A_l=dt3, B_l=A3, b_mn_l=False, K_l=r, accumulate=True)
            dA1 = torch.empty_like(A1); _g(2, xg, True, dt1, True, dA1, r, 0, plan, alpha=ws)
            dA3 = torch.empty_like(A3); _g(2, xg, True, dt3, True, dA3, r, 0, plan, alpha=ws)
            t1 = t13[:, :r]
            t3 = t13[:, r:]
            dB1 = torch.empty_like(B1); _g(2, t1, True, dg, True, dB1, F, 0, plan, alpha=ws)
            dB3 = torch.empty_like(B3); _g(2, t3, True, du, True, dB3, F, 0, plan, alpha=ws)
            grads.update({id(A1): dA1, id(B1): dB1, id(A3): dA3, id(B3): dB3})
        lora_grads = tuple(grads.get(k) for k in ctx.lora_ids) if ctx.n_lora else ()
        return (dx, dw1, dw2, dw3, None, None, None, None, None) + lora_grads


def grouped_swiglu_mlp(xg, w1, w2, w3, plan, lora=None, wgrad_scale=1.0, wgrad_out=None):
    tensors = []
    if lora:
        for name in ("w1", "w2", "w3"):
            if name in lora:
                tensors += [lora[name][0], lora[name][1]]
    ids = tuple(id(t) for t in tensors)
    return _GroupedSwiGLUMLP.apply(xg.contiguous(), w1, w2, w3, plan, lora, float(wgrad_scale), wgrad_out, ids, *tensors)


class _GroupedLinear(torch.autograd.Function):
    """y[rows of g] = x[rows of g] W_g (+ s (x A_g) B_g); W is [G,N,K] if trans_b else [G,K,N]."""

    @staticmethod
    def forward(ctx, x, w, plan, trans_b, A, B, scaling, wgrad_scale):
        x = x.contiguous()
        R, K = x.shape
        N = w.shape[1] if trans_b else w.shape[2]
        out = torch.empty(R, N, dtype=x.dtype, device=x.device)
        kw, t = {}, None
        if A is not None:
            r = A.shape[2]
            t = torch.empty(R, r, dtype=x.dtype, device=x.device)
            _g(1, x, False, A, True, t, r, K, plan, alpha=scaling)
            kw = dict(A_l=t, B_l=B, b_mn_l=True, K_l=r)
        _g(1, x, False, w, not trans_b, out, N, K, plan, **kw)
        ctx.plan, ctx.trans_b, ctx.scaling, ctx.ws = plan, trans_b, scaling, wgrad_scale
        ctx.save_for_backward(x, w, A, B, t)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w, A, B, t = ctx.saved_tensors
        plan, trans_b, ws = ctx.plan, ctx.trans_b, ctx.ws
        dy = dy.contiguous()
        R, K = x.shape
        N = dy.shape[1]
        dx = dw = dA = dB = None
        kw, dt = {}, None
        if A is not None:
            r = A.shape[2]
            dt = torch.empty(R, r, dtype=x.dtype, device=x.device)
            _g(1, dy, False, B, False, dt, r, N, plan, alpha=ctx.scaling)      # s * dy B^T
            kw = dict(A_l=dt, B_l=A, b_mn_l=False, K_l=r)
        if ctx.needs_input_grad[0]:
            dx = torch.empty(R, K, dtype=x.dtype, device=x.device)
            _g(1, dy, False, w, trans_b, dx, K, N, plan, **kw)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(w)
            if trans_b:
                _g(2, dy, True, x, True, dw, K, 0, plan, alpha=ws)
            else:
                _g(2, x, True, dy, True, dw, N, 0, plan, alpha=ws)
        if A is not None and ctx.needs_input_grad[4]:
            dA = torch.empty_like(A); _g(2, x, True, dt, True, dA, A.shape[2], 0, plan, alpha=ws)
        if B is not None and ctx.needs_input_grad[5]:
            dB = torch.empty_like(B); _g(2, t, True, dy, True, dB, N, 0, plan, alpha=ws)
        return dx, dw, None, None, dA, dB, None, None


def grouped_linear(x, w, plan, trans_b, lora=None, wgrad_scale=1.0):
    if lora is None:
        return _GroupedLinear.apply(x, w, plan, trans_b, None, None, 0.0, float(wgrad_scale))
    A, B, s = lora
    return _GroupedLinear.apply(x, w, plan, trans_b, A, B, float(s), float(wgrad_scale))


# ----------------------------------------------------------------------------------------------- small ops
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, rstd = ext.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dwp = ext.rmsnorm_bwd(x, w, dy.contiguous(), rstd)
        return dx, ext.rmsnorm_dw(dwp, w), None


def rmsnorm(x, weight, eps):
    return _RMSNorm.apply(x, weight, eps)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, theta):
        ctx.save_for_backward(positions)
        ctx.theta = theta
        return ext.rope(x, positions, theta, False)

    @staticmethod
    def backward(ctx, dy):
        (positions,) = ctx.saved_tensors
        return ext.rope(dy.contiguous(), positions, ctx.theta, True), None, None


def rope(x, positions, theta):
    return _Rope.apply(x, positions.int(), float(theta))


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ids = ids.long().contiguous()
        ctx.save_for_backward(ids)
        ctx.shape = weight.shape
        return ext.embedding(weight, ids)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        dtable = torch.zeros(ctx.shape, dtype=torch.float32, device=dout.device)
        ext.embedding_bwd(dout.contiguous(), ids, dtable)
        return None, dtable.to(dout.dtype)


def embedding(ids, weight):
    return _Embedding.apply(ids, weight)


def swiglu(g, u):
    return ext.swiglu_fwd(g.contiguous(), u.contiguous())


class _LinearCrossEntropy(torch.autograd.Function):
    """lm_head GEMM + softmax cross-entropy; the logits buffer is reused for its own gradient."""

    @staticmethod
    def forward(ctx, hidden, w_head, labels, ignore_index):
        hidden = hidden.contiguous()
        logits = mm_nt(hidden, w_head)
        out = ext.cross_entropy(logits, labels.long().contiguous(), ignore_index, 1.0)
        n = out[1]
        ctx.save_for_backward(hidden, w_head, logits, out[1].clone())
        loss_sum = out[0].clone()
        n = n.clone()
        ctx.mark_non_differentiable(n)
        return loss_sum, n

    @staticmethod
    def backward(ctx, dloss_sum, _dn):
        hidden, w_head, dlogits, n = ctx.saved_tensors
        # the kernel wrote d(mean loss)/dlogits; convert to d(loss_sum) and apply the incoming gradient
        dlogits.mul_((dloss_sum * n.clamp(min=1.0)).to(dlogits.dtype))
        dh = mm_nn(dlogits, w_head) if ctx.needs_input_grad[0] else None
        dw = mm_tn(dlogits, hidden) if ctx.needs_input_grad[1] else None
        return dh, dw, None, None


def cross_entropy_sum(hidden, w_head, labels, ignore_index=-100):
    return _LinearCrossEntropy.apply(hidden, w_head, labels, ignore_index)


def attention(q, k, v, cu_seqlens, max_seqlen=None):
    from . import attention_cuda
    return attention_cuda.attention(q, k, v, cu_seqlens, max_seqlen)


def adamw_multi(ps, gs, ms, vs, lr, b1, b2, eps, wd, step, grad_scale=1.0):
    ext.adamw(list(ps), list(gs), list(ms), list(vs), lr, b1, b2, eps, wd, int(step), float(grad_scale))
