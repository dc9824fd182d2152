"""Whole sub-blocks of the decoder layer as single autograd nodes with hand-written backward passes.

A decoder layer at these sizes is a few dozen kernels of 5-500 microseconds; with one autograd node per
operator the host cannot issue them as fast as the GPU retires them.  `attention_block` runs
RMSNorm -> q/k/v projections (+LoRA) -> RoPE -> causal GQA attention -> output projection (+LoRA)
-> residual add as ONE node: its forward and backward call the kernels directly, with no graph
bookkeeping in between.  The math is the same as composing the individual ops of `cuda_ops`.
"""
from __future__ import annotations

import os

import torch

from . import cuda_ops as C

ext = C.ext
# expert GEMMs wait for / deliver rows themselves (tile-wise overlap with the exchange) instead of separate kernels
GEMM_FUSION = os.environ.get("MDT_EP_GEMM_FUSION", "1") != "0"


def _lin_fwd(x2, W, A, B, s, residual=None):
    if A is None:
        return C.mm_nt(x2, W, residual=residual), None
    t = C.mm_nt(x2, A, alpha=s)                       # [M, r] = s * x A^T
    return C.mm_nt(x2, W, lora=(t, B), residual=residual), t


def _lin_bwd(dy2, xin, W, A, B, s, t, need_w, need_a, need_b, dx_out=None, accumulate=False):
    dt = C.mm_nn(dy2, B, alpha=s) if A is not None else None
    dx = C.mm_nn(dy2, W, out=dx_out, accumulate=accumulate, lora=(dt, A) if A is not None else None)
    dW = C.mm_tn(dy2, xin) if need_w else None
    dA = C.mm_tn(dt, xin) if (A is not None and need_a) else None
    dB = C.mm_tn(dy2, t) if (B is not None and need_b) else None
    return dx, dW, dA, dB


class _AttentionBlockNative(torch.autograd.Function):
    """Same sub-block with the kernel sequence issued from C++ (one binding call per direction)."""

    @staticmethod
    def forward(ctx, x, meta, *params):
        eps, theta, Hq, Hkv, d, positions, cu, max_seqlen, scalings = meta
        sc = [-1.0 if s is None else float(s) for s in scalings]
        res = ext.attention_block_fwd(x.contiguous(), list(params), sc, positions, cu, max_seqlen, eps, theta, Hq, Hkv, d,
                                      C.status_tensor(x.device))
        if any(ctx.needs_input_grad):
            ctx.meta, ctx.sc, ctx.n_params = meta, sc, len(params)
            ctx.save_for_backward(x, *res[1:], *params)
        return res[0]

    @staticmethod
    def backward(ctx, dy):
        eps, theta, Hq, Hkv, d, positions, cu, max_seqlen, scalings = ctx.meta
        saved = ctx.saved_tensors
        state, params = list(saved[:12]), list(saved[12:])
        needs = [bool(n) for n in ctx.needs_input_grad[2:]]
        res = ext.attention_block_bwd(dy, state, params, ctx.sc, needs, positions, cu, max_seqlen, theta, Hq, Hkv, d,
                                      C.status_tensor(dy.device))
        grads = tuple(g if (g.numel() and need) else None for g, need in zip(res[1:], needs))
        return (res[0], None) + grads


NATIVE_ISSUE = os.environ.get("MDT_NATIVE_BLOCKS", "1") != "0"


class _AttentionBlock(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, meta, *params):
        eps, theta, Hq, Hkv, d, positions, cu, max_seqlen, scalings = meta
        x2 = x.contiguous()
        T = x2.shape[0]
        ln_w = params[0]
        lins, i = [], 1
        for s in scalings:                                 # q, k, v, o
            if s is None:
                lins.append((params[i], None, None, 0.0, i)); i += 1
            else:
                lins.append((params[i], params[i + 1], params[i + 2], s, i)); i += 3
        xn, rstd = ext.rmsnorm_fwd(x2, ln_w, eps)
        q, tq = _lin_fwd(xn, *lins[0][:4])
        k, tk = _lin_fwd(xn, *lins[1][:4])
        v, tv = _lin_fwd(xn, *lins[2][:4])
        qr = ext.rope(q.view(T, Hq, d), positions, theta, False)
        kr = ext.rope(k.view(T, Hkv, d), positions, theta, False)
        v3 = v.view(T, Hkv, d)
        scale = float(d) ** -0.5
        o, lse = ext.attention_fwd(qr, kr, v3, cu, max_seqlen, scale)
        o2 = o.view(T, Hq * d)
        out, to = _lin_fwd(o2, *lins[3][:4], residual=x2)      # + x in the GEMM's epilogue
        if any(ctx.needs_input_grad):
            ctx.meta, ctx.n_params, ctx.lin_index = meta, len(params), [l[4] for l in lins]
            ctx.save_for_backward(x2, rstd, xn, qr, kr, v3, o, lse, tq, tk, tv, to, *params)
        return out

    @staticmethod
    def backward(ctx, dy):
        eps, theta, Hq, Hkv, d, positions, cu, max_seqlen, scalings = ctx.meta
        saved = ctx.saved_tensors
        x2, rstd, xn, qr, kr, v3, o, lse, tq, tk, tv, to = saved[:12]
        params = saved[12:]
        ln_w = params[0]
        T = x2.shape[0]
        need = ctx.needs_input_grad                           # index 0 = x, 1 = meta, 2.. = params
        grads = [None] * ctx.n_params

        def lin(j):
            i = ctx.lin_index[j]
            if scalings[j] is None:
                return params[i], None, None, 0.0, i
            return params[i], params[i + 1], params[i + 2], scalings[j], i

        def run(j, dy2, xin, t, dx_out=None, accumulate=False):
            W, A, B, s, i = lin(j)
            dx, dW, dA, dB = _lin_bwd(dy2, xin, W, A, B, s, t, need[2 + i], A is not None and need[3 + i],
                                      B is not None and need[4 + i], dx_out, accumulate)
            grads[i] = dW
            if A is not None:
                grads[i + 1], grads[i + 2] = dA, dB
            return dx

        dy2 = dy.contiguous()
        o2 = o.view(T, Hq * d)
        d_o = run(3, dy2, o2, to)
        scale = float(d) ** -0.5
        dq, dk, dv = ext.attention_bwd(qr, kr, v3, o, d_o.view(T, Hq, d), lse, cu, max_seqlen, scale)
        dq = ext.rope(dq, positions, theta, True).view(T, Hq * d)
        dk = ext.rope(dk, positions, theta, True).view(T, Hkv * d)
        d_xn = run(0, dq, xn, tq)
        run(1, dk, xn, tk, dx_out=d_xn, accumulate=True)
        run(2, dv.view(T, Hkv * d), xn, tv, dx_out=d_xn, accumulate=True)
        dx, dwp = ext.rmsnorm_bwd(x2, ln_w, d_xn, rstd, dy2)   # + dy: the residual connection's gradient
        if need[2]:
            grads[0] = ext.rmsnorm_dw(dwp, ln_w)
        return (dx, None) + tuple(grads)


def attention_block(layer, x, batch):
    """x + self_attn(input_layernorm(x)) for a `MixtralDecoderLayer` on CUDA (head_dim 128)."""
    attn = layer.self_attn
    params = [layer.input_layernorm.weight]
    scalings = []
    for lin in (attn.q_proj, attn.k_proj, attn.v_proj, attn.o_proj):
        params.append(lin.weight)
        if lin.lora_A is not None:
            params += [lin.lora_A["default"].weight, lin.lora_B["default"].weight]
            scalings.append(float(lin.scaling))
        else:
            scalings.append(None)
    meta = (layer.input_layernorm.eps, float(attn.cfg.rope_theta), attn.num_heads, attn.num_kv_heads, attn.head_dim,
            batch.positions, batch.cu_seqlens, int(batch.max_seqlen), tuple(scalings))
    return (_AttentionBlockNative if NATIVE_ISSUE else _AttentionBlock).apply(x, meta, *params)


# ---------------------------------------------------------------------------------------------------------
# MoE sub-block:  x + experts(router(post_attention_layernorm(x)))  as one node
# ---------------------------------------------------------------------------------------------------------
class _Ctx:
    """Stand-in for an autograd context, so that the forward/backward bodies of the per-op Functions can be
    run directly (no graph node) from inside a fused node."""

    def __init__(self, needs_input_grad):
        self.needs_input_grad = tuple(needs_input_grad)
        self.saved_tensors = ()

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_non_differentiable(self, *tensors):
        pass


def moe_block_supported(layer, x) -> bool:
    moe = layer.block_sparse_moe
    a, ex = moe.args, moe.experts
    if a.moe_jitter_eps is not None or a.uniform_expert_assignment or a.moe_loss_weight > 0 or ex.tp_group is not None:
        return False
    if a.moe_normalize_expert_weights not in (True, 1):
        return False
    if ex.ep_group is not None and ex.ep_size > 1:
        return ex._dispatch_impl(x) == "fused"
    return True


class _MoEBlock(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer, *params):
        moe = layer.block_sparse_moe
        ex, mlp, a = moe.experts, moe.experts.mlp, moe.args
        E, k = a.moe_num_experts, a.moe_top_k
        ln_w, Wr = params[0], params[1]
        lora_tensors = params[5:]
        x2 = x.contiguous()
        need = ctx.needs_input_grad
        grad_mode = any(need)
        xn, rstd = ext.rmsnorm_fwd(x2, ln_w, layer.post_attention_layernorm.eps)
        scores, wts, idx = ext.router_fwd(xn, Wr.contiguous(), k, True)
        with torch.set_grad_enabled(grad_mode):
            w1, w2, w3, lora, ws, wgrad_out = mlp.call_args(xn)
        # experts' own autograd body, run directly
        mneeds = [grad_mode, need[4], need[5], need[6], False, False, False, False, False] + [need[7 + i] for i in range(len(lora_tensors))]
        mctx = _Ctx(mneeds)
        ids = tuple(id(t) for t in lora_tensors)
        ep = ex.ep_group is not None and ex.ep_size > 1
        if not ep:
            plan = C.make_plan(idx, E)
            ex.last_tokens_per_expert = plan.tokens_per_expert
            xg = ext.gather_rows(xn, plan.src_slot, plan.padded_offsets, E, None, k)
            yg = C._GroupedSwiGLUMLP.forward(mctx, xg, w1, w2, w3, plan, lora, float(ws), wgrad_out, ids, *lora_tensors)
            ys = yg
            comb = ext.combine_rows(yg, plan.dest_row, wts, k, x2)      # + x
            eng = meta_c = expert_sorted = None
        else:
            if ex._fused is None:
                from ..parallel.fused_ep import FusedExpertParallel
                ex._fused = FusedExpertParallel.for_group(ex.ep_group, a, x2.device)
            eng = ex._fused
            n_slots = idx.numel()
            plan = C.make_plan(idx, E, 1, n_slots)
            ex.last_tokens_per_expert = plan.tokens_per_expert
            meta_c = eng.exchange_counts(plan.tokens_per_expert)
            eos = idx.reshape(-1).contiguous()
            expert_sorted = eos.index_select(0, plan.src_slot.long()) if grad_mode else None
            par = eng.next_phase()
            rplan = eng.recv_plan(meta_c)
            ext.gemm_rows_hint(n_slots)      # the receive buffers are sized for a capacity; expect about what was sent
            if GEMM_FUSION:
                # the expert GEMMs take part in the exchange: the first one waits for its row tiles as they arrive,
                # the down projection stores its result rows straight into the source ranks' buffers
                rr, rp, te = eng.fused_meta(meta_c)
                eng.dispatch(xn, plan.src_slot, eos, None, meta_c, k, par, wait=False)
                rplan.ep_wait, rplan.ep_scatter = eng.gemm_wait(par, te), eng.gemm_scatter(par, rr, rp)
                rplan.ep_clone_input, rplan.ep_meta = grad_mode, (rr, rp, te)
                H = x2.shape[1]
                C._GroupedSwiGLUMLP.forward(mctx, eng.wspace.recv_x(), w1, w2, w3, rplan, lora, float(ws), wgrad_out, ids, *lora_tensors)
                ys = eng.wait_rows(meta_c, par, n_slots, (H + 255) // 256 if H > 128 else 1, clone=grad_mode)
            else:
                eng.dispatch(xn, plan.src_slot, eos, None, meta_c, k, par)
                xr = eng.wspace.recv_x()
                if grad_mode:
                    xr = xr.clone()
                yg = C._GroupedSwiGLUMLP.forward(mctx, xr, w1, w2, w3, rplan, lora, float(ws), wgrad_out, ids, *lora_tensors)
                ys = eng.combine(yg, meta_c, par, n_slots, clone=grad_mode)
            ext.gemm_rows_hint(0)
            comb = ext.combine_rows(ys, plan.dest_row, wts, k, x2)      # + x
        if grad_mode:
            ctx.layer, ctx.plan, ctx.mctx, ctx.eng, ctx.meta_c, ctx.n_params = layer, plan, mctx, eng, meta_c, len(params)
            ctx.save_for_backward(x2, rstd, xn, wts, idx, ys, expert_sorted, ln_w, Wr)
        return comb

    @staticmethod
    def backward(ctx, dy):
        layer, plan, mctx, eng, meta_c = ctx.layer, ctx.plan, ctx.mctx, ctx.eng, ctx.meta_c
        x2, rstd, xn, wts, idx, ys, expert_sorted, ln_w, Wr = ctx.saved_tensors
        a = layer.block_sparse_moe.args
        E, k = a.moe_num_experts, a.moe_top_k
        need = ctx.needs_input_grad
        dy2 = dy.contiguous()
        d_rows = ext.gather_rows(dy2, plan.src_slot, plan.padded_offsets, E, wts.reshape(-1), k)   # gate-weighted, grouped order
        dwts = ext.combine_wgrad(ys, plan.dest_row, dy2, k)
        if eng is None:
            g = C._GroupedSwiGLUMLP.backward(mctx, d_rows)
            dxn = ext.combine_rows(g[0], plan.dest_row, None, k)
        else:
            par = eng.next_phase()
            rplan = mctx.plan
            n_slots = plan.dest_row.numel()
            ext.gemm_rows_hint(n_slots)
            if GEMM_FUSION:
                rr, rp, te = rplan.ep_meta
                eng.dispatch(d_rows, eng.identity(d_rows.shape[0]), expert_sorted, None, meta_c, 1, par, wait=False)
                rplan.ep_wait, rplan.ep_scatter, rplan.ep_clone_input = eng.gemm_wait(par, te), eng.gemm_scatter(par, rr, rp), False
                g = C._GroupedSwiGLUMLP.backward(mctx, eng.wspace.recv_x())
                if rplan.ep_scattered:
                    H = x2.shape[1]
                    back = eng.wait_rows(meta_c, par, n_slots, (H + 255) // 256 if H > 128 else 1, clone=False)
                else:
                    back = eng.combine(g[0].contiguous(), meta_c, par, n_slots, clone=False)
            else:
                eng.dispatch(d_rows, eng.identity(d_rows.shape[0]), expert_sorted, None, meta_c, 1, par)
                g = C._GroupedSwiGLUMLP.backward(mctx, eng.wspace.recv_x())
                back = eng.combine(g[0].contiguous(), meta_c, par, n_slots, clone=False)
            ext.gemm_rows_hint(0)
            dxn = ext.combine_rows(back, plan.dest_row, None, k)
        dxn = dxn.contiguous()
        _, dWr = ext.router_bwd(xn, Wr.contiguous(), idx, dwts, None, True, dxn)     # adds the router's input gradient to dxn
        dx, dwp = ext.rmsnorm_bwd(x2, ln_w, dxn, rstd, dy2)                          # + dy: the residual connection's gradient
        grads = [None] * ctx.n_params
        if need[2]:
            grads[0] = ext.rmsnorm_dw(dwp, ln_w)
        if need[3]:
            grads[1] = dWr.to(Wr.dtype)
        # the MLP works on [E, F, H] views of the [E*F, H] parameters
        grads[2], grads[3], grads[4] = (t.reshape(-1, t.shape[-1]) if t is not None else None for t in (g[1], g[2], g[3]))
        for i, gl in enumerate(g[9:]):
            grads[5 + i] = gl
        return (dx, None) + tuple(grads)


class _MoEBlockNative(torch.autograd.Function):
    """MoE sub-block without expert adapters, kernel sequence issued from C++ (local or fused expert-parallel)."""

    @staticmethod
    def _ep_args(eng, parity, H):
        w = eng.wspace
        eng.gemm_scatter(parity, None, None)      # makes sure the address tables exist
        ints = [w.my_base, w.rank, eng.count_epoch, eng.count_epoch & 1, parity, (H + 255) // 256 if H > 128 else 1]
        tens = [w.peer_base, eng._peer_out, eng._peer_arrive[parity], w.tile_counters(parity), w.recv_x(), w.recv_y(),
                eng.identity(w.capacity_slots)]
        return w.layout, ints, tens

    @staticmethod
    def forward(ctx, x, layer, *params):
        moe = layer.block_sparse_moe
        ex, mlp, a = moe.experts, moe.experts.mlp, moe.args
        ln_w, Wr = params[0], params[1]
        x2 = x.contiguous()
        grad_mode = any(ctx.needs_input_grad)
        with torch.set_grad_enabled(grad_mode):
            w1, w2, w3, _, ws, wgrad_out = mlp.call_args(x2)
        eng, layout, ints, tens = None, [], [], []
        is_ep = ex.ep_group is not None and ex.ep_size > 1
        if is_ep:
            if ex._fused is None:
                from ..parallel.fused_ep import FusedExpertParallel
                ex._fused = FusedExpertParallel.for_group(ex.ep_group, a, x2.device)
            eng = ex._fused
        # A block that is recomputed in the backward pass (layer._ckpt_mode: 1 = graph-free first pass, 2 = the
        # recomputation) keeps the results of its token exchange from the first pass, so that the recomputation needs
        # no second dispatch / down projection / combine: every rank skips them alike, no exchange epoch is used.
        ckpt_mode = getattr(layer, "_ckpt_mode", 0)
        stash = getattr(layer, "_moe_stash", None)
        if ckpt_mode == 2 and grad_mode and stash is not None:
            layer._moe_stash = None
            res = ext.moe_block_fwd(x2, ln_w, Wr.contiguous(), w1, w2, w3, layer.post_attention_layernorm.eps, a.moe_top_k,
                                    a.moe_num_experts, True, [], [], [], C.status_tensor(x2.device), 2, list(stash))
        else:
            if is_ep:
                assert x2.shape[0] * a.moe_top_k <= eng.wspace.capacity_slots, "more (token, choice) slots than the workspace was sized for"
                eng.count_epoch += 1
                layout, ints, tens = _MoEBlockNative._ep_args(eng, eng.next_phase(), x2.shape[1])
            make_stash = 1 if (ckpt_mode == 1 and not grad_mode) else 0
            res = ext.moe_block_fwd(x2, ln_w, Wr.contiguous(), w1, w2, w3, layer.post_attention_layernorm.eps, a.moe_top_k,
                                    a.moe_num_experts, grad_mode, layout, ints, tens, C.status_tensor(x2.device), make_stash, [])
            if make_stash:
                layer._moe_stash = res[1:]
        ex.last_tokens_per_expert = res[1]
        if grad_mode:
            ctx.layer, ctx.eng, ctx.ws, ctx.wgrad_out = layer, eng, float(ws), wgrad_out
            ctx.views = (w1, w2, w3)
            ctx.save_for_backward(x2, ln_w, Wr, *res)
        return res[0]

    @staticmethod
    def backward(ctx, dy):
        layer, eng = ctx.layer, ctx.eng
        a = layer.block_sparse_moe.args
        saved = ctx.saved_tensors
        x2, ln_w, Wr, state = saved[0], saved[1], saved[2], list(saved[3:])
        w1, w2, w3 = ctx.views
        layout, ints, tens = [], [], []
        if eng is not None:
            layout, ints, tens = _MoEBlockNative._ep_args(eng, eng.next_phase(), x2.shape[1])
        wg = list(ctx.wgrad_out) if ctx.wgrad_out is not None else []
        need = ctx.needs_input_grad
        dx, dln, dWr = ext.moe_block_bwd(dy, state, x2, ln_w, Wr.contiguous(), w1, w2, w3, wg, ctx.ws, a.moe_top_k, a.moe_num_experts,
                                         layout, ints, tens, C.status_tensor(dy.device), bool(need[2]), bool(need[3]))
        return dx, None, (dln if need[2] else None), (dWr if need[3] else None), None, None, None


def _native_moe_ok(layer) -> bool:
    """No expert adapters, and expert weights either frozen or owned by the module (direct gradient accumulation)."""
    ex = layer.block_sparse_moe.experts
    if getattr(ex, "lora", None) is not None:
        return False
    w = ex.mlp.w1
    return (not w.requires_grad) or isinstance(w, torch.nn.Parameter)


def moe_block(layer, x):
    """x + block_sparse_moe(post_attention_layernorm(x)) as one autograd node (local or fused-EP experts)."""
    moe = layer.block_sparse_moe
    mlp = moe.experts.mlp
    params = [layer.post_attention_layernorm.weight, moe.router.layer.weight, mlp.w1, mlp.w2, mlp.w3]
    lora = getattr(moe.experts, "lora", None)
    if lora is not None:
        for name in ("w1", "w2", "w3"):
            if name in lora.lora_A:
                params += [lora.lora_A[name], lora.lora_B[name]]
    if NATIVE_ISSUE and GEMM_FUSION and _native_moe_ok(layer):
        return _MoEBlockNative.apply(x, layer, *params[:5])
    return _MoEBlock.apply(x, layer, *params)
