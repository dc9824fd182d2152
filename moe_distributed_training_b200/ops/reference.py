"""Plain PyTorch statements of every op in the framework.

These functions serve two purposes: they are the fp32 oracles that the CUDA
kernels are tested against, and they are the path taken by CPU tensors (gloo
plumbing tests).  All of them are ordinary differentiable torch code, so
autograd provides the reference gradients as well.

Math follows the reference:
  * router: softmax over all experts -> top-k -> divide by the L1 norm
    (megablocks_utils/config_utils.py:255-284)
  * experts: (silu(x w1^T) * (x w3^T)) w2 with w2 stored [ffn, hidden]
    (megablocks_utils/sparse_mlp2.py:69-90)
  * LoRA on a grouped linear: Y = X W + (alpha/r) (X A) B with the intermediate
    X A scaled and rounded to the weight dtype (scattermoe_utils/kernels/ops.py:131-141)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

BLOCK_ROWS = 128  # expert row groups are padded to a multiple of this many rows


class _ScaleGradient(torch.autograd.Function):
    """Identity in forward, multiplies the gradient by `scale` in backward."""

    @staticmethod
    def forward(ctx, x, scale):
        ctx.scale = scale
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad * ctx.scale, None


def scale_gradient(x: torch.Tensor, scale: float) -> torch.Tensor:
    if scale == 1.0:
        return x
    return _ScaleGradient.apply(x, scale)



# ----------------------------------------------------------------------------
# routing plan
# ----------------------------------------------------------------------------
@dataclass
class RoutingPlan:
    """Placement of the T*k (token, choice) slots into an expert-grouped row buffer.

    Every expert's group starts on a BLOCK_ROWS boundary; rows between the end of
    a group and the next boundary are padding (src_slot == -1, contents zero).
    """
    tokens_per_expert: torch.Tensor  # [E] int32
    padded_offsets: torch.Tensor     # [E+1] int32, row where each group starts; [-1] = rows in use
    dest_row: torch.Tensor           # [T*k] int32, row of slot j (token j//k, choice j%k)
    src_slot: torch.Tensor           # [capacity] int32, slot held by a row or -1
    top_k: int
    num_experts: int
    capacity_rows: Optional[int] = None   # set when the plan describes a buffer it has no slot map for

    @property
    def capacity(self) -> int:
        return self.capacity_rows if self.capacity_rows is not None else self.src_slot.numel()


def plan_capacity(num_slots: int, num_experts: int, block: int = BLOCK_ROWS) -> int:
    """Upper bound (known on the host, no device sync) of padded rows for num_slots slots."""
    return max(block, ((num_slots + num_experts * (block - 1)) // block) * block)


def make_plan(top_experts: torch.Tensor, num_experts: int, block: int = BLOCK_ROWS,
              capacity: Optional[int] = None) -> RoutingPlan:
    """Counting sort of slots by expert id (stable), groups padded to `block` rows."""
    if top_experts.dim() == 1:
        top_experts = top_experts[:, None]
    T, k = top_experts.shape
    flat = top_experts.reshape(-1).long()
    n = flat.numel()
    cap = capacity if capacity is not None else plan_capacity(n, num_experts, block)
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts] if n else flat.new_zeros(num_experts)
    padded = ((counts + block - 1) // block) * block
    p_off = torch.zeros(num_experts + 1, dtype=torch.long, device=flat.device)
    p_off[1:] = torch.cumsum(padded, 0)
    off = torch.cumsum(counts, 0) - counts
    order = torch.argsort(flat, stable=True)
    rank_sorted = torch.arange(n, device=flat.device) - off[flat[order]]
    rank_in_expert = torch.empty_like(rank_sorted)
    rank_in_expert[order] = rank_sorted
    dest = p_off[flat] + rank_in_expert
    src_slot = torch.full((cap,), -1, dtype=torch.int32, device=flat.device)
    src_slot[dest] = torch.arange(n, device=flat.device, dtype=torch.int32)
    return RoutingPlan(counts.int(), p_off.int(), dest.int(), src_slot, k, num_experts)


# ----------------------------------------------------------------------------
# router
# ----------------------------------------------------------------------------
def router(x: torch.Tensor, w_router: torch.Tensor, top_k: int, normalize=True,
           jitter_eps: Optional[float] = None, training: bool = False):
    """scores = softmax(x Wr^T); (w, idx) = topk(scores); w /= ||w||_p."""
    if training and jitter_eps is not None:
        low, high = 1.0 - jitter_eps, 1.0 + jitter_eps
        x = x * (low + torch.rand_like(x) * (high - low))
    scores = F.linear(x, w_router).softmax(dim=-1)
    if top_k == 1:
        w, idx = scores.max(dim=-1, keepdim=True)
    else:
        w, idx = torch.topk(scores, top_k, dim=-1)
    if normalize is not None and normalize is not False:
        p = 1 if normalize is True else normalize
        w = w / torch.norm(w, p=p, dim=-1, keepdim=True)
    return scores, w, idx.int()


def load_balancing_loss(scores: torch.Tensor, top_experts: torch.Tensor, num_experts: int, top_k: int):
    """Switch-style auxiliary loss E * sum_e f_e * P_e (off by default, as in the reference)."""
    T = scores.shape[0]
    f = torch.bincount(top_experts.reshape(-1).long(), minlength=num_experts).to(scores.dtype) / max(T * top_k, 1)
    P = scores.mean(dim=0)
    return num_experts * torch.sum(f * P)


# ----------------------------------------------------------------------------
# permutation
# ----------------------------------------------------------------------------
def gather_rows(x: torch.Tensor, src_slot: torch.Tensor, top_k: int) -> torch.Tensor:
    """xg[r] = x[src_slot[r] // top_k], zero where src_slot[r] < 0."""
    valid = src_slot >= 0
    tok = torch.div(src_slot.clamp(min=0), top_k, rounding_mode="floor").long()
    out = x.index_select(0, tok)
    return out * valid[:, None].to(x.dtype)


def combine_rows(y: torch.Tensor, dest_row: torch.Tensor, weights: Optional[torch.Tensor], top_k: int) -> torch.Tensor:
    """out[t] = sum_c weights[t,c] * y[dest_row[t*k+c]] (fp32 accumulation)."""
    rows = y.index_select(0, dest_row.long()).view(-1, top_k, y.shape[-1]).float()
    if weights is not None:
        rows = rows * weights.float()[..., None]
    return rows.sum(dim=1).to(y.dtype)


# ----------------------------------------------------------------------------
# grouped GEMMs
# ----------------------------------------------------------------------------
def _groups(offsets: torch.Tensor, counts: Optional[torch.Tensor]):
    off = offsets.tolist()
    cnt = counts.tolist() if counts is not None else [off[i + 1] - off[i] for i in range(len(off) - 1)]
    return [(off[g], off[g] + cnt[g]) for g in range(len(cnt))]


def grouped_mm(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, trans_b: bool,
               counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[rows of g] = a[rows of g] @ (b[g]^T if trans_b else b[g]).

    b is [G, N, K] when trans_b else [G, K, N].  Rows outside every group are zero.
    """
    N = b.shape[1] if trans_b else b.shape[2]
    out = a.new_zeros(a.shape[0], N)
    for g, (s, e) in enumerate(_groups(offsets, counts)):
        if e > s:
            w = b[g].t() if trans_b else b[g]
            out[s:e] = a[s:e] @ w
    return out


def grouped_wgrad(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, num_groups: int,
                  counts: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[g] = a[rows of g]^T @ b[rows of g]  -> [G, a.shape[1], b.shape[1]] (fp32 accumulate)."""
    out = torch.zeros(num_groups, a.shape[1], b.shape[1], dtype=a.dtype, device=a.device)
    for g, (s, e) in enumerate(_groups(offsets, counts)):
        if e > s:
            out[g] = (a[s:e].float().t() @ b[s:e].float()).to(a.dtype)
    return out


def _lora_delta(x, A, B, scaling, offsets, counts):
    """scaling * (x A_g) B_g per group, with the intermediate rounded to x.dtype."""
    xa = grouped_mm(x, A, offsets, trans_b=False, counts=counts)
    xa = (xa.float() * scaling).to(x.dtype)
    return grouped_mm(xa, B, offsets, trans_b=False, counts=counts)


def grouped_linear(x, w, offsets, trans_b, counts=None, lora=None):
    """Grouped linear with optional per-group LoRA (A:[G,K,r], B:[G,r,N], scaling)."""
    y = grouped_mm(x, w, offsets, trans_b, counts)
    if lora is not None:
        A, B, scaling = lora
        y = y + _lora_delta(x, A, B, scaling, offsets, counts)
    return y


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    return (F.silu(g.float()) * u.float()).to(g.dtype)


def grouped_swiglu_mlp(xg, w1, w2, w3, offsets, counts=None, lora=None, wgrad_scale: float = 1.0):
    """Expert MLP on grouped rows.  w1, w3, w2: [G, F, H] (w2 stored transposed).

    lora: optional dict name -> (A, B, scaling) for any of "w1", "w2", "w3".
    wgrad_scale multiplies the gradients of w1, w2, w3 and of the LoRA factors (every
    parameter of an expert sees the tokens of all expert-parallel peers).
    """
    lora = {k: (scale_gradient(A, wgrad_scale), scale_gradient(B, wgrad_scale), s)
            for k, (A, B, s) in (lora or {}).items()}
    w1, w2, w3 = (scale_gradient(w, wgrad_scale) for w in (w1, w2, w3))
    g = grouped_linear(xg, w1, offsets, True, counts, lora.get("w1"))
    u = grouped_linear(xg, w3, offsets, True, counts, lora.get("w3"))
    h = swiglu(g, u)
    return grouped_linear(h, w2, offsets, False, counts, lora.get("w2"))


# ----------------------------------------------------------------------------
# dense layers
# ----------------------------------------------------------------------------
def linear(x, w, lora=None):
    """y = x w^T (+ scaling * (x A^T) B^T with peft layout A:[r,in], B:[out,r])."""
    y = F.linear(x, w)
    if lora is not None:
        A, B, scaling = lora
        xa = (F.linear(x, A).float() * scaling).to(x.dtype)
        y = y + F.linear(xa, B)
    return y


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (weight.float() * (xf * torch.rsqrt(var + eps))).to(x.dtype)


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE (HF convention).  x: [T, heads, d]; positions: [T]."""
    d = x.shape[-1]
    cos, sin = rope_cos_sin(positions, d, theta)
    cos, sin = cos[:, None, :], sin[:, None, :]
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def attention(q, k, v, cu_seqlens: torch.Tensor, scale: Optional[float] = None):
    """Causal GQA attention over packed sequences.

    q: [T, Hq, d]; k, v: [T, Hkv, d]; cu_seqlens: [B+1] int32 sequence boundaries.
    """
    T, Hq, d = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    scale = scale if scale is not None else d ** -0.5
    out = torch.empty_like(q)
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e <= s:
            continue
        qs = q[s:e].transpose(0, 1).float()                                  # [Hq, S, d]
        ks = k[s:e].transpose(0, 1).float().repeat_interleave(rep, dim=0)
        vs = v[s:e].transpose(0, 1).float().repeat_interleave(rep, dim=0)
        att = (qs @ ks.transpose(1, 2)) * scale
        S = e - s
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        out[s:e] = (att @ vs).transpose(0, 1).to(q.dtype)
    return out


def cross_entropy_sum(hidden: torch.Tensor, w_head: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """Sum of token CE losses (fp32 logits) and the number of counted tokens.

    `labels` are already shifted: labels[t] is the target of position t.
    """
    logits = F.linear(hidden, w_head).float()
    loss = F.cross_entropy(logits, labels.long(), ignore_index=ignore_index, reduction="sum")
    n = (labels != ignore_index).sum()
    return loss, n


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale: float = 1.0):
    """In-place decoupled-weight-decay Adam on one tensor (fp32 math, any storage dtype)."""
    gf = g.float() * grad_scale
    mf = m.float().mul_(beta1).add_(gf, alpha=1 - beta1)
    vf = v.float().mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    pf = p.float().mul_(1 - lr * weight_decay)
    denom = (vf / bc2).sqrt_().add_(eps)
    pf.addcdiv_(mf / bc1, denom, value=-lr)
    p.copy_(pf)
    m.copy_(mf)
    v.copy_(vf)
