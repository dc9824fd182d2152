"""Causal grouped-query attention over packed sequences on CUDA.

head_dim 128 (Mixtral) runs on the tcgen05 kernels of `csrc/attention.cu`.  Other head sizes are
only used by toy configurations; they go through torch's SDPA, stated here explicitly rather than
hidden as a fallback.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F


def _sdpa_backends():
    """Flash / memory-efficient SDPA (what the reference's `attn_implementation='sdpa'` selects under its torch 2.3),
    not the cuDNN backend: that one builds a new execution plan for every new sequence length (6-7 ms of host time
    per call), which one-sequence micro-batches of random length would pay on every call."""
    from torch.nn.attention import SDPBackend, sdpa_kernel
    return sdpa_kernel([SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH])


def sdpa_attention(q, k, v, cu_seqlens, max_seqlen=None):
    """Library path (torch SDPA): the baseline, and the route for head_dim != 128."""
    with _sdpa_backends():
        return _sdpa_attention(q, k, v, cu_seqlens, max_seqlen)


def _sdpa_attention(q, k, v, cu_seqlens, max_seqlen=None):
    T = q.shape[0]
    nseq = cu_seqlens.numel() - 1
    if nseq == 1:
        bounds = [0, T]
    elif max_seqlen is not None and max_seqlen * nseq == T:
        bounds = list(range(0, T + 1, max_seqlen))
    else:
        bounds = cu_seqlens.tolist()
    outs = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        o = F.scaled_dot_product_attention(q[s:e].transpose(0, 1)[None], k[s:e].transpose(0, 1)[None],
                                           v[s:e].transpose(0, 1)[None], is_causal=True, enable_gqa=True)
        outs.append(o[0].transpose(0, 1))
    return outs[0].contiguous() if len(outs) == 1 else torch.cat(outs, 0)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, scale):
        from .cuda_ops import ext
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = ext.attention_fwd(q, k, v, cu_seqlens, max_seqlen, scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.max_seqlen, ctx.scale = max_seqlen, scale
        return o

    @staticmethod
    def backward(ctx, dout):
        from .cuda_ops import ext
        q, k, v, o, lse, cu = ctx.saved_tensors
        dq, dk, dv = ext.attention_bwd(q, k, v, o, dout.contiguous(), lse, cu, ctx.max_seqlen, ctx.scale)
        return dq, dk, dv, None, None, None


def attention(q, k, v, cu_seqlens, max_seqlen=None):
    if q.shape[-1] != 128 or os.environ.get("MDT_ATTENTION_IMPL") == "sdpa":  # env switch: A/B timing against the library
        return sdpa_attention(q, k, v, cu_seqlens, max_seqlen)
    return _Attention.apply(q, k, v, cu_seqlens.int(), int(max_seqlen or q.shape[0]), float(q.shape[-1]) ** -0.5)
