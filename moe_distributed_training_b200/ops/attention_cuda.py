"""Causal grouped-query attention over packed sequences on CUDA."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def sdpa_attention(q, k, v, cu_seqlens, max_seqlen=None):
    """q [T, Hq, d], k/v [T, Hkv, d]; one causal attention problem per sequence in cu_seqlens."""
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


def attention(q, k, v, cu_seqlens, max_seqlen=None):
    return sdpa_attention(q, k, v, cu_seqlens, max_seqlen)
