"""Mixtral decoder-only model on packed (variable-length) token streams.

The reference trains Hugging Face's `MixtralForCausalLM`
(train_accelerate_fsdp2.py:67-72) and swaps each layer's `block_sparse_moe` for
its own MoE layer (megablocks_utils/shard_moe_utils.py:308-313).  This is an
own implementation with the same module/parameter names, so that HF Mixtral
safetensors map onto it one to one:

  model.embed_tokens.weight
  model.layers.{i}.input_layernorm.weight
  model.layers.{i}.self_attn.{q,k,v,o}_proj.weight
  model.layers.{i}.post_attention_layernorm.weight
  model.layers.{i}.block_sparse_moe.router.layer.weight      (HF: ...gate.weight)
  model.layers.{i}.block_sparse_moe.experts.mlp.w{1,2,3}     (HF: ...experts.{e}.w{1,2,3}.weight)
  model.norm.weight
  lm_head.weight

All heavy math goes through `ops`, i.e. the sm_100a kernels on CUDA tensors.
Tokens are kept as a packed `[T, hidden]` stream with `cu_seqlens` boundaries;
a `[B, S]` batch is the special case of B equal-length sequences.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..config import MixtralConfig, MoEArguments
from ..moe.layer import dMoE


class Linear(nn.Module):
    """Bias-free linear layer with optional LoRA factors in peft's naming.

    `lora_A.default.weight` is `[r, in]`, `lora_B.default.weight` is `[out, r]`
    and the layer computes `x W^T + (alpha/r) (x A^T) B^T`.
    """

    def __init__(self, in_features: int, out_features: int, dtype=None, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.lora_A: Optional[nn.ModuleDict] = None
        self.lora_B: Optional[nn.ModuleDict] = None
        self.scaling = 0.0

    def add_lora(self, r: int, alpha: float, dtype=None):
        dev, dt = self.weight.device, dtype or self.weight.dtype
        a, b = nn.Module(), nn.Module()
        a.weight = nn.Parameter(torch.empty(r, self.in_features, dtype=dt, device=dev))
        b.weight = nn.Parameter(torch.zeros(self.out_features, r, dtype=dt, device=dev))
        if dev.type != "meta":
            nn.init.kaiming_uniform_(a.weight, a=5 ** 0.5)
        self.lora_A = nn.ModuleDict({"default": a})
        self.lora_B = nn.ModuleDict({"default": b})
        self.scaling = alpha / r
        self.weight.requires_grad_(False)

    def forward(self, x):
        lora = None
        if self.lora_A is not None:
            lora = (self.lora_A["default"].weight, self.lora_B["default"].weight, self.scaling)
        return ops.linear(x, self.weight, lora)


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float, dtype=None, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


@dataclass
class PackedBatch:
    """Description of the packed token stream that flows through the decoder."""
    cu_seqlens: torch.Tensor   # [B+1] int32
    positions: torch.Tensor    # [T] int32, position of every token inside its sequence
    max_seqlen: int


class MixtralAttention(nn.Module):
    def __init__(self, cfg: MixtralConfig, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.num_heads, self.num_kv_heads, self.head_dim = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        h = cfg.hidden_size
        self.q_proj = Linear(h, self.num_heads * self.head_dim, dtype, device)
        self.k_proj = Linear(h, self.num_kv_heads * self.head_dim, dtype, device)
        self.v_proj = Linear(h, self.num_kv_heads * self.head_dim, dtype, device)
        self.o_proj = Linear(self.num_heads * self.head_dim, h, dtype, device)

    def forward(self, x: torch.Tensor, batch: PackedBatch) -> torch.Tensor:
        T = x.shape[0]
        q = self.q_proj(x).view(T, self.num_heads, self.head_dim)
        k = self.k_proj(x).view(T, self.num_kv_heads, self.head_dim)
        v = self.v_proj(x).view(T, self.num_kv_heads, self.head_dim)
        q = ops.rope(q, batch.positions, self.cfg.rope_theta)
        k = ops.rope(k, batch.positions, self.cfg.rope_theta)
        o = ops.attention(q, k, v, batch.cu_seqlens, batch.max_seqlen)
        return self.o_proj(o.reshape(T, self.num_heads * self.head_dim))


class MixtralDecoderLayer(nn.Module):
    def __init__(self, cfg: MixtralConfig, moe_args: MoEArguments, dtype=None, device=None):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.self_attn = MixtralAttention(cfg, dtype, device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)
        self.block_sparse_moe = dMoE(moe_args)

    def forward(self, x: torch.Tensor, batch: PackedBatch) -> torch.Tensor:
        fused = x.is_cuda and ops.get_backend() == "native" and x.dim() == 2 and os.environ.get("MDT_FUSED_BLOCKS", "1") != "0"
        if fused:
            from ..ops import fused_blocks
        if fused and self.self_attn.head_dim == 128:
            x = fused_blocks.attention_block(self, x, batch)      # one autograd node for the whole sub-block
        else:
            x = x + self.self_attn(self.input_layernorm(x), batch)
        if fused and fused_blocks.moe_block_supported(self, x):
            return fused_blocks.moe_block(self, x)
        moe_out, _ = self.block_sparse_moe(self.post_attention_layernorm(x))
        return x + moe_out


class MixtralModel(nn.Module):
    def __init__(self, cfg: MixtralConfig, moe_args: MoEArguments, dtype=None, device=None):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList(
            [MixtralDecoderLayer(cfg, moe_args, dtype, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor]
    hidden_states: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    num_tokens: Optional[torch.Tensor] = None


def moe_args_from_config(cfg: MixtralConfig, dtype: torch.dtype, device) -> MoEArguments:
    return MoEArguments(
        hidden_size=cfg.hidden_size, ffn_hidden_size=cfg.intermediate_size,
        moe_num_experts=cfg.num_local_experts, moe_top_k=cfg.num_experts_per_tok,
        bf16=dtype == torch.bfloat16, fp16=dtype == torch.float16, device=device,
        init_std=cfg.initializer_range, moe_loss_weight=cfg.router_aux_loss_coef)


def shift_labels(labels: torch.Tensor, cu_seqlens: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Next-token targets on a packed stream: target[t] = labels[t+1], none across a sequence end."""
    out = torch.full_like(labels, ignore_index)
    out[:-1] = labels[1:]
    ends = (cu_seqlens[1:] - 1).long()
    out[ends] = ignore_index
    return out


class MixtralForCausalLM(nn.Module):
    def __init__(self, cfg: MixtralConfig, moe_args: Optional[MoEArguments] = None,
                 dtype: torch.dtype = torch.float32, device="cpu"):
        super().__init__()
        self.config = cfg
        self.dtype_ = dtype
        moe_args = moe_args or moe_args_from_config(cfg, dtype, device)
        self.model = MixtralModel(cfg, moe_args, dtype, device)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, dtype, device)
        if torch.device(device).type != "meta":
            self.reset_parameters()
        # set by the parallel wrappers: runs one decoder layer (checkpointing, parameter gathering)
        self.layer_runner = None

    @torch.no_grad()
    def reset_parameters(self, seed: Optional[int] = None):
        """N(0, initializer_range) for every matrix, ones for the norms."""
        gen = None
        std = self.config.initializer_range
        for name, p in self.named_parameters():
            if p.device.type == "meta":
                continue
            if name.endswith("layernorm.weight") or name.endswith("model.norm.weight"):
                p.fill_(1.0)
            elif "lora_B" in name:
                p.zero_()
            elif "lora_A" in name:
                nn.init.kaiming_uniform_(p, a=5 ** 0.5)
            else:
                p.normal_(0.0, std, generator=gen)

    # ------------------------------------------------------------------
    @staticmethod
    def pack(input_ids: torch.Tensor, labels: Optional[torch.Tensor], cu_seqlens: Optional[torch.Tensor]):
        if input_ids.dim() == 2:
            B, S = input_ids.shape
            cu = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=input_ids.device)
            pos = torch.arange(S, dtype=torch.int32, device=input_ids.device).repeat(B)
            ids = input_ids.reshape(-1)
            lab = labels.reshape(-1) if labels is not None else None
            return ids, lab, PackedBatch(cu, pos, S)
        assert cu_seqlens is not None, "packed 1-D input needs cu_seqlens"
        cu = cu_seqlens.to(torch.int32)
        lens = (cu[1:] - cu[:-1]).long()
        T = input_ids.shape[0]
        starts = torch.repeat_interleave(cu[:-1].long(), lens, output_size=T)
        pos = (torch.arange(T, device=input_ids.device) - starts).int()
        return input_ids, labels, PackedBatch(cu, pos, 0)

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None,
                use_cache: bool = False, return_logits: bool = False) -> CausalLMOutput:
        ids, lab, batch = self.pack(input_ids, labels, cu_seqlens)
        if max_seqlen is not None:
            batch.max_seqlen = max_seqlen
        elif batch.max_seqlen == 0:
            batch.max_seqlen = int(ids.shape[0])
        runner = self.layer_runner
        x = runner.embed(ids) if runner is not None else ops.embedding(ids, self.model.embed_tokens.weight)
        for i, layer in enumerate(self.model.layers):
            x = runner.run_layer(i, layer, x, batch) if runner is not None else layer(x, batch)
        if runner is not None:
            return runner.head(x, lab, batch, return_logits)
        return self.head(x, lab, batch, return_logits)

    def head(self, x, lab, batch: PackedBatch, return_logits: bool = False) -> CausalLMOutput:
        x = self.model.norm(x)
        logits = self.lm_head(x) if return_logits else None
        if lab is None:
            return CausalLMOutput(None, x, logits)
        targets = shift_labels(lab, batch.cu_seqlens)
        loss_sum, n = ops.cross_entropy_sum(x, self.lm_head.weight, targets)
        loss = loss_sum / n.clamp(min=1).to(loss_sum.dtype)
        return CausalLMOutput(loss, x, logits, n)

    def moe_layers(self):
        return [l.block_sparse_moe for l in self.model.layers]
