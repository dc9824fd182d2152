"""Configuration dataclasses.

`MixtralConfig` mirrors the fields of the Hugging Face Mixtral `config.json` that
the training stack consumes.  `MoEArguments` is the configuration of one MoE
layer; it plays the role that megablocks' `Arguments` object plays in the
reference (built there by `get_moe_kwargs`, megablocks_utils/shard_moe_utils.py:26-46,
and instantiated at megablocks_utils/shard_moe_utils.py:250-253).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Optional

import torch


@dataclass
class MixtralConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: Optional[int] = None
    num_local_experts: int = 8
    num_experts_per_tok: int = 2
    rms_norm_eps: float = 1e-5
    rope_theta: float = 1e6
    max_position_embeddings: int = 32768
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False
    router_aux_loss_coef: float = 0.0  # the reference never computes the aux loss
    model_type: str = "mixtral"

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    # -- presets -----------------------------------------------------------
    @classmethod
    def mixtral_8x7b(cls) -> "MixtralConfig":
        return cls()

    @classmethod
    def tiny(cls) -> "MixtralConfig":
        """2-layer plumbing model used by the CPU/gloo tests."""
        return cls(
            vocab_size=1024, hidden_size=256, intermediate_size=512,
            num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            num_local_experts=4, num_experts_per_tok=2,
        )

    # -- HF config.json ----------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "MixtralConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    @classmethod
    def from_pretrained(cls, path: str) -> "MixtralConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        d = dataclasses.asdict(self)
        d["architectures"] = ["MixtralForCausalLM"]
        return d

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=2)

    def num_params(self) -> dict:
        h, f, e = self.hidden_size, self.intermediate_size, self.num_local_experts
        qd = self.num_attention_heads * self.head_dim
        kvd = self.num_key_value_heads * self.head_dim
        attn = h * qd * 2 + h * kvd * 2
        experts = 3 * h * f * e
        per_layer = attn + experts + e * h + 2 * h
        emb = self.vocab_size * h
        total = per_layer * self.num_hidden_layers + emb * (1 if self.tie_word_embeddings else 2) + h
        active = (attn + 3 * h * f * self.num_experts_per_tok + e * h) * self.num_hidden_layers + emb
        return {"total": total, "experts_per_layer": experts, "attention_per_layer": attn, "active_per_token": active}


@dataclass
class MoEArguments:
    """Configuration of one dropless MoE layer.

    Field names follow megablocks' `Arguments` so that code written against the
    reference's `get_moe_kwargs` keeps working.
    """
    hidden_size: int = 4096
    ffn_hidden_size: int = 14336
    moe_num_experts: int = 8
    moe_top_k: int = 2
    moe_expert_model_parallelism: bool = False
    expert_parallel_group: Any = None
    moe_normalize_expert_weights: Any = True  # True -> L1 (p=1); a number -> that p-norm; None -> off
    moe_loss_weight: float = 0.0
    moe_jitter_eps: Optional[float] = None
    moe_capacity_factor: int = 0  # dropless: never used
    memory_optimized_mlp: bool = False
    mlp_type: str = "mlp"
    mlp_impl: str = "sparse"  # "sparse" (block-padded grouped GEMM) | "scattermoe" (same kernels, LoRA capable)
    bias: bool = False
    return_bias: bool = False
    uniform_expert_assignment: bool = False
    fp16: bool = False
    bf16: bool = True
    device: Any = "cpu"
    init_std: float = 0.02
    # tensor-parallel slicing of every expert's FFN dim (use_tp_sharding)
    tensor_parallel_group: Any = None
    tensor_parallel_size: int = 1
    # which token-exchange implementation the EP layer uses: "nccl" = torch all_to_all_single
    # (works on gloo too), "fused" = in-kernel peer stores over NVLink.
    dispatch_impl: str = "auto"
    # most tokens one rank feeds into an MoE layer per call; sizes the symmetric receive buffers of the
    # fused exchange for the dropless worst case
    ep_max_tokens: int = 4096

    @property
    def dtype(self) -> torch.dtype:
        if self.bf16:
            return torch.bfloat16
        if self.fp16:
            return torch.float16
        return torch.float32


@dataclass
class LoraConfig:
    """Subset of peft.LoraConfig used by the reference (train_accelerate_fsdp2.py:259-266)."""
    r: int = 16
    lora_alpha: int = 16
    lora_dropout: float = 0.0
    bias: str = "none"
    target_modules: list = field(default_factory=lambda: ["q_proj", "k_proj", "v_proj", "o_proj"])
    task_type: str = "CAUSAL_LM"
    init_lora_weights: bool = True

    @property
    def scaling(self) -> float:
        return self.lora_alpha / self.r

    def to_dict(self) -> dict:
        d = dataclasses.asdict(self)
        d["peft_type"] = "LORA"
        return d
