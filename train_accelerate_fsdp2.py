"""FSDP2-style entry point: sharded dense parameters + expert-parallel dropless MoE.

    torchrun --nproc_per_node=8 --master-addr 127.0.0.1 train_accelerate_fsdp2.py \
        --use_megablocks_sharding True --gradient_accumulation_steps 16 --learning_rate 5e-5

Same flags as the reference script of this name (train_accelerate_fsdp2.py:48-65):
every keyword of `main` is a `--flag value` option.
"""
from moe_distributed_training_b200.cli import run
from moe_distributed_training_b200.train.run import run_training


def main(
    max_seq_length: int = 4096,
    load_model_dtype: str = "bfloat16",
    attn_implementation: str = "sdpa",
    per_device_train_batch_size: int = 1,
    gradient_accumulation_steps: int = 1,
    use_megablocks_sharding: bool = False,
    use_scattermoe: bool = False,
    use_tp_sharding: bool = False,
    lr_scheduler_type: str = "linear",
    num_epochs: int = 1,
    num_warmup_steps: int = 0,
    max_grad_norm: float = 1.0,
    learning_rate: float = 1e-5,
    truncate_model_for_debug: bool = False,
    expert_degree: int = None,
    use_lora: str = "none",
    debug: bool = False,
    model_name_or_path: str = "mistralai/Mixtral-8x7B-Instruct-v0.1",
    model_preset: str = "mixtral-8x7b",
    data_path: str = "data.json",
    num_synthetic_examples: int = 64,
    synthetic_min_len: int = 128,
    synthetic_max_len: int = 1024,
    device_type: str = "cuda",
    dispatch_impl: str = "auto",
    sync_each_batch: bool = False,
    activation_checkpointing: bool = True,
    seed: int = 0,
    save_path: str = None,
    resume_from: str = None,
    max_steps: int = 0,
    profile_trace: str = None,
    profile_steps: int = 2,
):
    kw = dict(locals())
    if kw.pop("debug"):
        kw["truncate_model_for_debug"] = True
    return run_training(**kw)


if __name__ == "__main__":
    run(main)
