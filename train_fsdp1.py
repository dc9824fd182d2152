"""FSDP1-style entry point (trainer-argument flags; expert parallelism over all ranks only).

    torchrun --nproc_per_node=8 --master-addr 127.0.0.1 train_fsdp1.py \
        --use_megablocks_sharding --per_device_train_batch_size 1 --gradient_accumulation_steps 16 \
        --learning_rate 5e-5 --lr_scheduler_type linear --num_train_epochs 1 --bf16 --save_strategy no

The reference's script of this name drives HF `SFTTrainer` under accelerate's FSDP1 plugin and
shards the experts with `ep_size = world_size` (train_fsdp1.py:17-98, accelerate.yaml).  Here the
same `TrainingArguments`-style flags are mapped onto the framework's engine: flat-parameter
sharding of everything except the expert-parallel MoE modules, which is what FSDP1 with
`ignored_modules` does there (train_fsdp1.py:94-96).
"""
from moe_distributed_training_b200.cli import run
from moe_distributed_training_b200.train.run import run_training


def main(
    use_megablocks_sharding: bool = False,
    truncate_model_for_debug: bool = False,
    accelerator_config: str = None,
    per_device_train_batch_size: int = 1,
    per_device_eval_batch_size: int = 1,
    evaluation_strategy: str = "no",
    gradient_accumulation_steps: int = 1,
    learning_rate: float = 5e-5,
    lr_scheduler_type: str = "linear",
    num_train_epochs: int = 1,
    warmup_steps: int = 0,
    max_grad_norm: float = 1.0,
    max_seq_length: int = 4096,
    bf16: bool = True,
    gradient_checkpointing: bool = True,
    logging_steps: int = 1,
    save_strategy: str = "no",
    output_dir: str = "./results",
    torch_dtype: str = "bfloat16",
    model_name_or_path: str = "mistralai/Mixtral-8x7B-Instruct-v0.1",
    model_preset: str = "mixtral-8x7b",
    data_path: str = "data.json",
    num_synthetic_examples: int = 64,
    device_type: str = "cuda",
    max_steps: int = 0,
    seed: int = 0,
):
    if evaluation_strategy != "no":
        raise ValueError("evaluation_strategy: only 'no' is supported (the reference runs no evaluation either)")
    sync_each_batch = True       # what the reference's accelerator_config.json sets (accelerator_config.json:1-4)
    if accelerator_config:
        import json
        with open(accelerator_config) as f:
            ga = json.load(f).get("gradient_accumulation_kwargs") or {}
        sync_each_batch = bool(ga.get("sync_each_batch", sync_each_batch))
    return run_training(
        max_seq_length=max_seq_length, load_model_dtype="bfloat16" if bf16 else torch_dtype,
        per_device_train_batch_size=per_device_train_batch_size,
        gradient_accumulation_steps=gradient_accumulation_steps,
        use_megablocks_sharding=use_megablocks_sharding, lr_scheduler_type=lr_scheduler_type,
        num_epochs=num_train_epochs, num_warmup_steps=warmup_steps, max_grad_norm=max_grad_norm,
        learning_rate=learning_rate, truncate_model_for_debug=truncate_model_for_debug,
        expert_degree=None, use_lora="none", model_name_or_path=model_name_or_path, model_preset=model_preset,
        data_path=data_path, num_synthetic_examples=num_synthetic_examples, device_type=device_type,
        sync_each_batch=sync_each_batch, seed=seed, max_steps=max_steps, activation_checkpointing=gradient_checkpointing,
        save_path=None if save_strategy == "no" else output_dir, sharding_strategy="fsdp1")


if __name__ == "__main__":
    run(main)
