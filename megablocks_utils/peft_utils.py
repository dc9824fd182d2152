"""Import path kept for users of the reference (`megablocks_utils.peft_utils`)."""
from moe_distributed_training_b200.peft.lora import ARTIFACTS, ParallelDroplessMLP, ParallelMLP  # noqa: F401
