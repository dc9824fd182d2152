"""Import path kept for users of the reference (`utils.prepare_peft`)."""
from moe_distributed_training_b200.peft.lora import prepare_peft  # noqa: F401
