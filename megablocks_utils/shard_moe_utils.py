"""Import path kept for users of the reference (`megablocks_utils.shard_moe_utils`)."""
from moe_distributed_training_b200.checkpoint.hf_safetensors import (  # noqa: F401
    assign_mlp_v2_weights, get_router_experts_sharded_safetensor)
from moe_distributed_training_b200.parallel.shard_moe import (  # noqa: F401
    DIM_EXPERT, FILE_SAFETENSOR_INDEX, KEY_DATA_PARALLEL, KEY_EXPERT_PARALLEL, KEY_EXPERTS, KEY_ROUTER,
    get_moe_kwargs, get_resolved_checkpoint_location, shard_moe)
