"""Import path kept for users of the reference (`megablocks_utils.config_utils`).

The reference's `update_mlp_registry()` patches megablocks classes at import time
(megablocks_utils/config_utils.py:71-284).  Here the MoE layer already has that behaviour,
so the function only reports which implementations exist.
"""
from moe_distributed_training_b200.moe.layer import MoE, ParallelDroplessMLP, dMoE  # noqa: F401
from moe_distributed_training_b200.moe.router import LearnedRouter  # noqa: F401


def get_mlp_weights(mod, name):
    """`[E_local, in, out]`-style view the grouped kernels consume (config_utils.py:28-35)."""
    w1, w2, w3 = mod.mlp.weight_views()
    return {"w1": w1, "w2": w2, "w3": w3}[name]


def get_mlp_weights_lora(mod, name):
    A, B, r, alpha, _, _ = mod.mlp._lora_pointers[name]
    return get_mlp_weights(mod, name), A, B, r, alpha


def get_mlp_device_mesh_pg(mod):
    """Process group over which `mod`'s experts are split (the reference takes the last mesh dimension of the
    weights' DTensor mesh, megablocks_utils/config_utils.py:63-69): the tensor-parallel group in the TP mode, else the
    expert-parallel group; None on a single rank."""
    args = mod.args
    if getattr(args, "tensor_parallel_group", None) is not None and args.tensor_parallel_size > 1:
        return args.tensor_parallel_group
    return args.expert_parallel_group if args.moe_expert_model_parallelism else None


def update_mlp_registry():
    return {"mlp": {"sparse": "SparseMLPv2", "scattermoe": "SparseMLPv2"}}
