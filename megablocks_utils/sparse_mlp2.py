"""Import path kept for users of the reference (`megablocks_utils.sparse_mlp2.SparseMLPv2`)."""
from moe_distributed_training_b200.moe.experts import SparseMLPv2  # noqa: F401
