"""Import-compatible names for code written against the reference's `megablocks_utils` package.

The implementations live in `moe_distributed_training_b200` (`parallel/shard_moe.py`, `moe/`, `peft/`); the modules
here re-export them under the reference's module and function names.
"""
