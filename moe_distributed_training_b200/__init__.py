"""Blackwell-native distributed fine-tuning of Mixture-of-Experts language models."""
from .config import LoraConfig, MixtralConfig, MoEArguments  # noqa: F401

__version__ = "0.1.0"
