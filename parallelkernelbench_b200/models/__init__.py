"""Composite blocks built from the fused ops."""
from .tp_mlp import TPMLPBlock, TPMLPConfig  # noqa: F401
