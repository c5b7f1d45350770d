"""Composite blocks built from the fused ops."""
from .tp_mlp import TPMLPBlock, TPMLPConfig  # noqa: F401
from .llama import FSDPLlama, LlamaConfig  # noqa: F401
from .moe_layer import EPMoELayer, MoEConfig  # noqa: F401
