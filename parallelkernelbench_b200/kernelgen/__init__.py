"""Prompt assembly and the generate -> evaluate -> feedback loop for candidate kernels written by a model.

Counterpart of the reference's kernel-generation tooling (reference: kernelgen/generate_kernel.py:239-363,
kernelgen/generate_kernel_agent.py:281-343, kernelgen/prompts.toml). No model client is bundled - there is no network
here - so the loop takes any callable ``propose(prompt, feedback) -> source``; :class:`ReplayProposer` replays files and
:class:`CommandProposer` pipes the prompt through an operator-supplied command (a local model runner, a script).
"""
from .agent import CommandProposer, ReplayProposer, extract_code, optimise  # noqa: F401
from .prompt import HARDWARE_PROFILES, build_prompt  # noqa: F401
