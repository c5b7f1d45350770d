"""Prompt assembly and the generate -> evaluate -> feedback loop for candidate kernels written by a model.

Counterpart of the reference's kernel-generation tooling (reference: kernelgen/generate_kernel.py:239-363,
kernelgen/generate_kernel_agent.py:281-343, kernelgen/prompts.toml). No provider SDK is bundled; the loop takes any callable
``propose(prompt, feedback) -> source``: :class:`ReplayProposer` replays files, :class:`CommandProposer` pipes the prompt
through an operator-supplied command (a local model runner, a script), and :class:`HttpProposer` posts it to a
chat-completions endpoint (a model server next to the GPUs, or a hosted one where there is a network).
"""
from .agent import CommandProposer, HttpProposer, ReplayProposer, extract_code, optimise  # noqa: F401
from .prompt import HARDWARE_PROFILES, build_prompt  # noqa: F401
