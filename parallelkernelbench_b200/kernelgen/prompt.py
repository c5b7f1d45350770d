"""Builds the task prompt for one op: what to compute, the reference implementation, the solution-file contract, the
building blocks this package offers and the hardware the kernel will run on."""
from __future__ import annotations

import inspect
import os
import textwrap
import tomllib

_TEMPLATE_FILE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "templates.toml")


def load_templates(path: str | None = None) -> dict:
    """The prompt templates (``contract``, ``[hardware]`` profiles, ``[precision]`` notes) from the packaged
    ``templates.toml``, with the entries of ``path`` - a file of the same layout - laid over them (reference:
    kernelgen/prompts.toml keeps its templates in TOML for the same reason: they are edited far more often than code)."""
    with open(_TEMPLATE_FILE, "rb") as fh:
        base = tomllib.load(fh)
    if path:
        with open(path, "rb") as fh:
            extra = tomllib.load(fh)
        for key, val in extra.items():
            if isinstance(val, dict) and isinstance(base.get(key), dict):
                base[key].update(val)
            else:
                base[key] = val
    return base


_T = load_templates()
HARDWARE_PROFILES = {k: v.rstrip("\n") for k, v in _T["hardware"].items()}
CONTRACT = _T["contract"].rstrip("\n")
PRECISION_NOTES = {k: v.rstrip("\n") for k, v in _T["precision"].items()}


def select_ops(selector: str) -> list[str]:
    """``"all"``, one op name or reference problem number, or a comma-separated / bracketed list of them
    (``"13"``, ``"allreduce,13"``, ``"[1, 8, 13]"``) -> op names in registry order, without duplicates
    (reference: kernelgen/generate_kernel.py:203-232 takes ``--problem all | [a,b] | id``)."""
    from ..workloads import registry

    sel = selector.strip()
    if sel == "all":
        return [s.name for s in registry.all_ops()]
    names = []
    for item in sel.strip("[]").split(","):
        item = item.strip()
        if item:
            name = registry.get(item).name
            if name not in names:
                names.append(name)
    if not names:
        raise ValueError(f"no op selected by {selector!r}")
    return names


def build_prompt(op: str, hardware: str = "b200_8", nproc: int = 8, feedback: str | None = None,
                 precision: str | None = None, templates: str | None = None) -> str:
    """The task prompt of one op. ``templates``: a TOML file whose entries replace the packaged templates."""
    from ..workloads import registry

    spec = registry.get(op)
    hw_profiles, contract, precision_notes = HARDWARE_PROFILES, CONTRACT, PRECISION_NOTES
    if templates:
        t = load_templates(templates)
        hw_profiles, contract, precision_notes = t["hardware"], t["contract"], t["precision"]
    parts = [f"# Task: a fast multi-GPU implementation of `{spec.name}`"
             + (f" (reference problems {', '.join(map(str, spec.problem_ids))})" if spec.problem_ids else ""),
             spec.doc or "", "## Hardware", hw_profiles[hardware].rstrip("\n"),
             "## Contract", contract.rstrip("\n").format(op=spec.name, nproc=nproc, atol=spec.atol, rtol=spec.rtol),
             "## Precision", precision_notes.get(precision or "", "").rstrip("\n"),
             "## Named shape configurations", "\n".join(f"- {k}: {v}" for k, v in spec.configs.items()),
             "## Input factory", _source(spec.make_inputs), "## Reference implementation (PyTorch + process group)",
             _source(spec.reference)]
    parts += ["## Worked examples (reference next to a solution file that passes the evaluation)", _examples_section(spec.name)]
    if feedback:
        parts += ["## Result of your previous attempt", feedback]
    return "\n\n".join(p for p in parts if p)


def _examples_section(current_op: str) -> str:
    """Reference/solution pairs of a few ops (the pair of the op being asked for is left out: it would be the answer)."""
    from ..workloads import registry
    from .examples import EXAMPLES, example_source

    out = []
    for op in EXAMPLES:
        if op == current_op:
            continue
        spec = registry.get(op)
        out.append(f"### `{op}`: reference\n{_source(spec.reference)}\n### `{op}`: solution file\n```python\n{example_source(op).rstrip()}\n```")
    return "\n\n".join(out)


def _source(fn) -> str:
    try:
        return "```python\n" + textwrap.dedent(inspect.getsource(fn)).rstrip() + "\n```"
    except (OSError, TypeError):
        return f"(source of {getattr(fn, '__name__', fn)!r} is not available)"
