"""Declarative op registry.

Every workload is one :class:`OpSpec`: how to build seeded inputs, the PyTorch + NCCL reference,
our implementation, tolerances, named shape configs and an algorithmic cost model for the roofline.
This replaces the reference's 87-way ``if/elif`` input factory and its per-problem files
(reference: utils/input_output_tensors.py:265-1881, reference/*.py) with data the harness can
enumerate; ``problem_ids`` records which reference problems a spec covers.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..harness.roofline import Cost
from ..utils.seeding import seed_for

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          "float16": torch.float16, "fp16": torch.float16, "float64": torch.float64, "fp64": torch.float64}


class RunCtx:
    """What an op implementation sees: the distributed context, a seeded RNG and (for "ours") comm."""

    def __init__(self, dist_ctx, op_name: str, trial: int = 0, dtype: torch.dtype = torch.bfloat16):
        self.dist = dist_ctx
        self.rank, self.world, self.device = dist_ctx.rank, dist_ctx.world, dist_ctx.device
        self.op_name, self.trial, self.dtype = op_name, trial, dtype
        self._comm = None
        self._gens: dict = {}
        self.cache: dict = {}     # per-job state of an implementation (fused-op objects, buffers)

    @property
    def comm(self):
        if self._comm is None:
            from ..parallel.comm import Comm

            self._comm = Comm(self.dist)
        return self._comm

    def gen(self, shared: bool = False, salt: int = 0) -> torch.Generator:
        """Generator seeded by (op, rank, trial); ``shared=True`` gives every rank the same stream."""
        key = (shared, salt)
        if key not in self._gens:
            g = torch.Generator(device=self.device)
            g.manual_seed(seed_for(self.op_name, 0 if shared else self.rank, self.trial) + 7777 * salt)
            self._gens[key] = g
        return self._gens[key]

    def randn(self, *shape, dtype=None, std: float = 1.0, shared: bool = False, salt: int = 0) -> torch.Tensor:
        x = torch.randn(*shape, device=self.device, dtype=torch.float32, generator=self.gen(shared, salt))
        return (x * std).to(dtype or self.dtype)

    def randint(self, lo: int, hi: int, shape, shared: bool = False, dtype=torch.int64, salt: int = 0) -> torch.Tensor:
        return torch.randint(lo, hi, tuple(shape), device=self.device, dtype=dtype, generator=self.gen(shared, salt))

    def rand(self, *shape, shared: bool = False, salt: int = 0) -> torch.Tensor:
        return torch.rand(*shape, device=self.device, generator=self.gen(shared, salt))


@dataclass
class OpSpec:
    name: str
    make_inputs: Callable[[RunCtx, dict], tuple]
    reference: Callable[..., Any]           # reference(rc, *inputs)
    ours: Callable[..., Any] | None         # ours(rc, *inputs); None = not implemented yet
    problem_ids: tuple = ()
    configs: dict = field(default_factory=lambda: {"default": {}})
    atol: float = 1e-2
    rtol: float = 1e-2
    cost: Callable[[dict, int], Cost] | None = None
    ours_needs_cuda: bool = False           # "ours" uses a CUDA kernel with no CPU twin
    group: str = "misc"
    doc: str = ""
    mutates_inputs: bool = False            # inputs must be re-created for every timed call
    heap_gib: Callable[[dict, int], float] | None = None   # symmetric-heap size this op needs (config, world) -> GiB
    explicit_only: bool = False             # engine-sized workload: part of "all" selections only when named
    tol_note: str = ""                      # why the gate is looser than 1e-2 / 1e-2 (required whenever it is)

    def tolerance(self, config_name: str = "default") -> tuple[float, float]:
        """(atol, rtol) of a named config: a config may carry its own ``atol`` / ``rtol`` keys (a lower-precision variant of
        the op), otherwise the op's values apply."""
        cfg = self.configs.get(config_name, {})
        return float(cfg.get("atol", self.atol)), float(cfg.get("rtol", self.rtol))

    def config(self, name: str = "default", overrides: dict | None = None) -> dict:
        if name not in self.configs:
            raise KeyError(f"op {self.name!r} has no config {name!r} (has {sorted(self.configs)})")
        cfg = dict(self.configs[name])
        cfg.update(overrides or {})
        return cfg


_REGISTRY: dict[str, OpSpec] = {}
_MODULES = ["collectives", "tp", "quant", "optim", "moe", "ulysses", "attention", "wild", "llama"]
_loaded = False


def register(spec: OpSpec) -> OpSpec:
    if spec.name in _REGISTRY:
        raise ValueError(f"duplicate op {spec.name}")
    _REGISTRY[spec.name] = spec
    return spec


def load_all() -> None:
    global _loaded
    if _loaded:
        return
    _loaded = True
    for m in _MODULES:
        try:
            importlib.import_module(f"{__package__}.{m}")
        except ModuleNotFoundError as e:
            if e.name != f"{__package__}.{m}":
                raise
    from . import tolerances

    tolerances.attach(_REGISTRY.values())


def get(name: str) -> OpSpec:
    load_all()
    if name in _REGISTRY:
        return _REGISTRY[name]
    # allow lookup by reference problem number ("13") as well
    if name.isdigit():
        for s in _REGISTRY.values():
            if int(name) in s.problem_ids:
                return s
    raise KeyError(f"unknown op {name!r}; known: {sorted(_REGISTRY)}")


def all_ops() -> list[OpSpec]:
    load_all()
    return [_REGISTRY[k] for k in sorted(_REGISTRY)]


def coverage() -> dict[int, list[str]]:
    """reference problem id -> ops that cover it."""
    cov: dict[int, list[str]] = {}
    for s in all_ops():
        for pid in s.problem_ids:
            cov.setdefault(pid, []).append(s.name)
    return cov


def parse_overrides(items: list[str] | None) -> dict:
    out: dict = {}
    for it in items or []:
        k, _, v = it.partition("=")
        try:
            out[k] = int(v)
        except ValueError:
            try:
                out[k] = float(v)
            except ValueError:
                out[k] = {"true": True, "false": False}.get(v.lower(), v)
    return out
