"""Op registry: inputs, reference, ours, tolerances and cost model per workload."""
from .registry import OpSpec, RunCtx, all_ops, coverage, get, load_all, register  # noqa: F401
