"""Builds the task prompt for one op: what to compute, the reference implementation, the solution-file contract, the
building blocks this package offers and the hardware the kernel will run on."""
from __future__ import annotations

import inspect
import textwrap

HARDWARE_PROFILES = {
    "b200_8": textwrap.dedent("""\
        8 x NVIDIA B200 (sm_100a) in one node, every pair connected at full NVLink 5 bandwidth through NVSwitch
        (900 GB/s per direction per GPU, in-switch reduction through multimem instructions); 148 SMs, 227 KB shared
        memory per CTA, 256 KB tensor memory per SM, 126 MB L2, 180 GB HBM3e at about 6.5 TB/s measured copy bandwidth;
        dense bf16 about 1.4-1.6 PFLOP/s measured. Matrix products belong on tcgen05.mma with accumulators in tensor
        memory and operands staged by TMA.
        Off-limits in any candidate (it runs on two or more ranks of a shared machine, and the evaluator refuses the file
        before building it): any TMA or bulk load with cluster multicast (local sources included - let each CTA fetch its
        own tile, or stage a remote tile in local memory first); the batched memcpy entry points of the CUDA runtime and
        driver (issue one cudaMemcpyAsync per copy or gather with a kernel); device traps and failing device asserts;
        any spin or wait without an iteration or time limit (on expiry record a status and return); changing clocks, power
        limits or any other GPU setting."""),
    "cpu_gloo": "CPU ranks over gloo and a shared-memory twin of the symmetric heap: correctness of the host logic only.",
}

CONTRACT = textwrap.dedent("""\
    Write ONE Python file that defines

        def solution(rc, *inputs): ...

    with the same inputs and the same outputs (types, shapes, dtypes, tuple/dict structure) as the reference below.
    `rc` gives rc.rank, rc.world, rc.device, rc.dtype and rc.comm, whose collectives run on a symmetric heap that every
    rank maps: all_reduce(x, op="sum", scale=1.0), all_gather(x) -> [W, ...], reduce_scatter(x), all_to_all(x[W, ...]),
    all_to_all_v(rows, counts, capacity), all_to_all_permute(x, scatter_dim, gather_dim), row_gather(shard, ids),
    broadcast / reduce / scatter / gather, barrier(); rc.comm.heap allocates tensors that peers can address.
    A result whose length is only known on the device may be returned as utils.ragged.Ragged(buffer, count[, dim]) - a capacity
    buffer and a device-side count, trimmed by the harness when it stores the output - so that no size has to come back to the
    host inside the timed call (never call .item() / .tolist() on the hot path).
    Kernels of this package: ops.gemm_bf16 (a @ w.T on tcgen05), ops.gemm_bf16_kn, ops.gemm_bf16_tn, ops.rmsnorm,
    ops.rope, ops.fp8_quantize_1x128 / fp8_dequantize_1x128, ops.attention.flash_attn_fwd / flash_attn_bwd /
    RingAttention, ops.tp.AllGatherGemm / GemmReduceScatterRMSNorm, ops.moe.MoEExchange / grouped_gemm.
    Your own CUDA kernel: utils.cuda_ext.compile_cuda_module(source_text, name) builds it for sm_100a (the package's device
    headers pkb/ptx.cuh - mbarrier, TMA, tcgen05, bounded waits - and pkb/symm.cuh - symmetric-heap view, cross-GPU barriers -
    are on the include path) and returns a ctypes library; call its extern "C" functions with tensor.data_ptr() and
    torch.cuda.current_stream().cuda_stream. Every device-side wait must be bounded; never trap or spin without a limit.
    The file is evaluated with
        python -m parallelkernelbench_b200.harness.launch eval --op {op} --nproc {nproc} --solution your_file.py --measure-perf
    which compares every rank's output with the reference within atol={atol}, rtol={rtol} over seeded trials and reports
    reference time / your time (device-timed, max over ranks). Aim for correctness first, then for the fewest launches and
    the fewest bytes over NVLink.""")


PRECISION_NOTES = {
    "bfloat16": "Inputs and outputs are bf16. Accumulate matrix products, reductions and normalisation statistics in fp32 and "
                "round once at the end; a sum over ranks must not depend on the order in which peers arrive.",
    "float32": "Inputs and outputs are fp32 (the CPU plumbing configuration): keep every reduction in fp32.",
}


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
                 precision: str | None = None) -> str:
    from ..workloads import registry

    spec = registry.get(op)
    parts = [f"# Task: a fast multi-GPU implementation of `{spec.name}`"
             + (f" (reference problems {', '.join(map(str, spec.problem_ids))})" if spec.problem_ids else ""),
             spec.doc or "", "## Hardware", HARDWARE_PROFILES[hardware],
             "## Contract", CONTRACT.format(op=spec.name, nproc=nproc, atol=spec.atol, rtol=spec.rtol),
             "## Precision", PRECISION_NOTES.get(precision or "", ""),
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
