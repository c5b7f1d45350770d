"""python -m parallelkernelbench_b200.kernelgen prompt --op OP|13|all|[a,b] [--out-dir DIR] | replay --op OP --candidates DIR"""
import argparse
import json
import sys

import os

from . import ReplayProposer, build_prompt, optimise
from .prompt import select_ops


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prompt")
    p.add_argument("--op", required=True)
    p.add_argument("--hardware", default="b200_8")
    p.add_argument("--nproc", type=int, default=8)
    p.add_argument("--precision", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--out-dir", default=None, help="write prompt_<op>.md per selected op instead of printing")
    r = sub.add_parser("replay", help="run the loop over recorded candidate files")
    r.add_argument("--op", required=True)
    r.add_argument("--candidates", required=True)
    r.add_argument("--workdir", default="logs/kernelgen")
    r.add_argument("--nproc", type=int, default=2)
    r.add_argument("--backend", default=None)
    r.add_argument("--dtype", default="bfloat16")
    r.add_argument("--config", default="default")
    a = ap.parse_args(argv)
    if a.cmd == "prompt":
        ops = select_ops(a.op)
        if a.out_dir:
            os.makedirs(a.out_dir, exist_ok=True)
        for op in ops:
            text = build_prompt(op, a.hardware, a.nproc, precision=a.precision)
            if a.out_dir:
                path = os.path.join(a.out_dir, f"prompt_{op}.md")
                with open(path, "w") as fh:
                    fh.write(text + "\n")
                print(path)
            else:
                if len(ops) > 1:
                    print(f"\n<!-- ===== {op} ===== -->")
                print(text)
        return 0
    out = optimise(a.op, ReplayProposer(a.candidates), a.workdir, nproc=a.nproc, backend=a.backend, dtype=a.dtype, config=a.config)
    print(json.dumps(out, indent=1))
    return 0 if out["solved"] else 1


if __name__ == "__main__":
    sys.exit(main())
