"""python -m parallelkernelbench_b200.kernelgen prompt --op OP | replay --op OP --candidates DIR"""
import argparse
import json
import sys

from . import ReplayProposer, build_prompt, optimise


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prompt")
    p.add_argument("--op", required=True)
    p.add_argument("--hardware", default="b200_8")
    p.add_argument("--nproc", type=int, default=8)
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
        print(build_prompt(a.op, a.hardware, a.nproc))
        return 0
    out = optimise(a.op, ReplayProposer(a.candidates), a.workdir, nproc=a.nproc, backend=a.backend, dtype=a.dtype, config=a.config)
    print(json.dumps(out, indent=1))
    return 0 if out["solved"] else 1


if __name__ == "__main__":
    sys.exit(main())
