"""python -m parallelkernelbench_b200.kernelgen prompt --op OP|13|all|[a,b] [--out-dir DIR] | replay --op OP --candidates DIR |
generate --op OP --command "CMD" (CMD reads the prompt on stdin and prints a candidate) |
generate --op OP --endpoint http://host:8000/v1 --model NAME (a chat-completions endpoint; key from $PKB_KERNELGEN_API_KEY)"""
import argparse
import json
import sys

import os

from . import CommandProposer, HttpProposer, ReplayProposer, build_prompt, optimise
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
    p.add_argument("--prompts", default=None, help="TOML file whose entries replace the packaged templates (kernelgen/templates.toml)")
    r = sub.add_parser("replay", help="run the loop over recorded candidate files")
    r.add_argument("--op", required=True)
    r.add_argument("--candidates", required=True)
    r.add_argument("--workdir", default="logs/kernelgen")
    r.add_argument("--nproc", type=int, default=2)
    r.add_argument("--backend", default=None)
    r.add_argument("--dtype", default="bfloat16")
    r.add_argument("--config", default="default")
    g = sub.add_parser("generate", help="run the loop with a command that reads the prompt on stdin and prints a candidate")
    g.add_argument("--op", required=True)
    g.add_argument("--command", default=None, help="e.g. 'python my_model_runner.py' (prompt on stdin, reply on stdout)")
    g.add_argument("--endpoint", default=None, help="base URL of a chat-completions endpoint, e.g. http://127.0.0.1:8000/v1")
    g.add_argument("--model", default=None, help="model name sent to --endpoint")
    g.add_argument("--api-key-env", default="PKB_KERNELGEN_API_KEY", help="environment variable holding the endpoint's key, if it needs one")
    g.add_argument("--max-tokens", type=int, default=16384)
    g.add_argument("--workdir", default="logs/kernelgen")
    g.add_argument("--prompts", default=None, help="TOML file whose entries replace the packaged templates")
    g.add_argument("--hardware", default="b200_8", help="hardware profile of the templates to quote")
    g.add_argument("--nproc", type=int, default=2)
    g.add_argument("--max-iters", type=int, default=4)
    g.add_argument("--resume", action="store_true", help="continue a previous run of this op in --workdir from its last feedback")
    g.add_argument("--measure-perf", action="store_true", help="time reference and candidate; the best matching candidate is kept by speed-up")
    g.add_argument("--backend", default=None)
    g.add_argument("--dtype", default="bfloat16")
    g.add_argument("--config", default="default")
    a = ap.parse_args(argv)
    if a.cmd == "prompt":
        ops = select_ops(a.op)
        if a.out_dir:
            os.makedirs(a.out_dir, exist_ok=True)
        for op in ops:
            text = build_prompt(op, a.hardware, a.nproc, precision=a.precision, templates=a.prompts)
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
    if a.cmd == "generate":
        rc = 0
        if bool(a.command) == bool(a.endpoint) or (a.endpoint and not a.model):
            ap.error("generate needs exactly one of --command or --endpoint (the latter with --model)")
        for op in select_ops(a.op):
            log_dir = os.path.join(a.workdir, f"{op}_exchanges")
            proposer = (CommandProposer(a.command, log_dir=log_dir) if a.command else
                        HttpProposer(a.endpoint, a.model, api_key_env=a.api_key_env, max_tokens=a.max_tokens, log_dir=log_dir))
            out = optimise(op, proposer, a.workdir,
                           nproc=a.nproc, max_iters=a.max_iters, backend=a.backend, dtype=a.dtype, config=a.config,
                           resume=a.resume, measure_perf=a.measure_perf, templates=a.prompts, hardware=a.hardware)
            print(json.dumps(out, indent=1))
            rc = rc or (0 if out["solved"] else 1)
        return rc
    out = optimise(a.op, ReplayProposer(a.candidates), a.workdir, nproc=a.nproc, backend=a.backend, dtype=a.dtype, config=a.config)
    print(json.dumps(out, indent=1))
    return 0 if out["solved"] else 1


if __name__ == "__main__":
    sys.exit(main())
