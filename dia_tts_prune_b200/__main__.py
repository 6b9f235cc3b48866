"""Command line of the framework: ``python -m dia_tts_prune_b200 <command>``.

  generate  --model DIR --prompt "1 2 3" [--prompt ...] [--max-new-tokens N] [--temperature T] ...
            continue prompts given as token ids with the model of DIR (chosen by its config.json)
  trace     --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
            replay a trace of steps from standard input and write the logits asked for (``bin/trace_run``)
  build     compile the CUDA libraries
"""

from __future__ import annotations

import argparse
import json
import os
import sys


def _cmd_build(a) -> int:
    from . import build
    for lib in build.build_all(force=a.force):
        print(lib)
    return 0


def _cmd_generate(a) -> int:
    from .registry import load_model
    model = load_model(a.model, dtype=a.dtype, max_tokens=a.max_tokens)
    if not hasattr(model, "generate") or not hasattr(model, "run_step"):
        print("generate: this command serves the language models; use the Dia API for speech", file=sys.stderr)
        return 2
    prompts = [[int(t) for t in p.replace(",", " ").split()] for p in a.prompt]
    outs = model.generate(prompts, max_new_tokens=a.max_new_tokens, temperature=a.temperature, top_p=a.top_p,
                          top_k=a.top_k, eos=a.eos, seed=a.seed)
    for o in outs:
        print(" ".join(str(t) for t in o))
    return 0


def _cmd_trace(a) -> int:
    """One JSON object per line on standard input: ``{"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}``.
    Runs the step on the state earlier steps left, writes the wanted logits (float32 little-endian, [wanted, vocab]) to
    ``<out>/<step>.f32`` and answers ``done <step>``."""
    import torch
    if a.dtype not in ("bfloat16", "float32"):
        print(f"trace: unknown dtype {a.dtype}", file=sys.stderr)
        return 2
    from .registry import load_model
    model = load_model(a.model, dtype=a.dtype, max_tokens=max(int(a.max_tokens), 1))
    if not hasattr(model, "run_step"):
        print("trace: the model of this folder has no step interface", file=sys.stderr)
        return 2
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        with torch.inference_mode():
            logits = model.run_step(step.get("entries", []), step.get("end", []))
        if logits.shape[0]:
            data = logits.to("cpu").numpy().astype("<f4", copy=False)
            tmp = os.path.join(a.out, f".{step['step']}.f32.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        else:
            torch.cuda.synchronize()
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="dia_tts_prune_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("build", help="compile the CUDA libraries in-tree")
    b.add_argument("--force", action="store_true")
    b.set_defaults(fn=_cmd_build)
    g = sub.add_parser("generate", help="continue token-id prompts with a language model")
    g.add_argument("--model", required=True)
    g.add_argument("--prompt", action="append", required=True, help="token ids separated by blanks or commas")
    g.add_argument("--dtype", default="bfloat16")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--max-tokens", type=int, default=4096, help="tokens the sequence state holds")
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=None)
    g.add_argument("--eos", type=int, default=None)
    g.add_argument("--seed", type=int, default=None)
    g.set_defaults(fn=_cmd_generate)
    t = sub.add_parser("trace", help="replay steps from standard input, write logits")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", default="bfloat16")
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, default=4096)
    t.set_defaults(fn=_cmd_trace)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
