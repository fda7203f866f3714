"""Command line of the framework.

    python -m llm_decoder.cli generate --model DIR --prompt 5,17,3 [--prompt ...] --max-new-tokens 16
                                       [--dtype bfloat16|float32] [--temperature T --top-k K --top-p P --seed S]
    python -m llm_decoder.cli trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   (bin/trace_run)

`trace` replays a schedule from standard input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Every entry brings the next tokens of a request; all entries of a step run as ONE batch through Engine.step (the step
function generation uses).  The logits at the wanted places go to <out>/<step>.f32 (little-endian float32,
[wanted, vocab]); requests named in "end" give back their pages and state slot; after every step `done <step>` is
printed.  The cache pool holds --max-tokens tokens and four state slots."""
import argparse
import json
import os
import sys


def _ensure_library():
    """A fresh checkout has no built library: compile the core subset now (in-tree, once)."""
    import importlib.util
    pkg = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("pa_b200_build", os.path.join(pkg, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ensure_core()


def trace_main(argv=None):
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--max-seqs", type=int, default=4)
    a = ap.parse_args(argv)
    _ensure_library()
    import numpy as np
    import torch

    from .engine import Engine
    from .registry import load_model
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    model = load_model(a.model, a.dtype, max_tokens=a.max_tokens, max_seqs=a.max_seqs)
    if not hasattr(model, "states"):
        print("this architecture has no ragged-batch step function", file=sys.stderr)
        return 4
    engine = Engine(model)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in step["entries"]]
        logits = engine.step(entries)
        if logits.shape[0]:
            path = os.path.join(a.out, f"{step['step']}.f32")
            logits.cpu().numpy().astype("<f4").tofile(path + ".part")
            os.replace(path + ".part", path)
        else:
            torch.cuda.synchronize()
        for rid in step.get("end", []):
            engine.finish(rid)
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


def generate_main(argv=None):
    ap = argparse.ArgumentParser(prog="generate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; may repeat")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--max-tokens", type=int, default=8192)
    ap.add_argument("--max-seqs", type=int, default=4)
    ap.add_argument("--max-batch-tokens", type=int, default=2048)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    _ensure_library()
    from .registry import load_model
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt]
    model = load_model(a.model, a.dtype, max_tokens=a.max_tokens, max_seqs=a.max_seqs)
    if hasattr(model, "states"):
        from .engine import generate
        outs = generate(model, prompts, a.max_new_tokens, max_batch_tokens=a.max_batch_tokens,
                        temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed)
    else:   # the fixed decoders: their own generate (equal-length prompts per call)
        outs = [model.generate(p, a.max_new_tokens, a.temperature) for p in prompts]
    for o in outs:
        print(",".join(str(t) for t in o))
    return 0


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in ("generate", "trace"):
        print(__doc__)
        return 2
    return (trace_main if argv[0] == "trace" else generate_main)(argv[1:])


if __name__ == "__main__":
    sys.exit(main())
