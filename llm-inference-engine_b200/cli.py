"""Command line of the package (bin/trace_run, bin/b200_generate).

trace:     replay a schedule of token steps through a model's engine and write the logits that the schedule asks for.
           Steps arrive on standard input, one JSON object a line:
               {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
           All entries of a step are one batch.  A request is admitted at its first entry and gives its pages and state slot back when a
           step lists it under "end".  For a step that wants something, OUT/<step>.f32 receives the logits [wanted, vocab] as little-endian
           fp32, in the order of the entries and of their "want"; after every step a line "done <step>" is printed.
generate:  continue prompts (lists of token ids) through the scheduler."""
import argparse
import importlib
import json
import os
import sys

import numpy as np


def _pkg(sub=None):
    base = __package__ or "llm-inference-engine_b200"
    return importlib.import_module(base + ("." + sub if sub else ""))


def _load(args, max_tokens, max_seqs):
    import torch

    if not torch.cuda.is_available():
        sys.exit("no CUDA device: this package has no CPU path")
    return _pkg("models").load_model(args.model, dtype=args.dtype, device="cuda:0", max_tokens=max_tokens, max_seqs=max_seqs)


def cmd_trace(args):
    import torch

    page = _pkg().KV_PAGE_SIZE
    pool = (args.max_tokens + page - 1) // page * page
    model = _load(args, pool, args.max_seqs)
    session = _pkg("serving").Session(model, pool, max_seqs=args.max_seqs)
    os.makedirs(args.out, exist_ok=True)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = []
        for e in step.get("entries", []):
            if not e["tokens"]:
                continue
            if e["id"] not in live:
                live[e["id"]] = session.open()
            entries.append((live[e["id"]], e["tokens"], e.get("want", [])))
        if entries:
            logits = session.feed(entries)
            if logits.shape[0]:
                logits.cpu().numpy().astype("<f4").tofile(os.path.join(args.out, f"{step['step']}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in step.get("end", []):
            if rid in live:
                session.close(live.pop(rid))
        print(f"done {step['step']}", flush=True)
    return 0


def cmd_generate(args):
    prompts = [[int(t) for t in p.split(",")] for p in args.prompt]
    longest = max(len(p) for p in prompts) + args.max_new_tokens
    page = _pkg().KV_PAGE_SIZE
    per_seq = (longest + page - 1) // page * page
    model = _load(args, max(per_seq, args.batch_tokens), args.max_seqs)
    session = _pkg("serving").Session(model, per_seq * min(len(prompts), args.max_seqs), max_seqs=args.max_seqs, max_batch_tokens=max(per_seq, args.batch_tokens))
    for p, out in zip(prompts, session.generate(prompts, args.max_new_tokens, top_k=args.top_k, end_id=args.end_id, chunk=args.chunk)):
        print(json.dumps({"prompt": p, "generated": out}))
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser(prog="b200llm", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("trace", "generate"):
        p = sub.add_parser(name)
        p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
        p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
        p.add_argument("--max-seqs", type=int, default=4, help="sequences alive at any time (state slots)")
    t = sub.choices["trace"]
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True, help="positions the page pool holds (rounded up to whole pages)")
    g = sub.choices["generate"]
    g.add_argument("--prompt", action="append", required=True, help="comma-separated token ids; repeat for several requests")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--top-k", type=int, default=1)
    g.add_argument("--end-id", type=int, default=-1)
    g.add_argument("--chunk", type=int, default=0, help="most prompt tokens a sequence brings to one iteration (0: no limit)")
    g.add_argument("--batch-tokens", type=int, default=2048, help="token budget of one iteration")
    args = ap.parse_args(argv)
    return {"trace": cmd_trace, "generate": cmd_generate}[args.cmd](args)


if __name__ == "__main__":
    sys.exit(main())
