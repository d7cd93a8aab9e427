"""Command line of the package.

    python -m koifish_b200.cli generate --model DIR --ids 5,17,3 --max-new-tokens 16 [--temperature T --top-k K --top-p P --seed S]
    python -m koifish_b200.cli trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N      (bin/trace_run)

`--model` is a checkpoint folder (config.json + *.safetensors); config.json selects the architecture through the model registry.
`generate` runs the prompt through the model's own generation loop and prints the new token ids.  `trace` replays a trace: it reads one
JSON object per line from standard input, {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}, feeds each entry's tokens to
the sequence slot of its request (the slot is acquired at the request's first step and released when the request ends), writes the
logits at the wanted places to <out>/<step>.f32 (float32, little-endian, [wanted, vocab]) and answers every step with "done <step>".
"""
import argparse
import json
import os
import sys

import numpy as np


def _open_model(args, max_seq_len, max_batch=1, gpt=None):
    from . import build as kb
    kb.build()  # in a fresh checkout the library is compiled here, once
    import koifish_b200 as kf
    ctx = kf.Context(0)
    model, tok = kf.from_pretrained(ctx, args.model, max_seq_len=max_seq_len, max_batch=max_batch, gpt=gpt)
    return ctx, model, tok


def cmd_generate(args):
    ids = [int(t) for t in args.ids.split(",") if t.strip()]
    ctx, model, _ = _open_model(args, max_seq_len=max(64, len(ids) + args.max_new_tokens + 1), gpt={"max_prefill": args.panel})
    if args.temperature > 0:
        model.set_sampler(args.temperature, args.top_k, args.top_p, args.seed)
    out, why = model.generate(ids, args.max_new_tokens, eos_id=args.eos_id)
    print(json.dumps({"tokens": out, "stop_reason": why}))
    return 0


def cmd_trace(args):
    import koifish_b200 as kf
    if args.dtype not in ("bfloat16", "float32"):
        print("unknown --dtype", file=sys.stderr)
        return 2
    panel = max(64, min(args.panel, args.max_tokens))
    gpt = {"max_prefill": panel, "logit_rows": panel}
    if args.dtype == "float32":
        gpt["compute_dtype"] = "float32"
    try:
        ctx, model, _ = _open_model(args, max_seq_len=max(64, args.max_tokens), max_batch=args.slots, gpt=gpt)
    except kf.KoifishError as e:
        if args.dtype == "float32" and "bf16 only" in str(e):
            print(str(e), file=sys.stderr)
            return 3  # this architecture has no 32-bit path
        raise
    os.makedirs(args.out, exist_ok=True)
    live = {}  # request id -> [slot, tokens so far]
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        rows = []
        for ent in step.get("entries", []):
            rid = ent["id"]
            if rid not in live:
                live[rid] = [model.acquire_slot(), 0]
            slot, done = live[rid]
            toks = list(ent["tokens"])
            want = sorted(set(int(w) for w in ent.get("want", [])))
            got = {}
            for lo in range(0, len(toks), panel):  # a step longer than the activation buffers goes through in panels
                part = toks[lo:lo + panel]
                sel = [w - lo for w in want if lo <= w < lo + len(part)]
                lg, _ = model.forward_rows(part, done + lo, slot=slot, rows=sel)
                for k, w in enumerate(sel):
                    got[w + lo] = lg[k]
            live[rid][1] = done + len(toks)
            rows += [got[int(w)] for w in ent.get("want", [])]
        if rows:
            np.stack(rows).astype("<f4").tofile(os.path.join(args.out, "%d.f32" % step["step"]))
        for rid in step.get("end", []):
            if rid in live:
                model.release_slot(live.pop(rid)[0])
        sys.stdout.write("done %d\n" % step["step"])
        sys.stdout.flush()
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser(prog="koifish_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate token ids from a prompt of token ids")
    g.add_argument("--model", required=True)
    g.add_argument("--ids", required=True, help="prompt token ids, comma separated")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--eos-id", type=int, default=-1)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=50)
    g.add_argument("--top-p", type=float, default=0.95)
    g.add_argument("--seed", type=int, default=42)
    g.add_argument("--panel", type=int, default=256, help="tokens per prefill panel")
    g.set_defaults(fn=cmd_generate)
    t = sub.add_parser("trace", help="replay a trace of steps from standard input and write logits")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", default="bfloat16")
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, default=4096)
    t.add_argument("--panel", type=int, default=512, help="tokens per forward panel")
    t.add_argument("--slots", type=int, default=4, help="sequence slots of the cache / state manager")
    t.set_defaults(fn=cmd_trace)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
