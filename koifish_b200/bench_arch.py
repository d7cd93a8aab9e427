"""Prefill and decode throughput of the Sipazen hybrid stack beside a Qwen3 stack of equal width, depth and active feed-forward width,
both bf16 with random weights (bench.py --compare-arch).  One JSON line per (model, size).

    prefill: a prompt of --prompt tokens through the model's own step function in panels, timed with CUDA events after 3 warm-up prompts
    decode : the device-resident greedy loop (one CUDA-graph replay per token) at context --prompt, after W warm-up tokens

The weights of every size exceed the 126 MB L2, so nothing is reused between steps.
"""
import json
import time

PRESETS = {
    # width, vocab, layers (m = state-space, a = latent attention), mixer sizes, experts
    "s": dict(width=1024, vocab=32768, pattern="mmamma",
              ssm=dict(heads=32, vdim=64, state=64, groups=1, norm_groups=1, conv=4),
              att=dict(heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256),
              moe=dict(experts=16, top=2, ff=512, shared=1024)),
    "m": dict(width=2048, vocab=65536, pattern="mmammama",
              ssm=dict(heads=64, vdim=64, state=128, groups=8, norm_groups=8, conv=4),
              att=dict(heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512),
              moe=dict(experts=64, top=6, ff=1408, shared=2816)),
    "l": dict(width=4096, vocab=65536, pattern="mmam",
              ssm=dict(heads=128, vdim=64, state=128, groups=8, norm_groups=8, conv=4),
              att=dict(heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512),
              moe=dict(experts=32, top=4, ff=2048, shared=4096)),
}


def sipazen_config(p):
    layers = []
    for ch in p["pattern"]:
        if ch == "m":
            mixer, typ = dict(p["ssm"]), "mamba2"
        else:
            a = p["att"]
            mixer, typ = dict(a, rot=dict(base=1e6, dims=a["rot_dim"]), scale=(a["dim"] + a["rot_dim"]) ** -0.5), "latent_attention"
        m = p["moe"]
        layers.append({"type": typ, "mixer": mixer,
                       "mlp": {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"]}, "expert": {"ff": m["ff"]}, "shared": {"ff": m["shared"]}}})
    return {"architecture": "Sipazen", "vocab": p["vocab"], "width": p["width"], "residual_mult": 0.7, "norm": {"eps": 1e-5, "groups": 4}, "layers": layers}


def run(args, ctx, stream):
    import numpy as np
    import torch
    import koifish_b200 as kf
    sizes = [s for s in args.arch_sizes.split(",") if s]
    P, panel = args.prompt, args.panel
    out = []
    for size in sizes:
        p = PRESETS[size]
        n_layer = len(p["pattern"])
        ff_active = p["moe"]["top"] * p["moe"]["ff"] + p["moe"]["shared"]
        cfgs = {
            "sipazen": {"hf_config": sipazen_config(p), "gpt": {"max_seq_len": P + args.steps + args.warmup + 64, "max_batch": 1, "max_prefill": panel},
                        "init": {"sigma": 0.02, "norm_sigma": 0.02}},
            "qwen3": kf.qwen3_config(n_layer, p["width"], (ff_active + 127) // 128 * 128, p["width"] // 128, max(1, p["width"] // 512), 128, p["vocab"], None, False,
                                     P + args.steps + args.warmup + 64, 1, 42, 1e6, max_prefill=panel),
        }
        for name, cfg in cfgs.items():
            model = kf.Model(ctx, cfg)
            model.init_random()
            toks = ((np.arange(P) * 37 + 11) % p["vocab"]).astype(np.int32)

            def prompt():
                nxt = None
                for lo in range(0, P, panel):
                    part = toks[lo:lo + panel]
                    last = lo + panel >= P
                    _, nxt = model.forward(part, np.arange(lo, lo + part.size), seq_mode=2, want_logits=False, want_next=last)
                return nxt

            for _ in range(3):
                prompt()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps, l0 = 3, ctx.launches
            e0.record(stream)
            for _ in range(reps):
                nxt = prompt()
            e1.record(stream)
            torch.cuda.synchronize()
            prefill_ms = e0.elapsed_time(e1) / reps
            prefill_launches = (ctx.launches - l0) / reps
            model.decode_loop(max(3, args.warmup), 1)
            torch.cuda.synchronize()
            l0 = ctx.launches
            e0.record(stream)
            model.decode_loop(args.steps, 1)
            e1.record(stream)
            torch.cuda.synchronize()
            decode_ms = e0.elapsed_time(e1) / args.steps
            info = model.info
            line = {"bench": "arch-compare", "model": name, "size": size, "width": p["width"], "layers": n_layer, "pattern": p["pattern"],
                    "weight_gb": round(info.weight_bytes / 1e9, 3), "prompt": P, "panel": panel,
                    "prefill_tok_s": round(P / (prefill_ms / 1e3), 1), "prefill_ms": round(prefill_ms, 3), "prefill_launches": prefill_launches,
                    "decode_tok_s": round(1e3 / decode_ms, 1), "decode_ms": round(decode_ms, 4), "decode_launches_per_token": (ctx.launches - l0) / args.steps,
                    "dtype": "bf16", "data": "synthetic", "steps": args.steps, "warmup": max(3, args.warmup), "timing": "cuda events, weights exceed L2"}
            print(json.dumps(line), flush=True)
            out.append(line)
            model.close()
            time.sleep(0.1)
    return out
