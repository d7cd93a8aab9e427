"""Small random Kivorax models for the tests: layer cards, a config.json, weights drawn on the bf16 grid (optionally shaped so that a fault
shows), bf16 bit patterns, random token lists."""
import numpy as np
import torch


# ------------------------------------------------------------------------------------------------------------ small models
def delta(heads=4, kv_heads=2, dim=12, vdim=10, conv=3, a_rank=6, g_rank=5):
    return {"type": "channel_delta", "mixer": dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, a_rank=a_rank, g_rank=g_rank)}


def gla(heads=3, dim=10, vdim=14, tau=8.0, a_rank=4):
    return {"type": "gla", "mixer": dict(heads=heads, dim=dim, vdim=vdim, tau=tau, a_rank=a_rank)}


def pair(heads=4, kv_heads=2, dim=12, vdim=20, coef=0.4, every=16, scale=None, width=24, blocks=3, conv=4):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale or dim ** -0.5)
    if every:
        left["q_temp"] = dict(coef=coef, every=every)
    return {"type": "parallel", "mixer": dict(left=left, right=dict(width=width, blocks=blocks, conv=conv))}


def moe(experts=5, top=2, ff=24):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def config(layers, width=48, vocab=96, eps=1e-5, scale=3.0, side=6):
    out = []
    for mixer, mlp in layers:
        d = dict(mixer)
        d["mlp"] = mlp
        out.append(d)
    cfg = {"architecture": "Kivorax", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps}, "layers": out}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def bf16_grid(t):
    return t.to(torch.bfloat16).to(torch.float32)


def weights(cfg, seed=0, q_gain=1.0, r1=0.5, a_log=-1.0, lam=0.0, dt_bias=0.0, side_gain=1.0, gla_bias=1.0):
    g = torch.Generator().manual_seed(seed)
    E, V, L = cfg["width"], cfg["vocab"], len(cfg["layers"])
    sd = (cfg.get("token_side") or {}).get("dim", 0)
    W = {}

    def mat(name, r, c, s=None):
        W[name] = bf16_grid(torch.randn(r, c, generator=g) * (s if s is not None else c ** -0.5))

    def vec(name, n, mean=0.0, s=0.3, shape=None):
        W[name] = bf16_grid(mean + s * torch.randn(n, generator=g)).reshape(shape or (n,))

    mat("embed", V, E, 1.0 / cfg["embedding"]["scale"])
    mat("head", V, E)
    vec("final.norm", E, 1.0)
    if sd:
        mat("side.embed", V, L * sd, side_gain)
    for i, ly in enumerate(cfg["layers"]):
        p, m = "l%d." % i, ly["mixer"]
        vec(p + "norm1", E, 1.0)
        W[p + "dwa"] = bf16_grid(torch.cat([0.3 * torch.randn(i + 1, generator=g) / (i + 1), torch.tensor([1.0])]))
        if sd:
            mat(p + "side.gate", sd, E, 1.0 / E ** 0.5)
            mat(p + "side.proj", E, sd)
            vec(p + "side.norm", E, 0.5)
        q = p + "mix."
        if ly["type"] == "channel_delta":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, c in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                mat(q + n, c, E)
                mat(q + n + ".conv", c, m["conv"], 0.6)
            mat(q + "b", H, E)
            vec(q + "A_log", H, a_log, 0.3)
            vec(q + "norm", dv, 1.0)
            mat(q + "a1", m["a_rank"], E)
            mat(q + "a2", H * dk, m["a_rank"])
            vec(q + "dt_bias", H * dk, dt_bias, 0.5)
            mat(q + "g1", m["g_rank"], E)
            mat(q + "g2", H * dv, m["g_rank"])
            mat(q + "o", E, H * dv)
        elif ly["type"] == "gla":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            mat(q + "q", H * dk, E), mat(q + "k", H * dk, E), mat(q + "v", H * dv, E), mat(q + "g", H * dv, E)
            mat(q + "o", E, H * dv)
            vec(q + "norm", dv, 1.0)
            mat(q + "a1", m["a_rank"], E)
            mat(q + "a2", H * dk, m["a_rank"])
            vec(q + "a2.b", H * dk, gla_bias, 0.5)
        else:
            a, r = m["left"], m["right"]
            H, G, dk, dv, Wd, B = a["heads"], a["kv_heads"], a["dim"], a["vdim"], r["width"], r["blocks"]
            mat(q + "left.q", H * dk, E, q_gain * E ** -0.5), mat(q + "left.k", G * dk, E), mat(q + "left.v", G * dv, E), mat(q + "left.g", H * dv, E)
            W[q + "left.r1"] = bf16_grid(r1 * (0.5 + torch.rand(H, generator=g)))
            W[q + "left.r2"] = bf16_grid(0.2 + torch.rand(H, generator=g))
            mat(q + "left.o", E, H * dv)
            vec(q + "left.out", E, 1.0), vec(q + "right.out", E, 1.0)
            mat(q + "right.y", Wd, E), vec(q + "right.y.b", Wd), mat(q + "right.x", Wd, E), vec(q + "right.x.b", Wd)
            mat(q + "right.conv", Wd, r["conv"], 0.6), vec(q + "right.conv.b", Wd)
            bs = Wd // B
            W[q + "right.ra"] = bf16_grid(torch.randn(B, bs, bs, generator=g) * bs ** -0.5)
            W[q + "right.ri"] = bf16_grid(torch.randn(B, bs, bs, generator=g) * bs ** -0.5)
            vec(q + "right.ra.b", Wd, shape=(B, bs)), vec(q + "right.ri.b", Wd, shape=(B, bs))
            vec(q + "right.lam", Wd, lam, 0.5)
            mat(q + "right.o", E, Wd)
        ml = ly["mlp"]
        if ml and ml["kind"] == "dense":
            mat(p + "mlp.up", ml["ff"], E), vec(p + "mlp.up.b", ml["ff"]), mat(p + "mlp.down", E, ml["ff"]), vec(p + "mlp.down.b", E)
        elif ml:
            mat(p + "mlp.router", ml["router"]["experts"], E, 1.0)  # wide logits: no near ties between experts
            for e in range(ml["router"]["experts"]):
                mat(p + "mlp.e%d.up" % e, ml["expert"]["ff"], E)
                mat(p + "mlp.e%d.down" % e, E, ml["expert"]["ff"])
    return W


def bits(t):
    return (t.contiguous().view(torch.int32).numpy().astype(np.uint32) >> 16).astype(np.uint16)


def tokens(n, vocab, seed):
    return np.random.RandomState(seed).randint(0, vocab, n).tolist()
