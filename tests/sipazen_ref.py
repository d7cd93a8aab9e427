"""A plain, slow restatement of the Sipazen design in float64 torch, one function per mechanism, for the tests.  It shares no code with
the library: weights come in as a dict name -> torch tensor, the configuration as the parsed config.json dict, and every sequence is run
whole (no cache, no state carried between calls), token by token where the design has a recurrence.

Notation: W is stored [out, in] and applied as x @ W.T; T tokens of one sequence at positions 0 .. T-1.
"""
import math

import torch

F = torch.float64


def rms_groups(x, w, groups, eps):
    """x [T, D] split into `groups` equal consecutive parts; each part divided by sqrt(mean(part^2) + eps); then times w."""
    T, D = x.shape
    p = x.reshape(T, groups, D // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(T, D) * w


def silu(z):
    return z * torch.sigmoid(z)


def mamba2(W, pre, mx, h, eps):
    """Selective state-space mixer.  h [T, width].  Returns [T, width]."""
    H, P, N, G, K = mx["heads"], mx["vdim"], mx["state"], mx["groups"], mx["conv"]
    inner = H * P
    T = h.shape[0]
    u = h @ W[pre + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    cw, cb = W[pre + "conv"], W[pre + "conv.b"]
    C = xbc.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=F), xbc], 0)
    conv = torch.zeros(T, C, dtype=F)
    for j in range(K):  # tap K-1 multiplies the current token
        conv += padded[j:j + T] * cw[:, j]
    xbc = silu(conv + cb)
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + W[pre + "dt_bias"], threshold=1e9)
    a = torch.exp(-torch.exp(W[pre + "A_log"]) * dt)  # [T, H]
    S = torch.zeros(H, N, P, dtype=F)
    y = torch.zeros(T, H, P, dtype=F)
    hpg = H // G
    for t in range(T):
        for hd in range(H):
            g = hd // hpg
            S[hd] = a[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ Cm[t, g] + W[pre + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    y = rms_groups(y, W[pre + "norm"], mx["norm_groups"], eps)
    return y @ W[pre + "o"].T


def rotate_half(v, pos, dims, base):
    """v [T, ..., R]; the first `dims` entries are rotated: entry i pairs with i + dims/2, angle pos * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * torch.arange(half, dtype=F) / dims)
    ang = pos.to(F)[:, None] * f[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def latent_attention(W, pre, mx, h, eps):
    """Attention over a compressed key/value latent with one shared rotated key part, a sink in the softmax and an output gate."""
    H, dn, dr, dv, r = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    T = h.shape[0]
    pos = torch.arange(T)
    q = (h @ W[pre + "q"].T).reshape(T, H, dn + dr)
    qn, qr = q[..., :dn], rotate_half(q[..., dn:], pos, mx["rot"]["dims"], mx["rot"]["base"])
    ckr = h @ W[pre + "dkv"].T
    c = rms_groups(ckr[:, :r], W[pre + "dkv.norm"], 1, eps)
    kr = rotate_half(ckr[:, r:], pos, mx["rot"]["dims"], mx["rot"]["base"])  # [T, dr]
    kn = (c @ W[pre + "uk"].T).reshape(T, H, dn)
    v = (c @ W[pre + "uv"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * mx["scale"]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        mxs = torch.maximum(s.max(-1).values, W[pre + "sink"][hd])
        e = torch.exp(s - mxs[:, None])
        den = e.sum(-1) + torch.exp(W[pre + "sink"][hd] - mxs)
        out[:, hd] = (e / den[:, None]) @ v[:, hd]
    out = out.reshape(T, H * dv) * torch.sigmoid(h @ W[pre + "g"].T)
    return out @ W[pre + "o"].T


def expert(W, pre, h):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def moe(W, pre, ml, h):
    """Routed experts (softmax over the chosen logits only) plus an always-on shared expert with a per-token sigmoid gate."""
    E, top = ml["router"]["experts"], ml["router"]["top"]
    logits = h @ W[pre + "router"].T + W[pre + "router.b"]
    val, idx = torch.topk(logits, top, dim=-1)
    wgt = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += wgt[t, j] * expert(W, "%se%d." % (pre, int(idx[t, j])), h[t:t + 1])[0]
    if ml.get("shared"):
        out = out + torch.sigmoid(h @ W[pre + "shared.sg"].T) * expert(W, pre + "shared.", h)
    return out


MIXERS = {"mamba2": mamba2, "latent_attention": latent_attention}


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  layers_out (a list) receives the residual stream after every layer."""
    W = {k: v.to(F) for k, v in W.items()}
    eps, ng, m = cfg["norm"]["eps"], cfg["norm"]["groups"], cfg["residual_mult"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, ly in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = rms_groups(x, W[p + "norm1"], ng, eps)
        y = MIXERS[ly["type"]](W, p + "mix.", ly["mixer"], h, eps)
        y = y * torch.sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        x = x + m * rms_groups(y, W[p + "norm1b"], ng, eps)
        if ly.get("mlp"):
            h = rms_groups(x, W[p + "norm2"], ng, eps)
            y = moe(W, p + "mlp.", ly["mlp"], h)
            y = y * torch.sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
            x = x + m * rms_groups(y, W[p + "norm2b"], ng, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_groups(x, W["final.norm"], ng, eps) @ W["head"].T
