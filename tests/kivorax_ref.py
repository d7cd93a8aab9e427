"""Plain float64 restatement of the Kivorax stack, one function per mechanism, token by token where the design is recurrent.

Notation: x_t is the residual row of token t (positions from 0), h_t its normed copy, W[name] the checkpoint tensors as float tensors.
Nothing here is shared with the library: it is the oracle of tests/test_gpu_kivorax.py and is itself checked for causality on the CPU.
"""
import math

import torch

F = torch.float64


def rms_unit(x, eps):
    """x scaled to unit root mean square over its last axis (eps inside the root)"""
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_t(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def short_conv(x, taps, bias=None):
    """per channel: out_t = sum_j taps[:, K-1-j] * x_{t-j}, inputs before the sequence are zero.  x [T, C], taps [C, K]"""
    T, C = x.shape
    K = taps.shape[1]
    out = torch.zeros(T, C, dtype=F)
    for t in range(T):
        for j in range(K):
            if t - j >= 0:
                out[t] += taps[:, K - 1 - j] * x[t - j]
    return out if bias is None else out + bias


def delta_rule(q, k, v, g, beta):
    """one head: S <- diag(g_t) S; u = beta_t (v_t - S^T k_t); S <- S + k_t u^T; o_t = S^T q_t.  q, k, g [T, dk]; v [T, dv]; beta [T]"""
    T, dk = q.shape
    S = torch.zeros(dk, v.shape[1], dtype=F)
    out = []
    for t in range(T):
        S = g[t].unsqueeze(1) * S
        u = beta[t] * (v[t] - k[t] @ S)
        S = S + k[t].unsqueeze(1) * u.unsqueeze(0)
        out.append(q[t] @ S)
    return torch.stack(out)


def decayed_outer_sum(q, k, v, a):
    """one head of gated linear attention: S <- diag(a_t) S + k_t v_t^T; o_t = S^T q_t"""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=F)
    out = []
    for t in range(q.shape[0]):
        S = a[t].unsqueeze(1) * S + k[t].unsqueeze(1) * v[t].unsqueeze(0)
        out.append(q[t] @ S)
    return torch.stack(out)


def mixer_channel_delta(W, p, m, h, eps):
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(dk)
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    step = torch.nn.functional.softplus((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).reshape(T, H, dk)
    g = torch.exp(-torch.exp(W[p + "A_log"]).reshape(1, H, 1) * step)
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, dv)
    heads = []
    for i in range(H):
        o = delta_rule(q[:, i // (H // G)], k[:, i // (H // G)], v[:, i], g[:, i], beta[:, i])
        heads.append(rms_unit(o, eps) * W[p + "norm"] * gate[:, i])
    return torch.cat(heads, -1) @ W[p + "o"].T


def mixer_gla(W, p, m, h, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, dk) / math.sqrt(dk)
    k = (h @ W[p + "k"].T).reshape(T, H, dk)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    a = torch.sigmoid((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]).pow(1.0 / m["tau"]).reshape(T, H, dk)
    heads = [rms_unit(decayed_outer_sum(q[:, i], k[:, i], v[:, i], a[:, i]), eps) * W[p + "norm"] for i in range(H)]
    return (torch.cat(heads, -1) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def attention_log_distance(W, p, m, h):
    """softmax attention, causal; score = t_i (q_i . k_j) scale - r1 ln(1 + r2 (i - j)), t_i = 1 + coef ln(floor((i + 1) / every) + 1)"""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, dk)
    k = (h @ W[p + "k"].T).reshape(T, G, dk)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    qt = m.get("q_temp")
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(T):
        temp = 1.0 + qt["coef"] * math.log((i + 1) // qt["every"] + 1) if qt else 1.0
        dist = torch.arange(i, -1, -1, dtype=F)  # i - j for j = 0 .. i
        for a in range(H):
            kv = a // (H // G)
            s = (k[: i + 1, kv] @ (q[i, a] * temp)) * m["scale"] - W[p + "r1"][a] * torch.log(1.0 + W[p + "r2"][a] * dist)
            out[i, a] = torch.softmax(s, 0) @ v[: i + 1, kv]
    return (out.reshape(T, H * dv) * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def gated_lru(W, p, m, h):
    """y = gelu(W_y h + b); u = conv(W_x h + b); per block r, i = sigmoid(block matrix u_b + b); a = exp(-8 r softplus(lam));
    s <- a s + sqrt(1 - a^2) i u; out = W_o (s * y)"""
    T = h.shape[0]
    Wd, B = m["width"], m["blocks"]
    y = gelu_t(h @ W[p + "y"].T + W[p + "y.b"])
    u = short_conv(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    ub = u.reshape(T, B, Wd // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ra"].reshape(B, Wd // B, Wd // B), ub) + W[p + "ra.b"].reshape(B, -1)).reshape(T, Wd)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ri"].reshape(B, Wd // B, Wd // B), ub) + W[p + "ri.b"].reshape(B, -1)).reshape(T, Wd)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(W[p + "lam"]))
    s = torch.zeros(Wd, dtype=F)
    rows = []
    for t in range(T):
        s = a[t] * s + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        rows.append(s * y[t])
    return torch.stack(rows) @ W[p + "o"].T


def mixer_parallel(W, p, m, h, eps):
    left = attention_log_distance(W, p + "left.", m["left"], h)
    right = gated_lru(W, p + "right.", m["right"], h)
    return 0.5 * (rms_unit(left, eps) * W[p + "left.out"] + rms_unit(right, eps) * W[p + "right.out"])


def feed_forward(W, p, f, h):
    if f["kind"] == "dense":
        return gelu_t(h @ W[p + "up"].T + W[p + "up.b"]) @ W[p + "down"].T + W[p + "down.b"]
    score = torch.softmax(h @ W[p + "router"].T, -1)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e in torch.argsort(score[t], descending=True, stable=True)[: f["router"]["top"]].tolist():
            out[t] += score[t, e] * (torch.relu(W["%se%d.up" % (p, e)] @ h[t]) ** 2 @ W["%se%d.down" % (p, e)].T)
    return out


def forward(cfg, W32, tokens, layers_out=None):
    """logits [T, vocab] (float64) of a whole sequence"""
    W = {k: v.to(F) for k, v in W32.items()}
    eps = cfg["norm"]["eps"]
    tok = torch.tensor(list(tokens), dtype=torch.long)
    x = W["embed"][tok] * cfg.get("embedding", {}).get("scale", 1.0)
    side = (cfg.get("token_side") or {}).get("dim", 0)
    history = [x]
    for n, layer in enumerate(cfg["layers"]):
        p = "l%d." % n
        h = rms_unit(x, eps) * W[p + "norm1"]
        mix = {"channel_delta": mixer_channel_delta, "gla": mixer_gla, "parallel": mixer_parallel}[layer["type"]](W, p + "mix.", layer["mixer"], h, eps)
        x = x + (mix + (feed_forward(W, p + "mlp.", layer["mlp"], h) if layer.get("mlp") else 0.0))
        if side:
            e = W["side.embed"][tok][:, n * side:(n + 1) * side]
            y = (gelu_t(x @ W[p + "side.gate"].T) * e) @ W[p + "side.proj"].T
            x = x + rms_unit(y, eps) * W[p + "side.norm"]
        history.append(x)
        x = sum(W[p + "dwa"][j] * history[j] for j in range(n + 2))
        if layers_out is not None:
            layers_out.append(x)
    return (rms_unit(x, eps) * W["final.norm"]) @ W["head"].T
