"""A plain float64 statement of the Solopel decoder: whole sequences, no cache, one function per mechanism, no code
of the engine.  ``cfg`` is the dict of config.json, ``w`` maps tensor names to tensors."""
import math

import torch

F64 = torch.float64


def t64(w):
    return {k: v.to(F64) for k, v in w.items()}


def unit(y, eps):
    """y divided by its root mean square over the last dimension, eps inside the root."""
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x, scale, eps):
    """RMS norm whose scale is stored around zero."""
    return unit(x, eps) * (1.0 + scale)


def causal_conv(u, taps_w):
    """y[t] = sum_j taps_w[:, j] * u[t - taps + 1 + j] per channel, zeros before the sequence; u [T, C], taps_w [C, taps]."""
    n = taps_w.shape[1]
    padded = torch.cat([torch.zeros(n - 1, u.shape[1], dtype=u.dtype), u], dim=0)
    return sum(taps_w[:, j] * padded[j:j + u.shape[0]] for j in range(n))


def causal_softmax(scores):
    """scores [..., T, T] (query, key): softmax over the keys at or before the query."""
    T = scores.shape[-1]
    hidden = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)
    return torch.softmax(scores.masked_fill(hidden, -math.inf), dim=-1)


def latent_weights(w, p, m, h, eps):
    """(softmax weights [H, T, T], values [T, H, dv]) of latent attention."""
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    c = unit(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    return causal_softmax(torch.einsum("ihd,jhd->hij", q, k) * m["scale"]), v


def latent_attention(w, p, m, h, eps):
    """Keys and values of every head come from one low-rank row per token; no positions."""
    a, v = latent_weights(w, p, m, h, eps)
    return torch.einsum("hij,jhe->ihe", a, v).reshape(h.shape[0], -1) @ w[p + "o"].T


def diff_lambda(w, p, diff):
    return torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + diff


def diff_weights(w, p, m, h):
    """(softmax weights [2, H, T, T], values [T, H, dv]) of the two maps of differential attention."""
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for name in ("q", "k", "v"):
        y = h @ w[p + name].T
        proj[name] = causal_conv(y, w[p + name + ".conv"]) if m.get("conv") else y
    q = proj["q"].view(T, H, 2, d)
    k = proj["k"].view(T, G, 2, d).repeat_interleave(H // G, dim=1)
    v = proj["v"].view(T, G, dv).repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihmd,jhmd->mhij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    return causal_softmax(s), v


def diff_attention(w, p, m, h, eps):
    """Two softmax maps per head over the same values; their difference, unit-normalised, gated per head."""
    T, H, dv = h.shape[0], m["heads"], m["vdim"]
    maps, v = diff_weights(w, p, m, h)
    a = torch.einsum("mhij,jhe->mihe", maps, v)
    o = a[0] - diff_lambda(w, p, m["diff"]) * a[1]
    o = unit(o, eps) * (1.0 - m["diff"])
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_ff(w, p, h):
    return gelu_tanh(h @ w[p + "up"].T) @ w[p + "down"].T


def gated_expert(w, p, x):
    g = x @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (x @ w[p + "up"].T)) @ w[p + "down"].T


def route(w, p, f, h):
    """(chosen experts [T, top], their weights [T, top]): the largest sigmoid scores, as they are."""
    scores = torch.sigmoid(h @ w[p + "router"].T)
    weights, chosen = torch.topk(scores, f["router"]["top"], dim=-1)
    return chosen, weights


def routed_ff(w, p, f, h):
    """Each chosen expert sees the token's input times its weight; a shared expert sees it as it is."""
    chosen, weights = route(w, p, f, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            out[t] += gated_expert(w, f"{p}e{e}.", (wt * h[t])[None])[0]
    if f.get("shared"):
        out = out + gated_expert(w, p + "shared.", h)
    return out


def layer(cfg, w, i, x):
    spec, p, eps = cfg["layers"][i], f"l{i}.", cfg["norm"]["eps"]
    h = offset_norm(x, w[p + "norm1"], eps)
    taps = (cfg.get("canon") or {}).get("taps") or 0
    seen = h + causal_conv(h, w[p + "canon1"]) if taps else h
    mix = latent_attention if spec["type"] == "latent_attention" else diff_attention
    x = x + torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"]) * mix(w, p + "mix.", spec["mixer"], seen, eps)
    f = spec.get("mlp")
    if f is not None:
        h = offset_norm(x, w[p + "norm2"], eps)
        y = dense_ff(w, p + "mlp.", h) if f["kind"] == "dense" else routed_ff(w, p + "mlp.", f, h)
        x = x + torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"]) * y
    return x


def order_of_runs(cfg):
    """(layer, pass or None): the pass is given at the first layer of each pass of the loop."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


def forward(cfg, w, tokens, after_runs=None):
    """float64 logits [T, vocab]; ``after_runs``: a list that takes the residual sum after every run of a layer."""
    w = t64(w)
    x0 = w["embed"][torch.tensor(list(tokens))]
    x = x0
    for i, t in order_of_runs(cfg):
        if t is not None:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(cfg, w, i, x)
        if after_runs is not None:
            after_runs.append(x)
    h = offset_norm(x, w["final.norm"], cfg["norm"]["eps"])
    return (h @ w["embed"].T) * cfg.get("logit_scale", 1.0)
