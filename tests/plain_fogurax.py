"""A plain, slow statement of the Fogurax design: whole sequences, no cache, float64, one function per mechanism.
It shares no code with the engine: it takes a plain configuration dict and a dict of tensors by name.

Notation.  D width, T tokens of one sequence at positions 0..T-1.  A linear weight W is stored [out, in] and applied
as x @ W^T.  rms(y) = sqrt(mean(y^2) + eps).

* layer:         h = x / rms(x) * w1;  x += m (mixer(h) + ff(h))  (one norm, both branches read it; m = residual_mult);
                 then, with e the layer's slice of the token's row of the side table:
                 y = Wp (gelu(Wg x) * e);  x += m y / rms(y) * ws
* attention:     q, k, v = Wq h + bq, ...; each channel of q, k, v then passes a causal convolution over ``conv`` tokens;
                 the first ``dims`` elements of every head of q and k turn in pairs (2i, 2i+1), at rates stretched
                 band by band (``llama3_rates``); then q and k are divided by their rms per head; causal softmax of
                 (q . k) scale; the head's output times sigmoid(Wg h)_head; Wo.
* attention_2:   q, k <- q / rms(q) * wq over the WHOLE projection (all heads at once), k alike; pairs (i, i + dims/2)
                 turn at rates blended by a ramp (``yarn_rates``), cos and sin times a magnitude; softmax over the keys
                 j <= i of the same block of ``mask.size`` positions; no gate.
* parallel:      left_scale * left(h) + right_scale * right(h).  left: the whole-projection norms, pairs (2i, 2i+1),
                 plain rates, softmax over the last ``mask.size`` keys, the per-head gate.  right: a recurrence with a
                 matrix state per head (``time_mix``).
* feed-forward:  dense Wd (silu(Wg h) * (Wu h)); or routed: s = sigmoid(Wr h), the ``top`` largest chosen,
                 out = sum over the chosen of expert_e(s_e h), plus shared(h).
* output:        logits = E (x / rms(x) * wf), E the embedding table.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


def rms_div(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def plain_rates(rot: dict) -> torch.Tensor:
    dims = int(rot["dims"])
    return float(rot["base"]) ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)


def llama3_rates(rot: dict) -> torch.Tensor:
    """Rates stretched band by band: short wavelengths stay, long ones are divided by ``factor``, between them a
    linear blend in original / wavelength."""
    f = plain_rates(rot)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for i in range(f.numel()):
        wl = 2.0 * math.pi / float(f[i])
        if wl < orig / high:
            continue
        if wl > orig / low:
            out[i] = f[i] / factor
        else:
            s = (orig / wl - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def yarn_rates(rot: dict):
    """(rates, magnitude): rates blended by a ramp over the pair index; cos and sin are multiplied by the magnitude."""
    f = plain_rates(rot)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    dims, base = int(rot["dims"]), float(rot["base"])
    factor, orig = float(sc["factor"]), float(sc["original"])

    def c(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(c(float(sc["fast"]))), 0)
    hi = min(math.ceil(c(float(sc["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=F64)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def turn(x: torch.Tensor, positions: torch.Tensor, rates: torch.Tensor, dims: int, layout: str,
         magnitude: float = 1.0) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` elements turn in pairs, (2i, 2i+1) for 'interleaved', (i, i + dims/2) for
    'half', by the angle position * rates[i]."""
    ang = positions.to(F64)[:, None] * rates[None, :]
    cos, sin = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    out = x.clone()
    if layout == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * cos - b * sin
        out[..., 1:dims:2] = b * cos + a * sin
    else:
        a, b = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = a * cos - b * sin
        out[..., dims // 2:dims] = b * cos + a * sin
    return out


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    pad = torch.cat([torch.zeros((taps - 1, u.shape[1]), dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j][None, :]
    return y


def visible(T: int, kind: str, size: int = 0) -> torch.Tensor:
    """[T, T] True where query i sees key j."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    m = j <= i
    if kind == "window":
        m = m & (i - j < size)
    elif kind == "chunk":
        m = m & (i // size == j // size)
    return m


def softmax_attention(q, k, v, scale: float, mask: torch.Tensor) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, vd] -> [T, H, vd]; head h reads key/value head h // (H / G)."""
    H, G = q.shape[1], k.shape[1]
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return torch.stack(out, dim=1)


def attention(h, m: dict, w: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w[p + n].T + w[p + n + ".b"] for n in ("q", "k", "v"))
    if m.get("conv"):
        q, k, v = (causal_conv(t, w[p + n + ".conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, vd)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        rates = llama3_rates(rot)
        q, k = (turn(t, pos, rates, int(rot["dims"]), "interleaved") for t in (q, k))
    q, k = rms_div(q, eps), rms_div(k, eps)
    o = softmax_attention(q, k, v, float(m["scale"]), visible(T, "causal"))
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * vd) @ w[p + "o"].T


def whole_norm(y: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm over a whole projection [T, heads * d], before it is split into heads."""
    return rms_div(y, eps) * weight


def attention_2(h, m: dict, w, p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = whole_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(T, H, d)
    k = whole_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, vd)
    rot = m.get("rot")
    if rot:
        rates, mag = yarn_rates(rot)
        q, k = (turn(t, torch.arange(T), rates, int(rot["dims"]), "half", mag) for t in (q, k))
    o = softmax_attention(q, k, v, float(m["scale"]), visible(T, "chunk", int(m["mask"]["size"])))
    return o.reshape(T, H * vd) @ w[p + "o"].T


def left_attention(h, m: dict, w, p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = whole_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(T, H, d)
    k = whole_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(T, G, d)
    v = (h @ w[p + "v"].T).reshape(T, G, vd)
    rot = m.get("rot")
    if rot:
        q, k = (turn(t, torch.arange(T), plain_rates(rot), int(rot["dims"]), "interleaved") for t in (q, k))
    o = softmax_attention(q, k, v, float(m["scale"]), visible(T, "window", int(m["mask"]["size"])))
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * vd) @ w[p + "o"].T


def time_mix(h, m: dict, w, p: str, eps: float) -> torch.Tensor:
    """A recurrence with a matrix state S [d, d] per head.  Each of r, k, v, g, w reads h blended with the token
    before, h + (h' - h) mu.  decay = exp(-exp(W2 tanh(W1 x_w) + w0));  o_t = (S + diag(u) k_t v_t^T)^T r_t;
    S <- diag(decay_t) S + k_t v_t^T;  out = Wo (o / rms(o) per head * norm * silu(Wg x_g))."""
    T, D = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros((1, D), dtype=h.dtype), h[:-1]], dim=0)
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in ("r", "k", "v", "g", "w")}
    r = (mix["r"] @ w[p + "r"].T).reshape(T, H, d)
    k = (mix["k"] @ w[p + "k"].T).reshape(T, H, d)
    v = (mix["v"] @ w[p + "v"].T).reshape(T, H, d)
    gate = silu(mix["g"] @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).reshape(T, H, d)
    u = w[p + "u"]
    S = torch.zeros((H, d, d), dtype=h.dtype)
    out = torch.zeros((T, H, d), dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    o = rms_div(out, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


def parallel_mixer(h, m: dict, w, p: str, eps: float) -> torch.Tensor:
    return float(m["left_scale"]) * left_attention(h, m["left"], w, p + "left.", eps) + \
        float(m["right_scale"]) * time_mix(h, m["right"], w, p + "right.", eps)


def gated_ff(h, w, p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(h, f: dict, w, p: str, chosen_out: Optional[list] = None, margins_out: Optional[list] = None) -> torch.Tensor:
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    pick = torch.topk(s, top, dim=-1).indices
    if chosen_out is not None:
        chosen_out.append(pick)
    if margins_out is not None and top < E:       # how far the last chosen score lies above the first one left out
        best = torch.topk(s, top + 1, dim=-1).values
        margins_out.append(best[:, top - 1] - best[:, top])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in pick[t].tolist():
            out[t] += gated_ff((s[t, e] * h[t])[None, :], w, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + gated_ff(h, w, p + "shared.")
    return out


MIXERS = {"attention": attention, "attention_2": attention_2, "parallel": parallel_mixer}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None,
            chosen_out: Optional[list] = None, margins_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence."""
    w = {k: v.to(F64) for k, v in weights.items() if v.is_floating_point()}
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    side = (cfg.get("token_side") or {}).get("dim", 0)
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["embed"][tok]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_div(x, eps) * w[p + "norm1"]
        a = MIXERS[layer["type"]](h, layer["mixer"], w, p + "mix.", eps)
        f = layer.get("mlp")
        if f is not None:
            a = a + (gated_ff(h, w, p + "mlp.") if f["kind"] == "dense" else routed_ff(h, f, w, p + "mlp.", chosen_out, margins_out))
        x = x + m * a
        if side:
            e = w["side.embed"][tok][:, i * side:(i + 1) * side]
            y = (gelu_tanh(x @ w[p + "side.gate"].T) * e) @ w[p + "side.proj"].T
            x = x + m * rms_div(y, eps) * w[p + "side.norm"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms_div(x, eps) * w["final.norm"]) @ w["embed"].T
