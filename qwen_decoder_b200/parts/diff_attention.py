"""Differential grouped-query attention: every head runs two softmax maps over the same values and keeps their
difference.

With h the mixer's input [T, D], H query heads over G key/value heads (query head i uses kv head i // (H / G)), a
per-map query/key size d and a value size vd:

    q = Wq h  [H, 2, d],   k = Wk h  [G, 2, d],   v = Wv h  [G, vd]         (a head's two maps side by side, no biases)
    each channel of q, k and v then passes a causal convolution over ``conv_taps`` tokens (no bias, no activation)
    s_m = (q_m . k_m) * scale,  then  cap * tanh(s_m / cap)  when ``softcap`` > 0;   p_m = causal softmax(s_m)
    a_m = p_m v                                                                  (m = 1, 2: the same values)
    lam = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                                  (one number for the layer)
    o = (a_1 - lam a_2) / sqrt(mean((a_1 - lam a_2)^2) + eps) * (1 - diff)         (over the head's vd values)
    out = Wo (o * sigmoid(Wg h)_head)                                             (one gate number per head)

No position enters the scores.  Cached per token: the convolved k (one row of 2d per kv head) and v; per request, in
its state row, the last ``conv_taps`` - 1 projected rows [q | k | v] before the convolution (float32).  q, k, v and
the gate are one stacked product with float32 sums; the convolution, scores, softmax weights, lam and the unit norm are
float32 in both engine dtypes (``csrc/attention_diff.cu``).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import kernels
from ..cache import FixedState, PagedKV
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, PagedCacheView, RunCacheView
from .linear import Linear


@register_part("mixer", "diff_attention")
class DiffAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, scale: float,
                 diff: float, eps: float, softcap: float = 0.0, conv_taps: int = 0, output_gate: bool = True,
                 window: Optional[int] = None, prefix: str = "mix.", weight_suffix: str = ""):
        if num_heads % num_kv_heads:
            raise ValueError("diff_attention: kv heads must divide heads")
        if v_dim > kernels.DIFF_MAX_VDIM:
            raise ValueError(f"diff_attention: value size {v_dim} exceeds {kernels.DIFF_MAX_VDIM}")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.v_dim = head_dim, v_dim
        self.scale, self.diff, self.eps, self.softcap = float(scale), float(diff), float(eps), float(softcap or 0.0)
        self.conv_taps, self.output_gate, self.window = int(conv_taps or 0), bool(output_gate), window
        self.prefix, self.sfx = prefix, weight_suffix
        H, G, d = num_heads, num_kv_heads, head_dim
        self.channels = H * 2 * d + G * 2 * d + G * v_dim
        pieces = [(f"{prefix}q", H * 2 * d), (f"{prefix}k", G * 2 * d), (f"{prefix}v", G * v_dim)]
        if self.output_gate:
            pieces.append((f"{prefix}g", H))
        self.qkvg = Linear(hidden_size, pieces, bias=False, weight_suffix=weight_suffix)
        self.out = Linear(H * v_dim, [(f"{prefix}o", hidden_size)], bias=False, weight_suffix=weight_suffix)
        self.conv_w = None
        self.lam = 0.0

    def cache_need(self):
        paged = PagedKV(self.num_kv_heads, 2 * self.head_dim, self.window, v_dim=self.v_dim)
        if self.conv_taps <= 1:
            return paged
        return (paged, FixedState(((self.conv_taps - 1) * self.channels,), torch.float32))

    def tensor_specs(self) -> List[TensorSpec]:
        p, d = self.prefix, self.head_dim
        H, G = self.num_heads, self.num_kv_heads
        specs = self.qkvg.tensor_specs() + self.out.tensor_specs()
        specs += [TensorSpec(f"{p}{n}", (d,), init="uniform:-0.3:0.3") for n in ("lq1", "lk1", "lq2", "lk2")]
        if self.conv_taps:
            specs += [TensorSpec(f"{p}{n}.conv", (c, self.conv_taps), init="uniform:-0.5:0.5")
                      for n, c in (("q", H * 2 * d), ("k", G * 2 * d), ("v", G * self.v_dim))]
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.qkvg.bind(source, dtype, device)
        self.out.bind(source, dtype, device)
        p = self.prefix
        f32 = lambda n: source.get(n).to(dtype=torch.float32)
        # one number for the layer, made once, in float32
        a = torch.exp((f32(f"{p}lq1") * f32(f"{p}lk1")).sum())
        b = torch.exp((f32(f"{p}lq2") * f32(f"{p}lk2")).sum())
        self.lam = float((a - b + torch.tensor(self.diff, dtype=torch.float32)).item())
        if self.conv_taps:
            self.conv_w = torch.cat([f32(f"{p}{n}.conv") for n in ("q", "k", "v")], dim=0).to(device).contiguous()

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        T, H, G, d, vd = x.shape[0], self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim
        paged: PagedCacheView = cache.paged if isinstance(cache, RunCacheView) else cache
        state = cache.state.state if isinstance(cache, RunCacheView) and self.conv_taps > 1 else None
        state_off = cache.state_off if isinstance(cache, RunCacheView) else 0
        u = self.qkvg.forward(x, out_dtype=torch.float32)                   # [T, q | k | v | gate]
        q = torch.empty((T, H * 2 * d), dtype=x.dtype, device=x.device)
        grp = paged.group
        kernels.diff_conv_write(u, H, G, d, vd, self.conv_w, state, state_off, ctx.token_request, ctx.cu_tokens,
                                ctx.state_slots, q, paged.kv, grp.slot_map, grp.page_size, ctx.num_requests,
                                paged.write)
        gate = u[:, self.channels:] if self.output_gate else None
        attn = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        kernels.diff_attention(q, attn, paged.kv, ctx, grp, H, G, d, vd, self.scale, self.softcap, self.lam, self.eps,
                               1.0 - self.diff, self.window or 0, gate)
        return self.out.forward_partial(attn)
