"""A recurrent mixer with a matrix state per head (linear attention with a per-channel, per-token decay).

With h the mixer's input [T, D], h' the row of the token before (zeros for a sequence's first token), H heads of size d:

    x_s = h + (h' - h) * mu_s               for s in r, k, v, g, w: each projection reads its own blend (``mu.<s>`` [D])
    r, k, v = Wr x_r, Wk x_k, Wv x_v         [H, d] each;     gate = silu(Wg x_g)   [H * d]
    w = exp(-exp(W2 tanh(W1 x_w) + w0))      the decay, per head and key channel (``w1`` [R, D], ``w2`` [H*d, R], ``w0``)
    per head:  o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          (the bonus u [H, d] for the current token only)
               S_t = diag(w_t) S_(t-1) + k_t v_t^T                 (S [d, d] starts at zero)
    out = Wo ((o / sqrt(mean(o^2) + eps) per head) * norm * gate)   (``norm`` [H * d])

Per request, one float32 state row: the heads' matrices S [H, d, d], then the last token's h [D].  The blends enter
their products rounded to the engine's dtype; the products' sums, the decay, the recurrence, the unit norm and the
gate are float32 in both engine dtypes (``csrc/time_mix.cu``).  The recurrence runs token by token in the tokens'
order, so a portion at once and token by token agree exactly.

``inner`` computes everything up to the output projection into a tensor the caller gives, times ``out_scale``.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..cache import FixedState
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, RunCacheView, StateCacheView
from .linear import Linear
from . import matmul_backend

BLENDS = ("r", "k", "v", "g", "w")


@register_part("mixer", "time_mix")
class TimeMix(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay_rank=None, eps: float = 1e-6,
                 prefix: str = "mix.", weight_suffix: str = "", output_projection: bool = True,
                 default_decay_rank: int = 32):
        """``decay_rank`` None: the rank R of the decay's low-rank product is whatever the stored ``w1`` [R, D] has
        (random weights then take ``default_decay_rank``)."""
        if head_dim > 256:
            raise ValueError("time_mix: the head size must be at most 256")
        self.default_decay_rank = int(default_decay_rank)
        self.hidden_size, self.num_heads, self.head_dim, self.decay_rank = hidden_size, num_heads, head_dim, decay_rank
        self.eps, self.prefix, self.sfx = float(eps), prefix, weight_suffix
        n = num_heads * head_dim
        self.inner_size = n
        self.proj = {s: Linear(hidden_size, [(f"{prefix}{s}", n)], bias=False, weight_suffix=weight_suffix)
                     for s in ("r", "k", "v", "g")}
        self.out = Linear(n, [(f"{prefix}o", hidden_size)], bias=False, weight_suffix=weight_suffix) \
            if output_projection else None
        self.out_stem = f"{prefix}o"
        self.mu = self.w1 = self.w2 = self.w0 = self.u = self.norm = None

    def state_size(self) -> int:
        return self.num_heads * self.head_dim * self.head_dim + self.hidden_size

    def paged_need(self):
        return None

    def cache_need(self):
        return FixedState((self.state_size(),), torch.float32)

    def tensor_specs(self) -> List[TensorSpec]:
        p, D, H, d, R = self.prefix, self.hidden_size, self.num_heads, self.head_dim, self.decay_rank
        specs = [s for lin in self.proj.values() for s in lin.tensor_specs()]
        R0 = self.default_decay_rank
        R = -1 if R is None else R
        if self.out is not None:
            specs += self.out.tensor_specs()
        specs += [TensorSpec(f"{p}mu.{s}", (D,), init="uniform:0:1") for s in BLENDS]
        specs += [TensorSpec(f"{p}w1{self.sfx}", (R, D), default_shape=(R0, D)),
                  TensorSpec(f"{p}w2{self.sfx}", (H * d, R), default_shape=(H * d, R0)),
                  TensorSpec(f"{p}w0", (H * d,), init="uniform:-2:0.5"),
                  TensorSpec(f"{p}u", (H, d), init="uniform:-0.5:0.5"), TensorSpec(f"{p}norm", (H * d,), init="around_one")]
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        for lin in list(self.proj.values()) + ([self.out] if self.out is not None else []):
            lin.bind(source, dtype, device)
        p = self.prefix
        f32 = lambda n: source.get(n).to(device=device, dtype=torch.float32).contiguous()
        self.mu = torch.stack([f32(f"{p}mu.{s}") for s in BLENDS]).contiguous()
        self.w1 = source.get(f"{p}w1{self.sfx}").to(device=device, dtype=dtype).contiguous()
        # kept as its transpose [R, H*d]: the decay's kernel reads neighbouring channels side by side
        self.w2 = source.get(f"{p}w2{self.sfx}").to(device=device, dtype=dtype).t().contiguous()
        if self.w1.shape[0] != self.w2.shape[0]:
            raise ValueError(f"time_mix: {p}w1 has rank {self.w1.shape[0]}, {p}w2 has {self.w2.shape[0]}")
        self.decay_rank = self.w1.shape[0]
        self.w0, self.u, self.norm = f32(f"{p}w0"), f32(f"{p}u"), f32(f"{p}norm")

    def inner(self, x: torch.Tensor, ctx, cache, out: torch.Tensor, out_scale: float = 1.0) -> None:
        """Everything before the output projection: out [T, H * d] (rows may be strided) in x's dtype."""
        T, D = x.shape
        H, d = self.num_heads, self.head_dim
        n = H * d
        if isinstance(cache, RunCacheView):
            st, off = cache.state, cache.state_off
        else:
            st, off = cache, 0
        assert isinstance(st, StateCacheView)
        state, prev_off = st.state, off + H * d * d
        blends = torch.empty((len(BLENDS), T, D), dtype=x.dtype, device=x.device)
        kernels.tm_shift_mix(x, self.mu, state, prev_off, ctx, blends)
        sums = torch.empty((4, T, n), dtype=torch.float32, device=x.device)       # r, k, v, gate logits
        for i, s in enumerate(("r", "k", "v", "g")):
            matmul_backend.linear(blends[i], self.proj[s].weight, None, sums[i])
        low = torch.empty((T, self.decay_rank), dtype=torch.float32, device=x.device)
        matmul_backend.linear(blends[4], self.w1, None, low)
        decay = torch.empty((T, n), dtype=torch.float32, device=x.device)
        kernels.tm_decay(low, self.w2, self.w0, decay)
        o = torch.empty((T, n), dtype=torch.float32, device=x.device)
        kernels.tm_scan(sums[0], sums[1], sums[2], decay, self.u, H, d, state, off, ctx, o, st.write)
        kernels.tm_finish(o, sums[3], self.norm, H, d, self.eps, out_scale, out, x, state, prev_off, ctx, st.write)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        y = torch.empty((x.shape[0], self.inner_size), dtype=x.dtype, device=x.device)
        self.inner(x, ctx, cache, y)
        return self.out.forward_partial(y)
