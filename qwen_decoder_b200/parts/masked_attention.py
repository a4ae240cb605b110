"""Grouped-query attention put together from options: biases, a short causal convolution on q, k and v, a norm of q
and k (over the whole projection with weights, or per head without), rotary positions, a mask (all earlier keys, the
last ``size``, or the keys of the query's own block of ``size`` positions), a per-head output gate.

With h the mixer's input [T, D], H query heads over G key/value heads (query head i reads key/value head
i // (H / G)), query/key size d and value size vd:

    q, k, v = Wq h (+ bq), Wk h (+ bk), Wv h (+ bv)
    ``conv_taps`` > 0: every channel c of q, k, v <- sum_j w[c, j] * (its value ``conv_taps`` - 1 - j tokens earlier),
        zeros before the sequence's start (``<q|k|v>.conv`` [channels, taps])
    ``qk_norm`` = "whole": q <- q / sqrt(mean(q^2) + eps) * wq with the mean over ALL H*d numbers of the token
        (``q.norm`` [H*d]), k alike (``k.norm`` [G*d]); before the rotation
    the first ``rotary_dim`` elements of every head of q and k turn by the token's position (the ``position`` part)
    ``qk_norm`` = "head": every head of q and k is divided by sqrt(mean(head^2) + eps), no weights; after the rotation
        (``norm_after_rotation``) or before it
    s_ij = (q_i . k_j) * scale for the keys j <= i that the mask lets through:
        "causal" all of them;  "window" those with i - j < size;  "chunk" those with j // size == i // size
        (blocks counted from position 0 of the sequence, wherever a prompt was cut)
    o_i = softmax_j(s_ij) v_j;   ``output_gate``: head h's o times sigmoid(Wg h)_h (``g`` [H, D]);   out = Wo [o of all heads]

Cached per token: k and v as they enter the scores; per request, in its state row, the last ``conv_taps`` - 1
projected rows [q | k | v] before the convolution (float32).  q, k, v and the gate logits are one stacked product with
float32 sums; convolution, norms, rotation, scores and softmax weights are float32 in both engine dtypes
(``csrc/qkv_prep.cu``, ``csrc/attention_sink.cu``).  A windowed mixer's pages are given back once the window has
passed them.

``inner`` computes everything up to the output projection into a tensor the caller gives (a column range of a wider
one, say), times ``out_scale``: a mixer that runs beside another one shares one output product with it.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..cache import FixedState, PagedKV
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, PagedCacheView, RunCacheView
from .linear import Linear
from .sink_attention import _TENSOR_CORES, sink_decode_splits

MASKS = ("causal", "window", "chunk")


@register_part("mixer", "masked_attention")
class MaskedAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: Optional[int] = None,
                 scale: Optional[float] = None, eps: float = 1e-6, bias: bool = False, conv_taps: int = 0,
                 qk_norm: str = "none", norm_after_rotation: bool = True, position=None, mask: str = "causal",
                 mask_size: int = 0, output_gate: bool = False, prefix: str = "mix.", weight_suffix: str = "",
                 bias_suffix: str = ".b", output_projection: bool = True):
        if num_heads % num_kv_heads:
            raise ValueError(f"masked_attention: kv heads ({num_kv_heads}) must divide heads ({num_heads})")
        if qk_norm not in kernels.QKV_NORMS or mask not in MASKS:
            raise ValueError(f"masked_attention: qk_norm must be one of {sorted(kernels.QKV_NORMS)}, mask one of {MASKS}")
        if mask != "causal" and mask_size < 1:
            raise ValueError(f"masked_attention: mask {mask!r} needs a size of at least 1")
        if head_dim % 2:
            raise ValueError("masked_attention: the head size must be even")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.v_dim = head_dim, v_dim or head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.eps, self.has_bias, self.conv_taps = float(eps), bool(bias), int(conv_taps or 0)
        self.qk_norm, self.norm_after = qk_norm, bool(norm_after_rotation)
        self.position, self.mask, self.mask_size = position, mask, int(mask_size or 0)
        self.output_gate, self.prefix, self.sfx = bool(output_gate), prefix, weight_suffix
        H, G, d, vd = num_heads, num_kv_heads, head_dim, self.v_dim
        self.channels = H * d + G * d + G * vd
        pieces = [(f"{prefix}q", H * d), (f"{prefix}k", G * d), (f"{prefix}v", G * vd)]
        self.qkv = Linear(hidden_size, pieces, bias=self.has_bias, weight_suffix=weight_suffix, bias_suffix=bias_suffix)
        # the gate has no bias: a product of its own rows, stacked under q, k, v when bound
        self.gate = Linear(hidden_size, [(f"{prefix}g", H)], bias=False, weight_suffix=weight_suffix) \
            if self.output_gate else None
        self.inner_size = H * vd
        self.out = Linear(H * vd, [(f"{prefix}o", hidden_size)], bias=False, weight_suffix=weight_suffix) \
            if output_projection else None
        self.out_stem = f"{prefix}o"
        self.conv_w = self.w_q_norm = self.w_k_norm = self.stacked = self.stacked_bias = None

    # ---- what it keeps -------------------------------------------------------
    def state_size(self) -> int:
        return (self.conv_taps - 1) * self.channels if self.conv_taps > 1 else 0

    def paged_need(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.mask_size if self.mask == "window" else None,
                       v_dim=self.v_dim)

    def cache_need(self):
        n = self.state_size()
        return (self.paged_need(), FixedState((n,), torch.float32)) if n else self.paged_need()

    # ---- tensors ---------------------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        p, H, G, d, vd = self.prefix, self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim
        specs = self.qkv.tensor_specs()
        if self.gate is not None:
            specs += self.gate.tensor_specs()
        if self.out is not None:
            specs += self.out.tensor_specs()
        if self.conv_taps:
            specs += [TensorSpec(f"{p}{n}.conv", (c, self.conv_taps), init="uniform:-0.5:0.5")
                      for n, c in (("q", H * d), ("k", G * d), ("v", G * vd))]
        if self.qk_norm == "whole":
            specs += [TensorSpec(f"{p}q.norm", (H * d,), init="around_one"),
                      TensorSpec(f"{p}k.norm", (G * d,), init="around_one")]
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.qkv.bind(source, dtype, device)
        self.stacked, self.stacked_bias = self.qkv.weight, self.qkv.bias
        if self.gate is not None:
            self.gate.bind(source, dtype, device)
            self.stacked = torch.cat([self.qkv.weight, self.gate.weight], dim=0).contiguous()
            if self.stacked_bias is not None:
                self.stacked_bias = torch.cat([self.stacked_bias, torch.zeros(self.num_heads, dtype=torch.float32,
                                                                              device=device)]).contiguous()
        if self.out is not None:
            self.out.bind(source, dtype, device)
        p = self.prefix
        f32 = lambda n: source.get(n).to(device=device, dtype=torch.float32).contiguous()
        if self.conv_taps:
            self.conv_w = torch.cat([f32(f"{p}{n}.conv") for n in ("q", "k", "v")], dim=0).contiguous()
        if self.qk_norm == "whole":
            self.w_q_norm, self.w_k_norm = f32(f"{p}q.norm"), f32(f"{p}k.norm")

    # ---- compute -----------------------------------------------------------------
    def inner(self, x: torch.Tensor, ctx, cache, out: torch.Tensor, out_scale: float = 1.0) -> None:
        """Everything before the output projection: out [T, H * vd] (rows may be strided) in x's dtype."""
        from . import matmul_backend
        H, G, d, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim
        T = x.shape[0]
        paged: PagedCacheView = cache.paged if isinstance(cache, RunCacheView) else cache
        state = cache.state.state if isinstance(cache, RunCacheView) and self.conv_taps > 1 else None
        state_off = cache.state_off if isinstance(cache, RunCacheView) else 0
        u = torch.empty((T, self.stacked.shape[0]), dtype=torch.float32, device=x.device)
        matmul_backend.linear(x, self.stacked, self.stacked_bias, u)      # [q | k | v | gate logits], float32 sums
        pos = self.position
        rope = (pos.rotary_dim, pos.pairing_code, pos.cos, pos.sin) if pos is not None else (0, 0, None, None)
        q = torch.empty((T, H * d), dtype=x.dtype, device=x.device)
        grp = paged.group
        kernels.qkv_prep(u, H, G, d, vd, self.conv_w, state, state_off, ctx, paged.write, self.qk_norm, self.norm_after,
                         self.w_q_norm, self.w_k_norm, self.eps, *rope, q, paged.kv, grp.slot_map, grp.page_size,
                         paged.write)
        gate = u[:, self.channels:] if self.output_gate else None
        window = self.mask_size if self.mask == "window" else 0
        chunk = self.mask_size if self.mask == "chunk" else 0
        ps = grp.page_size
        extra = dict(chunk=chunk, gate=gate, out_scale=out_scale)
        if _TENSOR_CORES and kernels.sink_mma_supported(x.dtype, H, G, d, vd):
            args = (H, G, d, vd, ps, self.scale, window, None)
            nd = T if ctx.all_decode else getattr(ctx, "num_decode", 0)
            if nd:
                keys = ctx.max_context if ctx.all_decode else ctx.decode_max_context
                reach = min(keys, window or keys, chunk or keys)
                splits = sink_decode_splits(nd * G, reach)
                kernels.sink_attention_mma(q, out, paged.kv, grp.block_table, ctx.cu_tokens, ctx.start_pos, nd, nd,
                                           *args, splits=splits, **extra)
            if nd < T:
                kernels.sink_attention_mma(q, out, paged.kv, grp.block_table[nd:], ctx.cu_tokens[nd:],
                                           ctx.start_pos[nd:], ctx.num_requests - nd, T - nd, *args, **extra)
            return
        kernels.sink_attention_generic(q, out, paged.kv, grp.block_table, ctx.token_request, ctx.positions, H, G, d, vd,
                                       ps, self.scale, window, None, **extra)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        attn = torch.empty((x.shape[0], self.inner_size), dtype=x.dtype, device=x.device)
        self.inner(x, ctx, cache, attn)
        return self.out.forward_partial(attn)
