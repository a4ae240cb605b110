"""Latent attention: queries and keys/values go through low-rank latents, and only one row per token is
cached, [normed key/value latent | rotated key part shared by all heads].

With h the mixer's input [T, D], H heads of ``nope_dim`` unrotated + ``rope_dim`` rotated query/key elements and
``v_dim`` value elements, latent sizes ``q_rank`` and ``kv_rank``:

    cq = rms(Wdq h) * w_dq            q = Wuq cq, per head [nope | rope]
    [c_raw | kr] = Wdkv h             c = rms(c_raw) * w_dkv;  kr and q's rope part rotated by position
    k_h = Wuk_h c,  v_h = Wuv_h c     score = (q_nope . k_h + q_rope . kr) * scale, causal softmax
    out = Wo ((heads' results) * sigmoid(Wg h))

Keys and values are never expanded: the query is carried into the latent space (Wuk_h^T q_nope), attention runs
over the cached rows, and Wuv_h is applied to the weighted sum of latents (``csrc/latent_attention.cu``).  Wdq,
Wdkv and Wg are one stacked product of h.  Norms, angles, scores and softmax weights are float32 in both engine
dtypes.  The plain norms here multiply by the stored weight (no offset); their eps is the layer's.

Variants, all constructor parameters: ``q_rank`` = 0 leaves the query latent out, q = Wq h (tensor ``<prefix>q``);
``rope_dim`` = 0 leaves the rotated part out (no position enters the scores, the cached row is c alone);
``output_gate`` = False leaves the sigmoid gate out.
"""
from __future__ import annotations

from typing import List, Optional

import os

import torch

from .. import kernels
from ..cache import PagedRows
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, PagedCacheView
from . import matmul_backend
from .linear import Linear

# From this many tokens on, the bfloat16 engine makes the per-head products with Wuk and Wuv as batched library
# products (as the framework does for every product of many tokens); below, the kernels read the weights themselves.
LIBRARY_TOKENS = 64
# Portions of prompts of at least this many tokens (the longest of the step) take the expanded form in bfloat16: keys
# and values of all heads are made from the cached rows of the requests' contexts by one product and an ordinary
# attention kernel runs over them.  A (token, key) pair then costs dn + dv products per head instead of 2 r, and a
# row of context one expansion: worth it from about twenty tokens per request.
EXPAND_TOKENS = int(os.environ.get("QD_LATENT_EXPAND_TOKENS", "32"))
EXPAND_MAX_BYTES = 4 << 30          # the expanded keys and values of a step; above it the absorbed form runs


def _hi_lo(x: torch.Tensor) -> torch.Tensor:
    """float32 [T, H, d] -> bfloat16 [H, T, 2 d]: every number as its bfloat16 rounding and what that left out,
    side by side, so that a bfloat16 product with a matrix stacked twice sees 16 bits of mantissa."""
    hi = x.to(torch.bfloat16)
    lo = (x - hi.float()).to(torch.bfloat16)
    return torch.cat((hi, lo), dim=-1).transpose(0, 1)


def attend_splits(ctas_without_split: int, max_keys: int) -> int:
    """CTAs that share one token's keys: enough to give every multiprocessor one, none with fewer than four
    tiles of 32 keys."""
    by_fill = max(1, kernels.sm_count() // max(1, ctas_without_split))
    by_work = max(1, (max_keys + 127) // 128)
    return max(1, min(by_fill, by_work, 64))


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, nope_dim: int, rope_dim: int, v_dim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, position=None, window: Optional[int] = None,
                 prefix: str = "self_attn.", weight_suffix: str = ".weight", output_gate: bool = True):
        if kv_rank > kernels.LATENT_MAX_RANK:
            raise ValueError(f"latent attention: kv_rank {kv_rank} exceeds {kernels.LATENT_MAX_RANK}")
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.nope_dim, self.rope_dim, self.v_dim = nope_dim, rope_dim, v_dim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.scale, self.eps, self.window = float(scale), float(eps), window
        self.position = position            # a Rotary over the rope part (its rotary_dim leading elements turn) or None
        self.prefix, self.sfx = prefix, weight_suffix
        H = num_heads
        self.output_gate = bool(output_gate)
        self.q_width = q_rank if q_rank else H * (nope_dim + rope_dim)      # the stacked product's first columns
        pieces = [(f"{prefix}dq", q_rank) if q_rank else (f"{prefix}q", self.q_width),
                  (f"{prefix}dkv", kv_rank + rope_dim)]
        if self.output_gate:
            pieces.append((f"{prefix}g", H * v_dim))
        self.down = Linear(hidden_size, pieces, bias=False, weight_suffix=weight_suffix)
        self.up_q = Linear(q_rank, [(f"{prefix}uq", H * (nope_dim + rope_dim))], bias=False,
                           weight_suffix=weight_suffix) if q_rank else None
        self.out = Linear(H * v_dim, [(f"{prefix}o", hidden_size)], bias=False, weight_suffix=weight_suffix)

    def cache_need(self):
        return PagedRows(self.kv_rank + self.rope_dim, self.window)

    def tensor_specs(self) -> List[TensorSpec]:
        p, s, H = self.prefix, self.sfx, self.num_heads
        specs = self.down.tensor_specs() + self.out.tensor_specs()
        if self.q_rank:
            specs += self.up_q.tensor_specs() + [TensorSpec(f"{p}dq.norm", (self.q_rank,), init="around_one")]
        return specs + [
            TensorSpec(f"{p}dkv.norm", (self.kv_rank,), init="around_one"),
            TensorSpec(f"{p}uk{s}", (H * self.nope_dim, self.kv_rank)),
            TensorSpec(f"{p}uv{s}", (H * self.v_dim, self.kv_rank))]

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        for lin in (self.down, self.up_q, self.out):
            if lin is not None:
                lin.bind(source, dtype, device)
        p, s = self.prefix, self.sfx
        f32 = lambda n: source.get(n).to(device=device, dtype=torch.float32).contiguous()
        self.w_dkv_norm = f32(f"{p}dkv.norm")
        self.w_dq_norm = f32(f"{p}dq.norm") if self.q_rank else self.w_dkv_norm       # unused without a query latent
        self.w_uk = source.get(f"{p}uk{s}").to(device=device, dtype=dtype).contiguous()
        self.w_uv = source.get(f"{p}uv{s}").to(device=device, dtype=dtype).contiguous()
        H = self.num_heads
        # for the batched library products: each matrix twice along its inner dimension, so that a float32 operand
        # can enter as [hi | lo] (two bfloat16 numbers per element) in ONE product with a float32 sum
        uk = self.w_uk.view(H, self.nope_dim, self.kv_rank)                                  # [H, dn, r]
        uv = self.w_uv.view(H, self.v_dim, self.kv_rank).transpose(1, 2)                     # [H, r, dv]
        self.w_uk_twice = torch.cat((uk, uk), dim=1).contiguous() if dtype == torch.bfloat16 else None
        self.w_uv_twice = torch.cat((uv, uv), dim=1).contiguous() if dtype == torch.bfloat16 else None
        self._no_table = torch.zeros((1, 0), dtype=torch.float32, device=device)
        # the expanded form's one matrix: a row of context -> [keys of all heads | values of all heads]
        self.w_ukv = torch.cat((self.w_uk, self.w_uv), dim=0).contiguous() if self._can_expand(dtype) else None

    def _can_expand(self, dtype) -> bool:
        return (dtype == torch.bfloat16 and self.rope_dim == 0 and not self.output_gate and not self.window
                and kernels.sink_mma_supported(dtype, self.num_heads, self.num_heads, self.nope_dim, self.v_dim))

    def _attend_expanded(self, q: torch.Tensor, attn: torch.Tensor, ctx, cache: PagedCacheView, nd: int,
                         lmax: int) -> None:
        """Requests nd.. of the step (rows cu_tokens[nd].. of q and attn): gather their contexts' rows, expand keys
        and values, attend with the tensor-core kernel for heads that each have their own keys (a page of one key:
        [keys of all heads | values of all heads] is a row of the product)."""
        H, dn, dv, r = self.num_heads, self.nope_dim, self.v_dim, self.kv_rank
        R = ctx.num_requests - nd
        T = q.shape[0]
        qb = torch.empty((T, H * dn), dtype=torch.bfloat16, device=q.device)
        kernels.round_rows(q, qb)
        rows = torch.empty((R * lmax, r), dtype=torch.bfloat16, device=q.device)
        kernels.latent_gather(cache.kv, cache.group.block_table[nd:], ctx.cu_tokens[nd:], ctx.start_pos[nd:], R, r,
                              rows, lmax)
        kv = torch.empty((R * lmax, H * (dn + dv)), dtype=torch.bfloat16, device=q.device)
        matmul_backend.linear(rows, self.w_ukv, None, kv)
        table = torch.arange(R * lmax, dtype=torch.int32, device=q.device).view(R, lmax)
        kernels.sink_attention_mma(qb, attn, kv, table, ctx.cu_tokens[nd:], ctx.start_pos[nd:], R,
                                   T - int(ctx.host_cu_tokens[nd]), H, H, dn, dv, 1, self.scale, 0, None)

    def forward(self, x: torch.Tensor, ctx, cache: PagedCacheView) -> torch.Tensor:
        T, H = x.shape[0], self.num_heads
        dn, dr, dv, r, qr = self.nope_dim, self.rope_dim, self.v_dim, self.kv_rank, self.q_rank
        pos = self.position
        rot = (pos.cos, pos.sin, pos.rotary_dim) if pos is not None else (self._no_table, self._no_table, 0)
        qw = self.q_width
        u = self.down.forward(x, out_dtype=torch.float32)                   # [T, qr (or q itself) | r + dr | H * dv]
        cq = torch.empty((T, qr), dtype=x.dtype, device=x.device)
        kernels.latent_prep(u, 0, qr, qw, r, dr, self.w_dq_norm, self.w_dkv_norm, self.eps, *rot, ctx.positions,
                            cache.group.slot_map, cq, cache.kv, cache.write)
        q = self.up_q.forward(cq, out_dtype=torch.float32) if qr else u[:, :qw]
        attn = torch.empty((T, H * dv), dtype=x.dtype, device=x.device)
        # rows 0 .. Ta-1 take the absorbed form: all of them, or the single tokens of a step whose portions expand
        Ta = T
        if self.w_ukv is not None and not ctx.all_decode and ctx.max_portion >= EXPAND_TOKENS:
            nd = getattr(ctx, "num_decode", 0)
            lmax = max(s + c1 - c0 for s, c0, c1 in zip(ctx.host_start_pos[nd:], ctx.host_cu_tokens[nd:],
                                                              ctx.host_cu_tokens[nd + 1:]))
            if (ctx.num_requests - nd) * lmax * H * (dn + dv) * 2 <= EXPAND_MAX_BYTES:
                self._attend_expanded(q, attn, ctx, cache, nd, lmax)
                Ta = nd
        if Ta:
            self._attend_absorbed(q[:Ta], u[:Ta, qw + r + dr:] if self.output_gate else None, attn[:Ta], ctx, cache, Ta)
        return self.out.forward_partial(attn)

    def _attend_absorbed(self, q: torch.Tensor, gate, attn: torch.Tensor, ctx, cache: PagedCacheView, T: int) -> None:
        """Rows 0 .. T-1 of the step: the queries take Wuk in, attention runs over the cached rows themselves, and
        Wuv expands the result."""
        H = self.num_heads
        dn, dr, dv, r = self.nope_dim, self.rope_dim, self.v_dim, self.kv_rank
        pos = self.position
        rot = (pos.cos, pos.sin, pos.rotary_dim) if pos is not None else (self._no_table, self._no_table, 0)
        x_dtype, dev = attn.dtype, attn.device
        positions, token_request = ctx.positions[:T], ctx.token_request[:T]
        qcat = torch.empty((T, H, r + dr), dtype=torch.float32, device=dev)
        library = x_dtype == torch.bfloat16 and T >= LIBRARY_TOKENS and matmul_backend.mode != "generic"
        pre = None
        if library:
            qn = _hi_lo(q.view(T, H, dn + dr)[:, :, :dn])                                   # [H, T, 2 dn]
            pre = torch.bmm(qn, self.w_uk_twice, out_dtype=torch.float32)                   # [H, T, r]
            matmul_backend.counters["library"] += 1
        kernels.latent_absorb(q, self.w_uk, qcat, H, dn, dr, r, *rot, positions, pre=pre)
        o_lat = torch.empty((T, H, r), dtype=torch.float32, device=dev)
        window = self.window or 0
        groups = -(-H // 8)
        keys = ctx.max_context if T == ctx.num_tokens else ctx.decode_max_context
        splits = attend_splits(T * groups, min(keys, window or keys))
        kernels.latent_attend(qcat, cache.kv, cache.group.block_table, token_request, positions, r, dr,
                              cache.group.page_size, self.scale, window, splits, o_lat)
        pre = None
        if library:
            pre = torch.bmm(_hi_lo(o_lat), self.w_uv_twice, out_dtype=torch.float32)        # [H, T, dv]
            matmul_backend.counters["library"] += 1
        kernels.latent_expand(o_lat, self.w_uv, gate, attn, dv, pre=pre)
