"""Several mixers side by side on the same input, added up with constant weights:

    out = sum_b scale_b * mixer_b(h)

Every branch is a registered mixer that can compute everything before its output projection into a given tensor
(``inner``) and tells what it keeps per token (``paged_need``) and per request (``state_size``).  Because
sum_b scale_b Wo_b y_b = [Wo_1 | Wo_2 | ...] [scale_1 y_1 ; scale_2 y_2 ; ...], the branches write their scaled y_b
into column ranges of ONE tensor and one product with the output matrices laid side by side finishes all of them.
At most one branch may keep pages; the per-request states follow one another in one float32 state row.

``branches``: a list of {"name": registered mixer, "params": its parameters (``prefix`` relative to this mixer's),
"scale": its weight}.
"""
from __future__ import annotations

from typing import List

import torch

from ..cache import FixedState
from ..config.registry import create_part, register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, PagedCacheView, RunCacheView, StateCacheView
from .linear import Linear


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    def __init__(self, hidden_size: int, branches, prefix: str = "mix.", weight_suffix: str = ""):
        if not branches:
            raise ValueError("side_by_side: at least one branch")
        self.hidden_size, self.prefix, self.sfx = hidden_size, prefix, weight_suffix
        self.mixers, self.scales = [], []
        for b in branches:
            p = dict(b["params"])
            p["prefix"] = prefix + p.get("prefix", "")
            p["output_projection"] = False
            m = create_part("mixer", b["name"], **p)
            if not (hasattr(m, "inner") and hasattr(m, "state_size") and hasattr(m, "paged_need")):
                raise ValueError(f"side_by_side: mixer {b['name']!r} cannot run beside another one")
            self.mixers.append(m)
            self.scales.append(float(b.get("scale", 1.0)))
        paged = [m.paged_need() for m in self.mixers if m.paged_need() is not None]
        if len(paged) > 1:
            raise ValueError("side_by_side: at most one branch may keep pages")
        self._paged = paged[0] if paged else None
        self.offsets, off = [], 0
        for m in self.mixers:                          # a branch's share of the state row follows the one before it
            self.offsets.append(off)
            off += m.state_size()
        self._state = off
        self.widths = [m.inner_size for m in self.mixers]
        self.out = Linear(sum(self.widths), [("out", hidden_size)], bias=False, weight_suffix="")

    def parts(self):
        return list(self.mixers)

    def cache_need(self):
        state = FixedState((self._state,), torch.float32) if self._state else None
        if self._paged is not None and state is not None:
            return (self._paged, state)
        return self._paged if self._paged is not None else state

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [s for m in self.mixers for s in m.tensor_specs()]
        specs += [TensorSpec(f"{m.out_stem}{self.sfx}", (self.hidden_size, m.inner_size)) for m in self.mixers]
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        for m in self.mixers:
            m.bind(source, dtype, device)
        ws = [source.get(f"{m.out_stem}{self.sfx}").to(device=device, dtype=dtype) for m in self.mixers]
        self.out.bind_tensor(torch.cat(ws, dim=1).contiguous())

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        if isinstance(cache, RunCacheView):
            paged, state, base, write = cache.paged, cache.state, cache.state_off, cache.write
        elif isinstance(cache, StateCacheView):
            paged, state, base, write = None, cache, 0, cache.write
        else:
            paged, state, base, write = cache, None, 0, getattr(cache, "write", True)
        y = torch.empty((x.shape[0], sum(self.widths)), dtype=x.dtype, device=x.device)
        lo = 0
        for m, scale, off, width in zip(self.mixers, self.scales, self.offsets, self.widths):
            view = RunCacheView(paged=paged if m.paged_need() is not None else None, state=state,
                                state_off=base + off, write=write)
            m.inner(x, ctx, view, y[:, lo:lo + width], out_scale=scale)
            lo += width
        return self.out.forward_partial(y)
