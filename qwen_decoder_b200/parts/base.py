"""Interfaces of the parts a layer is put together from.

A part has its sizes and constants as constructor parameters, declares the tensors
it needs by full name (``tensor_specs``), takes them in ``bind`` and computes in
``forward``.  No part knows which model it is in: a mixer sees the step's context
and a view of its own cache, nothing else.

Kinds of parts (each has a registry, see ``config.registry``):

* ``norm``          ``forward(stream, out_dtype, rows=None) -> normed [n, D]``
* ``position``      ``prepare(max_positions, device)``; a mixer asks it to ``rotate``
* ``mixer``         ``cache_need()``; ``forward(x [T, D], ctx, cache) -> delta [T, D]``
* ``feed_forward``  ``forward(x [T, D], ctx) -> delta [T, D]``
* ``block``         ``forward(stream, ctx, cache)``: the arrangement of the above
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import kernels
from ..weights.loader import TensorSource, TensorSpec


class Part:
    """Base of every part: tensors by name, bound once, then ``forward``."""

    # True if ``forward`` reads the host copies of the step's metadata (``ctx.host_cu_tokens``,
    # ``ctx.host_start_pos``, ``ctx.host_state_slots``): a loop over requests in Python.  A step that is
    # replayed as a CUDA graph has no such copies (nothing of it runs on the host), so a model with such
    # a part runs every step eagerly.  Parts that work from the device tensors alone leave it False.
    needs_host_metadata = False

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        pass

    def native_params(self) -> Optional[dict]:
        """The part's tensors and constants, if native code may stand in for its ``forward``: the native
        prompt loop (``parts/native_prompt.py``) runs a model only when every part of it answers.  None,
        the default, keeps the part's own path."""
        return None


class ResidualStream:
    """The residual sum of a step: ``x`` float32 [T, D], and a branch output ``delta`` that has
    not been added yet (the next norm's kernel adds it).  Blocks whose two branches read the same
    x leave a second output pending too (``delta2``), and a pending output may be one that joins
    unit-normalised: ``delta_unit`` = (u float32 [D], eps) means x += delta / sqrt(mean(delta^2) + eps) * u.
    A norm that takes only the plain form calls ``settle()`` first."""

    def __init__(self, x: torch.Tensor):
        self.x = x
        self.delta: Optional[torch.Tensor] = None
        self.delta_scale: Optional[torch.Tensor] = None     # float32 [D]: a layer scale on the pending branch
        self.delta_unit = None                              # (u, eps): the pending branch joins unit-normalised
        self.delta2: Optional[torch.Tensor] = None          # a second pending branch (plain)
        self.delta_gate: Optional[torch.Tensor] = None      # float32 logits [T, D]: the pending branch joins times their sigmoid
        self.delta_gate_bias: Optional[torch.Tensor] = None  # float32 [D]: added to every row of the logits first
        self.delta_mult = 1.0                               # a constant on what is pending (both outputs of a pair)
        self.origin: Optional[torch.Tensor] = None          # the embedding output, kept when a block reads it again

    def push(self, delta: torch.Tensor, scale: Optional[torch.Tensor] = None, unit=None,
             gate: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None, mult: float = 1.0) -> None:
        """Hand over a branch output (times ``scale`` along D, or times sigmoid(``gate`` + ``gate_bias``) element by
        element, if given; times the constant ``mult``); what is still pending is added first."""
        self.flush()
        if mult != 1.0 and (scale is not None or gate is not None):
            raise ValueError("a constant on a branch that has a layer scale or a gate is not supported")
        self.delta_mult = float(mult)
        self.delta = delta
        self.delta_scale = scale
        self.delta_unit = unit
        self.delta_gate = gate
        self.delta_gate_bias = gate_bias

    def push_pair(self, delta: torch.Tensor, delta2: torch.Tensor, mult: float = 1.0) -> None:
        """Hand over the outputs of two branches that read the same x (both times the constant ``mult``)."""
        self.flush()
        self.delta, self.delta2, self.delta_mult = delta, delta2, float(mult)

    def pending(self):
        """The pending outputs as (tensor, unit, constant) triples, for a kernel that adds up to two of them."""
        out = []
        if self.delta is not None:
            out.append((self.delta, self.delta_unit, self.delta_mult))
        if self.delta2 is not None:
            out.append((self.delta2, None, self.delta_mult))
        return out

    def clear(self) -> None:
        self.delta = self.delta_scale = self.delta_unit = self.delta2 = self.delta_gate = None
        self.delta_gate_bias = None
        self.delta_mult = 1.0

    def settle(self, gated_ok: bool = False) -> None:
        """Add what only ``flush`` can add (a second output, a unit-normalised one, and -- unless the caller's own
        kernel takes it, ``gated_ok`` -- a gated one); a plain pending delta stays."""
        if self.delta2 is not None or self.delta_unit is not None or self.delta_mult != 1.0 or \
                (self.delta_gate is not None and not gated_ok):
            self.flush()

    def flush(self) -> None:
        if self.delta is None and self.delta2 is None:
            return
        if self.delta_gate is not None:
            if self.delta2 is not None or self.delta_unit is not None or self.delta_scale is not None:
                raise ValueError("a gated branch beside a second, a scaled or a unit-normalised one is not supported")
            kernels.gated_add_norm(self.x, self.delta, self.delta_gate, gate_bias=self.delta_gate_bias)
        elif self.delta2 is None and self.delta_unit is None and self.delta_mult == 1.0:
            kernels.residual_add(self.x, self.delta, self.delta_scale)
        else:
            if self.delta_scale is not None:
                raise ValueError("a layer scale on a branch that joins unit-normalised or beside a second branch is not supported")
            kernels.add_tanh_norm(self.x, self.pending(), [])
        self.clear()


@dataclass
class PagedCacheView:
    """A mixer's view of its paged cache in this step."""
    kv: torch.Tensor            # [pages, 2, kv heads, page_size, head_dim]
    group: object               # engine.batch.GroupView
    write: bool                 # False when this run reads another run's cache


@dataclass
class StateCacheView:
    """A mixer's view of its fixed-size per-request state in this step."""
    state: torch.Tensor         # [slots, *shape]
    write: bool


@dataclass
class RunCacheView:
    """What a run of a layer sees when its need is a tuple: its pages and its per-request state row.  The owner of
    the need splits the row among its users by offset (a block keeps a convolution's inputs at the row's end, say,
    and hands the mixer a view with ``state_off`` / ``state_len`` set to the mixer's share)."""
    paged: Optional[PagedCacheView]
    state: Optional[StateCacheView]
    state_off: int = 0
    write: bool = True


class Mixer(Part):
    def cache_need(self):
        """``PagedKV``, ``FixedState`` or None."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, stream: ResidualStream, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_positions: int, device: torch.device) -> None:
        pass


class Block(Part):
    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        raise NotImplementedError
