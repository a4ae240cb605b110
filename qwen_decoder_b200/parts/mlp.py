"""SwiGLU feed-forward: h = silu(x W1^T) * (x W3^T); delta = h W2^T, no biases
(gpu_decoder.cu:457-497, swiglu_kernel gpu_kernels.cu:149-160, cpu_decoder.cpp:204-212;
W1 = gate_proj, W3 = up_proj, W2 = down_proj).  Gate and up are one stacked product.

``activation`` = "clamped" (with ``limit`` L and ``alpha`` a; the reference has silu only) gates instead with
g = min(x W1^T, L), u = clamp(x W3^T, -L, L), h = g * sigmoid(a g) * (u + 1); the stacked product then leaves
float32 sums and one elementwise kernel makes h.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import kernels
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import FeedForward
from . import matmul_backend
from .linear import Linear


ACTIVATIONS = {"silu": kernels.ACT_SILU, "clamped": kernels.ACT_CLAMPED}


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp.",
                 names: Sequence[str] = ("gate_proj", "up_proj", "down_proj"), weight_suffix: str = ".weight",
                 activation: str = "silu", limit: float = 0.0, alpha: float = 1.0):
        """``names``: what the gate, up and down matrices are called after ``prefix``."""
        if activation not in ACTIVATIONS:
            raise ValueError(f"gated feed-forward: activation must be one of {sorted(ACTIVATIONS)}, got {activation!r}")
        if activation == "clamped" and not limit > 0:
            raise ValueError("gated feed-forward: the clamped activation needs a positive limit")
        self.activation, self.limit, self.alpha = activation, float(limit), float(alpha)
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        g, u, d = names
        self.gate_up = Linear(hidden_size, [(f"{prefix}{g}", intermediate_size),
                                            (f"{prefix}{u}", intermediate_size)], bias=False,
                              weight_suffix=weight_suffix)
        self.down = Linear(intermediate_size, [(f"{prefix}{d}", hidden_size)], bias=False,
                           weight_suffix=weight_suffix)
        self._barrier = None

    def tensor_specs(self) -> List[TensorSpec]:
        return self.gate_up.tensor_specs() + self.down.tensor_specs()

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.gate_up.bind(source, dtype, device)
        self.down.bind(source, dtype, device)

    def native_params(self):
        if self.activation != "silu":
            return None
        return {"kind": "swiglu", "D": self.hidden_size, "F": self.intermediate_size, "wgu": self.gate_up.weight,
                "wd": self.down.weight}

    def reset_after_fault(self) -> None:
        """A launch whose wait for the other CTAs ran out may have left tiles counted: start from zero again."""
        if self._barrier is not None:
            self._barrier.zero_()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        if self.activation != "silu":
            h = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
            kernels.gated_act(self.gate_up.forward(x, out_dtype=torch.float32), h, ACTIVATIONS[self.activation],
                              self.limit, self.alpha)
            return self.down.forward_partial(h)
        if matmul_backend.mode == "auto" and kernels.ffn_stream_supported(x, self.gate_up.weight, self.down.weight):
            matmul_backend.counters["own"] += 1
            if self._barrier is None:       # this layer's own synchronisation words (zero once; each launch leaves them zero)
                self._barrier = torch.zeros(kernels.FFN_SYNC_WORDS, dtype=torch.int32, device=x.device)
            return kernels.ffn_stream(x, self.gate_up.weight, self.down.weight, self._barrier)   # one launch
        h = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        if matmul_backend.use_skinny(x, self.gate_up.weight):
            shares = kernels.swiglu_shares(x.shape[0], self.hidden_size, 2 * self.intermediate_size)
            if shares and self.intermediate_size % 4 == 0:
                # where the streamer keeps the tokens resident only for a share of K: partial sums, then SwiGLU
                kernels.swiglu_partial(kernels.gemm_skinny_partial(x, self.gate_up.weight, shares), h)
            else:
                kernels.gemm_skinny_swiglu(x, self.gate_up.weight, h)       # gate, up and SwiGLU in one kernel
            matmul_backend.counters["own"] += 1
        else:
            kernels.swiglu(self.gate_up.forward(x), h)
        return self.down.forward_partial(h)


PLAIN_ACTIVATIONS = {"gelu_tanh": kernels.ACT_GELU_TANH}


@register_part("feed_forward", "mlp")
class PlainMLP(FeedForward):
    """The ungated feed-forward: delta = Wdown act(Wup h), no biases; ``activation`` = "gelu_tanh" is
    0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).  The first product leaves float32 sums, one elementwise
    kernel makes the activation in the engine's dtype."""

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str = "mlp.", names: Sequence[str] = ("up", "down"),
                 weight_suffix: str = "", activation: str = "gelu_tanh"):
        if activation not in PLAIN_ACTIVATIONS:
            raise ValueError(f"feed-forward: activation must be one of {sorted(PLAIN_ACTIVATIONS)}, got {activation!r}")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        u, d = names
        self.up = Linear(hidden_size, [(f"{prefix}{u}", intermediate_size)], bias=False, weight_suffix=weight_suffix)
        self.down = Linear(intermediate_size, [(f"{prefix}{d}", hidden_size)], bias=False, weight_suffix=weight_suffix)

    def tensor_specs(self) -> List[TensorSpec]:
        return self.up.tensor_specs() + self.down.tensor_specs()

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.up.bind(source, dtype, device)
        self.down.bind(source, dtype, device)

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        h = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.plain_act(self.up.forward(x, out_dtype=torch.float32), h, PLAIN_ACTIVATIONS[self.activation])
        return self.down.forward_partial(h)
