"""RMSNorm: out = x / sqrt(mean(x^2) + eps) * w, statistics in float32, weight as ``w``
(not ``1 + w``), as the reference's rmsnorm_kernel (gpu_kernels.cu:32-67) and its CPU
form (cpu_decoder.cpp:48-53) — with eps a parameter where the reference has the
literal 1e-6 (gpu_kernels.cu:63).  The kernel also adds the residual branch that is
still pending on the stream, which the reference does in a separate residual_kernel
(gpu_kernels.cu:136-146).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Norm, ResidualStream


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float, prefix: str = "", tensor: str = "weight", offset: float = 0.0,
                 gain: float = 1.0):
        """``tensor``: the scale's name after ``prefix``.  ``offset``: the stored scale is kept around
        ``-offset`` and the norm multiplies by ``offset + w`` (1 for scales stored around zero).  ``gain``: one more
        constant factor on the output (a model that scales its logits by a constant puts it on the final norm)."""
        self.size = size
        self.eps = float(eps)
        self.prefix = prefix
        self.tensor = tensor
        self.offset = float(offset)
        self.gain = float(gain)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(f"{self.prefix}{self.tensor}", (self.size,),
                           init="around_one" if self.offset == 0.0 else "around_zero")]

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        # norm scales are used in float32 whatever they are stored in; the offset is added once, here
        w = source.get(f"{self.prefix}{self.tensor}").to(device=device, dtype=torch.float32)
        w = w + self.offset if self.offset != 0.0 else w
        self.weight = (w * self.gain if self.gain != 1.0 else w).contiguous()

    def native_params(self) -> Optional[dict]:
        return {"kind": "rmsnorm", "weight": self.weight, "eps": self.eps, "size": self.size}

    def launch_params(self, out: torch.Tensor):
        """This norm as the kernel that adds up to two pending outputs takes it."""
        return ("rms", self.weight, self.eps, out)

    def forward(self, stream: ResidualStream, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        stream.settle(gated_ok=True)
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=stream.x.device)
        if stream.delta_gate is not None:       # a branch that joins through a gate: added and normed in one launch
            kernels.gated_add_norm(stream.x, stream.delta, stream.delta_gate, self.weight, out, self.eps, rows=rows,
                                   write_back=rows is None, gate_bias=stream.delta_gate_bias)
            if rows is None:
                stream.clear()
            return out
        kernels.add_rmsnorm(stream.x, stream.delta, self.weight, out, self.eps, rows=rows,
                            write_back=rows is None, delta_scale=stream.delta_scale)
        if rows is None:
            stream.delta = None
            stream.delta_scale = None
        return out


@register_part("norm", "dyntanh")
class TanhNorm(Norm):
    """A norm without statistics: out = tanh(alpha * x) * w + b, element by element, with one learned number
    ``alpha`` and learned vectors w and b (float32 arithmetic).  Tensors: ``<prefix><tensor>`` (w),
    ``<prefix><tensor>.b``, ``<prefix><tensor>.alpha`` (a scalar).  The kernel adds what is pending on the stream
    (up to two branch outputs, also one that joins unit-normalised) before it takes the tanh."""

    def __init__(self, size: int, prefix: str = "", tensor: str = "weight"):
        self.size = size
        self.prefix = prefix
        self.tensor = tensor
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha = 1.0

    def tensor_specs(self) -> List[TensorSpec]:
        n = f"{self.prefix}{self.tensor}"
        return [TensorSpec(n, (self.size,), init="around_one"), TensorSpec(n + ".b", (self.size,), init="around_zero"),
                TensorSpec(n + ".alpha", (), init="uniform:0.4:1.2")]

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        n = f"{self.prefix}{self.tensor}"
        f32 = lambda name: source.get(name).to(device=device, dtype=torch.float32).contiguous()
        self.weight, self.bias = f32(n), f32(n + ".b")
        self.alpha = float(source.get(n + ".alpha").to(torch.float32).reshape(()).item())   # read once, at load time

    def launch_params(self, out: torch.Tensor):
        return (self.weight, self.bias, self.alpha, out)

    def forward(self, stream: ResidualStream, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if stream.delta_scale is not None:
            stream.flush()
        n = stream.x.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=stream.x.device)
        kernels.add_tanh_norm(stream.x, stream.pending(), [self.launch_params(out)], rows=rows,
                              write_back=rows is None)
        if rows is None:
            stream.clear()
        return out
