"""A feed-forward of routed experts with an optional shared expert.

    logits = Wr h + b (float32);  the ``top`` experts with the largest logits;  weights = softmax over those logits
    out = sum_k weight_k * expert_k(h)  +  sigmoid(wsg . h) * shared(h)
    expert(h) = Wdown (silu(Wgate h) * (Wup h)), no biases; the shared expert has the same form

Variants, all constructor parameters: ``routing`` = "softmax_all" takes scores = softmax(Wr h) over all outputs of
the router, chooses the ``top`` largest of score + correction (a learned vector, ``<prefix>correction``) and weighs
by the plain scores, not renormalised (no router bias); the last ``identity`` outputs of the router are identity
experts without tensors, expert(h) = h; ``activation`` = "clamped" with ``limit`` and ``alpha`` is the gate of
``parts.mlp`` (the shared expert has its own ``shared_limit``); ``shared_gate`` = False adds the shared expert in full.
``routing`` = "top_sigmoid" chooses the ``top`` largest logits and weighs each by its own sigmoid, not renormalised;
``router_bias`` = False leaves the router without a bias; ``weigh`` = "input" lets a pair's weight multiply the
expert's input instead of its output, out = sum_k expert_k(weight_k h) (the gate is not linear, so this differs):
since W (w h) = w (W h), the grouped product multiplies the pair's two sums by w before the gate.

Routing, ordering the (token, choice) pairs by expert, the grouped products and the weighted sum all stay on the
device (``csrc/moe.cu``): nothing is read back, so steps with routed experts replay as CUDA graphs.  The shared
expert is the dense gated feed-forward part with its own kernels.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import FeedForward
from . import matmul_backend
from .mlp import ACTIVATIONS, SwiGLU

ROUTINGS = {"top_softmax": kernels.MOE_ROUTE_TOP_SOFTMAX, "softmax_all": kernels.MOE_ROUTE_SOFTMAX_ALL,
            "top_sigmoid": kernels.MOE_ROUTE_TOP_SIGMOID}


@register_part("feed_forward", "moe")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, expert_size: int, num_experts: int, top: int, shared_size: int = 0,
                 prefix: str = "mlp.", weight_suffix: str = ".weight", names=("gate", "up", "down"),
                 routing: str = "top_softmax", identity: int = 0, activation: str = "silu", limit: float = 0.0,
                 alpha: float = 1.0, shared_limit: float = 0.0, shared_gate: bool = True, router_bias: bool = True,
                 weigh: str = "output"):
        outputs = num_experts + identity
        if not (1 <= top <= outputs) or top > kernels.MOE_MAX_TOP:
            raise ValueError(f"moe: top ({top}) must be between 1 and the router's outputs ({outputs}), at most {kernels.MOE_MAX_TOP}")
        if routing not in ROUTINGS or activation not in ACTIVATIONS or identity < 0:
            raise ValueError(f"moe: routing must be one of {sorted(ROUTINGS)}, activation one of {sorted(ACTIVATIONS)}, identity >= 0")
        self.hidden_size, self.expert_size, self.num_experts, self.top = hidden_size, expert_size, num_experts, top
        if weigh not in ("output", "input") or (weigh == "input" and identity):
            raise ValueError("moe: weigh must be 'output' or 'input' (and 'input' goes without identity experts)")
        self.identity, self.outputs = identity, outputs
        self.router_bias, self.weigh = bool(router_bias) and routing != "softmax_all", weigh
        self.routing, self.activation, self.limit, self.alpha = routing, activation, float(limit), float(alpha)
        self.prefix, self.sfx, self.names = prefix, weight_suffix, tuple(names)
        self.shared_gate = bool(shared_gate)
        self.shared = SwiGLU(hidden_size, shared_size, prefix=f"{prefix}shared.", names=self.names,
                             weight_suffix=weight_suffix, activation=activation, limit=shared_limit or limit,
                             alpha=alpha) if shared_size else None

    def tensor_specs(self) -> List[TensorSpec]:
        p, s, D, F = self.prefix, self.sfx, self.hidden_size, self.expert_size
        g, u, d = self.names
        specs = [TensorSpec(f"{p}router{s}", (self.outputs, D), init="uniform:-0.5:0.5")]
        if self.routing == "softmax_all":
            specs.append(TensorSpec(f"{p}correction", (self.outputs,), init="around_zero"))
        elif self.router_bias:
            specs.append(TensorSpec(f"{p}router.b", (self.outputs,), init="around_zero"))
        for e in range(self.num_experts):
            specs += [TensorSpec(f"{p}e{e}.{g}{s}", (F, D)), TensorSpec(f"{p}e{e}.{u}{s}", (F, D)),
                      TensorSpec(f"{p}e{e}.{d}{s}", (D, F))]
        if self.shared is not None:
            specs += self.shared.tensor_specs()
            if self.shared_gate:
                specs.append(TensorSpec(f"{p}shared.sg{s}", (1, D)))
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        p, s = self.prefix, self.sfx
        g, u, d = self.names
        get = lambda n: source.get(n).to(device=device, dtype=dtype)
        f32 = lambda n: source.get(n).to(device=device, dtype=torch.float32).contiguous()
        stack = lambda part: torch.stack([get(f"{p}e{e}.{part}{s}") for e in range(self.num_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack(g), stack(u), stack(d)          # [E, F, D], [E, F, D], [E, D, F]
        self.w_router = get(f"{p}router{s}").contiguous()
        self.b_router = self.correction = None
        if self.routing == "softmax_all":
            self.correction = f32(f"{p}correction")
        elif self.router_bias:
            self.b_router = f32(f"{p}router.b")
        self.w_sg = None
        if self.shared is not None:
            self.shared.bind(source, dtype, device)
            if self.shared_gate:
                self.w_sg = get(f"{p}shared.sg{s}").reshape(-1).contiguous()

    def reset_after_fault(self) -> None:
        if self.shared is not None:
            self.shared.reset_after_fault()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        T, D = x.shape
        E, top, F, O = self.num_experts, self.top, self.expert_size, self.outputs
        n = T * top
        dev = x.device
        idx = torch.empty((T, top), dtype=torch.int32, device=dev)
        wt = torch.empty((T, top), dtype=torch.float32, device=dev)
        sgate = torch.empty((T,), dtype=torch.float32, device=dev) if self.w_sg is not None else None
        if self.w_sg is None and self.b_router is None:
            # no bias, no gate vector: the logits are a plain product (float32 sums of the engine's operands), by
            # whichever kernel takes a product of this many tokens; then the choice
            logits = torch.empty((T, O), dtype=torch.float32, device=dev)
            matmul_backend.linear(x, self.w_router, None, logits)
            kernels.moe_choose(logits, top, idx, wt, ROUTINGS[self.routing], self.correction)
        else:
            kernels.moe_route(x, self.w_router, self.b_router, self.w_sg, top, idx, wt, sgate, ROUTINGS[self.routing],
                              self.correction)
        tile_rows = kernels.moe_tile_rows(n, E, D, F, x.dtype)   # rows of one expert a CTA takes
        max_tiles = n // tile_rows + E              # sum over experts of ceil(count / tile_rows) is at most this
        place = torch.empty((n,), dtype=torch.int32, device=dev)
        pair_at = torch.empty((n,), dtype=torch.int32, device=dev)
        meta = torch.empty((O + 2 + 3 * max_tiles,), dtype=torch.int32, device=dev)
        kernels.moe_sort(idx, O, tile_rows, max_tiles, place, pair_at, meta, with_weights=E)
        act_args = dict(num_outputs=O, act=ACTIVATIONS[self.activation], limit=self.limit, alpha=self.alpha,
                        in_scale=wt if self.weigh == "input" else None)
        act = torch.empty((n, F), dtype=x.dtype, device=dev)
        kernels.moe_gemm(x, pair_at, top, True, self.w_gate, self.w_up, act, meta, tile_rows, max_tiles, **act_args)
        y = torch.empty((n, D), dtype=torch.float32, device=dev)
        kernels.moe_gemm(act, pair_at, top, False, self.w_down, None, y, meta, tile_rows, max_tiles, num_outputs=O)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = torch.empty((T, D), dtype=torch.float32, device=dev)
        kernels.moe_combine(y, place, wt if self.weigh == "output" else None, shared, sgate, out,
                            idx=idx if self.identity else None, with_weights=E, h=x if self.identity else None, top=top)
        return out
