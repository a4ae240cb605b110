"""``Fogurax``: a decoder whose ``config.json`` lists its layers one by one.

A layer has ONE norm (RMS, plain weight) whose output both branches read, x += m (mixer(h) + ff(h)) with
h = norm1(x) and m = ``residual_mult``; then a per-layer token input joins: the layer's slice e of the token's row of
one side table gates a small projection of the new x, y = Wp (gelu(Wg x) * e), and x += m y / rms(y) * ws.
Three mixers:

* ``attention``: grouped-query attention with biases on q, k and v, a short causal convolution over ``conv`` tokens
  on every channel of q, k and v right after the projection, rotary positions on the first ``rot.dims`` elements of
  a head in adjacent pairs (rates stretched band by band by ``rot.scaling`` = factor, low, high, original), q and k
  then divided by their root mean square per head (no weight), all earlier keys visible, a per-head sigmoid gate on
  the output;
* ``attention_2``: no biases, q and k normed over the whole projection with weights before the rotation, half-split
  pairs (rates blended by a ramp, ``rot.scaling`` = factor, original, fast, slow, cosines and sines scaled), a query
  sees the keys of its own block of ``mask.size`` positions, no gate;
* ``parallel``: ``left_scale`` * left + ``right_scale`` * right on the same input: left is attention with the
  whole-projection norms, adjacent pairs at plain rates, the last ``mask.size`` keys visible and the output gate;
  right is the recurrent mixer with a matrix state per head (``parts/time_mix.py``).

Feed-forwards: dense gated (silu), or routed experts whose scores are sigmoids of the router's logits, the ``top``
largest chosen, not renormalised, multiplying the expert's input, plus a shared expert; or none.  The output matrix is
the embedding table.

Keys read from ``config.json``: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``residual_mult`` (optional, 1),
``token_side.dim`` (absent or null: no token input), ``layers[i].type`` / ``.mixer`` / ``.mlp`` (and, optional,
``max_positions``, ``eos_token_id`` and, in the recurrent mixer, ``rank``: the rank of the decay's low-rank product,
which otherwise is whatever the stored tensors ``w1`` [rank, width] and ``w2`` have).  Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.side.gate|proj|norm``, ``final.norm``; linear weights are [out, in] with no suffix, biases
``<tensor>.b``.  The numbers inside gelu are the design's and stand in code.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Tuple

from .model_config import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .veterax import DEFAULT_MAX_POSITIONS, _need

MIXERS = ("attention", "attention_2", "parallel")


def _check_rot(rot, dim: int, where: str, scaling_keys) -> None:
    if rot is None:
        return
    dims = _need(rot, "dims", where)
    if _need(rot, "base", where, float) <= 0:
        raise ConfigError(f"config.json: {where}.base must be positive")
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.dims ({dims}) must be even and at most dim ({dim})")
    sc = rot.get("scaling")
    if sc is not None:
        if scaling_keys is None:
            raise ConfigError(f"config.json: {where}.scaling: this mixer's rotation has no scaling")
        for k in scaling_keys:
            if _need(sc, k, f"{where}.scaling", float) <= 0:
                raise ConfigError(f"config.json: {where}.scaling.{k} must be positive")
        if "low" in scaling_keys and float(sc["low"]) == float(sc["high"]):
            raise ConfigError(f"config.json: {where}.scaling.low and .high must differ")


def _check_attention(m, where: str, masked: bool, scaling_keys) -> None:
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _need(m, k, where)
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.kv_heads ({m['kv_heads']}) must divide heads ({m['heads']})")
    if m["dim"] % 2:
        raise ConfigError(f"config.json: {where}.dim ({m['dim']}) must be even")
    _need(m, "scale", where, float)
    _check_rot(m.get("rot"), m["dim"], f"{where}.rot", scaling_keys)
    if masked:
        _need(m.get("mask"), "size", f"{where}.mask")
    conv = m.get("conv")
    if conv is not None and (isinstance(conv, bool) or not isinstance(conv, int) or conv < 0):
        raise ConfigError(f"config.json: {where}.conv must be a non-negative integer, got {conv!r}")


def _check_layer(i: int, layer) -> None:
    where = f"layers[{i}]"
    kind = layer.get("type") if isinstance(layer, Mapping) else None
    if kind not in MIXERS:
        raise ConfigError(f"config.json: {where}.type must be one of {MIXERS}, got {kind!r}")
    m = layer.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"config.json: {where}: required key 'mixer' is missing")
    if kind == "attention":
        _check_attention(m, f"{where}.mixer", False, ("factor", "low", "high", "original"))
    elif kind == "attention_2":
        _check_attention(m, f"{where}.mixer", True, ("factor", "original", "fast", "slow"))
    else:
        _check_attention(m.get("left"), f"{where}.mixer.left", True, None)
        for k in ("heads", "dim"):
            _need(m.get("right"), k, f"{where}.mixer.right")
        if m["right"]["dim"] > 256:
            raise ConfigError(f"config.json: {where}.mixer.right.dim must be at most 256")
        for k in ("left_scale", "right_scale"):
            _need(m, k, f"{where}.mixer", float)
    f = layer.get("mlp")
    if f is None:
        return
    fk = f.get("kind") if isinstance(f, Mapping) else None
    if fk == "dense":
        _need(f, "ff", f"{where}.mlp")
    elif fk == "moe":
        _need(f.get("expert"), "ff", f"{where}.mlp.expert")
        e = _need(f.get("router"), "experts", f"{where}.mlp.router")
        top = _need(f.get("router"), "top", f"{where}.mlp.router")
        if top > e:
            raise ConfigError(f"config.json: {where}.mlp.router.top ({top}) exceeds experts ({e})")
        if f.get("shared"):
            _need(f["shared"], "ff", f"{where}.mlp.shared")
    else:
        raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' or 'moe', got {fk!r}")


@dataclass(frozen=True)
class FoguraxConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    residual_mult: float
    side_dim: int                       # 0: no per-layer token input
    layers: Tuple[dict, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FoguraxConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, layer in enumerate(layers):
            _check_layer(i, layer)
        eps = _need(d.get("norm"), "eps", "norm", float)
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        mult = d.get("residual_mult")
        mult = 1.0 if mult is None else _need(d, "residual_mult", "config", float)
        side = d.get("token_side")
        side_dim = _need(side, "dim", "token_side") if side else 0
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        return cls(architecture=d.get("architecture") or d["architectures"][0],
                   vocab_size=_need(d, "vocab", "config"), hidden_size=_need(d, "width", "config"), norm_eps=eps,
                   residual_mult=mult, side_dim=side_dim, layers=tuple(copy.deepcopy(layer) for layer in layers),
                   max_position_embeddings=d.get("max_positions") or DEFAULT_MAX_POSITIONS, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
             "token_side": {"dim": self.side_dim} if self.side_dim else None,
             "layers": [copy.deepcopy(layer) for layer in self.layers]}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def _position(positions: dict, m: Mapping, pairing: str, scaling_kind) -> str:
    """The name under which the model keeps this mixer's rotation tables (mixers with equal rotations share them)."""
    rot = m.get("rot")
    if rot is None:
        return None
    sc = rot.get("scaling") if scaling_kind else None
    name = f"rot{rot['dims']}of{m['dim']}b{rot['base']!r}{pairing}" + \
        (f"{scaling_kind}" + "/".join(f"{k}={sc[k]!r}" for k in sorted(sc)) if sc else "")
    positions.setdefault(name, PartSpec("rotary", {
        "head_dim": m["dim"], "rotary_dim": rot["dims"], "base": rot["base"], "pairing": pairing,
        "scaling": dict(sc, kind=scaling_kind) if sc else None}))
    return name


def _attention_params(D: int, eps: float, m: Mapping, position, **options) -> dict:
    p = {"hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
         "v_dim": m["vdim"], "scale": m["scale"], "eps": eps, "position": position, "prefix": "mix.",
         "weight_suffix": ""}
    p.update(options)
    return p


def describe_fogurax(cfg: FoguraxConfig) -> ModelSpec:
    D, eps, L = cfg.hidden_size, cfg.norm_eps, len(cfg.layers)
    positions, layers = {}, []
    for i, layer in enumerate(cfg.layers):
        m, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            mixer = PartSpec("masked_attention", _attention_params(
                D, eps, m, _position(positions, m, "adjacent", "bands"), bias=True, conv_taps=m.get("conv") or 0,
                qk_norm="head", norm_after_rotation=True, mask="causal", output_gate=True))
        elif kind == "attention_2":
            mixer = PartSpec("masked_attention", _attention_params(
                D, eps, m, _position(positions, m, "half", "ramp"), qk_norm="whole", mask="chunk",
                mask_size=m["mask"]["size"], output_gate=False))
        else:
            left, right = m["left"], m["right"]
            lp = _attention_params(D, eps, left, _position(positions, left, "adjacent", None), qk_norm="whole",
                                   mask="window", mask_size=left["mask"]["size"], output_gate=True, prefix="left.")
            # the rank of the decay's low-rank product is the stored tensors' own, unless the file names one
            rp = {"hidden_size": D, "num_heads": right["heads"], "head_dim": right["dim"],
                  "decay_rank": right.get("rank"), "eps": eps, "prefix": "right.", "weight_suffix": ""}
            mixer = PartSpec("side_by_side", {"hidden_size": D, "prefix": "mix.", "weight_suffix": "", "branches": [
                {"name": "masked_attention", "params": lp, "scale": m["left_scale"]},
                {"name": "time_mix", "params": rp, "scale": m["right_scale"]}]})
        f = layer.get("mlp")
        if f is None:
            ff = None
        elif f["kind"] == "dense":
            ff = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": f["ff"], "prefix": "mlp.",
                                     "names": ("gate", "up", "down"), "weight_suffix": ""})
        else:
            shared = f.get("shared")
            ff = PartSpec("moe", {"hidden_size": D, "expert_size": f["expert"]["ff"],
                                  "num_experts": f["router"]["experts"], "top": f["router"]["top"],
                                  "shared_size": shared["ff"] if shared else 0, "routing": "top_sigmoid",
                                  "router_bias": False, "weigh": "input", "shared_gate": False, "prefix": "mlp.",
                                  "weight_suffix": ""})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block="parallel_side", mixer=mixer, feed_forward=ff,
            norms={"input": PartSpec("rmsnorm", {"size": D, "eps": eps, "tensor": "norm1"})},
            block_params={"size": D, "eps": eps, "side_dim": cfg.side_dim, "side_index": i, "side_table": "side.embed",
                          "side_table_shape": (cfg.vocab_size, L * cfg.side_dim), "prefix": "", "shared_norm": True,
                          "mult": cfg.residual_mult}))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding_tensor="embed", positions=positions, layers=layers,
        schedule=[ScheduleEntry(layer=i) for i in range(len(layers))],
        final_norm=PartSpec("rmsnorm", {"size": D, "eps": eps, "tensor": "norm"}), final_norm_prefix="final.",
        lm_head_tensor=None)


register_architecture("Fogurax", FoguraxConfig, describe_fogurax)
