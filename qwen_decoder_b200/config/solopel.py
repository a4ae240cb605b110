"""``Solopel``: a decoder whose ``config.json`` lists its layers one by one and runs a stretch of them several times.

A layer is pre-norm with gated branches: h = norm(x); x += sigmoid(Wg h + b) * branch(h), first the mixer and then
the feed-forward, with RMS norms whose scales are stored around zero (the norm multiplies by 1 + w).  The mixer reads
h + conv(h), a short causal convolution over ``canon.taps`` tokens per channel.  Mixers: ``latent_attention``
(keys and values of all heads expanded from one cached low-rank row per token; here without a query latent, without
positions and without an output gate) and ``attention`` (differential grouped-query attention: two softmax maps per
head over the same values, a short convolution on q, k and v, capped scores, a unit norm per head and a gate per
head).  Feed-forwards: dense ungated with the tanh form of gelu, or routed experts (the ``top`` largest sigmoid
scores, not renormalised, multiplying each expert's INPUT) with an optional shared expert, or none.  ``loop`` =
{start, stop, times}: layers start .. stop - 1 run ``times`` times in a row with the same weights and a cache of
their own per pass; before every pass x <- Win [x ; embedding output] + step[pass].  The output matrix is the
embedding table and the logits are multiplied by ``logit_scale``.

Keys read from ``config.json``: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` (optional: no
input convolution), ``loop`` (optional), ``logit_scale`` (optional, 1), ``layers[i].type`` / ``.mixer`` / ``.mlp``,
and, optional, ``max_positions`` and ``eos_token_id``.  Tensor names: ``embed``, ``loop.in``, ``loop.step``,
``l<i>.norm1|norm2|canon1|rg1|rg1.b|rg2|rg2.b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``; linear weights are
[out, in] with no suffix.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DEFAULT_MAX_POSITIONS = 1 << 17        # the design has no position limit of its own: the engine's, unless 'max_positions' says otherwise

_MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "vdim", "kv_rank"),
    "attention": ("heads", "kv_heads", "dim", "vdim"),
}


def _need(d, key: str, where: str, kind=int):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where}: required key '{key}' is missing")
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
        return v
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _count(d: Mapping[str, Any], key: str, where: str) -> int:
    """An optional non-negative integer (absent or null: 0)."""
    v = d.get(key)
    if v is None:
        return 0
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {where}.{key} must be a non-negative integer, got {v!r}")
    return v


def _check_layer(i: int, layer: Mapping[str, Any]) -> None:
    where = f"layers[{i}]"
    kind = layer.get("type") if isinstance(layer, Mapping) else None
    if kind not in _MIXER_KEYS:
        raise ConfigError(f"config.json: {where}.type must be one of {sorted(_MIXER_KEYS)}, got {kind!r}")
    m = layer.get("mixer")
    for k in _MIXER_KEYS[kind]:
        _need(m, k, f"{where}.mixer")
    _need(m, "scale", f"{where}.mixer", float)
    if kind == "attention":
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"config.json: {where}.mixer.kv_heads must divide heads")
        _need(m, "diff", f"{where}.mixer", float)
        _count(m, "conv", f"{where}.mixer")
        cap = m.get("softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
            raise ConfigError(f"config.json: {where}.mixer.softcap must be a non-negative number, got {cap!r}")
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
        if f.get("shared"):                     # absent, null or empty: no shared expert
            _need(f["shared"], "ff", f"{where}.mlp.shared")
    else:
        raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' or 'moe', got {fk!r}")


@dataclass(frozen=True)
class SolopelConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[dict, ...]
    canon_taps: int = 0                         # 0: the mixers read their input as it is
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    logit_scale: float = 1.0
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SolopelConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, layer in enumerate(layers):
            _check_layer(i, layer)
        eps = _need(d.get("norm"), "eps", "norm", float)
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        canon = d.get("canon")
        taps = _count(canon, "taps", "canon") if isinstance(canon, Mapping) else 0
        lp, loop = d.get("loop"), None
        if lp:
            start, stop = _count(lp, "start", "loop"), _need(lp, "stop", "loop")
            times = _need(lp, "times", "loop")
            if not (start < stop <= len(layers)):
                raise ConfigError(f"config.json: loop: start ({start}) < stop ({stop}) <= layers ({len(layers)}) must hold")
            loop = (start, stop, times)
        scale = d.get("logit_scale")
        scale = 1.0 if scale is None else _need(d, "logit_scale", "config", float)
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        return cls(architecture=d.get("architecture") or d["architectures"][0],
                   vocab_size=_need(d, "vocab", "config"), hidden_size=_need(d, "width", "config"), norm_eps=eps,
                   layers=tuple(copy.deepcopy(layer) for layer in layers), canon_taps=taps, loop=loop,
                   logit_scale=scale, max_position_embeddings=d.get("max_positions") or DEFAULT_MAX_POSITIONS,
                   eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale,
             "layers": [copy.deepcopy(layer) for layer in self.layers]}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.loop:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def describe_solopel(cfg: SolopelConfig) -> ModelSpec:
    D, eps = cfg.hidden_size, cfg.norm_eps
    norm = {"size": D, "eps": eps, "offset": 1.0}
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "num_heads": m["heads"], "nope_dim": m["dim"], "rope_dim": 0, "v_dim": m["vdim"],
                "q_rank": 0, "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps, "position": None,
                "output_gate": False, "prefix": "mix.", "weight_suffix": ""})
        else:
            mixer = PartSpec("diff_attention", {
                "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_dim": m["vdim"], "scale": m["scale"], "diff": m["diff"], "eps": eps,
                "softcap": m.get("softcap") or 0.0, "conv_taps": m.get("conv") or 0, "output_gate": True,
                "prefix": "mix.", "weight_suffix": ""})
        f = layer.get("mlp")
        if f is None:
            ff = None
        elif f["kind"] == "dense":
            ff = PartSpec("mlp", {"hidden_size": D, "intermediate_size": f["ff"], "prefix": "mlp.",
                                  "names": ("up", "down"), "weight_suffix": "", "activation": "gelu_tanh"})
        else:
            shared = f.get("shared")
            ff = PartSpec("moe", {"hidden_size": D, "expert_size": f["expert"]["ff"],
                                  "num_experts": f["router"]["experts"], "top": f["router"]["top"],
                                  "shared_size": shared["ff"] if shared else 0, "routing": "top_sigmoid",
                                  "router_bias": False, "weigh": "input", "shared_gate": False, "prefix": "mlp.",
                                  "weight_suffix": ""})
        norms = {"input": PartSpec("rmsnorm", dict(norm, tensor="norm1"))}
        if ff is not None:
            norms["post_mixer"] = PartSpec("rmsnorm", dict(norm, tensor="norm2"))
        layers.append(LayerSpec(prefix=f"l{i}.", block="pre_norm_gated", mixer=mixer, feed_forward=ff, norms=norms,
                                block_params={"size": D, "taps": cfg.canon_taps, "prefix": ""}))
    n = len(layers)
    if cfg.loop:
        start, stop, times = cfg.loop
        layers.append(LayerSpec(prefix="", block="loop_input", mixer=None, feed_forward=None, norms={},
                                block_params={"size": D, "passes": times, "prefix": ""}))
        schedule = [ScheduleEntry(layer=i) for i in range(start)]
        for t in range(times):
            schedule.append(ScheduleEntry(layer=n, visit=t))
            schedule += [ScheduleEntry(layer=i, visit=t) for i in range(start, stop)]
        schedule += [ScheduleEntry(layer=i) for i in range(stop, n)]
    else:
        schedule = [ScheduleEntry(layer=i) for i in range(n)]
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding_tensor="embed", positions={}, layers=layers, schedule=schedule,
        final_norm=PartSpec("rmsnorm", dict(norm, tensor="norm", gain=cfg.logit_scale)), final_norm_prefix="final.",
        lm_head_tensor=None)


register_architecture("Solopel", SolopelConfig, describe_solopel)
