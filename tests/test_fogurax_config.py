"""Fogurax's configuration, description, cache layout, position tables and the sizes a stored tensor gives (no GPU)."""
import copy
import math

import pytest
import torch

import fogurax_configs as fc
import plain_fogurax as pf
from qwen_decoder_b200.cache import CacheManager, FixedState, PagedKV
from qwen_decoder_b200.config import ConfigError, config_from_dict, describe_model
from qwen_decoder_b200.parts.model import build_model
from qwen_decoder_b200.parts.rotary import Rotary
from qwen_decoder_b200.weights.loader import TensorSource, WeightError, check_tensors


def test_round_trip_and_description():
    cfg = config_from_dict(fc.FA)
    assert cfg.architecture == "Fogurax" and cfg.vocab_size == 310 and cfg.hidden_size == 96 and cfg.side_dim == 6
    assert cfg.residual_mult == 0.7 and config_from_dict(cfg.to_dict()) == cfg
    spec = describe_model(cfg)
    assert spec.lm_head_tensor is None and len(spec.layers) == 5
    assert [l.block for l in spec.layers] == ["parallel_side"] * 5
    assert [l.mixer.name for l in spec.layers] == ["masked_attention", "side_by_side", "masked_attention",
                                                    "side_by_side", "masked_attention"]
    assert all(list(l.norms) == ["input"] and l.block_params["shared_norm"] for l in spec.layers)   # one norm a layer
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.name == "swiglu"
    assert spec.layers[2].feed_forward.params["weigh"] == "input" and spec.layers[2].feed_forward.params["routing"] == "top_sigmoid"
    assert [l.mixer.params.get("mask") for l in spec.layers] == ["causal", None, "chunk", None, "chunk"]
    assert spec.layers[1].mixer.params["branches"][0]["params"]["mask"] == "window"
    assert len(spec.positions) == 5          # five different rotations
    model = build_model(spec)
    names = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert names["l0.mix.q"] == (6 * 16, 96) and names["l0.mix.k"] == (3 * 16, 96) and names["l0.mix.v"] == (3 * 24, 96)
    assert names["l0.mix.q.b"] == (96,) and names["l0.mix.v.conv"] == (72, 2) and names["l0.mix.g"] == (6, 96)
    assert names["l0.mix.o"] == (96, 6 * 24) and "l0.mix.q.norm" not in names and "l0.mix.g.b" not in names
    assert names["l2.mix.q.norm"] == (64,) and names["l2.mix.k.norm"] == (16,) and "l2.mix.g" not in names
    assert "l2.mix.q.b" not in names and "l2.mix.q.conv" not in names
    assert names["l1.mix.left.q.norm"] == (96,) and names["l1.mix.left.g"] == (4, 96) and names["l1.mix.left.o"] == (96, 64)
    assert names["l1.mix.right.r"] == (40, 96) and names["l1.mix.right.mu.w"] == (96,) and names["l1.mix.right.u"] == (1, 40)
    assert names["l1.mix.right.w1"] == (5, 96) and names["l1.mix.right.w2"] == (40, 5) and names["l1.mix.right.o"] == (96, 40)
    assert names["l2.mlp.router"] == (5, 96) and "l2.mlp.router.b" not in names and "l2.mlp.shared.gate" not in names
    assert names["l3.mlp.shared.down"] == (96, 24) and names["l3.mlp.e3.up"] == (16, 96)
    assert "l0.norm2" not in names and names["l0.norm1"] == (96,) and names["l0.mlp.gate"] == (40, 96)
    assert names["side.embed"] == (310, 5 * 6) and names["l3.side.gate"] == (6, 96) and names["l3.side.proj"] == (96, 6)
    assert names["final.norm"] == (96,) and "lm_head.weight" not in names
    names_b = {s.name for s in build_model(describe_model(config_from_dict(fc.FB))).tensor_specs()}
    assert not any("side" in n for n in names_b) and "l0.mix.q.conv" not in names_b and "l3.mix.q.conv" in names_b


def test_cache_layout_pages_and_state_rows():
    model = build_model(describe_model(config_from_dict(fc.FA)))
    layout = model.cache_layout()
    needs = [g.need for g in layout.groups]
    # the windowed attention's pages go back behind the window; a blocked one keeps its pages
    assert PagedKV(3, 16, None, v_dim=24) in needs and PagedKV(4, 24, 11, v_dim=16) in needs
    assert PagedKV(2, 8, None, v_dim=16) in needs and PagedKV(1, 8, 40, v_dim=8) in needs and len(needs) == 5
    channels0 = 6 * 16 + 3 * 16 + 3 * 24
    assert layout.fixed_needs == [FixedState((1 * channels0,)),                       # two taps: one kept row
                                  FixedState((1 * 40 * 40 + 96,)),                  # a head's matrix and the last input
                                  FixedState((3 * 16 * 16 + 96,))]
    cm = CacheManager(layout, num_pages=8, page_size=16, max_requests=2)
    a = cm.open("a")
    cm.ensure(a, 40)
    cm.commit(a, 40)
    free = dict(zip([g.need for g in layout.groups], cm.free_pages()))
    assert free[PagedKV(3, 16, None, v_dim=24)] == 5 and free[PagedKV(4, 24, 11, v_dim=16)] == 6   # 40 tokens, the last 11
    cm.close(a)
    cm.check()


@pytest.mark.parametrize("scaling", [None, fc.bands(4.0, 1.0, 3.0, 64), fc.bands(6.0, 0.5, 5.0, 2048)])
def test_band_stretched_tables(scaling):
    rot = {"base": 500.0, "dims": 24}
    if scaling:
        rot["scaling"] = scaling
    part = Rotary(head_dim=32, rotary_dim=24, base=500.0, pairing="adjacent",
                  scaling=dict(scaling, kind="bands") if scaling else None)
    part.prepare(300, torch.device("cpu"))
    f = pf.llama3_rates(rot)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(part.cos.double(), torch.cos(ang), atol=1e-6)
    assert torch.allclose(part.sin.double(), torch.sin(ang), atol=1e-6)
    if scaling and scaling["original"] == 64:       # fast pairs stay, the slowest stretch in full, some lie between
        plain = pf.plain_rates(rot)
        assert f[0] == plain[0] and f[-1] == pytest.approx(float(plain[-1]) / scaling["factor"])
        assert any(float(plain[i]) / scaling["factor"] * 1.01 < float(f[i]) < float(plain[i]) * 0.99 for i in range(12))


@pytest.mark.parametrize("scaling", [None, fc.ramp(4.0, 64, 16.0, 2.0)])
def test_ramp_stretched_tables_with_half_split_pairs(scaling):
    rot = {"base": 500.0, "dims": 24}
    if scaling:
        rot["scaling"] = scaling
    part = Rotary(head_dim=32, rotary_dim=24, base=500.0, pairing="half", scaling=scaling)
    part.prepare(100, torch.device("cpu"))
    f, mag = pf.yarn_rates(rot)
    ang = torch.arange(100, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(part.cos.double(), torch.cos(ang) * mag, atol=1e-6)
    assert mag == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0 if scaling else 1.0)


def test_the_decay_rank_is_the_stored_tensors_own():
    """A file that does not name the rank: the tensors' shapes give it, and both tensors must agree."""
    cfg = copy.deepcopy(fc.FA)
    for layer in cfg["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("rank")
    model = build_model(describe_model(config_from_dict(cfg)))
    named = build_model(describe_model(config_from_dict(fc.FA)))
    shapes = {s.name: tuple(s.shape) for s in named.tensor_specs()}
    check_tensors(model.tensor_specs(), shapes)                                # ranks 5 and 9 fit a model that names none
    free = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert free["l1.mix.right.w1"] == (-1, 96) and free["l3.mix.right.w2"] == (48, -1)
    shapes["l1.mix.right.w1"] = (5, 95)
    with pytest.raises(WeightError) as e:
        check_tensors(model.tensor_specs(), shapes)
    assert "l1.mix.right.w1" in str(e.value)


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][2]["mixer"].pop("mask"), "size"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["layers"][1]["mixer"]["right"].pop("heads"), "heads"),
    (lambda c: c["layers"][2]["mlp"]["router"].__setitem__("top", 8), "top"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_errors_name_the_key(edit, word):
    cfg = copy.deepcopy(fc.FA)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)
