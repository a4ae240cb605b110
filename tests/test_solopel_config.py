"""Solopel's configuration, description, order of runs and cache layout (no GPU)."""
import copy

import pytest
import torch

import plain_solopel as ps
import solopel_configs as sc
from qwen_decoder_b200.cache import CacheManager, FixedState, PagedKV, PagedRows
from qwen_decoder_b200.config import ConfigError, config_from_dict, describe_model
from qwen_decoder_b200.parts.model import build_model


def test_round_trip_and_description():
    cfg = config_from_dict(sc.SA)
    assert cfg.architecture == "Solopel" and cfg.vocab_size == 310 and cfg.hidden_size == 96
    assert cfg.canon_taps == 4 and cfg.loop == (1, 3, 2) and cfg.logit_scale == 0.37
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = describe_model(cfg)
    assert spec.lm_head_tensor is None and len(spec.layers) == 6          # five layers and the loop's input step
    assert [l.mixer.name for l in spec.layers[:5]] == ["latent_attention", "diff_attention", "latent_attention",
                                                       "diff_attention", "latent_attention"]
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.name == "mlp"
    assert spec.layers[1].feed_forward.params["top"] == 2 and spec.layers[3].feed_forward.params["shared_size"] == 0
    model = build_model(spec)
    names = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert names["l0.mix.q"] == (3 * 24, 96) and names["l0.mix.uv"] == (3 * 16, 40) and names["l0.mix.dkv.norm"] == (40,)
    assert names["l1.mix.q"] == (6 * 2 * 8, 96) and names["l1.mix.k"] == (2 * 2 * 8, 96) and names["l1.mix.v"] == (2 * 24, 96)
    assert names["l1.mix.k.conv"] == (32, 2) and names["l3.mix.v.conv"] == (32, 4) and names["l1.mix.g"] == (6, 96)
    assert names["l1.mix.lq2"] == (8,) and names["l1.mix.o"] == (96, 6 * 24)
    assert names["l0.canon1"] == (96, 4) and names["l0.rg2.b"] == (96,) and names["l0.mlp.up"] == (136, 96)
    assert "l2.norm2" not in names and "l2.rg2" not in names and "l2.rg1" in names
    assert names["l1.mlp.shared.gate"] == (24, 96) and "l3.mlp.shared.gate" not in names
    assert names["l4.mlp.e5.down"] == (96, 24) and names["l1.mlp.router"] == (5, 96)
    assert names["loop.in"] == (96, 192) and names["loop.step"] == (2, 96) and names["final.norm"] == (96,)
    assert "head" not in names and "lm_head" not in names


def test_the_order_of_runs_follows_the_loop():
    spec = describe_model(config_from_dict(sc.SA))
    runs = [(e.layer, e.visit) for e in spec.schedule]
    n = 5                                                                 # the loop's input step is layer n
    assert runs == [(0, 0), (n, 0), (1, 0), (2, 0), (n, 1), (1, 1), (2, 1), (3, 0), (4, 0)]
    assert [i for i, _ in ps.order_of_runs(sc.SA)] == [l for l, _ in runs if l != n]
    # no loop: every layer once, no tensors of a loop
    spec = describe_model(config_from_dict(sc.SB))
    assert [e.layer for e in spec.schedule] == [0, 1, 2]
    assert not any(s.name.startswith("loop.") for s in build_model(spec).tensor_specs())
    # a loop of one pass still takes the embedding output in once
    one = copy.deepcopy(sc.SB)
    one["loop"] = {"start": 0, "stop": 3, "times": 1}
    spec = describe_model(config_from_dict(one))
    assert [e.layer for e in spec.schedule] == [3, 0, 1, 2]


def test_cache_layout_a_cache_per_pass_and_states_for_the_convolutions():
    model = build_model(describe_model(config_from_dict(sc.SA)))
    layout = model.cache_layout()
    needs = {g.need: len(g.entries) for g in layout.groups}
    # latent rows: layer 0 once (40), layer 2 in both passes (64), layer 4 once (24)
    assert needs[PagedRows(40)] == 1 and needs[PagedRows(64)] == 2 and needs[PagedRows(24)] == 1
    # keys of two maps side by side, values of another size; layer 1 runs twice
    assert needs[PagedKV(2, 16, None, v_dim=24)] == 2 and needs[PagedKV(4, 32, None, v_dim=8)] == 1
    sizes = sorted(f.shape[0] for f in layout.fixed_needs)
    width, taps = 96, 4
    ch1, ch3 = 6 * 16 + 2 * 16 + 2 * 24, 4 * 32 + 4 * 32 + 4 * 8
    want = [3 * width] * 4 + [(2 - 1) * ch1 + 3 * width] * 2 + [(4 - 1) * ch3 + 3 * width]
    assert sizes == sorted(want) and all(f.dtype == torch.float32 for f in layout.fixed_needs)
    cm = CacheManager(layout, num_pages=8, page_size=16, max_requests=2)
    a = cm.open("a")
    cm.ensure(a, 40)
    cm.commit(a, 40)
    assert cm.free_pages() == [5] * len(layout.groups)
    cm.close(a)
    cm.check()
    # two taps in the layers, none or one in the attention: the attention keeps no inputs of its own
    layout = build_model(describe_model(config_from_dict(sc.SB))).cache_layout()
    assert sorted(f.shape[0] for f in layout.fixed_needs) == [72, 72, 72]
    # one tap in the layers: a plain product per channel, no state at all for latent attention
    one = copy.deepcopy(sc.SB)
    one["canon"]["taps"] = 1
    layout = build_model(describe_model(config_from_dict(one))).cache_layout()
    assert layout.fixed_needs == []


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda c: c["loop"].__setitem__("stop", 7), "stop"),
    (lambda c: c.pop("norm"), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_errors_name_the_key(edit, word):
    cfg = copy.deepcopy(sc.SA)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_the_plain_statement_is_causal_and_uses_every_part():
    """The plain statement itself: a later token changes no earlier logits, and every tensor matters."""
    import tempfile
    folder = sc.make_folder(sc.SA, tempfile.mkdtemp(), seed=3)
    cfg, w = sc.read_folder(folder)
    seq = [5, 9, 200, 17, 3, 99, 41, 250, 8, 8, 61]
    base = ps.forward(cfg, w, seq)
    other = ps.forward(cfg, w, seq[:-1] + [7])
    assert torch.equal(base[:-1], other[:-1]) and not torch.equal(base[-1], other[-1])
    for name in sorted(w):
        if ".mlp.e" in name:
            continue                              # an expert that no token of this short sequence chose
        changed = dict(w)
        changed[name] = w[name] + 0.25
        assert not torch.allclose(ps.forward(cfg, changed, seq), base, atol=1e-9), name


def test_the_benchmark_models_describe():
    """``bench.py --micro solopel``: both sizes parse, unroll to eight layer runs beside a model of eight layers, and
    keep a cache and a state row per run."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
    import bench
    from qwen_decoder_b200.config import describe_model
    for size in ("S", "M"):
        solopel, other = bench.solopel_configs(size)
        spec = describe_model(solopel)
        runs = [e for e in spec.schedule if spec.layers[e.layer].block == "pre_norm_gated"]
        assert len(runs) == 8 == len(describe_model(other).schedule)
        assert sum(spec.layers[e.layer].block == "loop_input" for e in spec.schedule) == 2
    assert len(bench.solopel_configs("S", layers=2)[0].layers) == 2
