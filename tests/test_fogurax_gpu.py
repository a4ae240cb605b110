"""Fogurax in the engine against its plain float64 statement (``plain_fogurax``): each mechanism alone, every way of
cutting the work, batches, pages and state slots used again, keys far away and at the edges of windows, blocks, pages
and key tiles, the first tokens, long decoding, generation."""
import copy
import random

import numpy as np
import pytest
import torch

import fogurax_configs as fc
import plain_fogurax as pf
import trace_tools

pytestmark = pytest.mark.gpu

# max |logit difference| relative to the largest |logit|
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
# bfloat16: queries and keys are divided by their own length, so a token whose projection is short by cancellation
# carries the rounding of the projection's input many times over; one row in fifty may reach three times the
# tolerance (a lost key, a wrong page or a lost state moves most rows by far more).  float32: none.
STRAY = {"float32": 0.0, "bfloat16": 0.02}
# The recurrent mixer divides every head's output by its own root mean square: where a head's output is short by
# cancellation (one token in a few hundred) the rounding of the bfloat16 projections before it weighs many times as
# much; float32 shows the same places at 20 times its median error, still far inside its tolerance.
STRAY_FACTOR = 4.0
LENGTHS = {"A": [1, 2, 15, 16, 17, 33, 63, 64, 65, 150], "B": [3, 31, 32, 48, 97, 129, 210]}


def expected(cfg, w, seqs):
    return [pf.forward(cfg, w, s).numpy() for s in seqs]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> folder, config, weights, sequences, expected logits.  The bfloat16 runs get the same
    weights with routers that no rounding can flip (``fogurax_configs.steady_routing``)."""
    out = {}
    for i, (name, cfg) in enumerate(fc.CONFIGS.items()):
        rng = random.Random(900 + i)
        seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in LENGTHS[name]]
        for dtype, edit in (("float32", None), ("bfloat16", fc.steady_routing)):
            folder = fc.make_folder(cfg, str(tmp_path_factory.mktemp(f"f{name}{dtype}")), seed=83 + i, edit=edit)
            cfg_read, w = fc.read_folder(folder)
            out[name, dtype] = (folder, cfg_read, w, seqs, expected(cfg_read, w, seqs))
    return out


def make_runner(folder, dtype, max_tokens, page_size=16, max_requests=4, **kw):
    from qwen_decoder_b200.engine import ModelRunner
    pages = (max_tokens + page_size - 1) // page_size
    return ModelRunner.from_folder(folder, dtype=dtype, device="cuda:0", num_pages=pages, page_size=page_size,
                                   max_requests=max_requests, max_positions=pages * page_size, **kw)


def held(seqs):
    return max((len(s) + 63) // 64 * 64 for s in seqs)


def all_free(runner):
    runner.cache.check()
    assert runner.cache.free_pages() == [runner.cache.num_pages] * len(runner.cache.pools)


def run_all_ways(folder, dtype, seqs, want, tmp_path, max_tokens=128, tail=20, sizes=(7, 2, 24, 3, 2, 16, 5, 2, 31, 2),
                 stray=None, **kw):
    stray = STRAY[dtype] if stray is None else stray
    runner = make_runner(folder, dtype, max_tokens, **kw)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.portions(seqs, sizes=sizes),
                            trace_tools.decode_tail(seqs, tail=tail))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=stray, stray_factor=STRAY_FACTOR)
    all_free(runner)


SMALL = fc.attn(2, 1, 8, 8, conv=0)
ONE_LAYER = {
    # name: (mixer, feed-forward, token input, width, multiplier)
    "attention_four_taps": (fc.attn(4, 2, 16, 24, conv=4, scale=0.4), None, 0, 64, 0.6),
    "attention_three_taps_part_rotated_stretched": (
        fc.attn(2, 2, 24, 8, conv=3, rot_dims=10, base=37.0, scaling=fc.bands(3.0, 0.5, 4.0, 16)), None, 0, 64, 1.0),
    "attention_no_convolution_one_kv_head": (fc.attn(12, 1, 8, 16, conv=0), None, 0, 56, 0.25),
    "attention_wide_heads": (fc.attn(2, 1, 128, 128, conv=2, scale=0.05), None, 0, 64, 0.6),
    "attention_odd_pieces": (fc.attn(3, 3, 10, 6, conv=5, rot_dims=6), None, 0, 64, 0.6),
    "attention_many_heads_per_group": (fc.attn(40, 2, 8, 8, conv=2), None, 0, 64, 0.6),
    "blocks_of_five": (fc.attn2(4, 2, 16, 24, 5, scaling=fc.ramp(3.0, 16, 4.0, 0.5)), None, 0, 64, 0.6),
    "blocks_of_a_page": (fc.attn2(2, 2, 24, 8, 16, rot_dims=12, base=50.0), None, 0, 64, 0.6),
    "blocks_of_sixty_four_wide_heads": (fc.attn2(2, 1, 128, 64, 64, scaling=fc.ramp(8.0, 32, 8.0, 1.0), scale=0.06), None, 0, 64, 0.6),
    "blocks_longer_than_the_prompt": (fc.attn2(6, 3, 8, 8, 1000, rot_dims=4), None, 0, 48, 0.6),
    "window_of_one": (fc.par(2, 2, 8, 8, 1, 2, 8, 4), None, 0, 64, 0.6),
    "window_of_seven": (fc.par(4, 2, 16, 24, 7, 1, 16, 3, left_scale=1.5, right_scale=0.5, rot_dims=8), None, 0, 64, 0.6),
    "window_of_thirty_three": (fc.par(3, 1, 24, 8, 33, 3, 24, 7, left_scale=0.7, right_scale=1.4), None, 0, 72, 1.0),
    "window_past_the_prompt_recurrent_heads_of_64": (fc.par(2, 2, 64, 64, 500, 3, 64, 12), None, 0, 64, 0.6),
    "recurrent_head_of_136": (fc.par(2, 1, 8, 8, 20, 1, 136, 2, left_scale=0.1, right_scale=2.0), None, 0, 40, 0.6),
    "dense": (SMALL, fc.dense(88), 0, 64, 0.6),
    "token_input": (SMALL, None, 12, 64, 0.6),
    "token_input_of_one": (SMALL, fc.dense(24), 1, 72, 2.0),
    "experts": (SMALL, fc.moe(7, 3, 24), 0, 64, 0.6),
    "experts_one_of_many_and_shared": (SMALL, fc.moe(9, 1, 40, shared=56), 0, 64, 0.6),
    "experts_all_chosen": (SMALL, fc.moe(3, 3, 16, shared=8), 5, 64, 1.0),
    "a_width_of_no_whole_16_byte_rows": (fc.attn(3, 1, 12, 20, conv=2), fc.dense(50), 3, 100, 0.6),
    "all_of_it_on_a_narrow_width": (fc.par(2, 1, 16, 8, 9, 2, 8, 3, left_scale=0.9, right_scale=1.1), fc.moe(3, 2, 12, shared=20), 2, 36, 0.8),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_each_mechanism_alone(name, dtype, tmp_path):
    """One layer: one mixer with no feed-forward, or a small attention with one kind of feed-forward or the token
    input: a prompt at once, in portions, and its tail token by token."""
    mix, mlp, side, width, mult = ONE_LAYER[name]
    cfg = fc.one_layer(mix, mlp, width=width, side=side, mult=mult)
    folder = fc.make_folder(cfg, str(tmp_path / "m"), seed=sum(map(ord, name)), std=0.15,
                            edit=fc.steady_routing if dtype == "bfloat16" else None)
    cfg, w = fc.read_folder(folder)
    rng = random.Random(len(name))
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 2, 37, 90)]
    run_all_ways(folder, dtype, seqs, expected(cfg, w, seqs), tmp_path)


def test_the_experts_chosen_are_the_statements(tmp_path):
    """float32, random routers: the logits agree only if every token took the statement's experts; the statement
    itself moves by far more than the tolerance when one choice changes."""
    cfg = fc.one_layer(SMALL, fc.moe(6, 2, 24, shared=16), width=64)
    folder = fc.make_folder(cfg, str(tmp_path / "m"), seed=21, std=0.2)
    cfg, w = fc.read_folder(folder)
    rng = random.Random(5)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(80)]]
    want = expected(cfg, w, seqs)
    chosen = []
    pf.forward(cfg, w, seqs[0], chosen_out=chosen)
    assert len({tuple(sorted(r)) for r in chosen[0].tolist()}) > 4          # the choice depends on the token
    w2 = dict(w, **{"l0.mlp.router": torch.roll(w["l0.mlp.router"], 1, dims=0)})
    assert np.abs(pf.forward(cfg, w2, seqs[0]).numpy() - want[0]).max() > 0.02 * np.abs(want[0]).max()
    run_all_ways(folder, "float32", seqs, want, tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_and_decode_tail(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs), page_size=32 if name == "B" else 16)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=40))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_down_to_two_tokens(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs), page_size=16 if name == "B" else 24)     # 24: no divisor of a key tile
    for k, sizes in enumerate(((7, 2, 24, 3, 2, 16, 5, 2, 31, 2), (2,), (64, 1, 3), (1, 1, 2, 1))):
        tr = trace_tools.portions(seqs, sizes=sizes)
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype, tmp_path):
    """Unequal requests side by side, portions beside single tokens, in a pool of about two of the longest with three
    state slots: every page and every slot serves several requests in turn.  A key read from a page's former owner, a
    recurrent state or a convolution's kept inputs left over from a slot's former owner show against the statement."""
    folder, cfg, w, seqs, want = models[name, dtype]
    seqs2, want2 = seqs + seqs[::-1], want + want[::-1]
    max_tokens = 2 * held(seqs)
    runner = make_runner(folder, dtype, max_tokens, max_requests=3)
    tr = trace_tools.mixed(seqs2, max_tokens, seed=11, max_live=3)
    assert sum(len(s["entries"]) > 1 for s in tr.steps) > 5
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want2, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    all_free(runner)


def test_a_request_alone_and_in_a_batch_agree(models, tmp_path):
    """float32: the same rows from a batch of unequal requests and from each request alone differ by rounding
    of sums at most (far less than from the plain statement)."""
    folder, cfg, w, seqs, want = models["A", "float32"]
    runner = make_runner(folder, "float32", 4 * held(seqs))
    a = trace_tools.whole(seqs)
    ga = trace_tools.run_inprocess(runner, a, str(tmp_path / "a"))
    b = trace_tools.mixed(seqs, 4 * held(seqs), seed=3, max_live=4)
    gb = trace_tools.run_inprocess(runner, b, str(tmp_path / "b"))
    rows_a = {rp: ga[s][i] for s, rows in a.expect.items() for i, rp in enumerate(rows)}
    rows_b = {rp: gb[s][i] for s, rows in b.expect.items() for i, rp in enumerate(rows)}
    scale = max(float(np.abs(x).max()) for x in want)
    assert max(float(np.abs(rows_a[k] - rows_b[k]).max()) for k in rows_b) <= 3e-6 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_and_first_tokens(models, name, dtype, tmp_path):
    """Two tokens of prompt, then 300 tokens one by one across many pages, windows, blocks and key tiles: the windows
    pass over decoded tokens, pages behind them are given back, the recurrent state is carried 300 times; the first
    positions are compared one by one."""
    folder, cfg, w, _, _ = models[name, dtype]
    rng = random.Random(77)
    seq = [rng.randrange(cfg["vocab"]) for _ in range(302)]
    want = expected(cfg, w, [seq])
    runner = make_runner(folder, dtype, 320)
    tr = trace_tools.decode_tail([seq], tail=300)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    all_free(runner)


def _sharp(mix_kind, dtype):
    """One-layer models whose attention picks single keys: the query side is scaled up so that the statement's softmax
    puts most of its weight on one key.  A key that is lost, one position off, just inside or outside an edge, read
    from the wrong row of a page or turned by the wrong angle then moves the logits by far more than the tolerance."""
    f = 1.0 if dtype == "float32" else 0.45
    if mix_kind == "attention":        # unit-normed q and k: the scale alone sets the sharpness
        return fc.one_layer(fc.attn(4, 2, 16, 40, conv=3, base=200.0, scaling=fc.bands(4.0, 0.5, 3.0, 64), scale=2.2 * f),
                            None, vocab=400, width=48), None
    if mix_kind == "attention_2":
        cfg = fc.one_layer(fc.attn2(4, 2, 16, 40, 96, base=200.0, scaling=fc.ramp(4.0, 64, 16.0, 2.0), scale=1.0),
                           None, vocab=400, width=48)
        name = "l0.mix.q.norm"
    else:
        cfg = fc.one_layer(fc.par(4, 2, 16, 40, 130, 2, 16, 4, left_scale=1.5, right_scale=0.2, base=200.0, scale=1.0),
                           None, vocab=400, width=48)
        name = "l0.mix.left.q.norm"

    def sharpen(t):
        t[name] = (t[name].float() * 2.0 * f).to(torch.bfloat16)
    return cfg, sharpen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "attention_2", "parallel"])
def test_single_keys_far_back_and_at_the_edges(kind, dtype, tmp_path):
    """Hundreds of keys of which one matters, for each kind of mask: prompts that end just before, at and just after
    page, key-tile, window and block borders, their tails decoded token by token.  The statement itself is shown to
    depend on the edge: with a window or block one position longer its logits move by far more than the tolerance."""
    cfg, edit = _sharp(kind, dtype)
    folder = fc.make_folder(cfg, str(tmp_path / "m"), seed=5, std=0.2, edit=edit)
    cfg, w = fc.read_folder(folder)
    rng = random.Random(8)
    lengths = {"attention": (255, 256, 257, 400), "attention_2": (95, 96, 97, 193, 400), "parallel": (129, 130, 131, 400)}[kind]
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in lengths]
    want = expected(cfg, w, seqs)
    scale = max(float(np.abs(x).max()) for x in want)
    if kind != "attention":
        other = copy.deepcopy(cfg)
        m = other["layers"][0]["mixer"]
        (m if kind == "attention_2" else m["left"])["mask"]["size"] += 1
        moved = np.abs(pf.forward(other, w, seqs[-1]).numpy() - want[-1]).max(axis=-1)
        assert (moved > 3 * TOL["float32"] * scale).mean() > 0.1     # far above what the float32 run allows
    else:                               # a key more than a hundred positions back carries weight
        gone = dict(w)
        emb = w["embed"].clone()
        emb[seqs[-1][150]] = emb[seqs[-1][151]]
        gone["embed"] = emb
        moved = np.abs(pf.forward(cfg, gone, seqs[-1]).numpy()[300:] - want[-1][300:]).max(axis=-1)
        assert (moved > 3 * TOL["float32"] * scale).mean() > 0.1
    runner = make_runner(folder, dtype, 512)
    for i, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=36),
                            trace_tools.portions(seqs, sizes=(100, 2, 3, 64)))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{i}"))
        trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_over_a_long_context(dtype, tmp_path):
    """A thousand keys behind each decoded token of the convolved attention: its keys are shared among many CTAs whose
    partial results (values of a size that is no multiple of a warp) are added up and gated; alone and side by side."""
    cfg = fc.one_layer(fc.attn(4, 2, 32, 40, conv=4, base=5000.0, scale=0.9), fc.moe(3, 2, 16), vocab=150, width=64)
    folder = fc.make_folder(cfg, str(tmp_path / "m"), seed=12, std=0.15, edit=fc.steady_routing if dtype == "bfloat16" else None)
    cfg, w = fc.read_folder(folder)
    rng = random.Random(2)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1030, 1093)]
    want = [{p: row for p, row in enumerate(x) if p >= 940} for x in expected(cfg, w, seqs)]
    runner = make_runner(folder, dtype, 2304, page_size=32)
    tr = trace_tools.decode_tail(seqs, tail=70, keep=lambda r, p: p >= 940)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path / "o"))
    trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    tr = trace_tools.Trace()
    n0 = 1000
    tr.add([(r, 0, s[:n0], []) for r, s in enumerate(seqs)])
    for p in range(n0, 1030):
        tr.add([(r, p, s[p:p + 1], [0]) for r, s in enumerate(seqs)], end=[0, 1] if p == 1029 else [])
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path / "p"))
    trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    all_free(runner)


def test_the_tensor_core_kernel_and_the_float32_kernel_agree(models, tmp_path, monkeypatch):
    """bfloat16: the same model through the tensor-core attention and through the float32-arithmetic kernel."""
    from qwen_decoder_b200.parts import masked_attention
    folder, cfg, w, seqs, want = models["A", "bfloat16"]
    outs = []
    for on in (True, False):
        monkeypatch.setattr(masked_attention, "_TENSOR_CORES", on)
        runner = make_runner(folder, "bfloat16", held(seqs))
        tr = trace_tools.decode_tail(seqs, tail=10)
        outs.append(trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{on}")))
        trace_tools.compare(tr, outs[-1], want, TOL["bfloat16"], stray=STRAY["bfloat16"], stray_factor=STRAY_FACTOR)
    scale = max(float(np.abs(x).max()) for x in want)
    assert max(float(np.abs(outs[0][s] - outs[1][s]).max()) for s in outs[0]) <= 3e-2 * scale


def test_greedy_generation_through_the_engine(models):
    """``Engine.generate`` (scheduler, portions of prompts, batched decoding as replayed graphs, the sampler's
    argmax) against greedy decoding with the plain statement, for prompts of unequal length at once."""
    from qwen_decoder_b200.engine import Engine, SamplingParams
    folder, cfg, w, seqs, _ = models["A", "float32"]
    prompts = [seqs[2], seqs[5][:20], seqs[4], seqs[1], seqs[9][:50]]
    new = 12
    engine = Engine(folder, dtype="float32", max_batch=3, max_prefill_tokens_per_step=24, max_total_tokens=64,
                    num_pages=40, page_size=16, max_positions=256)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        seq = list(prompt)
        for _ in range(new):
            logits = pf.forward(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            assert float(top2[0] - top2[1]) > 1e-4, "a close call: choose another seed for this test"
            seq.append(int(torch.argmax(logits)))
        assert out == seq[len(prompt):]
    all_free(engine.runner)
    # bfloat16 with replayed graphs: every token the engine chose is, for the statement, the best one or within the
    # rounding of it (a near-tie may go either way, after which the statement follows the engine's sequence)
    folder, cfg, w, _, _ = models["A", "bfloat16"]
    e16 = Engine(folder, dtype="bfloat16", max_batch=4, max_prefill_tokens_per_step=32, max_total_tokens=64,
                 num_pages=40, page_size=16, max_positions=256)
    for prompt, out in zip(prompts, e16.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))):
        seq = list(prompt)
        assert len(out) == new
        for tok in out:
            logits = pf.forward(cfg, w, seq)[-1]
            assert float(logits.max() - logits[tok]) <= 2 * TOL["bfloat16"] * float(logits.abs().max())
            seq.append(tok)
    all_free(e16.runner)


def test_the_programs_take_the_folder(models, tmp_path):
    """``bin/decoder_main`` and ``bin/trace_run`` as separate processes on a Fogurax folder: the command line's greedy
    tokens are the statement's, and a replayed trace with four live requests in a small pool gives its logits."""
    import os
    import subprocess
    import sys
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
    folder, cfg, w, seqs, want = models["A", "float32"]
    prompts = [seqs[2], seqs[3]]
    stdin = "".join(" ".join(map(str, p)) + "\n" for p in prompts) + "\n"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "decoder_main"), folder, "8", "4096", "16", "64", "0",
                        "--dtype", "float32", "--max-new-tokens", "5", "--num-pages", "16", "--ignore-eos"],
                       input=stdin, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("[")]
    assert len(lines) == 2
    for p, line in zip(prompts, lines):
        got = [int(t) for t in line.split(")", 1)[1].split()]
        seq = list(p)
        for tok in got:
            logits = pf.forward(cfg, w, seq)[-1]
            assert float(logits.max() - logits[tok]) <= 1e-4 * float(logits.abs().max())
            seq.append(tok)
        assert len(got) == 5
    tr = trace_tools.mixed(seqs, max_tokens=2 * held(seqs), seed=9)
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(2 * held(seqs))], input=tr.lines(), capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr
    assert r.stdout.splitlines() == [f"done {s['step']}" for s in tr.steps]
    got = trace_tools.read_outputs(tr, str(out), cfg["vocab"])
    trace_tools.compare(tr, got, want, TOL["float32"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_models_drawn_at_random(seed, dtype, tmp_path):
    """Layers of any kind in any order with sizes, taps, windows, blocks, constants and feed-forwards drawn anew for
    every layer: whole, in portions, with decoded tails, and as mixed batches in a small pool with three state slots.
    A drawn model may hold a token at which the statement itself is ill-conditioned (a recurrent head's first output is
    one scalar times v, divided by its own size: where the scalar cancels, relative noise of 1e-7 in the weights moves
    the statement's logits by 6e-5), so float32 too lets one row in a hundred reach four times its tolerance here."""
    stray = max(STRAY[dtype], 0.01)
    cfg = fc.drawn(seed)
    folder = fc.make_folder(cfg, str(tmp_path / "m"), seed=100 + seed, std=0.13,
                            edit=fc.steady_routing if dtype == "bfloat16" else None)
    cfg, w = fc.read_folder(folder)
    rng = random.Random(seed)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 2, 19, 64, 65, 141)]
    want = expected(cfg, w, seqs)
    run_all_ways(folder, dtype, seqs, want, tmp_path, max_tokens=192, tail=30, page_size=16 if seed % 2 else 32, stray=stray)
    max_tokens = 2 * held(seqs)
    runner = make_runner(folder, dtype, max_tokens, max_requests=3)
    tr = trace_tools.mixed(seqs + seqs[::-1], max_tokens, seed=seed, max_live=3)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path / "mixed"))
    trace_tools.compare(tr, got, want + want[::-1], TOL[dtype], stray=stray, stray_factor=STRAY_FACTOR)
    all_free(runner)


LARGER = fc.config(420, 192, 1e-5, 0.8, 16, [
    (fc.attn(6, 2, 128, 96, conv=4, rot_dims=64, base=2e5, scaling=fc.bands(4.0, 1.0, 3.0, 256)), fc.dense(320)),
    (fc.attn2(4, 4, 64, 128, 128, rot_dims=32, base=1e4, scaling=fc.ramp(3.0, 256, 16.0, 2.0)), fc.moe(8, 2, 96, shared=64)),
    (fc.par(6, 3, 64, 64, 200, 3, 32, 24, left_scale=1.1, right_scale=0.9, base=5e5), fc.dense(256)),
    (fc.attn(4, 1, 64, 40, conv=3, rot_dims=64, base=1e3), fc.moe(6, 3, 64)),
])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_larger_model_with_long_prompts(dtype, tmp_path):
    """Heads of 128 and 64 with values of 96, 128, 64 and 40 (every form of the tensor-core kernel), groups of 1, 2, 3
    and 4 heads, prompts of up to 700 tokens over blocks of 128 and a window of 200: several key tiles per query tile,
    single tokens whose keys are shared among CTAs, every way of cutting, and a mixed batch in a small pool."""
    folder = fc.make_folder(LARGER, str(tmp_path / "m"), seed=31, std=0.1,
                            edit=fc.steady_routing if dtype == "bfloat16" else None)
    cfg, w = fc.read_folder(folder)
    rng = random.Random(14)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (700, 257, 384, 129, 513)]
    want = expected(cfg, w, seqs)
    run_all_ways(folder, dtype, seqs, want, tmp_path, max_tokens=704, tail=40, sizes=(100, 2, 3, 64, 200, 7))
    max_tokens = 1408
    runner = make_runner(folder, dtype, max_tokens, max_requests=3, page_size=32)
    tr = trace_tools.mixed(seqs, max_tokens, seed=5, max_live=3, prompt_frac=0.8, portion_sizes=(2, 9, 33, 64, 130))
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path / "mixed"))
    trace_tools.compare(tr, got, want, TOL[dtype], stray=STRAY[dtype], stray_factor=STRAY_FACTOR)
    all_free(runner)
