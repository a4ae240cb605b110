"""Solopel in the engine against its plain float64 statement (``plain_solopel``): each mechanism alone, every way
of cutting the work, batches, pages and state slots used again, far keys, long decoding, generation."""
import random

import numpy as np
import pytest
import torch

import plain_solopel as ps
import solopel_configs as sc
import trace_tools

pytestmark = pytest.mark.gpu

# max |logit difference| relative to the largest |logit|
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = {"A": [1, 2, 15, 16, 17, 33, 64, 65, 150], "B": [3, 31, 32, 48, 97, 130, 210]}


def expected(cfg, w, seqs):
    return [ps.forward(cfg, w, s).numpy() for s in seqs]


def clear_lambda(tensors) -> None:
    """Random small vectors make both exponentials about 1 and the layer's number about ``diff`` alone; these make
    them differ (about e^0.6 - e^-0.5), so that a wrong sign, a lost term or a swapped pair shows."""
    for name in list(tensors):
        if name.endswith(".lq1"):
            p, d = name[:-3], tensors[name].numel()
            tensors[p + "lq1"] = torch.full((d,), 0.6 / d ** 0.5, dtype=torch.bfloat16)
            tensors[p + "lk1"] = torch.full((d,), 1.0 / d ** 0.5, dtype=torch.bfloat16)
            tensors[p + "lq2"] = torch.full((d,), -0.5 / d ** 0.5, dtype=torch.bfloat16)
            tensors[p + "lk2"] = torch.full((d,), 1.0 / d ** 0.5, dtype=torch.bfloat16)


def edits(dtype):
    def edit(tensors):
        clear_lambda(tensors)
        if dtype == "bfloat16":
            sc.steady_routing(tensors)
    return edit


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(name, dtype) -> folder, config, weights, sequences, expected logits.  The bfloat16 runs get the same
    weights with routers that no rounding can flip (``solopel_configs.steady_routing``)."""
    out = {}
    for i, (name, cfg) in enumerate(sc.CONFIGS.items()):
        rng = random.Random(500 + i)
        seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in LENGTHS[name]]
        for dtype in ("float32", "bfloat16"):
            folder = sc.make_folder(cfg, str(tmp_path_factory.mktemp(f"s{name}{dtype}")), seed=40 + i, edit=edits(dtype))
            cfg_read, w = sc.read_folder(folder)
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
    assert runner.cache.slots.num_free == runner.cache.max_requests


SMALL = sc.latent(2, 8, 8, 16)
# name -> (mixer, feed-forward, taps of the layer's input convolution, loop)
ONE_LAYER = {
    "latent": (sc.latent(3, 16, 24, 40, scale=0.4), None, 3, None),
    "latent_many_heads": (sc.latent(11, 8, 16, 24), None, 3, None),
    "latent_two_head_tiles": (sc.latent(20, 8, 16, 32), None, 2, None),     # more heads than one 16-row tile holds
    "latent_no_input_conv": (sc.latent(2, 16, 8, 24), None, 0, None),
    "latent_one_tap": (sc.latent(2, 16, 8, 24), None, 1, None),
    "latent_five_taps": (sc.latent(2, 16, 8, 24), None, 5, None),
    "diff": (sc.attn(4, 4, 16, 32, diff=0.3, conv=3, softcap=20.0), None, 3, None),
    "diff_grouped": (sc.attn(6, 2, 8, 24, diff=0.2, conv=2, softcap=3.0, scale=0.7), None, 3, None),
    "diff_one_kv_head": (sc.attn(5, 1, 12, 20, diff=0.55, conv=4), None, 2, None),
    "diff_no_conv": (sc.attn(2, 2, 24, 8, diff=0.1, conv=0), None, 0, None),
    "diff_one_tap": (sc.attn(3, 3, 8, 40, diff=0.4, conv=1, softcap=50.0), None, 1, None),
    "diff_wide_values": (sc.attn(2, 1, 16, 136, diff=0.25, conv=2), None, 3, None),
    "diff_wide_keys": (sc.attn(2, 2, 72, 64, diff=0.35, conv=3, softcap=8.0), None, 3, None),
    "diff_one_head": (sc.attn(1, 1, 32, 32, diff=0.3, conv=3), None, 3, None),
    "dense": (SMALL, sc.dense(88), 3, None),
    "experts": (SMALL, sc.moe(7, 3, 24), 3, None),
    "experts_one": (SMALL, sc.moe(5, 1, 40), 3, None),
    "experts_shared": (SMALL, sc.moe(3, 1, 40, shared=56), 3, None),
    "experts_all": (SMALL, sc.moe(4, 4, 16, shared=8), 3, None),
    "loop_of_one": (sc.latent(2, 16, 8, 24), sc.dense(40), 3, (0, 1, 3)),
    "loop_once": (sc.attn(2, 1, 8, 16, conv=2), None, 2, (0, 1, 1)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ONE_LAYER))
def test_each_mechanism_alone(name, dtype, tmp_path):
    """One layer of one mixer (with no feed-forward, or a small mixer and one kind of feed-forward): a prompt at
    once, in portions, and its tail token by token."""
    mix, mlp, taps, loop = ONE_LAYER[name]
    cfg = sc.one_layer(mix, mlp, width=56 if "many" in name else 64, taps=taps, loop=loop)
    folder = sc.make_folder(cfg, str(tmp_path / "m"), seed=sum(map(ord, name)), std=0.15, edit=edits(dtype))
    cfg, w = sc.read_folder(folder)
    rng = random.Random(len(name))
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 2, 37, 90)]
    want = expected(cfg, w, seqs)
    runner = make_runner(folder, dtype, 128)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.portions(seqs), trace_tools.decode_tail(seqs, tail=20))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype])
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole_and_decode_tail(models, name, dtype, tmp_path):
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs), page_size=32 if name == "B" else 16)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=40))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype])
    all_free(runner)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_down_to_two_tokens(models, name, dtype, tmp_path):
    """Portions shorter than the convolutions' reach (two tokens under four taps; one token in the decoded tail): the
    kept inputs are moved on by less than they hold."""
    folder, cfg, w, seqs, want = models[name, dtype]
    runner = make_runner(folder, dtype, held(seqs))
    for k, sizes in enumerate(((7, 2, 24, 3, 2, 16, 5, 2, 31, 2), (2,), (64, 1, 3), (1, 1, 2, 1))):
        tr = trace_tools.portions(seqs, sizes=sizes)
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_batches_with_pages_and_slots_used_again(models, name, dtype, tmp_path):
    """Unequal requests side by side, portions beside single tokens, in a pool of about two of the longest and
    with three state slots: every page and slot serves several requests in turn.  Kept inputs that are not zeroed
    at hand-out (a new sequence starts after zeros), or a row read from a page's former owner, show against the
    plain statement."""
    folder, cfg, w, seqs, want = models[name, dtype]
    seqs2, want2 = seqs + seqs[::-1], want + want[::-1]
    max_tokens = 2 * held(seqs)
    runner = make_runner(folder, dtype, max_tokens, max_requests=3)
    tr = trace_tools.mixed(seqs2, max_tokens, seed=11, max_live=3)
    assert sum(len(s["entries"]) > 1 for s in tr.steps) > 5
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want2, TOL[dtype])
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
def test_long_decoding_and_first_tokens(models, dtype, tmp_path):
    """Two tokens of prompt, then 300 tokens one by one across many pages: the convolutions' kept inputs are moved
    on 300 times in every pass of the loop, the keys grow from 1; the first positions are compared one by one."""
    folder, cfg, w, _, _ = models["A", dtype]
    rng = random.Random(77)
    seq = [rng.randrange(cfg["vocab"]) for _ in range(302)]
    want = expected(cfg, w, [seq])
    runner = make_runner(folder, dtype, 320)
    tr = trace_tools.decode_tail([seq], tail=300)
    got = trace_tools.run_inprocess(runner, tr, str(tmp_path))
    trace_tools.compare(tr, got, want, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_larger_model_every_way_of_cutting(dtype, tmp_path):
    """Sizes that take the tensor-core kernels in bfloat16 (several tiles of tokens and keys, grouped heads, single
    tokens whose keys are shared among CTAs), prompts of up to 700 tokens: whole, with decoded tails, in portions,
    and as mixed batches in a pool of two of the longest."""
    folder = sc.make_folder(sc.SC, str(tmp_path / "m"), seed=91, edit=edits(dtype))
    cfg, w = sc.read_folder(folder)
    rng = random.Random(19)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (700, 129, 64, 333, 5)]
    want = expected(cfg, w, seqs)
    runner = make_runner(folder, dtype, 2 * held(seqs), page_size=64)
    both = seqs + seqs[::-1]
    keep = lambda r, p: p % 7 == 0 or p >= len(both[r]) - 40            # which rows are compared
    for k, tr in enumerate((trace_tools.whole(seqs, keep=keep), trace_tools.decode_tail(seqs, tail=36, keep=keep),
                            trace_tools.portions(seqs, sizes=(130, 2, 61, 3, 256), keep=keep),
                            trace_tools.mixed(both, 2 * held(seqs), seed=4, max_live=4, keep=keep, prompt_frac=0.85,
                                              portion_sizes=(2, 17, 64, 130)))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        trace_tools.compare(tr, got, (want + want[::-1]) if k == 3 else want, TOL[dtype],
                            stray=0.01 if dtype == "bfloat16" else 0.0)
    all_free(runner)


# kind -> (mixer, the factor on the queries in float32 and in bfloat16)
FAR = {
    "latent": (sc.latent(4, 16, 32, 32, scale=1.0), 6.0, 1.2),
    "diff": (sc.attn(4, 2, 16, 32, diff=0.3, conv=3, softcap=200.0, scale=1.0), 6.0, 2.5),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", sorted(FAR))
def test_one_far_key_stands_out(kind, dtype, tmp_path):
    """Attention among hundreds of keys with one that matters: the queries are scaled up so that the softmax picks
    single keys (the plain statement confirms that most weight sits on one key, often far back).  A key that is
    lost, read from the wrong row of a page, or one position off changes the logits by far more than the tolerance.
    Prompts end just before, at and just after page borders; the tail is decoded token by token."""
    mix, sharp32, sharp16 = FAR[kind]
    cfg = sc.one_layer(mix, None, vocab=400, width=48)

    # bfloat16 rounds q and the cached rows to 8 bits: scores of this size then move by tenths, and so would the
    # weights of a softmax as sharp as the float32 run's; its run is a little less sharp
    factor, peak = (sharp32, 0.5) if dtype == "float32" else (sharp16, 0.2)

    def sharpen(t):
        clear_lambda(t)
        t["l0.mix.q"] = (t["l0.mix.q"].float() * factor).to(torch.bfloat16)
    folder = sc.make_folder(cfg, str(tmp_path / "m"), seed=5, std=0.2, edit=sharpen)
    cfg, w = sc.read_folder(folder)
    rng = random.Random(8)
    seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (255, 256, 257, 400)]
    # how peaked the plain statement's attention is, and how far back its strongest keys lie
    w64 = ps.t64(w)
    eps, m = cfg["norm"]["eps"], cfg["layers"][0]["mixer"]
    h = ps.offset_norm(w64["embed"][torch.tensor(seqs[3])], w64["l0.norm1"], eps)
    seen = h + ps.causal_conv(h, w64["l0.canon1"])
    if kind == "latent":
        p, _ = ps.latent_weights(w64, "l0.mix.", m, seen, eps)
    else:
        p, _ = ps.diff_weights(w64, "l0.mix.", m, seen)
        p = p.reshape(-1, len(seqs[3]), len(seqs[3]))
    top_p, top_j = p[:, 200:, :].max(dim=-1)
    pos = torch.arange(len(seqs[3]))
    assert float(top_p.median()) > peak                                   # one key carries most of the weight
    assert float(((pos[200:][None, :] - top_j) > 100).float().mean()) > 0.2    # and it is often far back
    want = expected(cfg, w, seqs)
    runner = make_runner(folder, dtype, 512)
    for k, tr in enumerate((trace_tools.whole(seqs), trace_tools.decode_tail(seqs, tail=24),
                            trace_tools.portions(seqs, sizes=(100, 2, 3, 64)))):
        got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"o{k}"))
        # bfloat16: where two keys nearly tie, the rounding of q and of the cached rows shifts weight between them;
        # one row in a hundred may lie above the tolerance (a lost key would be above it many times over)
        trace_tools.compare(tr, got, want, TOL[dtype], stray=0.01 if dtype == "bfloat16" else 0.0)


def test_greedy_generation_through_the_engine(models):
    """``Engine.generate`` (scheduler, portions of prompts, batched decoding as replayed graphs, the sampler's
    argmax) against greedy decoding with the plain statement, for prompts of unequal length at once."""
    from qwen_decoder_b200.engine import Engine, SamplingParams
    folder, cfg, w, seqs, _ = models["A", "float32"]
    prompts = [seqs[2], seqs[5][:20], seqs[4], seqs[1], seqs[6][:50]]
    new = 12
    engine = Engine(folder, dtype="float32", max_batch=3, max_prefill_tokens_per_step=24, max_total_tokens=64,
                    num_pages=40, page_size=16, max_positions=256)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=new, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        seq = list(prompt)
        for _ in range(new):
            logits = ps.forward(cfg, w, seq)[-1]
            top2 = torch.topk(logits, 2).values
            assert float(top2[0] - top2[1]) > 1e-4, "a close call: choose another seed for this test"
            seq.append(int(torch.argmax(logits)))
        assert out == seq[len(prompt):]
    all_free(engine.runner)
    # bfloat16 with graphs: the same tokens whether a request runs alone or beside others
    folder = models["A", "bfloat16"][0]
    e16 = Engine(folder, dtype="bfloat16", max_batch=4, max_prefill_tokens_per_step=32, max_total_tokens=64,
                 num_pages=40, page_size=16, max_positions=256)
    together = e16.generate(prompts[:4], SamplingParams(max_new_tokens=new, ignore_eos=True))
    alone = [e16.generate([p], SamplingParams(max_new_tokens=new, ignore_eos=True))[0] for p in prompts[:4]]
    agree = sum(a == b for a, b in zip(together, alone))
    assert agree >= 3, (together, alone)       # a bfloat16 near-tie may flip one of them


@pytest.mark.parametrize("H,G,d,vd,ps,cap,window", [
    (8, 2, 128, 128, 16, 30.0, 0), (4, 4, 48, 96, 64, 50.0, 0), (6, 1, 64, 64, 24, 0.0, 0), (32, 1, 8, 16, 16, 2.0, 0),
    (3, 3, 72, 40, 32, 5.0, 100), (16, 2, 32, 128, 16, 0.0, 0)])
def test_tensor_core_attention_against_the_float32_kernel(H, G, d, vd, ps, cap, window):
    """The differential attention kernel on tensor cores (prompt portions at any start, single tokens with their
    keys shared among CTAs) against the one-warp-per-head float32 kernel, on the same scattered pages."""
    from qwen_decoder_b200 import kernels
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(H * 1000 + d)
    portions = [(0, 70), (100, 37), (500, 3), (64, 64), (31, 2)]          # (cached before, new tokens)
    singles = [0, 62, 63, 64, 899]                                         # cached before a single new token
    for reqs in (portions, [(c, 1) for c in singles]):
        R, T = len(reqs), sum(n for _, n in reqs)
        blocks = max((c + n + ps - 1) // ps for c, n in reqs)
        perm = torch.randperm(R * blocks + 3, generator=g)[:R * blocks].to(torch.int32).reshape(R, blocks)
        kv = (torch.randn((R * blocks + 3, G * ps * (2 * d + vd)), generator=g) * 0.7).to(torch.bfloat16).to(dev)
        q = (torch.randn((T, H * 2 * d), generator=g) * 1.5).to(torch.bfloat16).to(dev)
        gate = torch.randn((T, H + 3), generator=g).to(dev)[:, 1:H + 1]
        cu = torch.tensor([0] + list(np.cumsum([n for _, n in reqs])), dtype=torch.int32, device=dev)
        start = torch.tensor([c for c, _ in reqs], dtype=torch.int32, device=dev)
        token_req = torch.tensor([r for r, (_, n) in enumerate(reqs) for _ in range(n)], dtype=torch.int32, device=dev)
        pos = torch.tensor([c + i for c, n in reqs for i in range(n)], dtype=torch.int32, device=dev)
        bt = perm.to(dev).contiguous()
        args = (H, G, d, vd, ps, d ** -0.5, cap, 0.37, 1e-5, 0.7, window, gate)
        want = torch.empty((T, H * vd), dtype=torch.bfloat16, device=dev)
        kernels.diff_attention_generic(q, want, kv, bt, token_req, pos, *args)
        for splits in ((1, 3, 64) if T == R else (1,)):
            got = torch.full_like(want, float("nan"))
            kernels.diff_attention_mma(q, got, kv, bt, cu, start, R, T, *args, splits=splits)
            torch.cuda.synchronize()
            err = (got.float() - want.float()).abs().max().item()
            assert err <= 0.03 * want.float().abs().max().item(), (splits, err)


def _drawn_config(rng, routed: bool):
    """A model drawn at random near a small model's scale: three to six layers in any order, any loop."""
    n = rng.randint(3, 6)
    layers = []
    for _ in range(n):
        if rng.random() < 0.5:
            mix = sc.latent(rng.choice([2, 4, 6, 8]), rng.choice([16, 32, 48, 64]), rng.choice([16, 32, 64, 96]),
                            rng.choice([64, 96, 128, 192]))
        else:
            H = rng.choice([2, 4, 8])
            G = rng.choice([g for g in (1, 2, 4, 8) if H % g == 0])
            mix = sc.attn(H, G, rng.choice([16, 32, 48, 64]), rng.choice([32, 64, 96, 128]), diff=rng.choice([0.2, 0.3, 0.5]),
                          conv=rng.choice([2, 3, 4]), softcap=rng.choice([30.0, 50.0, None]))
        k = rng.random()
        mlp = None if k < 0.1 else sc.dense(rng.choice([256, 320, 512])) if k < 0.4 or not routed else \
            sc.moe(rng.choice([4, 8, 16]), rng.choice([1, 2]), rng.choice([64, 96]), shared=rng.choice([None, 96, 128]))
        layers.append((mix, mlp))
    loop = None
    if rng.random() < 0.8:
        a = rng.randint(0, n - 1)
        loop = (a, rng.randint(a + 1, n), rng.randint(1, 3))
    return sc.config(rng.choice([300, 640, 777, 1000]), rng.choice([128, 160, 224, 256, 320]), rng.choice([1e-6, 1e-5]),
                     rng.choice([2, 3, 4]), layers, loop=loop, logit_scale=rng.choice([0.5, 1.0, 0.37]))


@pytest.mark.parametrize("seed", range(6))
def test_models_drawn_at_random(seed, tmp_path):
    """Sizes, layer orders, loops and constants drawn at random, every way of cutting: float32 with routed experts
    (random routers: the choice is checked), bfloat16 with dense feed-forwards in their place (deep in a random
    model no router can be made safe from rounding)."""
    for dtype in ("float32", "bfloat16"):
        rng = random.Random(7000 + seed)
        cfg = _drawn_config(rng, routed=dtype == "float32")
        folder = sc.make_folder(cfg, str(tmp_path / dtype), seed=seed, edit=clear_lambda)
        cfg, w = sc.read_folder(folder)
        seqs = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (300, 70, 33, 150)]
        both = seqs + seqs[::-1]
        want = expected(cfg, w, seqs)
        runner = make_runner(folder, dtype, 2 * held(seqs))
        keep = lambda r, p: p % 5 == 0 or p >= len(both[r]) - 40
        for k, (tr, wnt) in enumerate((
                (trace_tools.whole(seqs, keep=keep), want), (trace_tools.decode_tail(seqs, tail=36, keep=keep), want),
                (trace_tools.portions(seqs, sizes=(40, 2, 17, 3, 100), keep=keep), want),
                (trace_tools.mixed(both, 2 * held(seqs), seed=seed, max_live=4, keep=keep, prompt_frac=0.8,
                                   portion_sizes=(2, 9, 33, 70)), want + want[::-1]))):
            got = trace_tools.run_inprocess(runner, tr, str(tmp_path / f"{dtype}{k}"))
            trace_tools.compare(tr, got, wnt, TOL[dtype])
        all_free(runner)
        del runner
