"""Small Fogurax configurations for the tests: every size and option differs between them and from layer to layer;
values that a model may happen to make equal or 1 are unequal or not 1 somewhere (and equal or 1 somewhere else)."""
import json
import os

import torch


def bands(factor, low, high, original):
    return {"factor": factor, "low": low, "high": high, "original": original}


def ramp(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def _rot(dim, rot_dims, base, scaling):
    r = {"base": base, "dims": rot_dims or dim}
    if scaling:
        r["scaling"] = scaling
    return r


def attn(heads, kv_heads, dim, vdim, conv=4, rot_dims=None, base=10000.0, scaling=None, scale=None):
    """Biases, a convolution over ``conv`` tokens, adjacent pairs, per-head unit norm after the rotation, a gate."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": _rot(dim, rot_dims, base, scaling),
         "scale": scale if scale is not None else dim ** -0.5}
    if conv:
        m["conv"] = conv
    return {"type": "attention", "mixer": m}


def attn2(heads, kv_heads, dim, vdim, block, rot_dims=None, base=10000.0, scaling=None, scale=None):
    """Whole-projection norms, half-split pairs, a query sees its own block of ``block`` positions."""
    return {"type": "attention_2", "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": block},
        "rot": _rot(dim, rot_dims, base, scaling), "scale": scale if scale is not None else dim ** -0.5}}


def par(heads, kv_heads, dim, vdim, window, rheads, rdim, rank, left_scale=1.0, right_scale=1.0, rot_dims=None,
        base=10000.0, scale=None):
    """Windowed attention beside the recurrent mixer."""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
            "rot": _rot(dim, rot_dims, base, None), "scale": scale if scale is not None else dim ** -0.5}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rheads, "dim": rdim, "rank": rank},
                                          "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def config(vocab, width, eps, mult, side, layers):
    c = {"architecture": "Fogurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
         "layers": [dict(mix, mlp=mlp) for mix, mlp in layers]}
    if side:
        c["token_side"] = {"dim": side}
    return c


# grouped heads in the convolved attention, values larger than keys, part of a head unrotated, two taps, a block that
# is no multiple of a page, a window shorter than a page, one recurrent head of a size that is no power of two, a
# layer without feed-forward, several experts per token, no shared expert in one layer, every layer another kind
FA = config(310, 96, 1e-6, 0.7, 6, [
    (attn(6, 3, 16, 24, conv=2, rot_dims=8, base=500.0, scaling=bands(4.0, 0.5, 3.0, 64), scale=0.3), dense(40)),
    (par(4, 4, 24, 16, 11, 1, 40, 5, left_scale=0.8, right_scale=1.3, base=77.0), None),
    (attn2(8, 2, 8, 16, 20, rot_dims=4, scaling=ramp(4.0, 64, 16.0, 2.0), scale=0.5), moe(5, 2, 24)),
    (par(3, 1, 8, 8, 40, 3, 16, 9, left_scale=1.0, right_scale=0.6, rot_dims=6), moe(4, 4, 16, shared=24)),
    (attn2(2, 2, 32, 8, 64, base=1e6), dense(56)),
])
# no token input, a multiplier of 1, one key/value head for many query heads, head sizes that are no whole 16-byte
# pieces (the float32 kernel serves them in bfloat16 too), heads of 128, no convolution and one of a single tap,
# a window longer than most prompts, a block of one position
FB = config(515, 128, 2e-5, 1.0, 0, [
    (attn(10, 1, 12, 20, conv=0, rot_dims=4, base=300.0), moe(7, 3, 32, shared=48)),
    (attn2(2, 1, 128, 20, 1, scaling=ramp(6.0, 128, 24.0, 1.5), scale=0.1), None),
    (par(5, 5, 72, 20, 150, 3, 64, 12, left_scale=1.25, right_scale=0.9, rot_dims=36), moe(2, 1, 64)),
    (attn(2, 2, 128, 64, conv=1, scaling=bands(6.0, 1.0, 3.0, 32), scale=0.08), dense(72)),
])
CONFIGS = {"A": FA, "B": FB}


def one_layer(mix, mlp, vocab=200, width=64, eps=3e-6, mult=0.6, side=0):
    return config(vocab, width, eps, mult, side, [(mix, mlp)])


def make_folder(cfg: dict, path: str, seed: int, std: float = 0.12, edit=None) -> str:
    """A model folder with random bfloat16 weights, large enough that attention and routing are far from uniform.
    ``edit(tensors)`` may change tensors before they are written."""
    from qwen_decoder_b200.config import config_from_dict, describe_model
    from qwen_decoder_b200.parts.model import build_model
    from qwen_decoder_b200.weights import random_tensors
    from qwen_decoder_b200.weights.safetensors_io import save_safetensors
    typed = config_from_dict(cfg)
    model = build_model(describe_model(typed))
    tensors = random_tensors(model.tensor_specs(), seed, torch.bfloat16, "cpu", std, 0.1)
    if edit is not None:
        edit(tensors)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(typed.to_dict(), f)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors, {"format": "pt"})
    return path


def read_folder(path: str):
    """(config dict, {name: tensor}) with no code of the engine."""
    from safetensors import safe_open
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt", device="cpu") as sf:
        tensors = {k: sf.get_tensor(k) for k in sf.keys()}
    return cfg, tensors


def steady_routing(tensors) -> None:
    """For runs in bfloat16: routers whose choice no rounding can flip.  The router has no bias, so its input must
    carry the choice: channel 0 of the embedding is made large and positive, and a router reads channel 0 only, with
    slopes that lie far apart.  Every token then takes the same experts, in a scrambled order, with weights (sigmoids
    of slope * normed channel) that still depend on the token, so every kernel of the routed path runs.  With random
    routers a bfloat16 run meets, every few hundred tokens, two scores closer than its rounding, takes the other
    expert and differs from the plain statement by an expert's whole output: the float32 runs keep the random routers
    and check the choice."""
    tensors["embed"][:, 0] = 6.0
    for name in list(tensors):
        if name.endswith("mlp.router"):
            n = tensors[name].shape[0]
            order = [n - 1 - j // 2 if j % 2 == 0 else j // 2 for j in range(n)]      # most preferred first
            r = torch.zeros_like(tensors[name])
            for j, e in enumerate(order):
                r[e, 0] = 0.25 * (n - 1 - j) - 0.3
            tensors[name] = r


def drawn(seed: int) -> dict:
    """A model drawn at random: three to six layers of any kind in any order, sizes, taps, windows, blocks, constants
    and feed-forwards drawn anew for every layer (head sizes even; some multiples of 8, some not)."""
    import random
    rng = random.Random(seed)
    width = rng.choice([40, 64, 72, 96, 104])
    layers = []
    for _ in range(rng.randint(3, 6)):
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 4])
        dim, vdim = rng.choice([8, 12, 16, 24, 32, 64]), rng.choice([8, 12, 16, 20, 40])
        rot_dims = rng.choice([dim, dim // 2 - (dim // 2) % 2 or 2, 4])
        base = rng.choice([50.0, 1000.0, 3e5])
        scale = rng.choice([dim ** -0.5, 0.3, 0.5])
        kind = rng.choice(["attention", "attention_2", "parallel"])
        if kind == "attention":
            sc = rng.choice([None, bands(rng.choice([2.0, 8.0]), rng.choice([0.5, 1.0]), rng.choice([2.0, 6.0]), rng.choice([16, 64]))])
            mix = attn(heads, kv, dim, vdim, conv=rng.choice([0, 1, 2, 3, 4]), rot_dims=rot_dims, base=base, scaling=sc, scale=scale)
        elif kind == "attention_2":
            sc = rng.choice([None, ramp(rng.choice([2.0, 5.0]), rng.choice([16, 64]), rng.choice([4.0, 16.0]), rng.choice([0.5, 2.0]))])
            mix = attn2(heads, kv, dim, vdim, rng.choice([1, 3, 16, 37, 64, 500]), rot_dims=rot_dims, base=base, scaling=sc, scale=scale)
        else:
            mix = par(heads, kv, dim, vdim, rng.choice([1, 5, 16, 50, 130, 500]), rng.choice([1, 2, 3]), rng.choice([8, 16, 24, 64]),
                      rng.choice([2, 7, 16]), left_scale=rng.choice([0.5, 1.0, 1.4]), right_scale=rng.choice([0.4, 1.0, 1.3]),
                      rot_dims=rot_dims, base=base, scale=scale)
        experts = rng.choice([2, 4, 6])
        mlp = rng.choice([None, dense(rng.choice([24, 40, 88])),
                          moe(experts, rng.randint(1, experts), rng.choice([12, 16, 40]), shared=rng.choice([None, 24]))])
        layers.append((mix, mlp))
    return config(rng.choice([150, 333]), width, rng.choice([1e-6, 1e-5, 1e-4]), rng.choice([0.3, 0.7, 1.0]),
                  rng.choice([0, 0, 3, 8]), layers)
