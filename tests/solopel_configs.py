"""Small Solopel configurations for the tests: every size and option differs between them and from layer to layer;
values that a model may happen to make equal or 1 are unequal or not 1 somewhere (and equal or 1 somewhere else)."""
import torch

from veterax_configs import make_folder, read_folder  # noqa: F401  (generic: any registered architecture)


def latent(heads, dim, vdim, kv_rank, scale=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale if scale is not None else dim ** -0.5}}


def attn(heads, kv_heads, dim, vdim, diff=0.3, conv=3, softcap=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": scale if scale is not None else dim ** -0.5}
    if conv:
        m["conv"] = conv
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def config(vocab, width, eps, taps, layers, loop=None, logit_scale=1.0):
    c = {"architecture": "Solopel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
         "layers": [dict(mix, mlp=mlp) for mix, mlp in layers]}
    if taps:
        c["canon"] = {"taps": taps}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# the loop starts after the first layer and holds both kinds of mixer; grouped heads (3 per kv head), values larger
# and smaller than keys, four taps in the layers and two in the attention, a small cap, two experts per token, a
# layer without feed-forward, experts with and without a shared one
SA = config(310, 96, 1e-5, 4, [
    (latent(3, 24, 16, 40, scale=0.3), dense(136)),
    (attn(6, 2, 8, 24, diff=0.2, conv=2, softcap=4.0, scale=0.5), moe(5, 2, 40, shared=24)),
    (latent(5, 16, 24, 64), None),
    (attn(4, 4, 16, 8, diff=0.45, conv=4), moe(3, 3, 16)),
    (latent(2, 32, 32, 24), moe(6, 1, 24, shared=56)),
], loop=(1, 3, 2), logit_scale=0.37)
# no loop, two taps, one kv head for all heads, attention without its convolution and without a cap, sizes that are
# no whole 16-byte pieces, one tap in one attention layer
SB = config(523, 72, 2e-6, 2, [
    (attn(4, 1, 20, 12, diff=0.6, conv=0), dense(100)),
    (latent(3, 12, 20, 36), moe(4, 2, 28, shared=20)),
    (attn(2, 2, 24, 40, diff=0.1, conv=1, softcap=30.0), moe(7, 1, 36)),
], logit_scale=1.0)
CONFIGS = {"A": SA, "B": SB}
# sizes nearer a real small model's, for the tensor-core paths: whole 16-byte pieces everywhere, four query heads per
# kv head, keys of 32 per map and values of 64, several tiles of tokens and of keys in one prompt, a loop of three
# layers run three times that ends at the last layer, three taps in the layers and four in the attention
SC = config(701, 256, 1e-6, 3, [
    (attn(8, 2, 32, 64, diff=0.25, conv=4, softcap=25.0), dense(384)),
    (latent(8, 32, 64, 96), moe(8, 2, 96, shared=128)),
    (attn(4, 4, 64, 32, diff=0.4, conv=2, softcap=40.0), moe(6, 1, 128)),
    (latent(4, 64, 32, 160, scale=0.11), dense(512)),
], loop=(1, 4, 3), logit_scale=0.6)


def one_layer(mix, mlp, vocab=200, width=64, eps=1e-5, taps=3, loop=None, logit_scale=0.8):
    return config(vocab, width, eps, taps, [(mix, mlp)], loop=loop, logit_scale=logit_scale)


def steady_routing(tensors) -> None:
    """For runs in bfloat16: routers whose choice no rounding can flip.  The router has no bias, so its input must
    carry the choice: channel 0 of the residual sum is made large and positive (the embedding's column, and in a loop
    the row of the pass's input matrix that makes channel 0 copies the embedding's), and a router reads channel 0 only,
    with slopes that lie far apart.  Every token then takes the same experts, in a scrambled order, with weights
    (sigmoids of slope * normed channel) that still depend on the token: every kernel of the routed path runs.  With
    random routers a bfloat16 run meets, every few hundred tokens, two logits closer than its rounding, takes the
    other expert and differs from the plain statement by an expert's whole output: the float32 runs keep the random
    routers and check the choice."""
    width = tensors["embed"].shape[1]
    tensors["embed"][:, 0] = 6.0
    if "loop.in" in tensors:
        tensors["loop.in"][0, :] = 0.0
        tensors["loop.in"][0, width] = 1.0
        tensors["loop.step"][:, 0] = 0.0
    for name in list(tensors):
        if name.endswith("mlp.router"):
            n = tensors[name].shape[0]
            order = [n - 1 - j // 2 if j % 2 == 0 else j // 2 for j in range(n)]      # most preferred first
            r = torch.zeros_like(tensors[name])
            for j, e in enumerate(order):
                r[e, 0] = 0.25 * (n - 1 - j) - 0.3
            tensors[name] = r
