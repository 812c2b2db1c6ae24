"""Small Gazezen configurations and random weights for them, made by the tests themselves.

The configurations differ in every size and constant: one to eight query heads a key/value head, key and value
widths that are equal, smaller and larger than one another, rotations of a part of a head, of a whole head and
none, windows shorter and longer than a cache page (and none), stretched and plain frequencies, one to four
experts a token (also all of them) with one to four groups of which one to three are kept, shared experts that
are smaller and larger than the routed ones (and none), layers without a feed-forward, looped ranges at the start,
in the middle and at the end of the stack run two and three times (and no loop), logits scaled and not.
`tensors(config, seed)` draws every tensor under its checkpoint name.
"""
import torch


def attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None, mlp=None):
    """`rot`: (base, dims) or None."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot is not None:
        mixer["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, window=None, scaling=None, mlp=None):
    """`scaling`: (factor, original, fast, slow) or None. The rotation takes the whole rotated part."""
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
             "rot": {"base": base, "dims": rot_dim}}
    if window is not None:
        mixer["mask"] = {"size": window}
    if scaling is not None:
        mixer["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def routed(experts, top, ff, groups=None, shared=None):
    """`groups`: (count, keep) or None."""
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


def model(vocab, width, eps, layers, logit_scale=None, loop=None, positions=None):
    config = {"architecture": "Gazezen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if logit_scale is not None:
        config["logit_scale"] = logit_scale
    if loop is not None:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
    if positions is not None:
        config["max_positions"] = positions
    return config


# a looped range in the middle (layers 1 and 2, twice); two heads a key/value head with values wider than keys; a
# latent layer whose frequencies are stretched over a ramp of several pairs; a layer without a feed-forward whose
# heads are rotated whole; three of four groups kept
SMALL_A = model(97, 64, 1e-5, [
    attention(4, 2, 16, 32, 0.3, window=40, rot=(10000.0, 8), mlp=routed(6, 2, 24, groups=(3, 2), shared=40)),
    latent(2, 16, 16, 16, 24, 0.2, 100.0, window=50, scaling=(4.0, 256.0, 8.0, 1.0), mlp=routed(4, 1, 16, shared=8)),
    attention(3, 1, 24, 16, 0.25, rot=(500.0, 24)),
    latent(3, 8, 8, 24, 40, 0.3, 5000.0, mlp=routed(8, 3, 16, groups=(4, 3), shared=24)),
], logit_scale=0.7, loop=(1, 3, 2), positions=700)

# no loop, logits as they are; widths that are no multiples of 16; a window shorter than a page and one far longer;
# a window of exactly a page without any rotation; every expert taken; one group of which one is kept; no shared
# expert; a single head
SMALL_B = model(131, 72, 3e-6, [
    attention(6, 2, 12, 20, 0.3, window=17, rot=(3000.0, 4), mlp=routed(5, 1, 20, shared=12)),
    latent(5, 12, 4, 20, 28, 0.35, 50.0, window=200, mlp=routed(3, 3, 16, groups=(1, 1))),
    attention(1, 1, 40, 24, 0.2, window=64, mlp=routed(4, 2, 24, groups=(2, 1), shared=40)),
    latent(1, 20, 12, 8, 16, 0.3, 1000.0, window=5, scaling=(2.0, 32.0, 4.0, 0.5)),
], positions=800)

# widths that the tensor-core kernels take; the looped range at the start, three times, the rest once; heads of 32, 64
# and 128 with groups of 2, 8 and 1 heads; latents of 64 and 128 with rotated parts of 32 and 64
WIDE = model(211, 256, 1e-5, [
    attention(8, 1, 64, 64, 0.2, window=150, rot=(10000.0, 32), mlp=routed(8, 2, 64, groups=(2, 1), shared=96)),
    latent(4, 32, 32, 64, 64, 0.2, 10000.0, window=100, scaling=(8.0, 128.0, 16.0, 1.0),
           mlp=routed(12, 4, 32, groups=(4, 2), shared=32)),
    attention(4, 2, 32, 64, 0.3, window=70, rot=(800.0, 32), mlp=routed(4, 1, 96, shared=64)),
    attention(2, 2, 128, 128, 0.12, rot=(20000.0, 64)),
    latent(8, 64, 64, 128, 128, 0.1, 50000.0, mlp=routed(16, 2, 48, groups=(4, 1), shared=128)),
], logit_scale=1.5, loop=(0, 2, 3), positions=1200)

# the looped range at the end; one layer only in the loop
TAIL = model(61, 48, 1e-6, [
    latent(2, 16, 8, 16, 32, 0.3, 200.0, window=30, mlp=routed(4, 2, 16, groups=(2, 2), shared=16)),
    attention(2, 2, 16, 16, 0.4, window=33, rot=(100.0, 16), mlp=routed(3, 2, 24, shared=8)),
], logit_scale=2.0, loop=(1, 2, 3), positions=600)

ALL = {"small_a": SMALL_A, "small_b": SMALL_B, "wide": WIDE, "tail": TAIL}


def tensors(config, seed, logits=4.0, sharp=1.0):
    """Every tensor of a model of `config`, bfloat16, under its checkpoint name. `logits` is about the standard
    deviation of the logits; `sharp` multiplies the query maps (sharper scores)."""
    generator = torch.Generator().manual_seed(seed)
    width, vocab = config["width"], config["vocab"]

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=generator) * std + mean).to(torch.bfloat16)

    def matrix(out, inner, gain=1.0):
        return normal(out, inner, std=gain / inner ** 0.5)

    out = {"embed": normal(vocab, width, std=1.0), "final.norm": normal(width, std=0.2, mean=1.0),
           "head": matrix(vocab, width, logits / float(config.get("logit_scale", 1.0)))}
    if "loop" in config:
        out["loop.step"] = normal(config["loop"]["times"], width, std=0.5)
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = normal(width, std=0.2, mean=1.0)
        out[p + "norm1b"] = normal(width, std=0.15, mean=0.5)
        if layer["type"] == "attention":
            groups = m["kv_heads"]
            out[p + "mix.q"] = matrix(heads * dim, width, 2.0 * sharp)
            out[p + "mix.k"] = matrix(groups * dim, width, 2.0)
            out[p + "mix.v"] = matrix(groups * vdim, width, 1.0)
            out[p + "mix.sink"] = normal(heads, std=1.0, mean=0.5)
        else:
            rank, rot = m["kv_rank"], m["rot_dim"]
            out[p + "mix.q"] = matrix(heads * (dim + rot), width, 2.0 * sharp)
            out[p + "mix.dkv"] = matrix(rank + rot, width, 2.0)
            out[p + "mix.dkv.norm"] = normal(rank, std=0.2, mean=1.0)
            out[p + "mix.uk"] = matrix(heads * dim, rank, 2.0)
            out[p + "mix.uv"] = matrix(heads * vdim, rank, 1.0)
        out[p + "mix.g"] = matrix(heads, width, 2.0)
        out[p + "mix.o"] = matrix(width, heads * vdim)
        mlp = layer["mlp"]
        if mlp:
            out[p + "norm2"] = normal(width, std=0.2, mean=1.0)
            out[p + "norm2b"] = normal(width, std=0.15, mean=0.5)
            out[p + "mlp.router"] = matrix(mlp["router"]["experts"], width, 2.0)
            names = [f"e{e}" for e in range(mlp["router"]["experts"])]
            sizes = [mlp["expert"]["ff"]] * len(names)
            if mlp.get("shared"):
                names.append("shared")
                sizes.append(mlp["shared"]["ff"])
            for name, ff in zip(names, sizes):
                out[p + f"mlp.{name}.up"] = matrix(ff, width, 2.0)
                out[p + f"mlp.{name}.down"] = matrix(width, ff, 2.0)
    return out
