"""Small Biropel configurations and random weights for them, made by the tests themselves.

The configurations differ in every size and constant: the order of the three kinds of layer, one to six query
heads a key/value head, key and value widths that are equal, smaller and larger than one another, rotations of a
part of a head and of a whole head, stretched and plain frequencies, windows shorter and longer than a cache
page, exactly a page and none, layers that read another layer's keys (the next layer, a later one, two layers
reading the same one), one to four residual lanes and none, state-space mixers with one to several groups, norm
parts and convolution taps (also one tap: no carried inputs), matrix memories of one to several heads, layers
without a feed-forward, a width that is no multiple of four. `tensors(config, seed)` draws every tensor under its checkpoint name.
"""
import torch


def attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None, scaling=None, softcap=None, q_temp=None,
              kv_from=None):
    """The dictionary of one softmax attention. `rot`: (base, dims); `scaling`: (factor, original, fast, slow);
    `q_temp`: (coef, every)."""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot is not None:
        mixer["rot"] = {"base": rot[0], "dims": rot[1]}
        if scaling is not None:
            mixer["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if softcap is not None:
        mixer["softcap"] = softcap
    if q_temp is not None:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def dense(ff):
    return {"kind": "dense", "ff": ff} if ff else None


def attention_layer(mixer, ff=None):
    return {"type": "attention", "mixer": mixer, "mlp": dense(ff)}


def state_space_layer(left, heads, vdim, state, groups, conv, norm_groups, ff=None):
    right = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": dense(ff)}


def matrix_memory_layer(left, heads, dim, vdim, gate_cap, ff=None):
    right = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}
    return {"type": "parallel_2", "mixer": {"left": left, "right": right}, "mlp": dense(ff)}


def model(vocab, width, eps, layers, streams=None, positions=None):
    config = {"architecture": "Biropel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        config["streams"] = streams
    if positions is not None:
        config["max_positions"] = positions
    return config


# every kind of layer; a layer that reads the keys of the layer before it, with a window of its own; values wider
# than keys; a state-space mixer of two groups, four taps and two norm parts; a layer without a feed-forward
SMALL_A = model(97, 64, 1e-5, [
    attention_layer(attention(4, 2, 16, 24, 0.3, window=40, rot=(10000.0, 8)), ff=48),
    attention_layer(attention(4, 2, 16, 24, 0.25, window=21, rot=(10000.0, 8), kv_from=0), ff=40),
    state_space_layer(attention(3, 1, 16, 16, 0.3, window=33, rot=(5000.0, 16), scaling=(4.0, 64.0, 8.0, 1.0),
                                softcap=20.0), heads=4, vdim=12, state=8, groups=2, conv=4, norm_groups=2, ff=56),
    matrix_memory_layer(attention(2, 2, 24, 8, 0.2, softcap=15.0, q_temp=(0.4, 16)), heads=2, dim=12, vdim=20,
                        gate_cap=10.0),
    matrix_memory_layer(attention(6, 1, 8, 8, 0.35, softcap=40.0, q_temp=(0.2, 50)), heads=3, dim=8, vdim=8,
                        gate_cap=6.0, ff=32),
], streams=2, positions=700)

# another order (the recurrent layers first); three lanes; widths that are no multiples of 16; a window shorter
# than a page and one of exactly a page; one tap (no carried inputs) and two taps; as many groups as heads and one
# norm part; two layers that read the keys of the same earlier layer, not the one right before them
SMALL_B = model(131, 72, 3e-6, [
    matrix_memory_layer(attention(1, 1, 20, 12, 0.3, softcap=25.0, q_temp=(0.3, 7)), heads=1, dim=20, vdim=36,
                        gate_cap=12.0, ff=40),
    state_space_layer(attention(2, 2, 12, 20, 0.3, window=17, rot=(300.0, 4), scaling=(2.0, 32.0, 4.0, 0.5),
                                softcap=10.0), heads=3, vdim=8, state=5, groups=3, conv=1, norm_groups=1, ff=24),
    attention_layer(attention(6, 3, 12, 8, 0.3, window=64, rot=(1000.0, 12)), ff=72),
    state_space_layer(attention(3, 3, 8, 8, 0.4, window=100, rot=(50.0, 8), softcap=35.0), heads=2, vdim=20,
                      state=12, groups=1, conv=2, norm_groups=4),
    attention_layer(attention(3, 3, 12, 8, 0.2, window=30, rot=(1000.0, 12), kv_from=2), ff=16),
    attention_layer(attention(6, 3, 12, 8, 0.3, rot=(1000.0, 12), kv_from=2)),
], streams=3, positions=800)

# one ordinary residual stream (no lanes)
PLAIN = model(61, 48, 1e-6, [
    state_space_layer(attention(2, 1, 16, 16, 0.3, window=50, rot=(100.0, 16), softcap=20.0), heads=2, vdim=16,
                      state=16, groups=1, conv=3, norm_groups=1, ff=64),
    attention_layer(attention(2, 2, 16, 16, 0.3, window=30, rot=(100.0, 8)), ff=32),
    matrix_memory_layer(attention(2, 1, 16, 16, 0.25, softcap=28.0, q_temp=(0.5, 32)), heads=2, dim=16, vdim=16,
                        gate_cap=8.0, ff=32),
], positions=600)

# a single lane (the mixing matrix is one number)
ONE_LANE = model(53, 40, 1e-5, [
    attention_layer(attention(2, 1, 8, 16, 0.35, window=25, rot=(100.0, 8)), ff=24),
    matrix_memory_layer(attention(2, 2, 8, 8, 0.35, softcap=22.0, q_temp=(0.3, 10)), heads=2, dim=8, vdim=8,
                        gate_cap=9.0, ff=24),
], streams=1, positions=600)

# widths that the tensor-core kernels take: heads of 64 and 128 with groups of 4, 1 and 2 heads, a window whose edge
# falls inside a tile; four lanes; a state of 64 rows and memories of 64 x 64
WIDE = model(211, 256, 1e-5, [
    attention_layer(attention(8, 2, 64, 64, 0.15, window=150, rot=(10000.0, 32)), ff=256),
    state_space_layer(attention(4, 4, 64, 64, 0.15, window=100, rot=(20000.0, 64), scaling=(8.0, 128.0, 16.0, 1.0),
                                softcap=25.0), heads=8, vdim=32, state=64, groups=2, conv=4, norm_groups=2, ff=128),
    attention_layer(attention(8, 2, 64, 64, 0.15, window=70, rot=(10000.0, 32), kv_from=0), ff=128),
    attention_layer(attention(2, 1, 128, 128, 0.1, rot=(50000.0, 64))),
    matrix_memory_layer(attention(4, 2, 64, 64, 0.12, softcap=25.0, q_temp=(0.25, 128)), heads=4, dim=64, vdim=64,
                        gate_cap=12.0, ff=256),
], streams=4, positions=1300)

# a width that is no multiple of four (no kernel takes its rows in pieces of several elements), three lanes
ODD = model(71, 50, 1e-5, [
    attention_layer(attention(2, 1, 10, 6, 0.3, window=45, rot=(100.0, 6)), ff=30),
    state_space_layer(attention(3, 1, 6, 10, 0.3, window=20, rot=(100.0, 6), softcap=12.0), heads=3, vdim=6, state=7,
                      groups=1, conv=3, norm_groups=3, ff=22),
    matrix_memory_layer(attention(2, 2, 6, 6, 0.3, softcap=12.0, q_temp=(0.3, 9)), heads=3, dim=7, vdim=5, gate_cap=7.0),
], streams=3, positions=600)

ALL = {"small_a": SMALL_A, "small_b": SMALL_B, "plain": PLAIN, "one_lane": ONE_LANE, "wide": WIDE, "odd": ODD}


def single(layer, vocab=67, width=48, eps=1e-5, streams=None, positions=900):
    """A model of one layer (a mechanism alone)."""
    return model(vocab, width, eps, [layer], streams=streams, positions=positions)


def tensors(config, seed, logits=4.0, sharp=1.0):
    """Every tensor of a model of `config`, bfloat16, under its checkpoint name. `logits` is about the standard
    deviation of the logits; `sharp` multiplies the query maps (sharper scores)."""
    generator = torch.Generator().manual_seed(seed)
    width, vocab = config["width"], config["vocab"]
    lanes = config.get("streams")

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=generator) * std + mean).to(torch.bfloat16)

    def matrix(out, inner, gain=1.0):
        return normal(out, inner, std=gain / inner ** 0.5)

    def softmax_attention(p, m, biased, gated):
        heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "q"] = matrix(heads * dim, width, 2.0 * sharp)
        if "kv_from" not in m:
            out[p + "k"] = matrix(groups * dim, width, 2.0)
            out[p + "v"] = matrix(groups * vdim, width, 1.0)
        if biased:
            for name, size in (("q", heads * dim), ("k", groups * dim), ("v", groups * vdim)):
                if name == "q" or "kv_from" not in m:
                    out[p + name + ".b"] = normal(size, std=0.5)
        if gated:
            out[p + "g"] = matrix(heads * vdim, width, 2.0)
        out[p + "o"] = matrix(width, heads * vdim)

    out = {"embed": normal(vocab, width, std=1.0), "embed.norm": normal(width, std=0.2, mean=1.0),
           "final.norm": normal(width, std=0.2, mean=1.0), "head": matrix(vocab, width, logits)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        numbers = ("1", "2") if layer["mlp"] else ("1",)
        for number in numbers:
            out[p + "norm" + number] = normal(width, std=0.2, mean=1.0)
            if lanes:
                out[p + f"hc{number}.in"] = normal(lanes, std=0.2, mean=1.0 / lanes)
                out[p + f"hc{number}.out"] = normal(lanes, std=0.3, mean=0.8)
                out[p + f"hc{number}.mix"] = (torch.eye(lanes) + 0.25 * torch.randn(lanes, lanes, generator=generator)
                                              ).to(torch.bfloat16)
        if layer["type"] == "attention":
            softmax_attention(p + "mix.", m, biased=True, gated=True)
        else:
            softmax_attention(p + "mix.left.", m["left"], biased=False, gated=False)
            out[p + "mix.left.out"] = normal(width, std=0.2, mean=1.0)
            out[p + "mix.right.out"] = normal(width, std=0.2, mean=1.0)
            r, q = m["right"], p + "mix.right."
            if layer["type"] == "parallel":
                heads, inner, span = r["heads"], r["heads"] * r["vdim"], r["groups"] * r["state"]
                out[q + "in"] = matrix(2 * inner + 2 * span + heads, width, 1.5)
                out[q + "conv"] = normal(inner + 2 * span, r["conv"], std=0.6)
                out[q + "conv.b"] = normal(inner + 2 * span, std=0.3)
                out[q + "dt_bias"] = normal(heads, std=1.0, mean=-0.5)
                out[q + "A_log"] = normal(heads, std=0.7, mean=-0.5)
                out[q + "D"] = normal(heads, std=0.3, mean=1.0)
                out[q + "norm"] = normal(inner, std=0.2, mean=1.0)
                out[q + "o"] = matrix(width, inner)
            else:
                heads, keys, values = r["heads"], r["heads"] * r["dim"], r["heads"] * r["vdim"]
                out[q + "q"] = matrix(keys, width, 2.0)
                out[q + "k"] = matrix(keys, width, 2.0)
                out[q + "v"] = matrix(values, width, 1.0)
                out[q + "g"] = matrix(values, width, 2.0)
                out[q + "o"] = matrix(width, values)
                out[q + "norm"] = normal(values, std=0.2, mean=1.0)
                out[q + "i"] = matrix(heads, width, 3.0)
                out[q + "i.b"] = normal(heads, std=1.0)
                out[q + "f"] = matrix(heads, width, 3.0)
                out[q + "f.b"] = normal(heads, std=1.0, mean=2.0)
        if layer["mlp"]:
            out[p + "mlp.up"] = matrix(layer["mlp"]["ff"], width, 1.5)
            out[p + "mlp.down"] = matrix(width, layer["mlp"]["ff"], 1.0)
    return out
