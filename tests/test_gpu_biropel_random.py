"""Random Biropel configurations (sizes that are no round numbers, the three kinds of layer in every order that the
draw gives, one to eight heads a key/value head, key and value widths with and without the tensor-core kernels'
multiples of 16, rotations of a part of a head, of a whole head and none, stretched and plain frequencies, windows
from 3 to 300 tokens or none, bounded scores and temperatures or none, borrowed keys wherever an earlier attention
layer fits, one to four lanes or none, state-space mixers and matrix memories of many shapes, layers without a
feed-forward) through the engine in both precisions against the plain implementation: a prompt in two portions, then
eight tokens decoded one by one, and the same request in a batch of two. Two of the draws run prompts of more than
1,024 tokens, so that the products of prompts take their tensor-memory kernel at these sizes and the windows pass
over many pages."""
import numpy as np
import pytest
import torch

import biropel_configs as configs
import plain_biropel

pytestmark = pytest.mark.gpu

DRAWS = 12


def draw(seed):
    rng = np.random.default_rng(5100 + seed)
    pick = lambda values: int(rng.choice(values))
    width = 8 * pick(range(5, 26)) + pick([0, 0, 4])

    def softmax_attention(kind, earlier):
        groups = pick([1, 1, 2, 3])
        heads = groups * pick([1, 2, 3, 4, 8])
        if rng.random() < 0.5:
            dim, vdim = pick([16, 32, 64, 128]), pick([16, 32, 48, 64, 96])      # widths of the tensor-core kernels
            if rng.random() < 0.6:
                vdim = dim
        else:
            dim, vdim = pick([4, 8, 12, 20, 24, 40]), pick([8, 12, 16, 24, 36, 72])
        window = pick([3, 17, 64, 65, 100, 128, 300]) if rng.random() < 0.75 else None
        rot = scaling = None
        if kind != "parallel_2" and rng.random() < 0.9:
            rot = (float(rng.choice([100.0, 10000.0, 1e6])), pick([d for d in (2, 4, 8, 12, 16, 32, 64, 128) if d <= dim]))
            if rng.random() < (0.8 if kind == "parallel" else 0.2):
                scaling = (float(rng.choice([2.0, 4.0, 8.0, 40.0])), float(rng.choice([32.0, 64.0, 512.0])),
                           float(rng.choice([4.0, 8.0, 32.0])), float(rng.choice([0.5, 1.0, 2.0])))
        bounded = rng.random() < (0.15 if kind == "attention" else 0.85)
        mixer = configs.attention(heads, groups, dim, vdim, float(rng.uniform(0.1, 0.5)),
                                  window=None if kind == "parallel_2" and rng.random() < 0.7 else window, rot=rot,
                                  scaling=scaling, softcap=float(rng.choice([5.0, 15.0, 30.0, 50.0])) if bounded else None,
                                  q_temp=(float(rng.uniform(0.1, 0.6)), pick([3, 16, 64, 256]))
                                  if rng.random() < (0.85 if kind == "parallel_2" else 0.1) else None)
        if kind == "attention" and earlier and rng.random() < 0.5:      # read an earlier layer's keys and values
            source = pick(earlier)
            other = layers[source]["mixer"]
            mixer.update(kv_heads=other["kv_heads"], heads=other["kv_heads"] * pick([1, 2, 4]), dim=other["dim"],
                         vdim=other["vdim"], kv_from=source)
            mixer.pop("rot", None)
            if "rot" in other:
                mixer["rot"] = dict(other["rot"])
        return mixer

    layers = []
    for _ in range(pick([2, 3, 3, 4, 5, 6])):
        kind = ["attention", "parallel", "parallel_2"][pick([0, 0, 1, 2])]
        ff = pick([8, 24, 40, 64, 100]) if rng.random() < 0.85 else None
        owners = [i for i, layer in enumerate(layers) if layer["type"] == "attention" and "kv_from" not in layer["mixer"]]
        left = softmax_attention(kind, owners)
        if kind == "attention":
            layers.append(configs.attention_layer(left, ff=ff))
        elif kind == "parallel":
            groups = pick([1, 1, 2, 3])
            heads = groups * pick([1, 2, 4])
            vdim = pick([4, 8, 12, 16, 32, 48, 64])
            parts = pick([p for p in (1, 2, 3, 4, 8) if (heads * vdim) % p == 0])
            layers.append(configs.state_space_layer(left, heads=heads, vdim=vdim, state=pick([4, 8, 16, 24, 48, 64, 128]),
                                                    groups=groups, conv=pick([1, 2, 3, 4, 4]), norm_groups=parts, ff=ff))
        else:
            layers.append(configs.matrix_memory_layer(left, heads=pick([1, 2, 3, 4, 6]), dim=pick([4, 8, 16, 24, 48, 64, 128]),
                                                      vdim=pick([4, 8, 16, 31, 32, 48, 64, 128]),
                                                      gate_cap=float(rng.choice([5.0, 15.0, 30.0])), ff=ff))
    return configs.model(pick(range(61, 400)), width, float(rng.choice([1e-6, 1e-5, 3e-5])), layers,
                         streams=pick([1, 2, 2, 3, 4]) if rng.random() < 0.85 else None, positions=1536)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(DRAWS))
def test_random_configuration(seed, dtype, record_property):
    from kidi_b200 import Engine, StepBatch
    config = draw(seed)
    tensors = configs.tensors(config, 900 + seed)
    engine = Engine.from_config(config, tensors=tensors, dtype=dtype, max_tokens=4096)
    rng = np.random.default_rng(seed)
    length = 1100 + 17 * seed if seed in (3, 8) else int(rng.integers(70, 330))
    tokens = rng.integers(0, config["vocab"], size=length).tolist()
    other = rng.integers(0, config["vocab"], size=int(rng.integers(1, 90))).tolist()
    want = plain_biropel.forward(config, tensors, tokens, dtype=torch.float64)
    head, cut = length - 8, int(rng.integers(1, length - 9))
    slot = engine.acquire()
    rows = [engine.step(StepBatch([slot], [tokens[:cut]], [list(range(cut))])).double().cpu(),
            engine.step(StepBatch([slot], [tokens[cut:head]], [list(range(head - cut))])).double().cpu()]
    rows += [engine.step(StepBatch([slot], [[token]], [[0]])).double().cpu() for token in tokens[head:]]
    engine.release(slot)
    got = torch.cat(rows)
    scale, level = float(want.abs().max()), float(want.pow(2).mean().sqrt())
    worst = float((got - want).abs().max()) / scale
    mean = float((got - want).pow(2).mean().sqrt()) / level
    record_property("largest and mean relative difference", (worst, mean))
    assert torch.isfinite(got).all()
    assert worst < (8e-5 if dtype == "float32" else 0.3) and mean < (2e-5 if dtype == "float32" else 0.06), \
        (seed, worst, mean, config)
    # the same request beside another one, on the slot and pages that were just given back
    slots = [engine.acquire(), engine.acquire()]
    both = engine.step(StepBatch(slots, [other, tokens[:head]], [[], list(range(head))])).double().cpu()
    last = engine.step(StepBatch(slots[1:], [[tokens[head]]], [[0]])).double().cpu()
    for used in slots:
        engine.release(used)
    beside = torch.cat([both, last])
    bound = 8e-5 if dtype == "float32" else 0.3
    assert float((beside - want[:head + 1]).abs().max()) / scale < bound, (seed, "in a batch")
    engine.cache.check()
