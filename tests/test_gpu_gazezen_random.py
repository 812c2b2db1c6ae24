"""Random Gazezen configurations (sizes that are no round numbers, one to eight heads a key/value head, key and value
widths with and without the tensor-core kernels' multiples of 16, rotations of a part of a head, of a whole head
and none, latents of 8 to 128, windows from 3 to 300 tokens or none, stretched and plain frequencies, one to six
experts a token in one to four groups, shared experts or none, layers without a feed-forward, looped ranges
anywhere in the stack or none, in every order that the draw gives) through the engine in both precisions against
the plain implementation: a prompt in two portions, then eight tokens decoded one by one. Two of the draws run
prompts of more than 1,024 tokens, so that the products of prompts take their tensor-memory kernel at these sizes
and the windows pass over many pages."""
import numpy as np
import pytest
import torch

import gazezen_configs
import plain_gazezen

pytestmark = pytest.mark.gpu

DRAWS = 10


def draw(seed):
    rng = np.random.default_rng(3200 + seed)
    pick = lambda values: int(rng.choice(values))
    width = 8 * pick(range(5, 26)) + pick([0, 0, 4])

    def feed_forward():
        if rng.random() < 0.15:
            return None
        groups = pick([1, 1, 2, 3, 4])
        per = pick([1, 2, 3, 4])
        keep = pick(range(1, groups + 1))
        top = pick(range(1, min(6, keep * per) + 1))
        shared = pick([8, 24, 40, 72]) if rng.random() < 0.7 else None
        return gazezen_configs.routed(groups * per, top, pick([8, 24, 40, 64]), groups=(groups, keep) if groups > 1 or rng.random() < 0.3 else None,
                                      shared=shared)

    layers = []
    for _ in range(pick([2, 3, 3, 4, 5, 6])):
        window = pick([3, 17, 64, 65, 100, 128, 300]) if rng.random() < 0.75 else None
        scale = float(rng.uniform(0.1, 0.5))
        if rng.random() < 0.5:
            groups = pick([1, 1, 2, 3])
            heads = groups * pick([1, 2, 3, 4, 8])
            if rng.random() < 0.5:
                dim, vdim = pick([16, 32, 48, 64]), pick([16, 32, 48, 80, 96])   # widths of the tensor-core kernels
            else:
                dim, vdim = pick([4, 8, 12, 20, 24, 40]), pick([8, 12, 16, 24, 36, 72])
            rot = (float(rng.choice([100.0, 10000.0, 1e6])), pick([d for d in (2, 4, 8, 12, 16, 32, 64) if d <= dim])) \
                if rng.random() < 0.85 else None
            layers.append(gazezen_configs.attention(heads, groups, dim, vdim, scale, window=window, rot=rot, mlp=feed_forward()))
        else:
            if rng.random() < 0.5:
                dim, rot_dim, vdim, rank = pick([16, 32, 64]), pick([16, 32, 64]), pick([16, 32, 64, 128]), pick([32, 64, 128])
            else:
                dim, rot_dim, vdim, rank = pick([4, 12, 20, 40]), pick([2, 4, 12, 24]), pick([8, 12, 36]), pick([8, 20, 28, 72])
            scaling = (float(rng.choice([2.0, 4.0, 8.0, 40.0])), float(rng.choice([32.0, 64.0, 512.0])),
                       float(rng.choice([4.0, 8.0, 32.0])), float(rng.choice([0.5, 1.0, 2.0]))) if rng.random() < 0.6 else None
            layers.append(gazezen_configs.latent(pick([1, 2, 3, 4, 8]), dim, rot_dim, vdim, rank, scale,
                                                 float(rng.choice([50.0, 10000.0, 1e6])), window=window, scaling=scaling,
                                                 mlp=feed_forward()))
    loop = None
    if rng.random() < 0.7:
        start = pick(range(len(layers)))
        loop = (start, pick(range(start + 1, len(layers) + 1)), pick([1, 2, 3]))
    return gazezen_configs.model(pick(range(61, 400)), width, float(rng.choice([1e-6, 1e-5, 3e-5])), layers,
                                 logit_scale=float(rng.choice([0.25, 1.0, 3.0])) if rng.random() < 0.7 else None,
                                 loop=loop, positions=1536)


# In bfloat16 a router's choice between experts whose scores lie closer together than the rounding of its input may
# fall the other way, and attention carries the difference to every later token. The plain model therefore takes
# the engine's choice at such a token, but only if tilting the scores by this factor towards it makes it the plain
# model's own choice; any other difference of choices stays a difference of logits.
CLOSE_CALL = 0.03


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(DRAWS))
def test_random_configuration(seed, dtype, record_property, monkeypatch):
    from kidi_b200 import Engine, StepBatch
    from kidi_b200.kernels import routed
    config = draw(seed)
    tensors = gazezen_configs.tensors(config, 50 + seed)
    length = 1100 if seed in (2, 5) else 60 + 31 * seed
    tokens = np.random.default_rng(seed).integers(0, config["vocab"], size=length + 8).tolist()
    calls, route = [], routed.route

    def recorded(x, *args, **kwargs):
        chosen, weight = route(x, *args, **kwargs)
        calls.append(chosen.clone())
        return chosen, weight

    monkeypatch.setattr(routed, "route", recorded)
    engine = Engine.from_config(config, tensors=tensors, dtype=dtype, max_tokens=4096)
    slot = engine.acquire()
    cut = length // 3
    rows = [engine.step(StepBatch([slot], [tokens[:cut]], [list(range(cut))])).double().cpu(),
            engine.step(StepBatch([slot], [tokens[cut:length]], [list(range(length - cut))])).double().cpu()]
    rows += [engine.step(StepBatch([slot], [[token]], None)).double().cpu() for token in tokens[length:]]
    engine.release(slot)
    engine.check_device_errors()
    got = torch.cat(rows)
    assert torch.isfinite(got).all()
    choices = None
    if dtype == "bfloat16":
        # every step calls the router once for every run of a layer with a feed-forward, in the order they run
        runs = sum(config["layers"][index]["mlp"] is not None for index, _ in plain_gazezen.run_order(config))
        assert runs == 0 or len(calls) == runs * len(rows)
        choices = [torch.cat([calls[step * runs + run].cpu() for step in range(len(rows))]) for run in range(runs)]
        assert all(chosen.shape[0] == len(tokens) for chosen in choices)
    want = plain_gazezen.forward(config, tensors, tokens, dtype=torch.float64, choices=choices, margin=CLOSE_CALL)
    worst_rows = (got - want).abs().max(-1).values / want.abs().max()
    largest = float(worst_rows.max())
    mean = float((got - want).pow(2).mean().sqrt() / want.pow(2).mean().sqrt())
    record_property("largest and mean relative difference", (largest, mean))
    assert largest < (1e-4 if dtype == "float32" else 0.4) and mean < (2e-5 if dtype == "float32" else 0.08), \
        (config, largest, mean)
