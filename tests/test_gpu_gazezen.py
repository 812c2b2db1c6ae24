"""Gazezen on the GPU against the plain implementation (tests/plain_gazezen.py, float64, whole sequences): each
mechanism alone, whole prompts, prompts then token-by-token decoding across page borders, portions down to two
tokens, batches of unequal requests against each alone, slots and pages that are used again, keys far away and
just inside and just outside a window (in prompts and decoded), a window that passes over decoded tokens, the
sink and the head gates made to matter, the first tokens of a sequence, a looped range with a cache per pass, and
greedy generation through `Engine.generate`, the command line and the trace runner. Weights and configurations
are the tests' own (tests/gazezen_configs.py)."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import gazezen_configs
import plain_gazezen

pytestmark = pytest.mark.gpu

# Bounds on a request's logits (the models' largest logits are 10 to 20): the largest difference relative to the
# largest logit, and the root mean square of the differences relative to that of the logits.
BOUND = {"float32": 2e-5, "bfloat16": 0.06}
LARGEST = {"float32": 8e-5, "bfloat16": 0.3}
GREEDY = {"float32": 2e-5, "bfloat16": 0.04}      # two logits closer than this (relative to the largest) may swap


def make(name, dtype, seed=1, max_tokens=2048, config=None, tensors=None):
    from kidi_b200 import Engine
    config = config or gazezen_configs.ALL[name]
    tensors = tensors or gazezen_configs.tensors(config, seed)
    engine = Engine.from_config(config, tensors=tensors, dtype=dtype, max_tokens=max_tokens)
    return engine, config, tensors


def prompt(config, length, seed):
    return np.random.default_rng(seed).integers(0, config["vocab"], size=length).tolist()


def plain(config, tensors, tokens):
    return plain_gazezen.forward(config, tensors, tokens, dtype=torch.float64)


def run(engine, slot, tokens, want=None):
    from kidi_b200 import StepBatch
    want = list(range(len(tokens))) if want is None else want
    return engine.step(StepBatch([slot], [list(tokens)], [want])).double().cpu()


def close(got, want, dtype, record=None, what="", slack=1.0):
    """Every row within the bounds in 32-bit. In bfloat16 a router's choice between two experts whose scores lie
    closer together than the rounding of its input may fall the other way, which moves that row's logits as a
    whole: one row in forty (at least one) may lie outside, and the bounds hold for the others."""
    assert torch.isfinite(got).all(), what
    scale, level = float(want.abs().max()), float(want.pow(2).mean().sqrt())
    worst_rows = (got - want).abs().max(-1).values / scale
    mean_rows = (got - want).pow(2).mean(-1)
    spared = 0 if dtype == "float32" else max(1, got.shape[0] // 40)
    kept = torch.argsort(worst_rows)[:max(1, got.shape[0] - spared)] if got.shape[0] > 1 else torch.arange(1)
    worst, mean = float(worst_rows[kept].max()), float(mean_rows[kept].mean().sqrt()) / level
    if record is not None:
        record(f"largest and mean relative difference {what}".strip(), (worst, mean))
    assert worst < slack * LARGEST[dtype] and mean < slack * BOUND[dtype], (what, worst, mean, scale)


def nearer(got, want, others, what, rows=slice(None)):
    """`got` lies nearer to `want` than to any model of `others` (plain models with one constant changed)."""
    right = float((got[rows] - want[rows]).pow(2).mean().sqrt())
    for index, other in enumerate(others):
        assert right < 0.5 * float((got[rows] - other[rows]).pow(2).mean().sqrt()), (what, index)


def in_steps(engine, tokens, sizes):
    slot = engine.acquire()
    rows, at = [], 0
    for size in sizes:
        rows.append(run(engine, slot, tokens[at:at + size]))
        at += size
    assert at == len(tokens)
    engine.release(slot)
    return torch.cat(rows)


def decoded(engine, tokens, head):
    slot = engine.acquire()
    rows = [run(engine, slot, tokens[:head])] + [run(engine, slot, [token]) for token in tokens[head:]]
    engine.release(slot)
    return torch.cat(rows)


# ------------------------------------------------------------------ each mechanism alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_small_kernels(dtype):
    """The exact gelu, the gate on heads, the vector added to every row, the constant on the logits, and the two
    layer norms around a residual sum in one kernel: each against its formula."""
    from kidi_b200.kernels import ops
    generator = torch.Generator().manual_seed(3)
    tolerance = 1e-6 if dtype == torch.float32 else 3e-2
    for count in (37, 4096 + 8):
        z = (torch.randn(count, generator=generator) * 3).to(dtype).cuda()
        want = plain_gazezen.gelu_erf(z.double().cpu())
        assert torch.allclose(ops.gelu(z).double().cpu(), want, atol=tolerance)
    assert abs(float(ops.gelu(torch.tensor([1.0], dtype=dtype).cuda())[0]) - 0.8413447) < (1e-6 if dtype == torch.float32 else 4e-3)
    for heads, width in ((3, 20), (4, 64)):
        x = torch.randn(9, heads * width, generator=generator).to(dtype).cuda()
        logits = (torch.randn(9, heads, generator=generator) * 3).to(dtype).cuda()
        want = (x.double().cpu().view(9, heads, width) * torch.sigmoid(logits.double().cpu())[:, :, None]).view(9, -1)
        assert torch.allclose(ops.head_gate(x.clone(), logits, heads, width).double().cpu(), want, atol=tolerance)
    stream = torch.randn(6, 40, generator=generator).cuda()
    vector = torch.randn(40, generator=generator).to(dtype).cuda()
    want = stream.double().cpu() + vector.double().cpu()
    ops.add_vector(stream, vector)
    assert torch.allclose(stream.double().cpu(), want, atol=1e-6)
    logits = torch.randn(5, 33, generator=generator).cuda()
    assert torch.allclose(ops.scale(logits.clone(), 0.37).cpu(), logits.cpu() * 0.37, atol=1e-6)
    for hidden in (40, 72, 256):
        residual = (torch.randn(11, hidden, generator=generator) * 2 + 0.7).cuda()
        delta = (torch.randn(11, hidden, generator=generator) * 5 - 1.0).to(dtype).cuda()
        inner, outer = ((torch.randn(hidden, generator=generator) * 0.3 + 1).cuda() for _ in range(2))
        summed = residual.double().cpu() + plain_gazezen.centred_norm(delta.double().cpu(), inner.double().cpu(), 1e-3)
        want = plain_gazezen.centred_norm(summed, outer.double().cpu(), 1e-5)
        got = ops.add_layernorm(residual, delta, outer, None, 1e-5, dtype, delta_weight=inner, delta_eps=1e-3)
        assert torch.allclose(residual.double().cpu(), summed, atol=2e-5)          # the stream itself stays 32-bit
        assert torch.allclose(got.double().cpu(), want, atol=2e-5 if dtype == torch.float32 else 4e-2)


def test_the_gelu_behind_a_product_of_few_rows():
    """The weight-streaming product with the exact gelu in its epilogue against gelu(x W^T), 1 to 64 rows."""
    from kidi_b200.kernels import skinny
    generator = torch.Generator().manual_seed(5)
    for rows, features, inner in ((1, 40, 64), (8, 96, 72), (33, 200, 256), (64, 24, 128)):
        x = torch.randn(rows, inner, generator=generator).to(torch.bfloat16).cuda()
        w = (torch.randn(features, inner, generator=generator) * 2 / inner ** 0.5).to(torch.bfloat16).cuda()
        want = plain_gazezen.gelu_erf(x.double().cpu() @ w.double().cpu().t())
        got = skinny.gemm(x, w, torch.bfloat16, activation="gelu").double().cpu()
        assert torch.allclose(got, want, atol=2e-2, rtol=1e-2), (rows, features, inner)
        assert float((got - want).abs().mean()) < 3e-3


@pytest.mark.parametrize("experts,top,groups,keep", [(6, 2, 3, 2), (10, 4, 2, 1), (12, 3, 4, 2), (16, 2, 4, 1), (5, 5, 1, 1),
                                                     (9, 1, 3, 3), (64, 6, 8, 3)])
def test_the_router_alone(experts, top, groups, keep):
    """Softmax over all experts, the best groups kept, the largest scores among them, divided by their sum: the
    choice and the weights of every row against the plain function. On some rows the groups matter: one of the
    largest scores lies in a group that is not kept."""
    from kidi_b200.kernels import routed
    generator = torch.Generator().manual_seed(experts + top)
    hidden, rows = 24, 200
    router = torch.randn(experts, hidden, generator=generator) * 0.8
    x = torch.randn(rows, hidden, generator=generator)
    scores = torch.softmax(x.double() @ router.double().t(), -1)
    chosen, weight = routed.route(x.cuda(), router.cuda(), top, True, "softmax", groups, keep, 1e-20)
    chosen, weight = chosen.cpu(), weight.double().cpu()
    limited = 0
    for row in range(rows):
        want = plain_gazezen.choose(scores[row], top, {"count": groups, "keep": keep} if groups > 1 else None)
        assert sorted(chosen[row].tolist()) == sorted(want.tolist()), row
        limited += sorted(want.tolist()) != sorted(torch.topk(scores[row], top).indices.tolist())
        picked = scores[row, chosen[row].long()]
        assert torch.allclose(weight[row], picked / picked.sum(), atol=1e-6)
    # the groups change some row's choice (they cannot where as many groups are kept as experts are taken)
    assert limited > 0 or keep == groups or keep >= top


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,groups,keep,rows,inter,shared", [
    (6, 2, 3, 2, 5, 24, 40), (4, 4, 1, 1, 300, 24, None), (16, 2, 4, 1, 200, 24, 8), (8, 3, 4, 3, 64, 40, 24),
    (4, 2, 2, 1, 150, 20, 36), (16, 2, 4, 2, 700, 64, 64)])
@pytest.mark.parametrize("lopsided", [False, True])
def test_routed_experts_alone(dtype, experts, top, groups, keep, rows, inter, shared, lopsided):
    """The feed-forward part alone (router, plain gelu experts weighted on their results, the shared expert added)
    on few rows and many, decoding and prompts, against the plain function. `lopsided`: every row chooses expert 0
    among its experts, so that one expert has several times the mean count of rows."""
    from types import SimpleNamespace
    from kidi_b200.parts.base import BuildEnv
    from kidi_b200.parts.routed import RoutedExperts
    from kidi_b200.parts.spec import PartSpec
    hidden = 64
    generator = torch.Generator().manual_seed(experts * 10 + top)
    w = {"m.router": torch.randn(experts, hidden, generator=generator) * 0.5}
    names = [f"e{e}" for e in range(experts)] + (["shared"] if shared else [])
    for name in names:
        ff = shared if name == "shared" else inter
        w[f"m.{name}.up"] = torch.randn(ff, hidden, generator=generator) * 0.3
        w[f"m.{name}.down"] = torch.randn(hidden, ff, generator=generator) * 0.3
    h = torch.randn(rows, hidden, generator=generator)
    if lopsided:
        w["m.router"][0, 0] = 2.0
        h[:, 0] += 4.0
    w = {name: tensor.to(dtype) for name, tensor in w.items()}
    h = h.to(dtype)
    mlp = {"router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}},
           "shared": {"ff": shared} if shared else None}
    want = plain_gazezen.routed_feed_forward(h.double(), {n: t.double() for n, t in w.items()}, "m.", mlp)
    part = RoutedExperts(PartSpec("routed_experts", {
        "hidden_size": hidden, "expert_size": inter, "experts": experts, "top": top, "score": "softmax",
        "renormalise": True, "renormalise_eps": 1e-20, "weight_on": "output", "groups": groups, "keep_groups": keep,
        "expert_form": "plain", "shared_size": shared}, "m."),
        BuildEnv(dtype=dtype, device=torch.device("cuda"), max_positions=16))
    bound = {"router": w["m.router"].cuda(),
             "experts.gate_up": torch.cat([w[f"m.e{e}.up"] for e in range(experts)]).cuda(),
             "experts.down": torch.cat([w[f"m.e{e}.down"] for e in range(experts)]).cuda()}
    if shared:
        bound["shared.up"], bound["shared.down"] = w["m.shared.up"].cuda(), w["m.shared.down"].cuda()
    part.bind(bound)
    tolerance = 2e-5 if dtype == torch.float32 else 0.08
    scale = float(want.abs().max())
    for decode in (False, True):
        ctx = SimpleNamespace(plan=SimpleNamespace(is_decode=decode))
        found = part.forward(h.cuda(), ctx).double().cpu()
        # a row whose choice is a close call may take another expert in bfloat16: at most a few rows differ
        bad = ((found - want).abs().max(-1).values > tolerance * scale).sum()
        assert int(bad) <= (0 if dtype == torch.float32 else max(1, rows // 50)), (decode, int(bad))


def one_attention(window, heads=2, kv_heads=1, dim=16, vdim=32, rot=(10000.0, 8), mlp=None, scale=0.4):
    return gazezen_configs.model(61, 48, 1e-5, [
        gazezen_configs.attention(heads, kv_heads, dim, vdim, scale, window=window, rot=rot, mlp=mlp)], positions=700)


def one_latent(window, heads=2, dim=16, rot_dim=16, vdim=16, rank=24, scaling=None, mlp=None, base=1000.0):
    return gazezen_configs.model(61, 48, 1e-5, [
        gazezen_configs.latent(heads, dim, rot_dim, vdim, rank, 0.3, base, window=window, scaling=scaling, mlp=mlp)],
        positions=700)


WINDOW_LAYERS = {
    "attention": lambda: one_attention(37),                                   # widths of the tensor-core kernels
    "attention, other widths": lambda: one_attention(37, heads=3, kv_heads=3, dim=12, vdim=20, rot=(300.0, 12)),
    "latent": lambda: one_latent(37),
    "latent, other widths": lambda: one_latent(37, heads=3, dim=12, rot_dim=4, vdim=20, rank=28),
    "latent, wide": lambda: one_latent(37, heads=2, dim=32, rot_dim=32, vdim=64, rank=64,
                                       scaling=(4.0, 64.0, 8.0, 1.0)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", sorted(WINDOW_LAYERS))
def test_window_edges(dtype, kind, record_property):
    """One layer with a window of 37. The plain model with a window one token shorter or longer differs clearly at
    the rows that are checked, so a key that is wrongly seen or missed at the edge shows. Checked in a whole prompt,
    in portions whose cuts fall before and after the edge, and decoded one by one over 120 tokens (the window
    passes over decoded tokens and page borders)."""
    config = WINDOW_LAYERS[kind]()
    tensors = gazezen_configs.tensors(config, 21, sharp=0.05)     # soft scores: every key of a window counts
    tokens = prompt(config, 200, 5)
    want = plain(config, tensors, tokens)
    wrong = []
    for window in (36, 38):
        other = copy.deepcopy(config)
        other["layers"][0]["mixer"]["mask"] = {"size": window}
        wrong.append(plain(other, tensors, tokens))
        moved = (wrong[-1][60:] - want[60:]).abs().max(-1).values / float(want.abs().max())
        assert float(moved.median()) > 20 * LARGEST["float32"], (window, float(moved.median()))
    assert torch.equal(wrong[0][:36], want[:36])                    # the first rows see everything either way
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    for got, what in ((in_steps(engine, tokens, (200,)), "whole"),
                      (in_steps(engine, tokens, (2, 2, 33, 1, 26, 64, 5, 67)), "portions"),
                      (decoded(engine, tokens, 80), "decoded")):
        close(got, want, dtype, record_property, what)
        nearer(got, want, wrong, what, slice(60, None))
    engine.cache.check()
    engine.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["attention", "latent"])
@pytest.mark.parametrize("window", [None, 445])
def test_far_keys_reach_the_last_rows(dtype, kind, window, record_property):
    """449 tokens, seven pages of the cache, soft scores (every key has its share of a row). Another token at
    position 2 moves those of the plain model's last rows that see it: all of them without a window, and with a
    window of 445 the rows up to position 446, while the last two rows stay as they are. So a far key that is lost, read from a wrong page, or kept a
    token too long shows: whole, and with the last eight tokens decoded one by one."""
    config = one_attention(window, heads=4, kv_heads=2) if kind == "attention" else one_latent(window, heads=4)
    tensors = gazezen_configs.tensors(config, 31, sharp=0.05)
    tokens = prompt(config, 449, 7)
    want = plain(config, tensors, tokens)
    other = plain(config, tensors, tokens[:2] + [(tokens[2] + 1) % config["vocab"]] + tokens[3:])
    seeing = slice(-8, None) if window is None else slice(-8, -2)
    moved = float((other[seeing] - want[seeing]).abs().max(-1).values.min()) / float(want.abs().max())
    record_property("what the far token moves at least", moved)
    assert moved > 20 * LARGEST["float32"]
    if window is not None:
        assert torch.equal(other[-2:], want[-2:])
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    slot = engine.acquire()
    whole = run(engine, slot, tokens)
    engine.release(slot)
    slot = engine.acquire()
    run(engine, slot, tokens[:-8], want=[])
    last = torch.cat([run(engine, slot, [token]) for token in tokens[-8:]])
    engine.release(slot)
    for got, what in ((whole[-8:], "whole"), (last, "decoded")):
        close(got, want[-8:], dtype, record_property, what)
        if dtype == "float32":
            nearer(got, want[-8:], [other[-8:]], what, seeing if window is None else slice(0, 6))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim,heads,kv_heads", [(16, 32, 4, 2), (12, 20, 3, 1), (64, 64, 2, 2)])
def test_the_sink_and_the_head_gates_matter(dtype, dim, vdim, heads, kv_heads, record_property):
    """One attention layer with large sinks. Plain models without the sink, with the sink multiplied by the
    score's scale, with the sink counted twice, and with gates that are all one half differ clearly; the engine
    agrees with the right one, in a prompt, in portions and decoded."""
    config = one_attention(50, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=(10000.0, dim // 2))
    tensors = gazezen_configs.tensors(config, 12, sharp=0.05)
    tensors["l0.mix.sink"] = (tensors["l0.mix.sink"].float() * 1.5 + 2.0).to(torch.bfloat16)
    tokens = prompt(config, 120, 9)
    want = plain(config, tensors, tokens)
    wrong = []
    for change in ("none", "scaled", "twice", "half"):
        other = dict(tensors)
        if change == "none":
            del other["l0.mix.sink"]
        elif change == "scaled":
            other["l0.mix.sink"] = tensors["l0.mix.sink"].double() * config["layers"][0]["mixer"]["scale"]
        elif change == "twice":
            other["l0.mix.sink"] = tensors["l0.mix.sink"].double() + math.log(2.0)
        else:
            other["l0.mix.g"] = torch.zeros_like(tensors["l0.mix.g"])
        wrong.append(plain(config, other, tokens))
        moved = (wrong[-1] - want).abs().max(-1).values / float(want.abs().max())
        assert float(moved.median()) > 20 * LARGEST["float32"], (change, float(moved.median()))
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    for got, what in ((in_steps(engine, tokens, (120,)), "whole"), (in_steps(engine, tokens, (1, 1, 2, 60, 3, 53)), "portions"),
                      (decoded(engine, tokens, 1), "decoded from the second token")):
        close(got, want, dtype, record_property, what)
        nearer(got, want, wrong, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stretched_frequencies_and_the_shared_rotated_key(dtype, record_property, monkeypatch):
    """One latent layer whose frequencies are stretched, over 300 positions. Plain models with plain frequencies,
    with the ramp one pair further along, and with cosine and sine left at length one differ clearly; the engine
    agrees with the right one."""
    config = one_latent(None, heads=2, dim=16, rot_dim=16, vdim=16, rank=24, scaling=(8.0, 64.0, 8.0, 1.0), base=10000.0)
    tensors = gazezen_configs.tensors(config, 14, sharp=0.3)
    tokens = prompt(config, 300, 3)
    want = plain(config, tensors, tokens)
    unscaled = copy.deepcopy(config)
    del unscaled["layers"][0]["mixer"]["rot"]["scaling"]
    shifted = copy.deepcopy(config)              # the ramp one pair further along
    shifted["layers"][0]["mixer"]["rot"]["scaling"].update(fast=2.0, slow=0.25)
    wrong = [plain(unscaled, tensors, tokens), plain(shifted, tensors, tokens)]
    stretched = plain_gazezen.frequencies
    monkeypatch.setattr(plain_gazezen, "frequencies", lambda rot, dtype: (stretched(rot, dtype)[0], 1.0))
    wrong.append(plain(config, tensors, tokens))             # the right frequencies, cosine and sine of length one
    monkeypatch.setattr(plain_gazezen, "frequencies", stretched)
    for index, other in enumerate(wrong):
        moved = (other[100:] - want[100:]).abs().max(-1).values / float(want.abs().max())
        assert float(moved.median()) > 20 * LARGEST["float32"], (index, float(moved.median()))
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    for got, what in ((in_steps(engine, tokens, (300,)), "whole"), (in_steps(engine, tokens, (150, 2, 148)), "portions"),
                      (decoded(engine, tokens, 260), "decoded")):
        close(got, want, dtype, record_property, what)
        nearer(got, want, wrong, what, slice(100, None))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_looped_range_keeps_a_cache_per_pass(dtype, record_property):
    """Two layers, the second run three times: each pass has keys of its own, so decoding after a prompt agrees
    with the whole sequence only if no pass reads or overwrites another's. Plain models with the passes' vectors
    in another order, or added at every layer of the range, differ clearly."""
    config = gazezen_configs.model(61, 48, 1e-5, [
        gazezen_configs.attention(2, 1, 16, 16, 0.4, window=45, rot=(100.0, 16),
                                  mlp=gazezen_configs.routed(4, 2, 16, groups=(2, 1), shared=16)),
        gazezen_configs.latent(2, 16, 8, 16, 32, 0.3, 200.0, window=30),
        gazezen_configs.attention(2, 2, 16, 16, 0.4, rot=(100.0, 8))], loop=(1, 3, 3), positions=600, logit_scale=0.5)
    tensors = gazezen_configs.tensors(config, 5)
    tokens = prompt(config, 160, 2)
    want = plain(config, tensors, tokens)
    turned = dict(tensors)
    turned["loop.step"] = tensors["loop.step"].flip(0)
    once = copy.deepcopy(config)
    once["loop"]["times"] = 2
    wrong = [plain(config, turned, tokens), plain(once, tensors, tokens)]
    for other in wrong:
        assert float(((other - want).abs().max(-1).values / want.abs().max()).median()) > 20 * LARGEST["float32"]
    engine, _, _ = make(None, dtype, config=config, tensors=tensors)
    for got, what in ((in_steps(engine, tokens, (160,)), "whole"), (in_steps(engine, tokens, (3, 70, 2, 85)), "portions"),
                      (decoded(engine, tokens, 60), "decoded")):
        close(got, want, dtype, record_property, what)
        nearer(got, want, wrong, what)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens(dtype, record_property):
    """Sequences of one, two and three tokens, and a sequence that starts in portions of one and two tokens: the
    first row sees itself and the sink only."""
    engine, config, tensors = make("small_a", dtype, seed=6)
    for length in (1, 2, 3):
        tokens = prompt(config, length, length)
        close(in_steps(engine, tokens, (length,)), plain(config, tensors, tokens), dtype, record_property, f"{length} tokens")
    tokens = prompt(config, 12, 8)
    close(in_steps(engine, tokens, (1, 1, 2, 1, 2, 5)), plain(config, tensors, tokens), dtype, record_property, "short portions")
    close(decoded(engine, tokens, 1), plain(config, tensors, tokens), dtype, record_property, "decoded from the start")


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(gazezen_configs.ALL))
def test_whole_prompts_and_decoding(name, dtype, record_property):
    """A whole prompt in one step (its first tokens included), then the same request with its last 100 tokens one
    by one (past page borders of the cache and past the windows), then in portions of 2 to 64 tokens."""
    engine, config, tensors = make(name, dtype)
    tokens = prompt(config, 230, 11)
    want = plain(config, tensors, tokens)
    assert float(want.abs().max()) > 5
    close(in_steps(engine, tokens, (230,)), want, dtype, record_property, "whole")
    close(decoded(engine, tokens, 130), want, dtype, record_property, "decoded")
    close(in_steps(engine, tokens, (2, 3, 64, 61, 2, 1, 17, 80)), want, dtype, record_property, "portions")
    engine.cache.check()
    engine.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, record_property):
    """400 tokens decoded one by one after a prompt of 20: every window passes over decoded tokens only, and the
    cache grows by six pages while decoding."""
    engine, config, tensors = make("small_b", dtype, seed=3)
    tokens = prompt(config, 420, 13)
    close(decoded(engine, tokens, 20), plain(config, tensors, tokens), dtype, record_property, "decoded")
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small_a", "wide"])
def test_batches_of_unequal_requests(name, dtype, record_property):
    """Requests of 1, 70 and 131 tokens start together and are decoded together; the shortest ends first and a new
    request takes its slot and pages at once. Every request's logits equal those it gets alone."""
    from kidi_b200 import StepBatch
    engine, config, tensors = make(name, dtype, seed=2, max_tokens=2048)
    slot = engine.acquire()                     # a request that ran before leaves keys and pages behind
    run(engine, slot, prompt(config, 200, 3))
    engine.release(slot)
    requests = [prompt(config, n, 20 + n) for n in (9, 78, 139)]
    starts = [1, 70, 131]
    want = [plain(config, tensors, tokens) for tokens in requests]
    slots = [engine.acquire() for _ in requests]
    got = [[] for _ in requests]
    logits = engine.step(StepBatch(slots, [r[:s] for r, s in zip(requests, starts)],
                                   [list(range(s)) for s in starts])).double().cpu()
    at = 0
    for i, s in enumerate(starts):
        got[i].append(logits[at:at + s])
        at += s
    live = [0, 1, 2]
    for step in range(8):
        logits = engine.step(StepBatch([slots[i] for i in live], [[requests[i][starts[i] + step]] for i in live],
                                       [[0] for _ in live])).double().cpu()
        for row, i in enumerate(live):
            got[i].append(logits[row:row + 1])
        if step == 3:
            engine.release(slots[0])
            live = [1, 2]
            other = engine.acquire()
            assert other == slots[0]
            fresh = prompt(config, 66, 77)
            close(run(engine, other, fresh), plain(config, tensors, fresh), dtype, None, "a reused slot")
            engine.release(other)
    for i in range(3):
        found = torch.cat(got[i])
        close(found, want[i][:found.shape[0]], dtype, record_property, f"request {i} in a batch")
    engine.cache.check()


def test_batches_and_portions_leave_32_bit_logits_alone():
    """In 32-bit a request's logits alone, in a batch, and in portions agree far below the bound against the
    plain model (the sums run in the same order whatever else the step holds)."""
    from kidi_b200 import StepBatch
    engine, config, tensors = make("small_a", "float32", seed=4)
    a, b = prompt(config, 90, 1), prompt(config, 33, 2)
    sa, sb = engine.acquire(), engine.acquire()
    both = engine.step(StepBatch([sa, sb], [a, b], [list(range(90)), list(range(33))])).double().cpu()
    engine.release(sa), engine.release(sb)
    alone = in_steps(engine, a, (90,))
    parts = in_steps(engine, a, (50, 40))
    scale = float(alone.abs().max())
    assert float((both[:90] - alone).abs().max()) < 4e-6 * scale
    assert float((parts - alone).abs().max()) < 4e-6 * scale


def test_which_kernels_run(record_property):
    """The bfloat16 engine takes the tensor-core attention kernels where a layer's widths allow (prompts and
    decoding) and the general kernel elsewhere; the 32-bit engine takes the general kernels and the 32-bit product
    only. The forms agree within rounding."""
    from kidi_b200.kernels import ops
    engine, config, tensors = make("wide", "bfloat16", seed=3)
    tokens = prompt(config, 300, 5)
    want = plain(config, tensors, tokens)
    slot = engine.acquire()
    with ops.record_launches() as names:
        run(engine, slot, tokens[:299], want=[])
    record_property("prompt kernels", sorted(set(names)))
    assert "attention_generic" not in names and any(name.startswith("attention_prefill") for name in names)
    assert "latent_pack" in names                      # a prompt from position 0: keys and values unfolded per head
    with ops.record_launches() as names:
        last = run(engine, slot, tokens[299:])
    record_property("decode kernels", sorted(set(names)))
    assert "attention_generic" not in names and names.count("expert_slots") == 8       # four layer runs loop thrice
    assert any(name.startswith("latent_attention[mma.sync") for name in names)     # decoding reads the latents alone
    engine.release(slot)
    close(last, want[299:], "bfloat16", record_property, "decoded", slack=2.0)
    engine32, _, _ = make("wide", "float32", seed=3)
    slot = engine32.acquire()
    with ops.record_launches() as names:
        run(engine32, slot, tokens)
    assert "library_mm" not in names and "library_bmm" not in names
    assert not any("tensor" in name or "tcgen05" in name or "skinny" in name or "mma" in name for name in names)


def teacher_forced(config, tensors, request, tokens, bound):
    """(close calls, misses): tokens whose two best logits lie closer than the bound (either may be taken), and
    tokens that are not the plain model's choice although it was clear."""
    logits = plain(config, tensors, list(request) + list(tokens))[len(request) - 1:-1].numpy()
    close_calls = misses = 0
    for place, token in enumerate(tokens):
        row = logits[place]
        best, second = np.sort(row)[-1], np.sort(row)[-2]
        margin = bound * float(np.abs(row).max())
        if best - second >= margin:
            misses += token != int(np.argmax(row))
        else:
            close_calls += 1
            misses += row[token] < best - margin
    return close_calls, misses


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("use_graph", [True, False])
@pytest.mark.parametrize("name", ["small_b", "wide"])
def test_greedy_generation_through_the_engine(name, dtype, use_graph):
    """`Engine.generate`: batches of unequal prompts, decode steps replayed as a captured graph (with padding rows:
    three live sequences in four rows), slots reused by the next batch."""
    config = gazezen_configs.ALL[name]
    tensors = gazezen_configs.tensors(config, 7, logits=12.0)
    engine, _, _ = make(None, dtype, config=config, tensors=tensors, max_tokens=2048)
    requests = [prompt(config, n, 40 + n) for n in (5, 1, 70, 12, 33)]
    found = engine.generate(requests, max_new_tokens=12, ignore_eos=True, max_active=3, use_graph=use_graph)
    counts = [teacher_forced(config, tensors, r, t, GREEDY[dtype]) for r, t in zip(requests, found)]
    close_calls, misses = sum(c for c, _ in counts), sum(m for _, m in counts)
    # in bfloat16 a router's close call may fall the other way and cost that token
    assert all(len(tokens) == 12 for tokens in found) and close_calls <= 30 and misses <= (0 if dtype == "float32" else 2)
    again = engine.generate(requests[:2], max_new_tokens=12, ignore_eos=True, use_graph=use_graph)
    if dtype == "float32":
        assert again == found[:2]
    engine.cache.check()
    assert not engine.cache.slots.held
    engine.check_device_errors()


def write_folder(folder, config, tensors):
    from kidi_b200.weights.safetensors_io import write_safetensors
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(str(folder / "model.safetensors"), tensors, metadata={"format": "pt"})


def test_the_command_line_generates(tmp_path, capsys):
    import kidi_b200
    config = gazezen_configs.SMALL_A
    tensors = gazezen_configs.tensors(config, 8, logits=12.0)
    write_folder(tmp_path / "model", config, tensors)
    requests = [prompt(config, n, n) for n in (4, 19)]
    (tmp_path / "in.jsonl").write_text("".join(json.dumps({"token_ids": r, "id": str(i)}) + "\n"
                                              for i, r in enumerate(requests)))
    code = kidi_b200.main(["generate", "-m", str(tmp_path / "model"), "-i", str(tmp_path / "in.jsonl"), "-o",
                           str(tmp_path / "out.jsonl"), "--max-new-tokens", "6", "--ignore-eos", "--precision", "fp32"])
    assert code == 0, capsys.readouterr().err
    records = [json.loads(line) for line in (tmp_path / "out.jsonl").read_text().splitlines()]
    assert len(records) == 2
    for record in records:
        request = requests[int(record["id"])]
        assert teacher_forced(config, tensors, request, record["token_ids"], LARGEST["float32"]) == (0, 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_runner_replays_a_model_folder(tmp_path, dtype, record_property):
    """bin/trace_run on a Gazezen folder: three unequal requests start together (one of a single token), are decoded
    together until the shorter ones end, a step in which nothing is wanted, then a fourth request on what they gave
    back. `--max-tokens` is the tokens they hold, with no allowance for partly filled pages."""
    import os
    import subprocess
    import sys
    config = gazezen_configs.SMALL_A
    tensors = gazezen_configs.tensors(config, 9)
    write_folder(tmp_path / "model", config, tensors)
    a, b, c, d = (prompt(config, n, 60 + n) for n in (1, 75, 133, 90))
    want = {name: plain(config, tensors, tokens) for name, tokens in (("a", a), ("b", b), ("c", c), ("d", d))}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a, "want": [0]}, {"id": "b", "tokens": b[:70], "want": [0, 69]},
                                     {"id": "c", "tokens": c[:129], "want": [5, 128]}], "end": ["a"]}]
    for index in range(5):
        entries = [{"id": "b", "tokens": [b[70 + index]], "want": [0] if index != 2 else []}]
        if index < 4:
            entries.append({"id": "c", "tokens": [c[129 + index]], "want": [0] if index != 2 else []})
        steps.append({"step": 1 + index, "entries": entries, "end": ["c"] if index == 3 else ["b"] if index == 4 else []})
    steps.append({"step": 6, "entries": [{"id": "d", "tokens": d, "want": [0, 45, 89]}], "end": ["d"]})
    out = tmp_path / "out"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    result = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "model"), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(1 + 75 + 133)],
        input="\n".join(json.dumps(step) for step in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert result.returncode == 0, result.stderr
    assert result.stdout.split() == [word for step in steps for word in ("done", str(step["step"]))]
    read = lambda step: torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(-1, config["vocab"])).double()
    assert not (out / "3.f32").exists()                      # nothing was wanted in that step
    assert read(0).shape[0] == 5 and read(2).shape[0] == 2 and read(5).shape[0] == 1 and read(6).shape[0] == 3
    # the rows of all steps under one bound (in bfloat16 one row may rest on a router's close call)
    close(torch.cat([read(0), read(2), read(5), read(6)]),
          torch.cat([torch.stack([want["a"][0], want["b"][0], want["b"][69], want["c"][5], want["c"][128]]),
                     torch.stack([want["b"][71], want["c"][130]]), want["b"][74:75], want["d"][[0, 45, 89]]]),
          dtype, record_property, "prompts together, decoded together, the last one alone, on reused pages", slack=2.0)
