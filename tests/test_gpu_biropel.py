"""Biropel on the GPU against the plain implementation (tests/plain_biropel.py, float64, whole sequences): each
mechanism alone (the lanes' kernels, the short convolution with carried inputs, the recurrence kernel, one layer of
each kind against plain models with one constant changed), whole prompts, prompts then token-by-token decoding
across page borders, portions down to two tokens, batches of unequal requests against each alone, slots and pages
that are used again, keys far away and just inside and just outside a window (in prompts and decoded), windows that
pass over decoded tokens, layers that read another layer's keys, the first tokens of a sequence, and greedy
generation through `Engine.generate`, the command line and the trace runner. Weights and configurations are the
tests' own (tests/biropel_configs.py)."""
import copy
import json
import types

import numpy as np
import pytest
import torch

import biropel_configs as configs
import plain_biropel

pytestmark = pytest.mark.gpu

# Bounds on a request's logits (the models' largest logits are 10 to 20): the largest difference relative to the
# largest logit, and the root mean square of the differences relative to that of the logits.
BOUND = {"float32": 2e-5, "bfloat16": 0.06}
LARGEST = {"float32": 8e-5, "bfloat16": 0.3}
GREEDY = {"float32": 2e-5, "bfloat16": 0.04}      # two logits closer than this (relative to the largest) may swap


def make(config, dtype, seed=1, max_tokens=2048, tensors=None, **weights):
    from kidi_b200 import Engine
    tensors = tensors or configs.tensors(config, seed, **weights)
    return Engine.from_config(config, tensors=tensors, dtype=dtype, max_tokens=max_tokens), tensors


def prompt(config, length, seed):
    return np.random.default_rng(seed).integers(0, config["vocab"], size=length).tolist()


def plain(config, tensors, tokens):
    return plain_biropel.forward(config, tensors, tokens, dtype=torch.float64)


def run(engine, slot, tokens, want=None):
    from kidi_b200 import StepBatch
    want = list(range(len(tokens))) if want is None else want
    return engine.step(StepBatch([slot], [list(tokens)], [want])).double().cpu()


def close(got, want, dtype, record=None, what="", slack=1.0):
    assert torch.isfinite(got).all(), what
    scale, level = float(want.abs().max()), float(want.pow(2).mean().sqrt())
    worst = float((got - want).abs().max()) / scale
    mean = float((got - want).pow(2).mean().sqrt()) / level
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
    return in_steps(engine, tokens, [head] + [1] * (len(tokens) - head))


def changed(config, path, value):
    other = copy.deepcopy(config)
    node = other
    for key in path[:-1]:
        node = node[key]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return other


# ------------------------------------------------------------------ the kernels alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_lanes_kernels(dtype):
    """The weighted sum of lanes with its norm, the update of all lanes at once (from one matrix that stands for
    every lane, then in place), the sum of two normalised rows, the sigmoid gate and the squared relu."""
    from kidi_b200.kernels import ops
    generator = torch.Generator().manual_seed(3)
    loose = 1e-5 if dtype == torch.float32 else 3e-2
    for count, rows, hidden in ((1, 5, 40), (2, 9, 72), (3, 4, 256), (8, 3, 24), (2, 7, 30)):
        lanes = torch.randn(count, rows, hidden, generator=generator).cuda()
        read = torch.randn(count, generator=generator).cuda()
        weight = (torch.randn(hidden, generator=generator) * 0.3 + 1).to(dtype).cuda()
        u = (read.double().cpu()[:, None, None] * lanes.double().cpu()).sum(0)
        want = plain_biropel.rms_norm(u, weight.double().cpu(), 1e-5)
        assert torch.allclose(ops.lanes_rmsnorm(lanes, read, weight, 1e-5, dtype).double().cpu(), want, atol=loose)
        index = torch.tensor([rows - 1, 0], dtype=torch.int32).cuda()
        total = plain_biropel.rms_norm(lanes.double().cpu().sum(0), weight.double().cpu(), 1e-5)[[rows - 1, 0]]
        assert torch.allclose(ops.lanes_rmsnorm(lanes, None, weight, 1e-5, dtype, row_index=index).double().cpu(), total,
                              atol=loose)
        mix = torch.randn(count, count, generator=generator).cuda()
        write = torch.randn(count, generator=generator).cuda()
        y = torch.randn(rows, hidden, generator=generator).to(dtype).cuda()
        new = torch.einsum("st,srh->trh", mix.double().cpu(), lanes.double().cpu()) \
            + write.double().cpu()[:, None, None] * y.double().cpu()[None]
        target = torch.empty_like(lanes)
        ops.lanes_mix(lanes, target, mix, write, y)
        assert torch.allclose(target.double().cpu(), new, atol=1e-5)
        ops.lanes_mix(lanes, lanes, mix, write, y)                      # in place
        assert torch.allclose(lanes.double().cpu(), new, atol=1e-5)
        one = torch.randn(rows, hidden, generator=generator).cuda()     # one matrix that stands for every lane
        ops.lanes_mix(one.unsqueeze(0).expand(count, rows, hidden), target, mix, write, y)
        new = mix.double().cpu().sum(0)[:, None, None] * one.double().cpu()[None] \
            + write.double().cpu()[:, None, None] * y.double().cpu()[None]
        assert torch.allclose(target.double().cpu(), new, atol=1e-5)
        # update and read in one kernel: the same bits as the two kernels, also at picked rows (which leave the lanes)
        before = torch.randn(count, rows, hidden, generator=generator).cuda()
        apart = torch.empty_like(before)
        ops.lanes_mix(before, apart, mix, write, y)
        fused = before.clone()
        got = ops.lanes_mix_rmsnorm(fused, fused, mix, write, y, read, weight, 1e-5, dtype)
        assert torch.equal(fused, apart) and torch.equal(got, ops.lanes_rmsnorm(apart, read, weight, 1e-5, dtype))
        kept = before.clone()
        got = ops.lanes_mix_rmsnorm(kept, kept, mix, write, y, None, weight, 1e-5, dtype, row_index=index)
        assert torch.equal(kept, before) and torch.equal(got, ops.lanes_rmsnorm(apart, None, weight, 1e-5, dtype, row_index=index))
        a, b = (torch.randn(rows, hidden, generator=generator).mul(3).to(dtype).cuda() for _ in range(2))
        wa, wb = (torch.randn(hidden, generator=generator).mul(0.3).add(1).cuda() for _ in range(2))
        want = 0.5 * plain_biropel.rms_norm(a.double().cpu(), wa.double().cpu(), 1e-4) \
            + 0.5 * plain_biropel.rms_norm(b.double().cpu(), wb.double().cpu(), 1e-4)
        assert torch.allclose(ops.normed_pair_sum(a, b, wa, wb, 1e-4).double().cpu(), want, atol=1e-5)
        gate = torch.randn(rows, hidden, generator=generator).mul(3).to(dtype).cuda()
        want = a.double().cpu() * torch.sigmoid(gate.double().cpu())
        assert torch.allclose(ops.sigmoid_gate(a.clone(), gate).double().cpu(), want, atol=loose)
        want = torch.relu(b.double().cpu()) ** 2
        assert torch.allclose(ops.relu_squared(b).double().cpu(), want, atol=loose, rtol=1e-2)


def step_tables(lengths, starts, slots):
    """The device tables of a step that brings `lengths[b]` tokens to sequences that hold `starts[b]`."""
    row_seq, row_pos, row0, cursor = [], [], [], 0
    for index, (count, start) in enumerate(zip(lengths, starts)):
        row0.append(cursor)
        row_seq += [index] * count
        row_pos += list(range(start, start + count))
        cursor += count
    as_int = lambda values: torch.tensor(values, dtype=torch.int32).cuda()
    return types.SimpleNamespace(row_seq=as_int(row_seq), row_pos=as_int(row_pos), seq_slot=as_int(slots),
                                 seq_start=as_int(starts), seq_row0=as_int(row0), seq_len=as_int(lengths))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 9])
def test_the_short_convolution_carries_its_inputs(dtype, taps):
    """Two sequences in portions of unequal sizes (also shorter than the taps) against the convolution over each
    whole sequence; a slot's state is zero at the start."""
    from kidi_b200.kernels import scalar_recurrence as kernels
    generator = torch.Generator().manual_seed(taps)
    channels, lengths = 37, (23, 11)
    inputs = [torch.randn(n, channels, generator=generator).to(dtype) for n in lengths]
    weight = torch.randn(channels, taps, generator=generator)
    bias = torch.randn(channels, generator=generator)
    want = [torch.nn.functional.silu(plain_biropel.causal_conv(x.double(), weight.double(), bias.double())) for x in inputs]
    state = torch.zeros(5, max(taps - 1, 1), channels, dtype=dtype).cuda() if taps > 1 else None
    got, done = [[], []], [0, 0]
    for sizes in ((1, 3), (2, 1), (5, 2), (1, 1), (14, 4)):
        live = [b for b in (0, 1) if done[b] < lengths[b]]
        pieces = [inputs[b][done[b]:done[b] + sizes[b]] for b in live]
        tables = step_tables([len(piece) for piece in pieces], [done[b] for b in live], [3 if b == 0 else 1 for b in live])
        packed = torch.cat([torch.zeros(sum(len(p) for p in pieces), 3, dtype=dtype), torch.cat(pieces)], 1).cuda()
        out = kernels.short_conv(packed[:, 3:], weight.cuda(), bias.cuda(), state, silu=True, tables=tables,
                                 seqs=len(live), one_token=all(len(piece) == 1 for piece in pieces)).double().cpu()
        at = 0
        for b, piece in zip(live, pieces):
            got[b].append(out[at:at + len(piece)])
            at += len(piece)
            done[b] += len(piece)
    assert done == list(lengths)
    for b in (0, 1):
        assert torch.allclose(torch.cat(got[b]), want[b], atol=1e-5 if dtype == torch.float32 else 5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,k_heads,dim,vdim,extra", [(4, 2, 8, 12, 0), (3, 3, 20, 36, 1), (2, 1, 64, 64, 0),
                                                         (1, 1, 130, 5, 1), (6, 2, 5, 33, 0)])
def test_the_recurrence_kernel(dtype, heads, k_heads, dim, vdim, extra):
    """S_t = a_t S + b_t k_t (v_t, 1)^T, o_t = S_t^T (c q_t), in portions, against the loop over each sequence; the
    state of a slot carries from step to step, and portions change nothing (the same bits in 32-bit)."""
    from kidi_b200.kernels import scalar_recurrence as kernels
    generator = torch.Generator().manual_seed(dim)
    lengths, slots = (37, 1, 18), (2, 0, 4)
    total = sum(lengths)
    k = torch.randn(total, k_heads * dim, generator=generator).to(dtype)
    q = torch.randn(total, k_heads * dim, generator=generator).to(dtype)
    v = torch.randn(total, heads * vdim, generator=generator).to(dtype)
    coef = torch.stack([torch.rand(total, heads, generator=generator) * 0.5 + 0.5,
                        torch.rand(total, heads, generator=generator), torch.zeros(total, heads)], -1).contiguous()
    want, at = [], 0
    for count in lengths:
        out = torch.zeros(count, heads, vdim + extra, dtype=torch.float64)
        for h in range(heads):
            g = h // (heads // k_heads)
            S = torch.zeros(dim, vdim + extra, dtype=torch.float64)
            for t in range(count):
                row = at + t
                value = torch.cat([v[row, h * vdim:(h + 1) * vdim].double(), torch.ones(extra, dtype=torch.float64)])
                S = coef[row, h, 0].double() * S + coef[row, h, 1].double() * torch.outer(k[row, g * dim:(g + 1) * dim].double(), value)
                out[t, h] = S.t() @ (0.5 * q[row, g * dim:(g + 1) * dim].double())
        want.append(out.reshape(count, -1))
        at += count
    results = []
    for cuts in ((37, 1, 18), (5, 1, 2), None):
        state = torch.zeros(6, heads, dim, vdim + extra).cuda()
        pieces, done = [[] for _ in lengths], [0] * len(lengths)
        while any(d < n for d, n in zip(done, lengths)):
            live = [b for b, n in enumerate(lengths) if done[b] < n]
            sizes = [min(lengths[b] - done[b], cuts[b] if cuts else 1 + (done[b] * 7 + b) % 19) for b in live]
            rows = torch.cat([torch.arange(sum(lengths[:b]) + done[b], sum(lengths[:b]) + done[b] + n) for b, n in zip(live, sizes)])
            tables = step_tables(sizes, [done[b] for b in live], [slots[b] for b in live])
            out = kernels.scalar_recurrence(k[rows].cuda(), q[rows].cuda(), v[rows].cuda(), coef[rows].contiguous().cuda(),
                                            state, heads=heads, k_heads=k_heads, q_heads=k_heads, dim=dim, vdim=vdim,
                                            extra=extra, q_scale=0.5, tables=tables, seqs=len(live)).cpu()
            at = 0
            for b, n in zip(live, sizes):
                pieces[b].append(out[at:at + n])
                at += n
                done[b] += n
        results.append([torch.cat(p) for p in pieces])
    for found in results:
        for b in range(len(lengths)):
            assert torch.allclose(found[b].double(), want[b], atol=2e-4 * dim ** 0.5, rtol=1e-4)
            assert torch.equal(found[b], results[0][b])


# ------------------------------------------------------------------ one layer of each kind
LEFT = dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3)
LAYERS = {
    "attention": configs.attention_layer(configs.attention(**LEFT, window=37, rot=(1000.0, 8)), ff=40),
    "state_space": configs.state_space_layer(
        configs.attention(**LEFT, window=70, rot=(1000.0, 16), scaling=(4.0, 64.0, 8.0, 1.0), softcap=8.0),
        heads=4, vdim=12, state=8, groups=2, conv=4, norm_groups=2, ff=40),
    "matrix_memory": configs.matrix_memory_layer(
        configs.attention(**LEFT, softcap=8.0, q_temp=(0.6, 16)), heads=2, dim=12, vdim=20, gate_cap=6.0, ff=40),
}
# what must not be confused with what: (path into the layer, other value); None removes the key
OTHERS = {
    "attention": [(("mixer", "mask", "size"), 36), (("mixer", "mask", "size"), 38), (("mixer", "rot", "dims"), 16),
                  (("mixer", "rot", "base"), 500.0), (("mixer", "scale"), 0.25)],
    "state_space": [(("mixer", "left", "mask", "size"), 69), (("mixer", "left", "mask", "size"), 71),
                    (("mixer", "left", "softcap"), 4.0), (("mixer", "left", "softcap"), None),
                    (("mixer", "left", "rot", "scaling"), None), (("mixer", "left", "rot", "scaling", "factor"), 2.0),
                    (("mixer", "left", "rot", "scaling", "fast"), 2.0), (("mixer", "right", "norm_groups"), 1),
                    (("mixer", "right", "norm_groups"), 4)],
    "matrix_memory": [(("mixer", "left", "q_temp", "every"), (17, 48)), (("mixer", "left", "q_temp", "coef"), 0.3),
                      (("mixer", "left", "q_temp"), None), (("mixer", "left", "softcap"), None),
                      (("mixer", "left", "mask"), {"size": 150}), (("mixer", "right", "gate_cap"), 3.0)],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("lanes", [None, 2])
@pytest.mark.parametrize("kind", sorted(LAYERS))
def test_one_layer_alone(kind, lanes, dtype, record_property):
    """A model of one layer, whole, in portions and decoded over three pages, against the plain model and against
    plain models with a window one token shorter and longer, another bound on the scores, other frequencies, another
    temperature, other norm parts or another gate bound: the engine's logits must lie nearer to the right one."""
    config = configs.single(LAYERS[kind], streams=lanes)
    engine, tensors = make(config, dtype, seed=11, sharp=3.0, logits=6.0)
    tokens = prompt(config, 200, 21)
    want = plain(config, tensors, tokens)
    # (a pair of values: the finer one for 32-bit, the coarser one where bfloat16 rounding would drown the finer)
    others = [plain(changed(config, ("layers", 0) + path, value[dtype == "bfloat16"] if isinstance(value, tuple) else value),
                    tensors, tokens) for path, value in OTHERS[kind]]
    if kind == "attention":              # without the gate, without the biases, the gate taken per head
        for drop in (["l0.mix.g"], ["l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b"]):
            without = {name: torch.zeros_like(t) if name in drop else t for name, t in tensors.items()}
            others.append(plain(config, without, tokens))
    if lanes:                            # the mixing matrix read [to, from]
        swapped = {name: t.t().contiguous() if name.endswith(".mix") else t for name, t in tensors.items()}
        others.append(plain(config, swapped, tokens))
    for what, got in (("whole", in_steps(engine, tokens, [200])),
                      ("in portions", in_steps(engine, tokens, [61, 2, 3, 64, 1, 30, 39])),
                      ("decoded", decoded(engine, tokens, 50))):
        close(got, want, dtype, record_property, f"{kind} {what}")
        nearer(got, want, others, f"{kind} {what}", rows=slice(100, 200))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_recurrent_states_start_as_the_design_says(dtype):
    """A matrix memory whose running maximum started at minus infinity instead of zero, or a state-space mixer whose
    state or carried inputs were not zero at a sequence's start, would show in the first tokens: sequences of one to
    five tokens, in a slot that a longer sequence has just used."""
    for kind in ("matrix_memory", "state_space"):
        config = configs.single(LAYERS[kind], streams=2)
        engine, tensors = make(config, dtype, seed=5, logits=6.0)
        slot = engine.acquire()
        run(engine, slot, prompt(config, 90, 1))
        engine.release(slot)
        for length in (1, 2, 3, 5):
            tokens = prompt(config, length, 30 + length)
            assert engine.acquire() == slot
            got = run(engine, slot, tokens)
            engine.release(slot)
            close(got, plain(config, tensors, tokens), dtype, what=f"{kind}, {length} tokens")
            close(decoded(engine, tokens, 1), plain(config, tensors, tokens), dtype, what=f"{kind}, {length} tokens decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 445])
def test_far_keys_reach_the_last_rows(dtype, window, record_property):
    """Sharp scores over 600 tokens: the last rows attend to single keys up to nine pages back. Changing the
    sequence's first forty tokens moves them in the plain model (without a window) or leaves them alone (behind a
    window of 445), and the engine follows in both cases, whole and decoded."""
    mixer = configs.attention(2, 1, 16, 16, 0.5, window=window, rot=(10000.0, 8))
    config = configs.single(configs.attention_layer(mixer), positions=700)
    engine, tensors = make(config, dtype, seed=13, sharp=6.0, logits=6.0)
    tokens = prompt(config, 600, 3)
    other = prompt(config, 40, 4) + tokens[40:]
    want, moved = plain(config, tensors, tokens), plain(config, tensors, other)
    shift = float((want[560:] - moved[560:]).abs().max()) / float(want.abs().max())
    record_property("what the first forty tokens move the last rows by", shift)
    assert shift > 0.2 if window is None else shift == 0.0
    for sequence, expected in ((tokens, want), (other, moved)):
        close(in_steps(engine, sequence, [600])[560:], expected[560:], dtype, record_property, "whole")
        close(decoded(engine, sequence, 560)[560:], expected[560:], dtype, record_property, "decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_borrowed_keys(dtype, record_property):
    """Two layers read the keys and values of an earlier one with windows and queries of their own. Against plain
    models in which they read another layer's, or have other windows."""
    base = configs.attention(4, 2, 16, 16, 0.3, window=40, rot=(1000.0, 8))
    config = configs.model(67, 48, 1e-5, [
        configs.attention_layer(base, ff=32),
        configs.attention_layer(dict(base, mask={"size": 70}), ff=32),
        configs.attention_layer(dict(base, mask={"size": 25}, kv_from=0), ff=32),
        configs.attention_layer(dict(base, mask={"size": 90}, kv_from=1)),
    ], streams=2, positions=600)
    engine, tensors = make(config, dtype, seed=17, sharp=3.0, logits=6.0)
    tokens = prompt(config, 260, 8)
    want = plain(config, tensors, tokens)
    others = []
    for path, value in ((("layers", 2, "mixer", "kv_from"), 1), (("layers", 3, "mixer", "kv_from"), 0),
                        (("layers", 2, "mixer", "mask", "size"), (40, 60)), (("layers", 3, "mixer", "mask", "size"), (70, 20))):
        # (a pair of values: the finer one for 32-bit, the coarser one where bfloat16 rounding would drown the finer)
        value = value[dtype == "bfloat16"] if isinstance(value, tuple) else value
        others.append(plain(changed(config, path, value), tensors, tokens))
    for what, got in (("whole", in_steps(engine, tokens, [260])), ("in portions", in_steps(engine, tokens, [100, 2, 93, 65])),
                      ("decoded", decoded(engine, tokens, 120))):
        close(got, want, dtype, record_property, what)
        nearer(got, want, others, what, rows=slice(130, 260))


# ------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(configs.ALL))
def test_whole_prompts_portions_and_decoding(name, dtype, record_property):
    config = configs.ALL[name]
    engine, tensors = make(config, dtype, seed=2)
    tokens = prompt(config, 330 if name == "wide" else 210, 9)
    want = plain(config, tensors, tokens)
    close(in_steps(engine, tokens, [len(tokens)]), want, dtype, record_property, "whole")
    close(in_steps(engine, tokens, [63, 2, 64, 1, 3, len(tokens) - 133]), want, dtype, record_property, "in portions")
    close(decoded(engine, tokens, len(tokens) - 140), want, dtype, record_property, "decoded past every window")
    for length in (1, 2, 3):
        few = prompt(config, length, 50 + length)
        close(in_steps(engine, few, [length]), plain(config, tensors, few), dtype, what=f"{length} tokens")
    engine.cache.check()
    assert not engine.cache.slots.held


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small_a", "small_b", "wide"])
def test_batches_of_unequal_requests(name, dtype, record_property):
    """Requests of unequal lengths start together, are decoded together, the shorter ones leave and their slots and
    pages go to the next batch at once: every request as if it ran alone."""
    from kidi_b200 import StepBatch
    config = configs.ALL[name]
    engine, tensors = make(config, dtype, seed=4, max_tokens=1024)
    lengths = [(1, 70, 131, 40), (150, 3, 66), (90, 64)]
    seen = set()
    for batch, sizes in enumerate(lengths):
        requests = [prompt(config, n + 6 + 3 * i, 100 * batch + i) for i, n in enumerate(sizes)]
        want = [plain(config, tensors, r) for r in requests]
        slots = [engine.acquire() for _ in requests]
        if batch:
            assert seen & set(slots)                       # slots (and their pages) are used again
        seen |= set(slots)
        heads = list(sizes)
        logits = engine.step(StepBatch(slots, [r[:n] for r, n in zip(requests, heads)],
                                       [list(range(n)) for n in heads])).double().cpu()
        got, at = [], 0
        for n in heads:
            got.append([logits[at:at + n]])
            at += n
        done = list(heads)
        live = list(range(len(requests)))
        while live:
            step = engine.step(StepBatch([slots[b] for b in live], [[requests[b][done[b]]] for b in live],
                                         [[0]] * len(live))).double().cpu()
            for row, b in enumerate(live):
                got[b].append(step[row:row + 1])
                done[b] += 1
            for b in [b for b in live if done[b] == len(requests[b])]:
                engine.release(slots[b])
            live = [b for b in live if done[b] < len(requests[b])]
        for b, expected in enumerate(want):
            close(torch.cat(got[b]), expected, dtype, record_property, f"batch {batch}, request {b}")
    engine.cache.check()
    assert not engine.cache.slots.held


def test_batches_and_portions_leave_32_bit_logits_alone():
    """In 32-bit a request's logits are the same alone, in a batch and in portions (within 4e-6 of the largest)."""
    from kidi_b200 import StepBatch
    config = configs.SMALL_A
    engine, tensors = make(config, "float32", seed=6)
    a, b = prompt(config, 150, 1), prompt(config, 77, 2)
    alone = in_steps(engine, a, [150])
    cut = in_steps(engine, a, [64, 2, 83, 1])
    slots = [engine.acquire(), engine.acquire()]
    both = engine.step(StepBatch(slots, [b, a], [[76], list(range(150))])).double().cpu()[1:]
    for slot in slots:
        engine.release(slot)
    scale = float(alone.abs().max())
    assert float((alone - cut).abs().max()) <= 4e-6 * scale and float((alone - both).abs().max()) <= 4e-6 * scale


def test_which_kernels_run(record_property):
    """The bfloat16 engine takes the tensor-core attention kernels for the attention layers whose widths allow it
    (prompts and decoding, also with borrowed keys); the 32-bit engine takes the general kernels and the 32-bit
    product only."""
    from kidi_b200.kernels import ops
    config = configs.WIDE
    engine, tensors = make(config, "bfloat16", seed=3)
    tokens = prompt(config, 300, 5)
    want = plain(config, tensors, tokens)
    slot = engine.acquire()
    with ops.record_launches() as names:
        run(engine, slot, tokens[:299], want=[])
    record_property("prompt kernels", sorted(set(names)))
    assert sum(name.startswith("attention_prefill") for name in names) >= 3
    assert names.count("scalar_recurrence") == 2 and names.count("lanes_mix_rmsnorm") == 8 and "short_conv_state" in names
    with ops.record_launches() as names:
        last = run(engine, slot, tokens[299:])
    record_property("decode kernels", sorted(set(names)))
    assert sum(name.startswith("attention_decode") for name in names) >= 3
    engine.release(slot)
    close(last, want[299:], "bfloat16", record_property, "decoded", slack=2.0)
    engine32, _ = make(config, "float32", seed=3)
    slot = engine32.acquire()
    with ops.record_launches() as names:
        run(engine32, slot, tokens)
    assert "library_mm" not in names
    assert not any("tensor" in name or "tcgen05" in name or "skinny" in name or "mma" in name for name in names)


# ------------------------------------------------------------------ generation, the command line, the trace runner
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
@pytest.mark.parametrize("name", ["small_b", "wide", "plain"])
def test_greedy_generation_through_the_engine(name, dtype, use_graph):
    """`Engine.generate`: batches of unequal prompts, decode steps replayed as a captured graph (with padding rows:
    three live sequences in four rows), slots reused by the next batch."""
    config = configs.ALL[name]
    tensors = configs.tensors(config, 7, logits=12.0)
    engine, _ = make(config, dtype, tensors=tensors, max_tokens=2048)
    requests = [prompt(config, n, 40 + n) for n in (5, 1, 70, 12, 33)]
    found = engine.generate(requests, max_new_tokens=12, ignore_eos=True, max_active=3, use_graph=use_graph)
    counts = [teacher_forced(config, tensors, r, t, GREEDY[dtype]) for r, t in zip(requests, found)]
    close_calls, misses = sum(c for c, _ in counts), sum(m for _, m in counts)
    assert all(len(tokens) == 12 for tokens in found) and close_calls <= 30 and misses == 0
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
    config = configs.SMALL_A
    tensors = configs.tensors(config, 8, logits=12.0)
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


def test_a_random_model_folder_runs(tmp_path):
    """`write_random_model` draws every tensor the design declares (the lanes' mixing matrices near the identity)
    and the engine loads the folder it wrote."""
    import kidi_b200
    from safetensors import safe_open
    folder = kidi_b200.write_random_model(configs.SMALL_B, str(tmp_path / "model"), seed=3)
    engine = kidi_b200.Engine.load(folder, dtype="bfloat16", max_tokens=512)
    with safe_open(f"{folder}/model.safetensors", "pt") as handle:
        tensors = {name: handle.get_tensor(name) for name in handle.keys()}
    tokens = prompt(configs.SMALL_B, 80, 1)
    got = in_steps(engine, tokens, [80])
    want = plain(configs.SMALL_B, tensors, tokens)
    assert float((got - want).abs().max()) < 0.1 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_trace_runner_replays_a_model_folder(tmp_path, dtype, record_property):
    """bin/trace_run on a Biropel folder: three unequal requests start together (one of a single token), are decoded
    together until the shorter ones end, a step in which nothing is wanted, then a fourth request on what they gave
    back. `--max-tokens` is the tokens they hold, with no allowance for partly filled pages."""
    import os
    import subprocess
    import sys
    config = configs.SMALL_A
    tensors = configs.tensors(config, 9)
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
    close(torch.cat([read(0), read(2), read(5), read(6)]),
          torch.cat([torch.stack([want["a"][0], want["b"][0], want["b"][69], want["c"][5], want["c"][128]]),
                     torch.stack([want["b"][71], want["c"][130]]), want["b"][74:75], want["d"][[0, 45, 89]]]),
          dtype, record_property, "prompts together, decoded together, the last one alone, on reused pages", slack=2.0)
