"""Gazezen without a GPU: its typed configuration, the registry, the tensors its parts declare, the order in which a
looped range runs, a random model folder through the command line, and the plain implementation's mechanisms
against closed forms worked out by hand."""
import copy
import json
import math

import pytest
import torch

import gazezen_configs
import plain_gazezen


def test_the_configuration_round_trips_and_is_chosen_by_its_name():
    from kidi_b200.config.gazezen import GazezenConfig
    from kidi_b200.registry import registered_architectures, resolve_architecture
    assert "Gazezen" in registered_architectures()
    for config in gazezen_configs.ALL.values():
        assert resolve_architecture(config).config_type is GazezenConfig
        typed = GazezenConfig.from_dict(config)
        written = copy.deepcopy(config)
        for layer in written["layers"]:                  # a single group of which one is kept is not written out
            if layer["mlp"] and layer["mlp"]["router"].get("groups") == {"count": 1, "keep": 1}:
                del layer["mlp"]["router"]["groups"]
        assert typed.to_dict() == written
        assert GazezenConfig.from_dict(typed.to_dict()) == typed
    typed = GazezenConfig.from_dict(gazezen_configs.SMALL_A)
    first, second = typed.layers[0], typed.layers[1]
    assert (first.type, first.heads, first.kv_heads, first.dim, first.vdim, first.window) == ("attention", 4, 2, 16, 32, 40)
    assert (first.rot_base, first.rot_dims, first.rot_scaling) == (10000.0, 8, None)
    assert (first.mlp.experts, first.mlp.top, first.mlp.groups, first.mlp.keep_groups, first.mlp.shared_ff) == (6, 2, 3, 2, 40)
    assert (second.type, second.rot_dim, second.kv_rank, second.rot_scaling.factor, second.rot_scaling.original) == \
        ("latent_attention", 16, 24, 4.0, 256.0)
    assert typed.layers[2].mlp is None and typed.layers[2].window is None
    assert typed.loop == (1, 3, 2) and typed.logit_scale == 0.7
    plain = GazezenConfig.from_dict(gazezen_configs.SMALL_B)
    assert plain.loop is None and plain.logit_scale == 1.0 and plain.layers[2].rot_base is None
    assert (plain.layers[1].mlp.groups, plain.layers[1].mlp.keep_groups, plain.layers[1].mlp.shared_ff) == (1, 1, None)


def test_the_order_of_a_looped_range():
    from kidi_b200.config.gazezen import GazezenConfig
    order = lambda config: list(GazezenConfig.from_dict(config).run_order())
    assert order(gazezen_configs.SMALL_A) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert order(gazezen_configs.SMALL_B) == [(0, None), (1, None), (2, None), (3, None)]
    assert order(gazezen_configs.WIDE) == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None),
                                           (3, None), (4, None)]
    assert order(gazezen_configs.TAIL) == [(0, None), (1, 0), (1, 1), (1, 2)]
    for config in gazezen_configs.ALL.values():           # the plain implementation counts the same way
        assert plain_gazezen.run_order(config) == order(config)


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.update(vocab="many"), "vocab"),
    (lambda c: c["layers"][0].update(type="recurrence"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3, kv_heads=2), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("rot"), "rot"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not supported"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "feed-forward sizes"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=6), "equal groups"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
])
def test_refused_configurations(change, message):
    from kidi_b200.config.gazezen import GazezenConfig
    from kidi_b200.errors import KidiError
    config = copy.deepcopy(gazezen_configs.SMALL_A)
    change(config)
    with pytest.raises(KidiError) as caught:
        GazezenConfig.from_dict(config)
    assert message in str(caught.value)


def test_declared_tensors_are_the_checkpoint_names():
    from kidi_b200.engine.model import declared_parameters
    from kidi_b200.registry import spec_from_config
    for config in gazezen_configs.ALL.values():
        _, _, spec = spec_from_config(config)
        declared = {}
        for prefix, parameter in declared_parameters(spec):
            assert parameter.alias_of is None
            for name, shape in (parameter.sources or ((parameter.name, parameter.shape),)):
                declared[prefix + name] = tuple(shape)
        made = {name: tuple(tensor.shape) for name, tensor in gazezen_configs.tensors(config, 1).items()}
        assert declared == made
    _, _, spec = spec_from_config(gazezen_configs.SMALL_A)
    assert [entry.layer for entry in spec.schedule] == [0, 1, 2, 1, 2, 3]
    assert [entry.offset[1] if entry.offset else None for entry in spec.schedule] == [None, 0, None, 1, None, None]
    assert "feed_forward" not in spec.layers[2].parts and spec.layers[1].parts["feed_forward"].kind == "routed_experts"
    assert spec.layers[0].parts["mixer"].kind == "attention" and spec.layers[1].parts["mixer"].kind == "latent_attention"


def test_a_random_model_folder_through_the_command_line(tmp_path, capsys):
    import kidi_b200
    from kidi_b200.weights.loader import Checkpoint
    (tmp_path / "config.json").write_text(json.dumps(gazezen_configs.SMALL_A))
    assert kidi_b200.main(["random-model", "--config", str(tmp_path / "config.json"), "-o", str(tmp_path / "model"),
                           "--seed", "3"]) == 0, capsys.readouterr().err
    held = Checkpoint(str(tmp_path / "model"))
    assert held.shape("l0.mlp.e5.down") == (64, 24) and held.shape("l0.mlp.shared.up") == (40, 64)
    assert held.shape("l1.mix.dkv") == (24 + 16, 64) and held.shape("l0.mix.sink") == (4,)
    assert held.shape("loop.step") == (2, 64) and "l2.norm2" not in held and "l1.mix.sink" not in held
    held.close()
    assert kidi_b200.main(["inspect", "-m", str(tmp_path / "model")]) == 0
    assert "Gazezen" in capsys.readouterr().out


# ------------------------------------------------------------------ the plain mechanisms against closed forms
def test_the_plain_norms():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    weight = torch.tensor([1.0, 2.0, 0.5, -1.0], dtype=torch.float64)
    # mean 3, squared deviations 4, 1, 0, 9: variance 3.5
    want = torch.tensor([-2.0, -1.0, 0.0, 3.0], dtype=torch.float64) / math.sqrt(3.5 + 0.5) * weight
    assert torch.allclose(plain_gazezen.centred_norm(x, weight, 0.5), want[None])
    # mean square 12.5
    assert torch.allclose(plain_gazezen.rms_weighted(x, weight, 3.5), x / 4.0 * weight)


def test_the_plain_rotation_pairs_halves_and_leaves_the_rest():
    rot = {"base": 100.0, "dims": 4}
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0] = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], dtype=torch.float64)
    y = plain_gazezen.rotate(x, rot)
    assert torch.equal(y[0], x[0])                                          # position 0
    for position in (1, 2):
        for i, f in enumerate((1.0, 100.0 ** -0.5)):                        # entry i with entry i + 2
            a = position * f
            u, v = x[position, 0, i], x[position, 0, i + 2]
            assert abs(float(y[position, 0, i]) - float(u * math.cos(a) - v * math.sin(a))) < 1e-12
            assert abs(float(y[position, 0, i + 2]) - float(v * math.cos(a) + u * math.sin(a))) < 1e-12
        assert y[position, 0, 4:].tolist() == [5.0, 6.0]


def test_the_plain_stretched_frequencies():
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64.0, "fast": 4.0, "slow": 1.0}}
    freq, factor = plain_gazezen.frequencies(rot, torch.float64)
    plain, one = plain_gazezen.frequencies({"base": 10000.0, "dims": 16}, torch.float64)
    assert one == 1.0 and abs(factor - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    # the pair at which a frequency makes t turns in 64 positions: 16 ln(64 / (2 pi t)) / (2 ln 10000)
    lo = math.floor(16 * math.log(64 / (2 * math.pi * 4.0)) / (2 * math.log(10000.0)))
    hi = math.ceil(16 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(10000.0)))
    assert (lo, hi) == (0, 3)
    for i in range(8):
        ramp = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(float(freq[i]) - float(plain[i]) * (ramp / 4.0 + 1.0 - ramp)) < 1e-15
    assert float(freq[0]) == float(plain[0]) and abs(float(freq[7]) - float(plain[7]) / 4.0) < 1e-18
    # a ramp that would have no length still divides by a little
    steep = dict(rot, scaling={"factor": 2.0, "original": 64.0, "fast": 1.0, "slow": 1.0})
    freq, _ = plain_gazezen.frequencies(steep, torch.float64)
    assert torch.isfinite(freq).all()


def test_the_plain_window_and_sink():
    seen = plain_gazezen.window_mask(6, 3)
    assert seen[5].tolist() == [False, False, False, True, True, True]
    assert seen[1].tolist() == [True, True, False, False, False, False]
    assert plain_gazezen.window_mask(4, None)[3].all() and not plain_gazezen.window_mask(4, None)[0, 1]
    scores = torch.tensor([[0.0, math.log(2.0), 5.0]], dtype=torch.float64)
    mask = torch.tensor([[True, True, False]])
    weights = plain_gazezen.softmax_rows(scores, mask, torch.tensor(math.log(3.0), dtype=torch.float64))
    assert torch.allclose(weights, torch.tensor([[1.0 / 6.0, 2.0 / 6.0, 0.0]], dtype=torch.float64))   # 1 + 2 + 3
    assert torch.allclose(plain_gazezen.softmax_rows(scores, mask), torch.tensor([[1 / 3, 2 / 3, 0.0]], dtype=torch.float64))


def test_the_plain_router_keeps_groups_and_divides_by_the_sum():
    scores = torch.tensor([0.30, 0.05, 0.02, 0.25, 0.20, 0.18], dtype=torch.float64)
    pick = lambda top, groups: sorted(plain_gazezen.choose(scores, top, groups).tolist())
    assert pick(2, None) == [0, 3]
    assert pick(2, {"count": 3, "keep": 1}) == [0, 1]          # group 0 holds the best score: only its experts
    assert pick(2, {"count": 3, "keep": 2}) == [0, 3]          # groups 0 and 1 (bests 0.30 and 0.25)
    assert pick(3, {"count": 2, "keep": 1}) == [0, 1, 2]       # halves: bests 0.30 and 0.25
    assert pick(3, {"count": 2, "keep": 2}) == [0, 3, 4]
    generator = torch.Generator().manual_seed(4)
    w = {"router": torch.tensor([[2.0, 0.0], [0.0, 0.0], [1.0, 0.0], [-3.0, 0.0]], dtype=torch.float64)}
    for name in ("e0", "e1", "e2", "e3", "shared"):
        w[f"{name}.up"] = torch.randn(5, 2, generator=generator, dtype=torch.float64)
        w[f"{name}.down"] = torch.randn(2, 5, generator=generator, dtype=torch.float64)
    h = torch.tensor([[1.0, -0.4]], dtype=torch.float64)
    mlp = {"router": {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}, "shared": {"ff": 5}}
    out = plain_gazezen.routed_feed_forward(h, w, "", mlp)
    s = torch.softmax(torch.tensor([2.0, 0.0, 1.0, -3.0], dtype=torch.float64), 0)      # over all four experts
    gelu = lambda z: 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))
    run = lambda name: gelu(h @ w[f"{name}.up"].t()) @ w[f"{name}.down"].t()
    want = (s[0] * run("e0") + s[1] * run("e1")) / (s[0] + s[1]) + run("shared")         # group 0: experts 0 and 1
    assert torch.allclose(out, want)
    assert abs(float(plain_gazezen.gelu_erf(torch.tensor(1.0, dtype=torch.float64))) - 0.8413447460685429) < 1e-12


def test_the_plain_model_adds_a_vector_before_each_pass():
    """The streams after every layer run: a looped layer counts each time, and with the mixers and feed-forwards
    silenced (zero weights behind them) the stream only gathers the passes' vectors."""
    config = gazezen_configs.TAIL
    tensors = gazezen_configs.tensors(config, 2)
    for name in tensors:
        if name.endswith("norm1b") or name.endswith("norm2b"):
            tensors[name] = torch.zeros_like(tensors[name])
    streams = []
    tokens = [3, 9, 27]
    plain_gazezen.forward(config, tensors, tokens, streams=streams)
    assert len(streams) == 4
    x = tensors["embed"].double()[tokens]
    steps = tensors["loop.step"].double()
    assert torch.allclose(streams[0], x) and torch.allclose(streams[1], x + steps[0])
    assert torch.allclose(streams[3], x + steps.sum(0))
