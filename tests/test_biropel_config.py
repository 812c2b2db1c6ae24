"""Biropel without a GPU: the typed configuration (round trip, refusals), the registry, the tensors a model
declares, and the plain implementation's mechanisms against closed forms and against each other."""
import copy
import math

import pytest
import torch

import biropel_configs
import plain_biropel
from kidi_b200 import KidiError
from kidi_b200.config.biropel import BiropelConfig
from kidi_b200.engine.model import declared_parameters
from kidi_b200.registry import registered_architectures, spec_from_config


@pytest.mark.parametrize("name", list(biropel_configs.ALL))
def test_configuration_round_trip(name):
    config = biropel_configs.ALL[name]
    typed = BiropelConfig.from_dict(config)
    assert typed.to_dict() == config
    assert BiropelConfig.from_dict(typed.to_dict()) == typed
    assert "Biropel" in registered_architectures()


@pytest.mark.parametrize("name", list(biropel_configs.ALL))
def test_declared_tensors_are_the_checkpoints(name):
    """The tensors the model declares (fused parameters as their sources) are exactly the tests' own checkpoint."""
    config = biropel_configs.ALL[name]
    _, _, spec = spec_from_config(config)
    declared = {}
    for prefix, parameter in declared_parameters(spec):
        for source, shape in (parameter.sources or ((parameter.name, parameter.shape),)):
            declared[prefix + source] = tuple(shape)
    made = {key: tuple(value.shape) for key, value in biropel_configs.tensors(config, 0).items()}
    assert declared == made


def test_the_schedule_names_borrowed_caches():
    _, _, spec = spec_from_config(biropel_configs.SMALL_B)
    assert [entry.cache_from for entry in spec.schedule] == [None, None, None, None, 2, 2]
    assert spec.layers[4].parts["mixer"].params["own_kv"] is False
    assert spec.layers[2].parts["mixer"].params["own_kv"] is True
    assert spec.layers[0].arrangement.kind == "hyper_connections"
    _, _, plain = spec_from_config(biropel_configs.PLAIN)
    assert plain.layers[0].arrangement.kind == "pre_norm"


def change(config, path, value):
    changed = copy.deepcopy(config)
    node = changed
    for key in path[:-1]:
        node = node[key]
    if value is None:
        node.pop(path[-1], None)
    else:
        node[path[-1]] = value
    return changed


@pytest.mark.parametrize("path,value", [
    (("vocab",), None), (("norm", "eps"), 0.0), (("streams",), 9), (("layers", 0, "type"), "conv"),
    (("layers", 0, "mixer", "heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 7),
    (("layers", 0, "mixer", "rot", "dims"), 18), (("layers", 0, "mixer", "mask", "size"), 0),
    (("layers", 1, "mixer", "kv_from"), 1), (("layers", 1, "mixer", "kv_from"), 3),
    (("layers", 1, "mixer", "kv_heads"), 4), (("layers", 1, "mixer", "rot", "base"), 20000.0),
    (("layers", 2, "mixer", "right", "groups"), 3), (("layers", 2, "mixer", "right", "norm_groups"), 5),
    (("layers", 2, "mixer", "left", "rot", "scaling", "factor"), 0.0), (("layers", 3, "mixer", "right", "gate_cap"), 0.0),
    (("layers", 3, "mixer", "left", "q_temp", "every"), 0), (("layers", 0, "mlp", "kind"), "moe"),
    (("layers", 3, "mixer", "left", "kv_from"), 0),
])
def test_refused_configurations(path, value):
    with pytest.raises(KidiError):
        BiropelConfig.from_dict(change(biropel_configs.SMALL_A, path, value))


def test_optional_keys():
    """No mask: every earlier token; no rot: no rotation; no softcap, no q_temp, no streams, no feed-forward."""
    config = biropel_configs.single(biropel_configs.attention_layer(biropel_configs.attention(2, 1, 8, 8, 0.3)))
    typed = BiropelConfig.from_dict(config)
    layer = typed.layers[0]
    assert (layer.attention.window, layer.attention.rot_base, layer.attention.softcap, layer.attention.q_temp,
            layer.ff, typed.streams) == (None,) * 6
    _, _, spec = spec_from_config(config)
    assert not spec.positions and spec.layers[0].parts.get("feed_forward") is None


# ------------------------------------------------------------------ the plain implementation's mechanisms
def test_plain_mask_and_temperature():
    seen = plain_biropel.visible(6, 3)
    assert seen.tolist() == [[j <= i and i - j < 3 for j in range(6)] for i in range(6)]
    assert plain_biropel.visible(4, None).tolist() == [[j <= i for j in range(4)] for i in range(4)]
    temp = plain_biropel.query_temperature(10, 0.5, 4, torch.float64)
    assert temp[:3].tolist() == [1.0, 1.0, 1.0]                      # floor((p + 1) / 4) = 0 up to p = 2
    assert abs(float(temp[3]) - (1 + 0.5 * math.log(2))) < 1e-12 and abs(float(temp[7]) - (1 + 0.5 * math.log(3))) < 1e-12


def test_plain_frequencies():
    plain, factor = plain_biropel.frequencies({"base": 100.0, "dims": 8})
    assert factor == 1.0 and torch.allclose(plain, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=torch.float64))
    stretched, factor = plain_biropel.frequencies({"base": 100.0, "dims": 8, "scaling": {
        "factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0}})
    assert abs(factor - (0.1 * math.log(4.0) + 1)) < 1e-12
    # pair_of(8) = 8 ln(64 / 16 pi) / (2 ln 100) = 0.21 -> lo 0; pair_of(1) = 2.02 -> hi 3: ramp 0, 1/3, 2/3, 1
    ramp = torch.tensor([0.0, 1 / 3, 2 / 3, 1.0], dtype=torch.float64)
    assert torch.allclose(stretched, plain / 4.0 * ramp + plain * (1 - ramp))


def test_plain_rotation_pairs_halves():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0] = 1.0                                       # entry 0 is paired with entry 2 of the 4 rotated ones
    x[:, 0, 5] = 7.0
    turned = plain_biropel.rotate(x, {"base": 10.0, "dims": 4})
    for p in range(3):
        assert abs(float(turned[p, 0, 0]) - math.cos(p)) < 1e-12 and abs(float(turned[p, 0, 2]) - math.sin(p)) < 1e-12
        assert float(turned[p, 0, 1]) == 0.0 and float(turned[p, 0, 5]) == 7.0


def test_plain_convolution_is_causal_and_ends_on_the_current_token():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    weight = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    y = plain_biropel.causal_conv(x, weight, torch.tensor([0.5], dtype=torch.float64))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5, 345.5]


def test_plain_recurrences_against_their_sums():
    """One head, closed forms: the state-space read-out is a decayed sum over the past; the matrix memory with
    constant gates is a normalised, decayed sum."""
    generator = torch.Generator().manual_seed(0)
    T, D = 7, 6
    h = torch.randn(T, D, generator=generator, dtype=torch.float64)
    mixer = {"heads": 1, "vdim": 2, "state": 3, "groups": 1, "conv": 1, "norm_groups": 1}
    tensors = {"in": torch.randn(2 * 2 + 2 * 3 + 1, D, generator=generator, dtype=torch.float64),
               "conv": torch.ones(2 + 6, 1, dtype=torch.float64), "conv.b": torch.zeros(8, dtype=torch.float64),
               "dt_bias": torch.tensor([0.3], dtype=torch.float64), "A_log": torch.tensor([-0.2], dtype=torch.float64),
               "D": torch.tensor([0.7], dtype=torch.float64), "norm": torch.ones(2, dtype=torch.float64),
               "o": torch.eye(2, dtype=torch.float64)}
    got = plain_biropel.state_space(h, tensors, "", mixer, 1e-6)
    proj = h @ tensors["in"].t()
    z, rest, dt = proj[:, :2], torch.nn.functional.silu(proj[:, 2:10]), torch.nn.functional.softplus(proj[:, 10] + 0.3)
    x, B, C = rest[:, :2], rest[:, 2:5], rest[:, 5:8]
    rate = math.exp(-0.2)
    want = torch.zeros(T, 2, dtype=torch.float64)
    for t in range(T):
        y = 0.7 * x[t]
        for u in range(t + 1):
            y = y + torch.exp(-rate * dt[u + 1:t + 1].sum()) * dt[u] * (B[u] @ C[t]) * x[u]
        y = y * torch.nn.functional.silu(z[t])
        want[t] = y / torch.sqrt((y * y).mean() + 1e-6)
    assert torch.allclose(got, want, atol=1e-10)


def test_the_command_line_writes_and_inspects_a_folder(tmp_path, capsys):
    """`random-model` draws every declared tensor (the lanes' mixing matrices near the identity) and `inspect` reads
    the folder back; neither needs a GPU."""
    import json

    import kidi_b200
    from safetensors import safe_open
    (tmp_path / "config.json").write_text(json.dumps(biropel_configs.SMALL_B))
    folder = tmp_path / "model"
    assert kidi_b200.main(["random-model", "--config", str(tmp_path / "config.json"), "-o", str(folder), "--seed", "4"]) == 0
    assert kidi_b200.main(["inspect", "-m", str(folder)]) == 0
    printed = capsys.readouterr().out
    assert "architecture: Biropel" in printed and "layers: 6 (run order: 6 entries)" in printed
    with safe_open(str(folder / "model.safetensors"), "pt") as handle:
        names = set(handle.keys())
        mixing = handle.get_tensor("l0.hc1.mix").float()
    assert names == set(biropel_configs.tensors(biropel_configs.SMALL_B, 0))
    assert mixing.shape == (3, 3) and float((mixing - torch.eye(3)).abs().max()) < 0.6
