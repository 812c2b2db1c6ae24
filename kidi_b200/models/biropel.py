"""Biropel as a `ModelSpec`.

A decoder-only stack: token embeddings pass an RMS norm; every layer is a pre-norm block (RMS norms) around a
mixer and, where it has one, a dense feed-forward W_down relu(W_up h)^2; a final RMS norm and a head. With
`streams` the residual stream is kept as that many lanes that every sublayer reads as one weighted sum and writes
back through a mixing matrix (the `hyper_connections` arrangement), and the final norm reads the lanes' sum.
Three kinds of layer:

* "attention": grouped-query softmax attention with biases on q, k and v, queries and keys rotated on the first
  part of a head, a sliding window, and an element-wise sigmoid gate (computed from the mixer's input) on the
  concatenated heads. A layer with `kv_from` has no key and value projections and reads the named layer's cache.
* "parallel": softmax attention (no biases, no gate; stretched rotation frequencies, bounded scores, a sliding
  window) beside a state-space mixer with one decay per head; each result is RMS-normed over the width with a
  weight of its own and the mixer's result is half their sum.
* "parallel_2": softmax attention without rotation (queries and keys divided by their root mean square per head, a
  query temperature that grows with the position, bounded scores, every earlier token visible) beside a matrix
  memory with exponential gates, combined the same way.

Tensor names: `embed`, `embed.norm`, `final.norm`, `head`, and per layer `l<i>.norm1`, `l<i>.norm2`,
`l<i>.hc{1,2}.{in,out,mix}`, `l<i>.mlp.{up,down}`, `l<i>.mix.{q,q.b,k,k.b,v,v.b,g,o}` or
`l<i>.mix.left.{q,k,v,o}`, `l<i>.mix.{left,right}.out`, and `l<i>.mix.right.{in,conv,conv.b,dt_bias,A_log,D,norm,o}`
or `l<i>.mix.right.{q,k,v,g,o,norm,i,i.b,f,f.b}`.

This file maps a `BiropelConfig` to parts and their parameters; nothing here computes.
"""
from __future__ import annotations

from ..config.biropel import ATTENTION, PARALLEL_STATE_SPACE, BiropelConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture


def rotation_name(attention) -> str:
    scaling = attention.rot_scaling
    stretch = f"_{scaling.factor!r}_{scaling.original!r}_{scaling.fast!r}_{scaling.slow!r}" if scaling else ""
    return f"rot_{attention.rot_base!r}_{attention.rot_dims}_{attention.dim}{stretch}"


def build_spec(config: BiropelConfig) -> ModelSpec:
    hidden, eps = config.width, config.norm_eps
    norm = lambda name, prefix="": PartSpec("rms_norm", {"size": hidden, "eps": eps, "weight_name": name}, prefix)
    positions, layers = {}, []

    def softmax_attention(attention, prefix: str, *, biased: bool, gated: bool, unit_qk: bool) -> PartSpec:
        position = temperature = None
        if attention.rot_base is not None:
            position = rotation_name(attention)
            positions.setdefault(position, PartSpec("rotary", {
                "head_dim": attention.dim, "rotary_dim": attention.rot_dims, "theta": attention.rot_base,
                "max_positions": config.max_positions,
                "scaling": attention.rot_scaling.to_dict() if attention.rot_scaling is not None else None}))
        if attention.q_temp is not None:
            temperature = f"q_temp_{attention.q_temp[0]!r}_{attention.q_temp[1]}"
            positions.setdefault(temperature, PartSpec("query_temperature", {
                "coef": attention.q_temp[0], "every": attention.q_temp[1], "max_positions": config.max_positions}))
        return PartSpec("attention", {
            "hidden_size": hidden, "num_heads": attention.heads, "num_kv_heads": attention.kv_heads,
            "head_dim": attention.dim, "value_dim": attention.vdim, "scale": attention.scale,
            "window": attention.window, "ring": False, "position": position, "query_scale": temperature,
            "score_softcap": attention.softcap, "qkv_bias": biased, "output_gate": gated,
            "own_kv": attention.kv_from is None, "qk_norm": unit_qk, "qk_norm_weight": False, "qk_norm_eps": eps,
            "q_name": "q", "k_name": "k", "v_name": "v", "o_name": "o", "gate_name": "g", "q_bias_name": "q.b",
            "k_bias_name": "k.b", "v_bias_name": "v.b"}, prefix)

    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        mix = prefix + "mix."
        if layer.type == ATTENTION:
            mixer = softmax_attention(layer.attention, mix, biased=True, gated=True, unit_qk=False)
        else:
            right = layer.right
            if layer.type == PARALLEL_STATE_SPACE:
                left = softmax_attention(layer.attention, mix + "left.", biased=False, gated=False, unit_qk=False)
                other = PartSpec("mamba2", {"hidden_size": hidden, "num_heads": right.heads, "vdim": right.vdim,
                                            "state": right.state, "groups": right.groups, "conv": right.conv,
                                            "norm_groups": right.norm_groups, "eps": eps}, mix + "right.")
            else:
                left = softmax_attention(layer.attention, mix + "left.", biased=False, gated=False, unit_qk=True)
                other = PartSpec("mlstm", {"hidden_size": hidden, "num_heads": right.heads, "dim": right.dim,
                                           "vdim": right.vdim, "gate_cap": right.gate_cap, "eps": eps}, mix + "right.")
            mixer = PartSpec("parallel_mixers", {"hidden_size": hidden, "eps": eps, "left": left, "right": other,
                                                 "left_norm_name": "left.out", "right_norm_name": "right.out"}, mix)
        parts = {"input_norm": norm("norm1", prefix), "mixer": mixer}
        if layer.ff is not None:
            parts["post_norm"] = norm("norm2", prefix)
            parts["feed_forward"] = PartSpec("dense_mlp", {
                "hidden_size": hidden, "intermediate_size": layer.ff, "activation": "relu_squared", "up_name": "up",
                "down_name": "down"}, prefix + "mlp.")
        arrangement = PartSpec("hyper_connections", {"hidden_size": hidden, "streams": config.streams}, prefix) \
            if config.streams is not None else PartSpec("pre_norm")
        layers.append(LayerSpec(arrangement=arrangement, parts=parts))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=hidden,
        max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": hidden, "name": "embed"}, ""),
        embedding_norm=norm("embed.norm"),
        positions=positions,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(index, cache_from=layer.attention.kv_from)
                       for index, layer in enumerate(config.layers)),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"hidden_size": hidden, "vocab_size": config.vocab, "name": "head"}, ""),
        eos_token_ids=config.eos_token_ids,
    )


register_architecture("Biropel", BiropelConfig, build_spec)
