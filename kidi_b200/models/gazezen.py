"""Gazezen as a `ModelSpec`.

A decoder-only stack whose layers put a layer norm (weight, no bias) before and behind each sublayer,
x <- x + norm1b(mixer(norm1(x))), x <- x + norm2b(ff(norm2(x))), around one of two mixers and, where a layer has
one, a feed-forward of routed experts with a shared expert. Mixer "attention": grouped-query softmax attention
over a sliding window, queries and keys rotated on part of a head (halves paired), a learned sink per head in the
softmax denominator, a sigmoid gate per head and token on the result. Mixer "latent_attention": attention over a
cached latent with one rotated key part for all heads (halves paired, frequencies stretched for long sequences),
a sliding window, the same gate. The experts are W_down gelu(W_up h); the router takes a softmax over all experts,
keeps the best groups of neighbouring experts, chooses the largest scores among them and divides the chosen
scores by their sum. A range of layers may run several times in a row with the same weights and a cache per pass;
a learned vector per pass is added to the stream before the pass's first layer. The logits are the head's
product times a constant.

Tensor names: `embed`, `loop.step`, `final.norm`, `head`, and per layer `l<i>.norm1`, `norm1b`, `norm2`, `norm2b`,
`l<i>.mix.{q,k,v,sink,g,o}` or `l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}`, `l<i>.mlp.{router,e<j>.up,e<j>.down,
shared.up,shared.down}`.

This file maps a `GazezenConfig` to parts and their parameters; nothing here computes.
"""
from __future__ import annotations

from ..config.gazezen import ATTENTION, GazezenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..registry import register_architecture

# Constants the design fixes.
RENORMALISE_EPS = 1e-20      # added to the sum that the chosen experts' scores are divided by
LOOP_STEPS = "loop_steps"    # the shared table of one vector per pass of the looped range


def rotation_name(layer) -> str:
    scaling = layer.rot_scaling
    stretch = f"_{scaling.factor!r}_{scaling.original!r}_{scaling.fast!r}_{scaling.slow!r}" if scaling else ""
    width = layer.dim if layer.type == ATTENTION else layer.rot_dim
    return f"rot_{layer.rot_base!r}_{layer.rot_dims}_{width}{stretch}"


def build_spec(config: GazezenConfig) -> ModelSpec:
    hidden, eps = config.width, config.norm_eps
    norm = lambda name, prefix="": PartSpec("layer_norm", {"size": hidden, "eps": eps, "weight_name": name,
                                                           "bias": False}, prefix)
    positions, layers = {}, []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}."
        position = None
        if layer.rot_base is not None:
            position = rotation_name(layer)
            positions.setdefault(position, PartSpec("rotary", {
                "head_dim": layer.dim if layer.type == ATTENTION else layer.rot_dim, "rotary_dim": layer.rot_dims,
                "theta": layer.rot_base, "max_positions": config.max_positions,
                "scaling": layer.rot_scaling.to_dict() if layer.rot_scaling is not None else None}))
        if layer.type == ATTENTION:
            mixer = PartSpec("attention", {
                "hidden_size": hidden, "num_heads": layer.heads, "num_kv_heads": layer.kv_heads, "head_dim": layer.dim,
                "value_dim": layer.vdim, "scale": layer.scale, "window": layer.window, "position": position,
                "sink": True, "head_gate": True, "q_name": "q", "k_name": "k", "v_name": "v", "o_name": "o",
                "sink_name": "sink", "gate_name": "g"}, prefix + "mix.")
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": hidden, "num_heads": layer.heads, "dim": layer.dim, "rot_dim": layer.rot_dim,
                "vdim": layer.vdim, "q_rank": None, "kv_rank": layer.kv_rank, "scale": layer.scale, "eps": eps,
                "position": position, "window": layer.window, "ring": False, "rotation_layout": "half",
                "head_gate": True}, prefix + "mix.")
        parts = {"input_norm": norm("norm1", prefix), "mixer": mixer, "mixer_out_norm": norm("norm1b", prefix)}
        mlp = layer.mlp
        if mlp is not None:
            parts["post_norm"] = norm("norm2", prefix)
            parts["feed_forward_out_norm"] = norm("norm2b", prefix)
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden_size": hidden, "expert_size": mlp.expert_ff, "experts": mlp.experts, "top": mlp.top,
                "score": "softmax", "renormalise": True, "renormalise_eps": RENORMALISE_EPS, "weight_on": "output",
                "groups": mlp.groups, "keep_groups": mlp.keep_groups, "expert_form": "plain",
                "shared_size": mlp.shared_ff}, prefix + "mlp.")
        layers.append(LayerSpec(arrangement=PartSpec("sandwich_norm"), parts=parts))
    schedule = tuple(ScheduleEntry(index, offset=(LOOP_STEPS, number) if number is not None else None)
                     for index, number in config.run_order())
    shared = {}
    if config.loop is not None:
        shared[LOOP_STEPS] = PartSpec("stream_offsets", {"hidden_size": hidden, "count": config.loop[2],
                                                         "name": "loop.step"}, "")
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab,
        hidden_size=hidden,
        max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": config.vocab, "hidden_size": hidden, "name": "embed"}, ""),
        positions=positions,
        shared=shared,
        layers=tuple(layers),
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"hidden_size": hidden, "vocab_size": config.vocab, "name": "head",
                                      "logit_scale": config.logit_scale}, ""),
        eos_token_ids=config.eos_token_ids,
    )


register_architecture("Gazezen", GazezenConfig, build_spec)
