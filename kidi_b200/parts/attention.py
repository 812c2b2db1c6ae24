"""Grouped-query attention as a mixer.

The reference's Qwen3 attention (src/kidi/layers/qwen3.cpp:13-56): one fused
projection to q, k and v heads; an optional per-head RMSNorm on q and k followed by
rotary encoding (norm before rotation, one weight vector for all heads); scores
scaled by 1/sqrt(head_dim); query head h reads key/value head h // (heads/kv_heads);
an output projection. What this part adds is the causal rule, an optional window
and the cache: key u is visible from position p when u <= p and, with a window W,
u > p - W.

Parameters (`spec.params`): hidden_size, num_heads, num_kv_heads, head_dim, qk_norm
(bool), qk_norm_eps, position (name of a rotary encoding in `env.positions`, or None),
window (tokens, or None), scale (None: 1/sqrt(head_dim)), qkv_bias and out_bias (bool,
default false: the reference's Qwen3 projections carry none, src/kidi/layers/qwen3.cpp:14-15;
its Linear has the option, src/kidi/layers/linear.cpp:181-190), score_softcap (a score s
becomes cap * tanh(s / cap); default none) and score_slopes (one number per head: head h adds
slope * (key position - query position) to its scores; default none). The last two have no
counterpart in the reference's Qwen3; they are there so that an architecture that bounds or
shifts its scores is a specification, not a change to the kernels' arguments: every attention kernel takes the
bound; layers with slopes run on the general attention kernel in either precision.

Three more, none of them in the reference's Qwen3: value_dim (the width of a value head, default
head_dim: the output projection then takes num_heads * value_dim columns); sink (bool): a learned
number per head, tensor `sink_name` [num_heads], whose exponential joins the softmax denominator
(a key that every row sees, with that score as it is, unscaled, and no value); head_gate (bool):
head h's result is multiplied by sigmoid(W_g x)_h, W_g the tensor `gate_name` [num_heads, hidden],
its rows fused behind q, k and v into the one projection. Tensor names under the prefix are the
parameters q_name, k_name, v_name, o_name, sink_name, gate_name (and q_bias_name, k_bias_name, v_bias_name).

Further parameters: output_gate (bool): the concatenated heads are multiplied element by element by
sigmoid(W_g x), W_g the tensor `gate_name` [num_heads * value_dim, hidden], its rows fused into the one projection
like a head gate's (a layer has one kind of gate or none); own_kv (default true; false: the layer has no key and
value projections and reads, with its own queries, the keys and values that the layer named by the schedule
entry's `cache_from` wrote: rotated keys as that layer's cache holds them); ring (default true; false: a
windowed layer keeps every page and the window is a mask, so that prompts may continue cached sequences and
another layer may read the cache); qk_norm_weight (default true; false: the per-head norm of q and k divides by
the root mean square and has no weight); query_scale (name of a position part with a `table` of one factor per
position: q is multiplied by its position's factor after norm and rotation).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from ..cache.sequence_cache import KVRequest
from ..errors import invalid_argument, unsupported
from ..kernels import ops
from ..kernels.attention import AttentionLauncher
from .base import Part
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec


@register_part("mixer", "attention")
class Attention(Part):
    accepts_row_scaled = True     # x may lack its norm's factor: the q/k/v product applies it
    takes_sink = True             # the output product may add its result to the residual stream itself

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.heads = int(spec.param("num_heads"))
        self.kv_heads = int(spec.param("num_kv_heads"))
        self.head_dim = int(spec.param("head_dim"))
        self.qk_norm = bool(spec.param("qk_norm", False))
        self.qkv_bias = bool(spec.param("qkv_bias", False))
        self.out_bias = bool(spec.param("out_bias", False))
        self.eps = float(spec.param("qk_norm_eps", 1e-6))
        self.window = spec.param("window", None)
        self.value_dim = int(spec.param("value_dim", self.head_dim))
        self.has_sink = bool(spec.param("sink", False))
        self.has_gate = bool(spec.param("head_gate", False))
        self.output_gate = bool(spec.param("output_gate", False))
        self.own_kv = bool(spec.param("own_kv", True))
        self.ring = bool(spec.param("ring", True))
        self.norm_weight = bool(spec.param("qk_norm_weight", True))
        if self.has_gate and self.output_gate:
            raise invalid_argument("an attention layer has a gate per head or a gate per element, not both")
        self.names = {key: spec.param(key + "_name", default) for key, default in (
            ("q", "q_proj.weight"), ("k", "k_proj.weight"), ("v", "v_proj.weight"), ("o", "o_proj.weight"),
            ("sink", "sinks"), ("gate", "gate_proj.weight"), ("q_bias", "q_proj.bias"), ("k_bias", "k_proj.bias"),
            ("v_bias", "v_proj.bias"))}
        scale = spec.param("scale", None)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(self.head_dim))
        if self.hidden <= 0 or self.heads <= 0 or self.kv_heads <= 0 or self.heads % self.kv_heads or self.head_dim <= 0:
            raise invalid_argument("invalid attention dimensions")
        if self.head_dim > 256 or not 0 < self.value_dim <= 256:
            raise unsupported(f"head widths {self.head_dim} and {self.value_dim}: the kernels take 1 to 256")
        if self.window is not None and int(self.window) <= 0:
            raise invalid_argument("an attention window must be positive")
        name = spec.param("position", None)
        self.position = env.positions[name] if name is not None else None
        if self.position is not None and self.position.head_dim != self.head_dim:
            raise invalid_argument("the rotary encoding was built for another head width")
        self.q_width = self.heads * self.head_dim
        self.kv_width = self.kv_heads * self.head_dim
        self.v_width = self.kv_heads * self.value_dim
        self.out_width = self.heads * self.value_dim
        # The fused projection's rows: q, k, v, then one gate row a head, then zero rows up to a multiple of 8
        # (so that the rows of its result start on 16-byte boundaries).
        self.gate_width = self.heads if self.has_gate else self.out_width if self.output_gate else 0
        self.gate_begin = self.q_width + (self.kv_width + self.v_width if self.own_kv else 0)
        self.fused_width = self.gate_begin + self.gate_width
        scale_name = spec.param("query_scale", None)
        self.query_scale = env.positions[scale_name] if scale_name is not None else None
        self.sinks = None
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm = self.k_norm = None
        # Optional: scores bounded by score_softcap * tanh(s / score_softcap); scores of head h shifted by
        # score_slopes[h] * (key position - query position) (a list with one number per head).
        self.softcap = float(spec.param("score_softcap", 0.0) or 0.0)
        slopes = spec.param("score_slopes", None)
        if slopes is not None and len(slopes) != self.heads:
            raise invalid_argument("score_slopes needs one number per attention head")
        if self.softcap < 0:
            raise invalid_argument("score_softcap must be positive")
        self.slopes = torch.tensor([float(value) for value in slopes], dtype=torch.float32, device=env.device) \
            if slopes is not None else None
        self.launcher = AttentionLauncher(heads=self.heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
                                          scale=self.scale, window=self.window, softcap=self.softcap,
                                          slopes=self.slopes)

    def parameter_specs(self) -> List[ParamSpec]:
        n = self.names
        sources = [(n["q"], (self.q_width, self.hidden))]
        biases = [(n["q_bias"], (self.q_width,))]
        if self.own_kv:
            sources += [(n["k"], (self.kv_width, self.hidden)), (n["v"], (self.v_width, self.hidden))]
            biases += [(n["k_bias"], (self.kv_width,)), (n["v_bias"], (self.v_width,))]
        if self.gate_width:
            sources.append((n["gate"], (self.gate_width, self.hidden)))
        specs = [
            ParamSpec("qkv_proj.weight", (self.fused_width, self.hidden), sources=tuple(sources)),
            ParamSpec(n["o"], (self.hidden, self.out_width)),
        ]
        if self.qkv_bias:
            specs.append(ParamSpec("qkv_proj.bias", (self.gate_begin,), sources=tuple(biases)))
        if self.out_bias:
            specs.append(ParamSpec("o_proj.bias", (self.hidden,)))
        if self.qk_norm and self.norm_weight:
            specs.append(ParamSpec("q_norm.weight", (self.head_dim,), init=("one_plus_normal", 0.1)))
            specs.append(ParamSpec("k_norm.weight", (self.head_dim,), init=("one_plus_normal", 0.1)))
        if self.has_sink:
            specs.append(ParamSpec(n["sink"], (self.heads,), init=("normal", 1.0)))
        return specs

    def bind(self, tensors) -> None:
        fused = tensors["qkv_proj.weight"]
        if self.fused_width % 8:
            pad = torch.zeros((8 - self.fused_width % 8, self.hidden), dtype=fused.dtype, device=fused.device)
            fused = torch.cat([fused, pad], dim=0).contiguous()
        bias = tensors.get("qkv_proj.bias")
        if bias is not None and bias.shape[0] != fused.shape[0]:      # gate rows and padding rows carry no bias
            bias = torch.cat([bias.float(), torch.zeros(fused.shape[0] - bias.shape[0], dtype=torch.float32,
                                                        device=bias.device)])
        self.qkv = Linear(fused, bias)
        self.out = Linear(tensors[self.names["o"]], tensors.get("o_proj.bias"))
        if self.qk_norm and not self.norm_weight:
            self.q_norm = self.k_norm = torch.ones(self.head_dim, dtype=torch.float32, device=fused.device)
        elif self.qk_norm:
            self.q_norm, self.k_norm = tensors["q_norm.weight"], tensors["k_norm.weight"]
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()
        if self.has_sink:
            self.sinks = tensors[self.names["sink"]].float().contiguous()

    def cache_requests(self) -> list:
        window = int(self.window) if self.window is not None and self.ring else None
        return [KVRequest(self.kv_heads, self.head_dim, window,
                          value_dim=self.value_dim if self.value_dim != self.head_dim else None)]

    def launch_signature(self, rows: int, longest: int) -> tuple:
        """The choices a captured decode step of `rows` sequences of at most `longest` tokens
        freezes for this part (the form of its decode kernel)."""
        return self.launcher.launch_signature(self.env.dtype, rows, longest, self.env.device)

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        view = views[0]
        plan = ctx.plan
        if owns_cache and not self.own_kv:
            raise invalid_argument("an attention layer without key and value projections reads another layer's cache "
                                   "(the schedule entry's `cache_from`)")
        qkv = self.qkv.forward(x)
        position = self.position
        rotate = dict(cos=position.cos, sin=position.sin, rotary_dim=position.rotary_dim) if position is not None \
            else dict(cos=None, sin=None, rotary_dim=0)
        if self.query_scale is not None:
            rotate["q_scale"] = self.query_scale.table
        common = dict(heads=self.heads, kv_heads=self.kv_heads if self.own_kv else 0, head_dim=self.head_dim,
                      value_dim=self.value_dim)
        ring = view.ring_pages > 0
        extras = {}
        if self.has_sink:
            extras["sinks"] = self.sinks
        if self.has_gate:
            extras["gate"] = qkv[:, self.gate_begin:self.gate_begin + self.heads]
        if self.value_dim != self.head_dim:
            extras["value_dim"] = self.value_dim
        # A ring that is written before attention would lose keys that the step's
        # earlier rows still need; it is written afterwards unless the step is one
        # token per sequence. A full-history cache is written first.
        store_first = owns_cache and (not ring or plan.is_decode)
        if not owns_cache and ring and not plan.is_decode:
            raise unsupported("a layer that reads another layer's windowed cache takes one token per step")
        # One token per sequence on the tensor-core path: the attention kernel takes the rows as
        # the projection left them and does norm, rotation and the cache write itself.
        fused = owns_cache and store_first and self.value_dim == self.head_dim and self.query_scale is None \
            and self.launcher.fuses_rotation(plan, qkv, kv_view=view, q_norm=self.q_norm, k_norm=self.k_norm, **rotate)
        if not fused:
            ops.rope_store(qkv, q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, tables=ctx.tables, kv_view=view,
                           store=store_first, **rotate, **common)
        attended = torch.empty((qkv.shape[0], self.out_width), dtype=qkv.dtype, device=qkv.device)
        keys_in_step = owns_cache and not plan.is_decode
        rotation = dict(q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, store=True, **rotate) if fused else None
        self.launcher.run(ctx, qkv, attended, kv_view=view, keys_in_step=keys_in_step, rotation=rotation,
                          step_rows_cached=store_first and not fused, q_only=not self.own_kv, **extras)
        if owns_cache and not store_first:
            ops.rope_store(qkv, q_norm=None, k_norm=None, eps=self.eps, tables=ctx.tables, kv_view=view, store=True,
                           transform=False, cos=None, sin=None, rotary_dim=0, **common)
        if self.output_gate:
            ops.sigmoid_gate(attended, qkv[:, self.gate_begin:self.gate_begin + self.out_width])
        return self.out.forward(attended, sink=sink)
