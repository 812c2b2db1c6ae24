"""How a layer's parts are wired around the residual stream.

`pre_norm` is the reference's Qwen3 block (src/kidi/layers/qwen3.cpp:111-122):
    h = x + mixer(input_norm(x));  out = h + feed_forward(post_norm(h))
Each sum is handed to the stream as a pending delta and formed by the next norm, in
32-bit.

Interface of an arrangement: `__init__(spec, env, parts)` with the layer's parts by
role name, `children()`, and `forward(stream, ctx, views, owns_cache)`. Optionally
`first_norm()` (the norm it applies to the stream first) and, with the class attribute
`supports_next_norm`, `forward(..., next_norm=...)`: the norm that reads the stream after
this layer, so that the layer's last product can prepare the rows for it.

Norms between two products need no launch of their own when both products run on the
weight-streaming kernel (`ResidualSink`, `RowScaled` in parts/base.py): the product before
the norm adds its result to the stream and prepares the rows, the product after applies
each row's factor. The arrangement only makes the offers; parts that do not know them
get and return plain matrices.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..errors import invalid_argument
from .base import Part, ResidualSink, ResidualStream, plain_rows
from .registry import register_part
from .spec import ParamSpec


import os

# Which norms are folded into the products around them: "all", "post" (the norm after the mixer only),
# "none".
FOLD_NORMS = os.environ.get("KIDI_B200_FOLD_NORMS", "all")


def normed_for(norm: Part, stream: ResidualStream, consumer: Part):
    """The stream's rows normalised by `norm`, as a `RowScaled` where `consumer` takes one."""
    if getattr(consumer, "accepts_row_scaled", False) and hasattr(norm, "prepared_weight"):
        return norm.forward(stream, scaled=True)
    return plain_rows(norm.forward(stream))


def sink_for(part: Part, stream: ResidualStream, norm):
    """The offer to `part` to add its result to the stream itself, for `norm` to find prepared."""
    if norm is not None and FOLD_NORMS != "none" and getattr(part, "takes_sink", False) and hasattr(norm, "prepared_weight"):
        return {"sink": ResidualSink(stream, norm)}
    return {}


@register_part("arrangement", "pre_norm")
class PreNormBlock(Part):
    """Optional parts: without `feed_forward` (and `post_norm`) the block has its first sublayer only;
    `token_input` adds a function of the rows' token ids to the stream after the sublayers; `stream_mix`
    then replaces the stream by a function of the streams that earlier layers left."""

    ROLES = {"input_norm": "norm", "mixer": "mixer"}
    OPTIONAL_ROLES = {"post_norm": "norm", "feed_forward": "feed_forward", "token_input": "token_input",
                      "stream_mix": "stream_mix"}

    def __init__(self, spec, env, parts: Dict[str, Part]):
        super().__init__(spec, env)
        self.input_norm = parts["input_norm"]
        self.mixer = parts["mixer"]
        self.post_norm = parts.get("post_norm")
        self.feed_forward = parts.get("feed_forward")
        self.token_input = parts.get("token_input")
        self.stream_mix = parts.get("stream_mix")
        if (self.post_norm is None) != (self.feed_forward is None):
            raise invalid_argument("a pre-norm block has a feed-forward and the norm before it, or neither")

    def children(self):
        return tuple(part for part in (self.input_norm, self.mixer, self.post_norm, self.feed_forward,
                                       self.token_input, self.stream_mix) if part is not None)

    def cache_requests(self) -> list:
        return self.mixer.cache_requests()

    supports_next_norm = True

    def first_norm(self) -> Part:
        return self.input_norm

    def forward(self, stream: ResidualStream, ctx, views, owns_cache: bool, next_norm=None) -> None:
        if self.stream_mix is not None:
            self.stream_mix.begin(stream, ctx)
        if self.token_input is not None or self.stream_mix is not None:
            next_norm = None          # the stream changes once more before the next layer's norm reads it
        stream.add(self.mixer.forward(normed_for(self.input_norm, stream, self.mixer), ctx, views, owns_cache,
                                      **sink_for(self.mixer, stream, self.post_norm)))
        if self.feed_forward is not None:
            stream.add(self.feed_forward.forward(normed_for(self.post_norm, stream, self.feed_forward), ctx,
                                                 **sink_for(self.feed_forward, stream,
                                                            next_norm if FOLD_NORMS == "all" else None)))
        if self.token_input is not None:
            self.token_input.forward(stream, ctx, mix=self.stream_mix)
        elif self.stream_mix is not None:
            self.stream_mix.forward(stream, ctx)


@register_part("arrangement", "parallel")
class ParallelBlock(Part):
    """One norm, and both sublayers read its output: h = norm(x), x <- x + (mixer(h) + feed_forward(h)).
    The feed-forward is optional. Both results are added to the 32-bit stream: the feed-forward's at once,
    the mixer's as the pending delta that the next norm adds while it normalises."""

    ROLES = {"input_norm": "norm", "mixer": "mixer"}
    OPTIONAL_ROLES = {"feed_forward": "feed_forward"}

    def __init__(self, spec, env, parts: Dict[str, Part]):
        super().__init__(spec, env)
        self.input_norm = parts["input_norm"]
        self.mixer = parts["mixer"]
        self.feed_forward = parts.get("feed_forward")

    def children(self):
        return tuple(part for part in (self.input_norm, self.mixer, self.feed_forward) if part is not None)

    def cache_requests(self) -> list:
        return self.mixer.cache_requests()

    def first_norm(self) -> Part:
        return self.input_norm

    def forward(self, stream: ResidualStream, ctx, views, owns_cache: bool) -> None:
        from ..kernels import ops
        normed = plain_rows(self.input_norm.forward(stream))
        mixed = self.mixer.forward(normed, ctx, views, owns_cache)
        if self.feed_forward is not None:
            ops.add_cast(stream.hidden, self.feed_forward.forward(normed, ctx), None)
        stream.add(mixed)


@register_part("arrangement", "sandwich_norm")
class SandwichNormBlock(Part):
    """A norm before and a norm behind each sublayer:
        x <- x + mixer_out_norm(mixer(input_norm(x)));  x <- x + feed_forward_out_norm(feed_forward(post_norm(x)))
    The feed-forward (with its two norms) is optional. The norms behind the sublayers have a weight and no bias
    (`delta_weight()`); a sublayer's result goes to the stream together with its norm, and the norm that reads the
    stream next normalises the result, forms the 32-bit sum and normalises the sum in one kernel."""

    ROLES = {"input_norm": "norm", "mixer": "mixer", "mixer_out_norm": "norm"}
    OPTIONAL_ROLES = {"post_norm": "norm", "feed_forward": "feed_forward", "feed_forward_out_norm": "norm"}

    def __init__(self, spec, env, parts: Dict[str, Part]):
        super().__init__(spec, env)
        self.input_norm = parts["input_norm"]
        self.mixer = parts["mixer"]
        self.mixer_out_norm = parts["mixer_out_norm"]
        self.post_norm = parts.get("post_norm")
        self.feed_forward = parts.get("feed_forward")
        self.feed_forward_out_norm = parts.get("feed_forward_out_norm")
        if len({self.post_norm is None, self.feed_forward is None, self.feed_forward_out_norm is None}) != 1:
            raise invalid_argument("a sandwich block has a feed-forward with the norms before and behind it, or none")
        for norm in (self.mixer_out_norm, self.feed_forward_out_norm):
            if norm is not None and not hasattr(norm, "delta_weight"):
                raise invalid_argument("the norm behind a sublayer must be one that a residual delta can pass")

    def children(self):
        return tuple(part for part in (self.input_norm, self.mixer, self.mixer_out_norm, self.post_norm,
                                       self.feed_forward, self.feed_forward_out_norm) if part is not None)

    def cache_requests(self) -> list:
        return self.mixer.cache_requests()

    def first_norm(self) -> Part:
        return self.input_norm

    def forward(self, stream: ResidualStream, ctx, views, owns_cache: bool) -> None:
        mixed = self.mixer.forward(plain_rows(self.input_norm.forward(stream)), ctx, views, owns_cache)
        stream.add(mixed, normed_by=self.mixer_out_norm)
        if self.feed_forward is not None:
            result = self.feed_forward.forward(plain_rows(self.post_norm.forward(stream)), ctx)
            stream.add(result, normed_by=self.feed_forward_out_norm)


@register_part("arrangement", "hyper_connections")
class HyperConnectionBlock(Part):
    """A pre-norm block over a residual stream that is kept as `streams` lanes x_1 .. x_s (all equal to what the
    embedding left, at the first such block). Sublayer q (1: the mixer, 2: the feed-forward, optional) reads one
    weighted sum of the lanes and writes its result back into every lane while the lanes mix:

        u = sum_s in_q[s] x_s;   y = sublayer(norm(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y    (all t at once)

    The sum that a norm reads is formed in the norm's kernel, and so is the update of the lanes before it (it waits
    in `ResidualStream.lane_update` for the next norm, as a residual delta does); lanes, sums and updates are 32-bit. After the last block the stream is the sum of the lanes (the norm before the head reads
    that sum). Parameters: hidden_size, streams, and the tensor names under the prefix: in1, out1, mix1, in2, out2,
    mix2 (defaults hc1.in, hc1.out, hc1.mix, hc2.in, hc2.out, hc2.mix)."""

    ROLES = {"input_norm": "norm", "mixer": "mixer"}
    OPTIONAL_ROLES = {"post_norm": "norm", "feed_forward": "feed_forward"}
    MAX_STREAMS = 8

    def __init__(self, spec, env, parts: Dict[str, Part]):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.streams = int(spec.param("streams"))
        if not 1 <= self.streams <= self.MAX_STREAMS:
            raise invalid_argument(f"a stream is kept as 1 to {self.MAX_STREAMS} lanes")
        self.input_norm = parts["input_norm"]
        self.mixer = parts["mixer"]
        self.post_norm = parts.get("post_norm")
        self.feed_forward = parts.get("feed_forward")
        if (self.post_norm is None) != (self.feed_forward is None):
            raise invalid_argument("a block has a feed-forward and the norm before it, or neither")
        for norm in (self.input_norm, self.post_norm):
            if norm is not None and not getattr(norm, "reads_lanes", False):
                raise invalid_argument("the norms of a block over several lanes must be able to read lanes")
        self.names = {key: spec.param(key + "_name", default) for key, default in (
            ("in1", "hc1.in"), ("out1", "hc1.out"), ("mix1", "hc1.mix"), ("in2", "hc2.in"), ("out2", "hc2.out"),
            ("mix2", "hc2.mix"))}
        self.weights: Dict[str, torch.Tensor] = {}

    def children(self):
        return tuple(part for part in (self.input_norm, self.mixer, self.post_norm, self.feed_forward)
                     if part is not None)

    def parameter_specs(self) -> List[ParamSpec]:
        count, n = self.streams, self.names
        specs = []
        for number in ("1", "2") if self.feed_forward is not None else ("1",):
            specs += [ParamSpec(n["in" + number], (count,), init=("one_plus_normal", 0.2)),
                      ParamSpec(n["out" + number], (count,), init=("one_plus_normal", 0.2)),
                      ParamSpec(n["mix" + number], (count, count), init=("eye_plus_normal", 0.1))]
        return specs

    def bind(self, tensors) -> None:
        self.weights = {key: tensors[name].float().contiguous() for key, name in self.names.items() if name in tensors}

    def cache_requests(self) -> list:
        return self.mixer.cache_requests()

    def first_norm(self) -> Part:
        return self.input_norm

    def _write(self, stream: ResidualStream, number: str, result: torch.Tensor) -> None:
        """The update waits for the norm that reads the lanes next, which applies it in its own kernel."""
        stream.apply_lane_update()
        stream.lane_update = (self.weights["mix" + number], self.weights["out" + number], result.contiguous())

    def forward(self, stream: ResidualStream, ctx, views, owns_cache: bool) -> None:
        if stream.lanes is None:
            pending = stream.take_pending()
            if pending is not None:
                from ..kernels import ops
                ops.add_cast(stream.hidden, pending, None)
            stream.lanes = stream.hidden.unsqueeze(0).expand(self.streams, *stream.hidden.shape)
        elif stream.lanes.shape[0] != self.streams:
            raise invalid_argument("every block of a model keeps the stream as the same number of lanes")
        normed = self.input_norm.forward(stream, read=self.weights["in1"])
        self._write(stream, "1", self.mixer.forward(normed, ctx, views, owns_cache))
        if self.feed_forward is not None:
            normed = self.post_norm.forward(stream, read=self.weights["in2"])
            self._write(stream, "2", self.feed_forward.forward(normed, ctx))
