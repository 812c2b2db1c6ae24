"""Depth average: what goes on to the next layer is a weighted sum of the embedding output and of every
layer's result so far.

With X_0 the embedding output and X_(i+1) the result of layer i, layer i hands on
x = sum_{j <= i+1} w_i[j] X_j, with a weight vector of its own (i + 2 numbers). The sum is 32-bit.

The X_j are kept in `ResidualStream.kept` [layers + 2, rows, hidden]: row 0 is X_0; a layer works in place on
row i + 1 (which starts as the sum that the layer before handed on) and the sum it hands on is written to row
i + 2, so nothing is copied but the embedding output, once.

Parameters: index (i), layers (how many layers mix, which sizes the store), name (the weights' tensor name).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..errors import invalid_argument
from ..kernels import ops
from .base import Part, ResidualStream
from .registry import register_part
from .spec import ParamSpec


@register_part("stream_mix", "depth_average")
class DepthAverage(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.index = int(spec.param("index"))
        self.layers = int(spec.param("layers"))
        self.name = spec.param("name", "weight")
        if not 0 <= self.index < self.layers:
            raise invalid_argument("a depth average's index lies outside its layers")
        self.weight: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.name, (self.index + 2,), init=("last_one", 0.2))]

    def bind(self, tensors) -> None:
        self.weight = tensors[self.name].float().contiguous()

    def begin(self, stream: ResidualStream, ctx) -> None:
        """Before the layer runs: the first layer sets the store up and keeps the embedding output."""
        if stream.kept is None:
            if self.index != 0:
                raise invalid_argument("the first layer of a depth average must have index 0")
            rows, hidden = stream.hidden.shape
            count = (self.layers + 2) * rows * hidden
            stream.kept = ctx.workspace("kept_streams", count)[:count].view(self.layers + 2, rows, hidden)
            stream.kept[0].copy_(stream.hidden)
            stream.kept[1].copy_(stream.hidden)
            stream.hidden = stream.kept[1]
            stream.kept_count = 1
        if stream.kept_count != self.index + 1:
            raise invalid_argument("the layers of a depth average must run in the order of their indices")

    def forward(self, stream: ResidualStream, ctx, addend=None) -> None:
        """After the layer: the stream (with its pending delta, and with `addend` = (y, weight, eps) added as
        y / rms(y) * weight) is X_(index+1); the weighted sum replaces it."""
        x = stream.hidden
        if stream.pending is not None:
            ops.add_cast(x, stream.take_pending(), None)
        mixed = stream.kept[self.index + 2]
        y, weight, eps = addend if addend is not None else (None, None, 0.0)
        ops.add_normed_mix(x, y, weight, eps, kept=stream.kept, mix=self.weight, mixed=mixed)
        stream.hidden = mixed
        stream.kept_count = self.index + 2
        stream.prepared = None


@register_part("shared", "stream_offsets")
class StreamOffsets(Part):
    """A table [count, hidden] of learned vectors of which the run order names one at some of its positions
    (`ScheduleEntry.offset`): `add(stream, index)` adds row `index` to every row of the stream, in 32-bit, before
    that position's layer runs: the vector that marks the pass of a range of layers that runs several times, say.
    Parameters: hidden_size, count, name (the tensor's name, default "weight")."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.count = int(spec.param("count"))
        self.name = spec.param("name", "weight")
        if self.hidden <= 0 or self.count <= 0:
            raise invalid_argument("a table of stream offsets needs a positive width and count")
        self.table = None

    def parameter_specs(self):
        return [ParamSpec(self.name, (self.count, self.hidden), init=("normal", 0.1))]

    def bind(self, tensors) -> None:
        self.table = tensors[self.name]

    def add(self, stream: ResidualStream, index: int) -> None:
        if not 0 <= index < self.count:
            raise invalid_argument(f"the run order names stream offset {index} of {self.count}")
        # A delta that is still pending is added by the next norm; the order of the two additions does not matter.
        stream.prepared = None
        ops.add_vector(stream.hidden, self.table[index])
