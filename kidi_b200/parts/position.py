"""Position encodings.

`rotary` is the reference's table: freq_i = 1 / theta^(2i/d) for i < d/2,
angle = float(position) * freq_i, cos and sin of it, all in 32-bit, positions from
0 (src/kidi/model/qwen3.cpp:138-157). A mixer that rotates its queries and keys looks
the encoding up by name in `env.positions` and hands `cos`/`sin` to its kernel.

With `scaling` = {factor, original, fast, slow} the table is stretched for sequences longer than the `original`
length the frequencies were meant for (the scheme known as YaRN): pair i completes original * f_i / (2 pi) turns
over that length; pairs that turn more often than `fast` keep their frequency, pairs that turn less often than
`slow` have it divided by `factor`, and a linear ramp over the pair index blends between the two,
    turns_to_pair(t) = n ln(original / (2 pi t)) / (2 ln theta),   n the rotary width
    lo = max(floor(turns_to_pair(fast)), 0),  hi = min(ceil(turns_to_pair(slow)), n - 1)
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),   f_i <- f_i / factor * ramp_i + f_i (1 - ramp_i)
and cosine and sine are both multiplied by 0.1 ln(factor) + 1.

`learned_positions` is a table with a vector per position that is added to the embeddings
(times `scale`, default 1), in 32-bit; mixers read nothing from it. Parameters: hidden_size,
max_positions, scale, name (the table's tensor name under the prefix, default "weight").

`query_temperature` is a factor per position that an attention layer multiplies its queries by (named in the
layer's `query_scale`): 1 + coef * ln(floor((p + 1) / every) + 1) at position p, so that scores sharpen step by
step as a sequence grows. Parameters: coef, every, max_positions. The table is 32-bit, built once.

Interface of a position encoding: `on_embeddings(stream, ctx)` (may change the
embeddings; rotary does nothing there) and whatever its mixers agree to read from it
(`cos`, `sin`, `rotary_dim` here).
"""
from __future__ import annotations

import torch

from ..errors import invalid_argument
from ..kernels import ops
from .base import Part
from .registry import register_part
from .spec import ParamSpec


@register_part("position", "rotary")
class RotaryEncoding(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec.param("head_dim"))
        self.rotary_dim = int(spec.param("rotary_dim", self.head_dim))
        self.theta = float(spec.param("theta"))
        self.max_positions = int(spec.param("max_positions"))
        scaling = spec.param("scaling", None)
        self.scaling = {key: float(scaling[key]) for key in ("factor", "original", "fast", "slow")} if scaling else None
        if self.scaling is not None and (self.scaling["factor"] <= 0 or self.scaling["original"] <= 0
                                         or self.scaling["fast"] <= 0 or self.scaling["slow"] <= 0 or self.theta <= 1):
            raise invalid_argument("a stretched rotary encoding needs positive constants and a base above 1")
        if self.rotary_dim <= 0 or self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise invalid_argument("the rotary width must be even and at most the head width")
        self._tables = None

    def _build(self):
        # Built at first use, on the host in 32-bit, then moved to the device once.
        if self._tables is None:
            half = self.rotary_dim // 2
            # The reference takes the power with the C library's 32-bit powf, which rounds correctly
            # in all but rare cases; a vectorised 32-bit power may be one unit off in the last
            # place, which the position multiplies (1e-4 in the cosine at position 1,000). So the
            # power is taken in 64-bit from the 32-bit base and exponent and rounded once.
            index = torch.arange(half, dtype=torch.float32)
            exponent = (2.0 * index) / torch.tensor(float(self.rotary_dim), dtype=torch.float32)
            power = torch.pow(torch.tensor(self.theta, dtype=torch.float32).double(), exponent.double()).float()
            frequency = 1.0 / power
            factor = 1.0
            if self.scaling is not None:
                import math
                s, n = self.scaling, float(self.rotary_dim)
                pair = lambda turns: n * math.log(s["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
                lo = max(math.floor(pair(s["fast"])), 0)
                hi = min(math.ceil(pair(s["slow"])), self.rotary_dim - 1)
                ramp = torch.clamp((index.double() - lo) / max(hi - lo, 0.001), 0.0, 1.0)
                frequency = (frequency.double() / s["factor"] * ramp + frequency.double() * (1.0 - ramp)).float()
                factor = 0.1 * math.log(s["factor"]) + 1.0
            angle = torch.arange(self.max_positions, dtype=torch.float32)[:, None] * frequency[None, :]
            self._tables = ((torch.cos(angle) * factor).contiguous().to(self.env.device),
                            (torch.sin(angle) * factor).contiguous().to(self.env.device))
        return self._tables

    @property
    def cos(self) -> torch.Tensor:
        return self._build()[0]

    @property
    def sin(self) -> torch.Tensor:
        return self._build()[1]

    def on_embeddings(self, stream, ctx) -> None:
        return None


@register_part("position", "learned_positions")
class LearnedPositions(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.max_positions = int(spec.param("max_positions"))
        self.scale = float(spec.param("scale", 1.0))
        self.name = spec.param("name", "weight")
        if self.hidden <= 0 or self.max_positions <= 0:
            raise invalid_argument("a position table needs a positive width and length")
        self.table = None

    def parameter_specs(self):
        return [ParamSpec(self.name, (self.max_positions, self.hidden), init=("normal", 0.05))]

    def bind(self, tensors) -> None:
        self.table = tensors[self.name]

    def on_embeddings(self, stream, ctx) -> None:
        ops.add_table_rows(stream.hidden, self.table, ctx.tables.row_pos, self.scale)


@register_part("position", "query_temperature")
class QueryTemperature(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.coef = float(spec.param("coef"))
        self.every = int(spec.param("every"))
        self.max_positions = int(spec.param("max_positions"))
        if self.every <= 0 or self.max_positions <= 0:
            raise invalid_argument("a query temperature needs a positive interval and length")
        self._table = None

    @property
    def table(self) -> torch.Tensor:
        """float32 [max_positions] on the device: the factor of each position (computed in 64-bit, rounded once)."""
        if self._table is None:
            position = torch.arange(self.max_positions, dtype=torch.float64)
            factor = 1.0 + self.coef * torch.log(torch.floor((position + 1.0) / self.every) + 1.0)
            self._table = factor.float().contiguous().to(self.env.device)
        return self._table

    def on_embeddings(self, stream, ctx) -> None:
        return None
