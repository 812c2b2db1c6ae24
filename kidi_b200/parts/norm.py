"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * w.

The reference's RmsNorm (src/kidi/layers/gemma4.cpp:23-67; op contract
src/kidi/ops/context.cpp:1043-1082; arithmetic
src/kidi/runtime/mps/eager_kernels.metal:65-87). The norm is also where the residual
stream takes its pending delta: sum and normalisation run in one kernel, in 32-bit.

Parameters of `rms_norm`: size, eps, weight_name (the tensor's name under the prefix, default "weight") and
weight_offset (default 0): the stored tensor plus this number is the weight, so a weight that a model stores
around zero has weight_offset 1: y = x / sqrt(mean(x^2) + eps) * (1 + w).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import Part, ResidualStream, RowScaled
from .registry import register_part
from .spec import ParamSpec


@register_part("norm", "rms_norm")
class RMSNorm(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.param("size"))
        self.eps = float(spec.param("eps"))
        self.weight_name = spec.param("weight_name", "weight")
        self.offset = float(spec.param("weight_offset", 0.0))
        self.weight: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        init = ("normal", 0.1) if self.offset else ("one_plus_normal", 0.1)
        return [ParamSpec(self.weight_name, (self.size,), init=init)]

    def bind(self, tensors) -> None:
        self.weight = tensors[self.weight_name]
        if self.offset:           # the sum is formed once, in 32-bit
            self.weight = (self.weight.float() + self.offset).contiguous()

    def prepared_weight(self) -> Optional[torch.Tensor]:
        """The weight vector a product needs to prepare rows for this norm (`ResidualSink`), or
        None when this norm does not take prepared rows."""
        return self.weight if self.env.dtype == torch.bfloat16 and not self.offset else None

    reads_lanes = True            # a stream kept as several lanes is read as a weighted sum of them

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, scaled: bool = False,
                out_dtype: Optional[torch.dtype] = None, read: Optional[torch.Tensor] = None):
        """Adds the stream's pending delta and returns the normalised rows in the
        engine dtype (or `out_dtype`). With `rows` (int32 indices) only those rows are produced and the
        stream itself is left untouched. With `scaled` the caller takes a `RowScaled` too:
        when the product before has prepared the rows (added its result to the stream, multiplied
        by this norm's weight, summed the squares) there is nothing left to launch. A stream that is kept as
        several lanes is read as sum_s read[s] * lane_s (`read` float32 [lanes]; None: the plain sum) and
        normalised in the same kernel."""
        if stream.lanes is not None:
            if self.offset and self.weight.dtype != torch.float32:
                raise RuntimeError("a norm with a weight offset keeps its weight in 32-bit")
            if stream.lane_update is not None:        # the lanes' waiting update and this read in one kernel
                mix, write, y = stream.lane_update
                target = stream.lane_target()
                normed = ops.lanes_mix_rmsnorm(stream.lanes, target, mix, write, y, read, self.weight, self.eps,
                                               out_dtype or self.env.dtype, row_index=rows)
                if rows is None:
                    stream.lanes, stream.lane_update = target, None
                return normed
            return ops.lanes_rmsnorm(stream.lanes, read, self.weight, self.eps, out_dtype or self.env.dtype,
                                     row_index=rows)
        prepared = stream.take_prepared(self) if rows is None else None
        if prepared is not None:
            ready = RowScaled(prepared[0], prepared[1], self.size, self.eps)
            return ready if scaled else ready.plain()
        return ops.add_rmsnorm(stream.hidden, stream.take_pending(), self.weight, self.eps,
                               out_dtype or self.env.dtype, row_index=rows)


@register_part("norm", "layer_norm")
class LayerNorm(Part):
    """y = (x - mean(x)) / sqrt(mean((x - mean)^2) + eps) * w + b over each row, in 32-bit, in the kernel
    that also forms the residual sum. Parameters: size, eps, weight_name and bias_name (tensor names under
    the prefix; default "weight" and "bias"), bias (default true; false: the norm has a weight only).

    A norm without bias can also stand behind a sublayer, x <- x + norm(sublayer(...)): the arrangement hands
    the sublayer's result to the stream with `normed_by=` this part, and the norm that reads the stream next
    normalises the delta, adds it and normalises the sum in one kernel (`delta_weight`)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.param("size"))
        self.eps = float(spec.param("eps"))
        self.weight_name = spec.param("weight_name", "weight")
        self.bias_name = spec.param("bias_name", "bias")
        self.has_bias = bool(spec.param("bias", True))
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.weight_name, (self.size,), init=("one_plus_normal", 0.1))]
        if self.has_bias:
            specs.append(ParamSpec(self.bias_name, (self.size,), init=("normal", 0.1)))
        return specs

    def bind(self, tensors) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()
        self.bias = tensors[self.bias_name].float().contiguous() if self.has_bias else None

    def delta_weight(self):
        """(weight, eps) for a kernel that applies this norm to a residual delta before adding it."""
        if self.has_bias:
            raise RuntimeError("a norm behind a sublayer has no bias")
        return self.weight, self.eps

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, scaled: bool = False):
        delta, delta_norm = stream.take_pending_normed()
        weight, eps = delta_norm.delta_weight() if delta_norm is not None else (None, 0.0)
        if rows is not None and delta is not None:
            # Only some rows are wanted and the stream stays as it is: the delta goes back for whoever reads it next.
            stream.pending, stream.pending_norm = delta, delta_norm
        return ops.add_layernorm(stream.hidden, delta, self.weight, self.bias, self.eps, self.env.dtype,
                                 row_index=rows, delta_weight=weight, delta_eps=eps)
