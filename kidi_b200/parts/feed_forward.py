"""Gated feed-forward: y = (act(x Wg^T) * (x Wu^T)) Wd^T.

The reference's GatedFeedForward (src/kidi/layers/gemma4.cpp:164-225): one fused
projection to [gate | up] (gate = first I columns), the activation on the gate times
up, then the down projection; no biases. SiLU is g / (1 + exp(-g))
(src/kidi/runtime/mps/eager_kernels.metal:129-137).

Parameters: hidden_size, intermediate_size, activation, gate_name, up_name, down_name (tensor names under the
prefix; default gate_proj.weight, up_proj.weight, down_proj.weight). Activations:

* "silu": y = silu(g) * u;
* "bounded_swish": g <- min(g, limit), u <- clamp(u, -limit, limit), y = g * sigmoid(alpha * g) * (u + up_shift),
  with the parameters limit, alpha (default 1.702) and up_shift (default 1).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..errors import invalid_argument, unsupported
from ..kernels import ops
from .base import Part, RowScaled
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec


@register_part("feed_forward", "gated_mlp")
class GatedFeedForward(Part):
    accepts_row_scaled = True     # x may lack its norm's factor: the gate/up product applies it
    takes_sink = True             # the down product may add its result to the residual stream itself

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.inter = int(spec.param("intermediate_size"))
        self.activation = spec.param("activation", "silu")
        if self.activation not in ("silu", "bounded_swish"):
            raise unsupported(f"gated feed-forward activation '{self.activation}' is not built "
                              f"(silu and bounded_swish are)")
        if self.activation == "bounded_swish":
            self.limit = float(spec.param("limit"))
            self.alpha = float(spec.param("alpha", 1.702))
            self.up_shift = float(spec.param("up_shift", 1.0))
            if not self.limit > 0:
                raise invalid_argument("the bound of a bounded gate must be positive")
        self.gate_name = spec.param("gate_name", "gate_proj.weight")
        self.up_name = spec.param("up_name", "up_proj.weight")
        self.down_name = spec.param("down_name", "down_proj.weight")
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def parameter_specs(self) -> List[ParamSpec]:
        return [
            ParamSpec("gate_up_proj.weight", (2 * self.inter, self.hidden), sources=(
                (self.gate_name, (self.inter, self.hidden)),
                (self.up_name, (self.inter, self.hidden)))),
            ParamSpec(self.down_name, (self.hidden, self.inter)),
        ]

    def bind(self, tensors) -> None:
        self.gate_up = Linear(tensors["gate_up_proj.weight"])
        self.down = Linear(tensors[self.down_name])

    def forward(self, x, ctx, sink=None) -> Optional[torch.Tensor]:
        from ..kernels import skinny, tcgen05
        if self.activation == "bounded_swish":
            both = self.gate_up.forward(x)
            return self.down.forward(ops.bounded_gate(both, self.limit, self.alpha, self.up_shift), sink=sink)
        factors = None
        if isinstance(x, RowScaled):
            if skinny.supports(x.values, self.gate_up.weight) and x.values.shape[0] <= skinny.MAX_ROWS:
                x, factors = x.values, x.factors
            else:
                x = x.plain()
        if factors is not None or skinny.fits(x, self.gate_up.weight):
            gated = skinny.gemm_silu_gate(x, self.gate_up.weight, factors=factors)
        elif tcgen05.MIN_GATED_ROWS <= x.shape[0] <= tcgen05.MAX_GATED_ROWS and tcgen05.fits(x, self.gate_up.weight):
            gated = tcgen05.gemm_silu_gate(x, self.gate_up.weight)
        else:
            gated = ops.silu_gate(self.gate_up.forward(x))
        return self.down.forward(gated, sink=sink)


@register_part("feed_forward", "dense_mlp")
class DenseFeedForward(Part):
    """y = act(x Wu^T) Wd^T with one up and one down projection and no gate. Parameters: hidden_size,
    intermediate_size, activation, eps (of the activation's norms), up_name, down_name, act_name (tensor names
    under the prefix). Activations:

    * "poly_norm": a N(z) + b N(z^2) + c N(z^3) + e, powers element by element, N(u) = u / sqrt(mean(u^2) + eps)
      over the intermediate values of a token, and (a, b, c, e) a tensor of four numbers;
    * "relu_squared": max(z, 0)^2 (no tensor of its own)."""

    ACTIVATIONS = ("poly_norm", "relu_squared")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.inter = int(spec.param("intermediate_size"))
        self.activation = spec.param("activation")
        if self.activation not in self.ACTIVATIONS:
            raise unsupported(f"dense feed-forward activation '{self.activation}' is not built "
                              f"({', '.join(self.ACTIVATIONS)} are)")
        self.eps = float(spec.param("eps", 1e-6))
        self.up_name = spec.param("up_name", "up_proj.weight")
        self.down_name = spec.param("down_name", "down_proj.weight")
        self.act_name = spec.param("act_name", "act")
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None
        self.coefficients: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.up_name, (self.inter, self.hidden)),
                 ParamSpec(self.down_name, (self.hidden, self.inter))]
        if self.activation == "poly_norm":
            specs.append(ParamSpec(self.act_name, (4,), init=("normal", 0.5)))
        return specs

    def bind(self, tensors) -> None:
        self.up = Linear(tensors[self.up_name])
        self.down = Linear(tensors[self.down_name])
        if self.activation == "poly_norm":
            self.coefficients = tensors[self.act_name].float().contiguous()

    def forward(self, x, ctx, sink=None) -> Optional[torch.Tensor]:
        if self.activation == "relu_squared":
            from ..kernels import skinny
            if self.up.bias is None and skinny.fits(x, self.up.weight):     # few rows: the activation in the epilogue
                return self.down.forward(skinny.gemm(x, self.up.weight, x.dtype, activation="relu_squared"))
            z = self.up.forward(x)
            return self.down.forward(ops.relu_squared(z, out=z))
        z = self.up.forward(x)
        return self.down.forward(ops.poly_norm(z, self.coefficients, self.eps))
