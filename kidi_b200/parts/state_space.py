"""A selective state-space mixer with one decay per head (Mamba-2, the scalar-decay form of the state-space
duality) as a mixer.

With h the mixer's input, H heads of e values, N state rows, G groups (head j reads group j // (H / G)) and
inner = H e, one projection gives [z: inner | x: inner | B: G N | C: G N | dt: H]. x, B and C together pass a short
causal convolution per channel (taps `conv`, a bias) and SiLU. Then per head, with step = softplus(dt + dt_bias):

    S_t = exp(-exp(A_log) step) S_(t-1) + step B_t x_t^T         S: [N, e]
    y_t = S_t^T C_t + D x_t

y (heads concatenated) is multiplied by silu(z), divided by its root mean square in `norm_groups` equal parts,
multiplied by a weight [inner] and projected by W_o. What a sequence keeps, as fixed-size state per cache slot:
S in 32-bit floats and the convolution's last taps - 1 inputs. Steps, decays, state, read-out and norm are 32-bit; so
is the result of dt's projection (a product of its own, H rows), since its rounding would be multiplied by the decay rate
inside an exponential.

Parameters (`spec.params`): hidden_size, num_heads, vdim, state, groups, conv (taps), norm_groups, eps, and the
tensor names under the prefix: in, conv, conv_bias, dt_bias, a_log, skip, norm, o.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..errors import invalid_argument, unsupported
from ..kernels import scalar_recurrence as kernels
from .base import Part, plain_rows
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec

NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "skip": "D",
         "norm": "norm", "o": "o"}


@register_part("mixer", "mamba2")
class StateSpaceMixer(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.heads = int(spec.param("num_heads"))
        self.vdim = int(spec.param("vdim"))
        self.state = int(spec.param("state"))
        self.groups = int(spec.param("groups", 1))
        self.taps = int(spec.param("conv"))
        self.norm_groups = int(spec.param("norm_groups", 1))
        self.eps = float(spec.param("eps"))
        if min(self.hidden, self.heads, self.vdim, self.state, self.groups, self.norm_groups) <= 0:
            raise invalid_argument("invalid state-space dimensions")
        self.inner = self.heads * self.vdim
        if self.heads % self.groups or self.inner % self.norm_groups:
            raise invalid_argument("a state-space mixer's heads split into equal groups and its rows into equal parts")
        if self.state > kernels.MAX_DIM:
            raise unsupported(f"a state of {self.state} rows a head exceeds {kernels.MAX_DIM}, the most the kernel takes")
        if not 1 <= self.taps <= kernels.MAX_TAPS:
            raise unsupported(f"the short convolution takes 1 to {kernels.MAX_TAPS} taps")
        self.channels = self.inner + 2 * self.groups * self.state          # what the convolution runs over
        self.width = 2 * self.inner + 2 * self.groups * self.state + self.heads
        self.names = {key: spec.param(key + "_name", default) for key, default in NAMES.items()}
        self.projection: Optional[Linear] = None
        self.step_projection: Optional[Linear] = None
        self.out: Optional[Linear] = None

    def parameter_specs(self) -> List[ParamSpec]:
        n = self.names
        return [
            ParamSpec(n["in"], (self.width, self.hidden)),
            ParamSpec(n["conv"], (self.channels, self.taps), init=("normal", 0.5)),
            ParamSpec(n["conv_bias"], (self.channels,), init=("normal", 0.1)),
            ParamSpec(n["dt_bias"], (self.heads,), init=("normal", 1.0)),
            ParamSpec(n["a_log"], (self.heads,), init=("normal", 0.5)),
            ParamSpec(n["skip"], (self.heads,), init=("one_plus_normal", 0.1)),
            ParamSpec(n["norm"], (self.inner,), init=("one_plus_normal", 0.1)),
            ParamSpec(n["o"], (self.hidden, self.inner)),
        ]

    def bind(self, tensors) -> None:
        n = self.names
        def padded(matrix):        # rows of a product's result start on 16-byte boundaries
            extra = -matrix.shape[0] % 8
            pad = torch.zeros((extra, self.hidden), dtype=matrix.dtype, device=matrix.device)
            return torch.cat([matrix, pad], dim=0).contiguous()

        fused, main = tensors[n["in"]], self.width - self.heads
        self.projection, self.step_projection = Linear(padded(fused[:main])), Linear(padded(fused[main:]))
        self.out = Linear(tensors[n["o"]])
        # everything that enters the recurrence beside the projections is 32-bit
        for key in ("conv", "conv_bias", "dt_bias", "a_log", "skip", "norm"):
            setattr(self, key, tensors[n[key]].float().contiguous())

    def cache_requests(self) -> list:
        requests = [StateRequest((self.heads, self.state, self.vdim), torch.float32)]
        if self.taps > 1:
            requests.append(StateRequest((self.taps - 1, self.channels)))
        return requests

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        if not owns_cache:
            raise invalid_argument("a state-space layer keeps a state of its own")
        plan = ctx.plan
        x = plain_rows(x)
        projected = self.projection.forward(x)
        steps = self.step_projection.forward(x, out_dtype=torch.float32)
        inner, span = self.inner, self.groups * self.state
        z = projected[:, :inner]
        mixed = kernels.short_conv(projected[:, inner:inner + self.channels], self.conv, self.conv_bias,
                                   views[1] if self.taps > 1 else None, silu=True, tables=ctx.tables, seqs=plan.n_seqs,
                                   one_token=plan.is_decode)
        coef = kernels.state_space_gates(steps[:, :self.heads], self.dt_bias, self.a_log)
        values = mixed[:, :inner]
        read = kernels.scalar_recurrence(mixed[:, inner:inner + span], mixed[:, inner + span:], values, coef, views[0],
                                         heads=self.heads, k_heads=self.groups, q_heads=self.groups, dim=self.state,
                                         vdim=self.vdim, tables=ctx.tables, seqs=plan.n_seqs)
        gated = kernels.state_space_finish(read, values, z, self.skip, self.norm, heads=self.heads, vdim=self.vdim,
                                           parts=self.norm_groups, eps=self.eps)
        return self.out.forward(gated)
