"""A matrix memory with exponential gates (the mLSTM of xLSTM) as a mixer.

With h the mixer's input, H heads, d the width of a query or key head and e the width of a value head:

    q = W_q h / sqrt(d),  k = W_k h  [H, d],   v = W_v h  [H, e]
    i = cap tanh((W_i h + b_i) / cap),   f = logsigmoid(cap tanh((W_f h + b_f) / cap))      (log gates, one a head)
    m_t = max(f_t + m_(t-1), i_t)                                                            (m_0 = 0)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Each head's o is divided by its root mean square; the heads are concatenated, multiplied by a weight [H e] and by
sigmoid(W_g h), and projected by W_o. What a sequence keeps, as fixed-size 32-bit state per cache slot: S with n as
one more column, [H, d, e + 1], and m [H]. Gates, the maximum, the state, the read-out and the norm are 32-bit.

Parameters (`spec.params`): hidden_size, num_heads, dim, vdim, gate_cap, eps, and the tensor names under the prefix:
q, k, v, g, o, norm, i, i_bias, f, f_bias.
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

NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "i_bias": "i.b", "f": "f",
         "f_bias": "f.b"}
NORMALISER_FLOOR = 1e-6       # added to the read-out's denominator


@register_part("mixer", "mlstm")
class MatrixMemory(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.heads = int(spec.param("num_heads"))
        self.dim = int(spec.param("dim"))
        self.vdim = int(spec.param("vdim"))
        self.cap = float(spec.param("gate_cap"))
        self.eps = float(spec.param("eps"))
        if min(self.hidden, self.heads, self.dim, self.vdim) <= 0 or not self.cap > 0:
            raise invalid_argument("invalid matrix-memory dimensions")
        if self.dim > kernels.MAX_DIM:
            raise unsupported(f"a memory of {self.dim} rows a head exceeds {kernels.MAX_DIM}, the most the kernel takes")
        self.qk_width, self.v_width = self.heads * self.dim, self.heads * self.vdim
        self.width = 2 * self.qk_width + 2 * self.v_width + 2 * self.heads      # [q | k | v | g | i | f]
        self.names = {key: spec.param(key + "_name", default) for key, default in NAMES.items()}
        self.projection: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.norm = None

    def parameter_specs(self) -> List[ParamSpec]:
        n, hidden = self.names, self.hidden
        return [
            ParamSpec("qkvgif", (self.width, hidden), sources=(
                (n["q"], (self.qk_width, hidden)), (n["k"], (self.qk_width, hidden)), (n["v"], (self.v_width, hidden)),
                (n["g"], (self.v_width, hidden)), (n["i"], (self.heads, hidden)), (n["f"], (self.heads, hidden)))),
            ParamSpec("if.bias", (2 * self.heads,), init=("normal", 1.0), sources=(
                (n["i_bias"], (self.heads,)), (n["f_bias"], (self.heads,)))),
            ParamSpec(n["norm"], (self.v_width,), init=("one_plus_normal", 0.1)),
            ParamSpec(n["o"], (hidden, self.v_width)),
        ]

    def bind(self, tensors) -> None:
        n = self.names
        fused = tensors["qkvgif"]
        rows = fused.shape[0] + (-fused.shape[0] % 8)      # rows of the product's result start on 16-byte boundaries
        if rows != fused.shape[0]:
            pad = torch.zeros((rows - fused.shape[0], self.hidden), dtype=fused.dtype, device=fused.device)
            fused = torch.cat([fused, pad], dim=0).contiguous()
        bias = torch.zeros(rows, dtype=torch.float32, device=fused.device)
        bias[self.width - 2 * self.heads:self.width] = tensors["if.bias"].float()
        self.projection, self.out = Linear(fused, bias), Linear(tensors[n["o"]])
        self.norm = tensors[n["norm"]].float().contiguous()

    def cache_requests(self) -> list:
        return [StateRequest((self.heads, self.dim, self.vdim + 1), torch.float32),
                StateRequest((self.heads,), torch.float32)]

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        if not owns_cache:
            raise invalid_argument("a matrix-memory layer keeps a state of its own")
        plan = ctx.plan
        projected = self.projection.forward(plain_rows(x))
        qk, v = self.qk_width, self.v_width
        gates = 2 * qk + 2 * v
        coef = kernels.matrix_memory_gates(projected, gates, gates + self.heads, self.cap, views[1], heads=self.heads,
                                           tables=ctx.tables, seqs=plan.n_seqs)
        read = kernels.scalar_recurrence(projected[:, qk:2 * qk], projected[:, :qk], projected[:, 2 * qk:2 * qk + v],
                                         coef, views[0], heads=self.heads, k_heads=self.heads, q_heads=self.heads,
                                         dim=self.dim, vdim=self.vdim, extra=1, q_scale=float(self.dim) ** -0.5,
                                         tables=ctx.tables, seqs=plan.n_seqs)
        gated = kernels.matrix_memory_finish(read, coef, self.norm, projected[:, 2 * qk + v:2 * qk + 2 * v],
                                             heads=self.heads, vdim=self.vdim, eps=self.eps)
        return self.out.forward(gated)
