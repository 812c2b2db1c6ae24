"""A matrix memory with exponential gates (the mLSTM of xLSTM) as a mixer.

With h the mixer's input, H heads, d the width of a query or key head and e the width of a value head:

    q = W_q h / sqrt(d),  k = W_k h  [H, d],   v = W_v h  [H, e]
    i = cap tanh((W_i h + b_i) / cap),   f = logsigmoid(cap tanh((W_f h + b_f) / cap))      (log gates, one a head)
    m_t = max(f_t + m_(t-1), i_t)                                                            (m_0 = 0)
    S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Each head's o is divided by its root mean square; the heads are concatenated, multiplied by a weight [H e] and by
sigmoid(W_g h), and projected by W_o. What a sequence keeps, as fixed-size 32-bit state per cache slot: S with n as
one more column, [H, d, e + 1], and m [H]. Gates, the maximum, the state, the read-out and the norm are 32-bit; so are
the results of the two gate projections (a product of their own, 2 H rows): a log gate of up to `gate_cap` rounded to
bfloat16 would be off by up to a sixteenth, which the exponential turns into six per cent of a write strength.

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
        self.width = 2 * self.qk_width + 2 * self.v_width                       # [q | k | v | g]; [i | f] apart
        self.names = {key: spec.param(key + "_name", default) for key, default in NAMES.items()}
        self.projection: Optional[Linear] = None
        self.gate_projection: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.norm = None

    def parameter_specs(self) -> List[ParamSpec]:
        n, hidden = self.names, self.hidden
        return [
            ParamSpec("qkvg", (self.width, hidden), sources=(
                (n["q"], (self.qk_width, hidden)), (n["k"], (self.qk_width, hidden)), (n["v"], (self.v_width, hidden)),
                (n["g"], (self.v_width, hidden)))),
            ParamSpec("if", (2 * self.heads, hidden), sources=((n["i"], (self.heads, hidden)), (n["f"], (self.heads, hidden)))),
            ParamSpec("if.bias", (2 * self.heads,), init=("normal", 1.0), sources=(
                (n["i_bias"], (self.heads,)), (n["f_bias"], (self.heads,)))),
            ParamSpec(n["norm"], (self.v_width,), init=("one_plus_normal", 0.1)),
            ParamSpec(n["o"], (hidden, self.v_width)),
        ]

    def bind(self, tensors) -> None:
        n = self.names
        def padded(matrix):        # rows of a product's result start on 16-byte boundaries
            extra = -matrix.shape[0] % 8
            if not extra:
                return matrix
            pad = torch.zeros((extra, self.hidden), dtype=matrix.dtype, device=matrix.device)
            return torch.cat([matrix, pad], dim=0).contiguous()

        gates = padded(tensors["if"])
        bias = torch.zeros(gates.shape[0], dtype=torch.float32, device=gates.device)
        bias[:2 * self.heads] = tensors["if.bias"].float()
        self.projection, self.gate_projection = Linear(padded(tensors["qkvg"])), Linear(gates, bias)
        self.out = Linear(tensors[n["o"]])
        self.norm = tensors[n["norm"]].float().contiguous()

    def cache_requests(self) -> list:
        return [StateRequest((self.heads, self.dim, self.vdim + 1), torch.float32),
                StateRequest((self.heads,), torch.float32)]

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        if not owns_cache:
            raise invalid_argument("a matrix-memory layer keeps a state of its own")
        plan = ctx.plan
        x = plain_rows(x)
        projected = self.projection.forward(x)
        qk, v = self.qk_width, self.v_width
        gates = self.gate_projection.forward(x, out_dtype=torch.float32)
        coef = kernels.matrix_memory_gates(gates, 0, self.heads, self.cap, views[1], heads=self.heads,
                                           tables=ctx.tables, seqs=plan.n_seqs)
        read = kernels.scalar_recurrence(projected[:, qk:2 * qk], projected[:, :qk], projected[:, 2 * qk:2 * qk + v],
                                         coef, views[0], heads=self.heads, k_heads=self.heads, q_heads=self.heads,
                                         dim=self.dim, vdim=self.vdim, extra=1, q_scale=float(self.dim) ** -0.5,
                                         tables=ctx.tables, seqs=plan.n_seqs)
        gated = kernels.matrix_memory_finish(read, coef, self.norm, projected[:, 2 * qk + v:2 * qk + 2 * v],
                                             heads=self.heads, vdim=self.vdim, eps=self.eps)
        return self.out.forward(gated)
