"""Attention whose keys and values are linear maps of a cached latent, as a mixer.

A token leaves one row in the cache: its latent c = RMSNorm(first `kv_rank` rows of W_dkv h) and, from the last
`rot_dim` rows of W_dkv h, one rotated key part that all heads share. Queries pass a latent of their own,
c_q = RMSNorm(W_dq h), q = W_uq c_q, laid out per head as [dim plain | rot_dim rotated]. Head i's plain key is
W_uk[i] c, its value W_uv[i] c; a score is (q_plain . k_plain + q_rot . k_rot) * scale, the softmax is causal
(key u is visible from position p when u <= p and, with a window W, u > p - W), and W_o maps the concatenated
heads back. The rotation pairs entries 2i and 2i+1 of the rotated part (the named position encoding gives the
angles).

Two forms compute the same thing. Folded: the key map is folded into the query (q_lat = W_uk[i]^T q_plain, per
head) and the value map is applied to the weighted sum of latents, so attention reads the cached rows only and
never materialises per-head keys or values: decoding, prompts that continue cached sequences, and everything in
32-bit (bfloat16 with widths in multiples of 16 on the tensor cores, a page of cached rows read once for 16 heads;
else on the general kernel). Unfolded: for bfloat16 prompts that start at position 0 every head's keys and values are computed from
the latents of the step's own rows, packed with the queries into the matrix that this package's tensor-core prompt
attention kernels take (values zero-padded to the key width, W_o's columns padded to match), and attention costs
dim + rot_dim + vdim multiply-adds per score instead of 2 kv_rank + rot_dim.

A layer with `kv_from` set has no W_dkv and reads the cache of the layer that is named as its cache source in
the schedule; its own W_uk, W_uv, queries and mask apply.

Parameters (`spec.params`): hidden_size, num_heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, eps, position
(name of a rotary encoding of head width rot_dim), window (tokens or None), owns_latent (False: no W_dkv), and
the tensor names under the prefix: dq, dq_norm, uq, dkv, dkv_norm, uk, uv, o (and q, gate).

Variants, all parameters: q_rank None: no query latent, q = W_q h with the tensor `q_name`. rotation_layout
"half": entry i of the rotated part is paired with entry i + rotary width / 2 instead of entries 2i and 2i + 1;
since a score is a dot product, which does not change when queries and keys are reordered alike, the rows of W_q
and W_dkv that make the rotated parts are reordered once at load and the kernels rotate neighbours as ever.
head_gate: head i's result is multiplied by sigmoid(W_g h)_i (tensor `gate_name`, [num_heads, hidden]).
ring (default true): a window is kept as a ring of pages (one token a step); false: every page is kept and the
window is a mask, so that prompts and portions of prompts run over a window too. Without a query latent the
projections of h (q, the latent with the shared key part, the gate) are one product.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import KVRequest
from ..errors import invalid_argument, unsupported
from ..kernels import attention as attention_kernels
from ..kernels import latent as latent_kernels
from ..kernels import ops
from .base import Part, plain_rows
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec

NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
         "o": "o", "q": "q", "gate": "g"}


def neighbour_order(width: int, rotary: int) -> torch.Tensor:
    """The order of a rotated part's entries in which the pairs (i, i + rotary/2) of its first `rotary` entries
    become neighbours (2i, 2i + 1): new[2i] = old[i], new[2i + 1] = old[i + rotary/2]; the rest stay."""
    half = rotary // 2
    order = torch.arange(width)
    order[0:rotary:2] = torch.arange(half)
    order[1:rotary:2] = torch.arange(half) + half
    return order


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.heads = int(spec.param("num_heads"))
        self.dim = int(spec.param("dim"))
        self.rot_dim = int(spec.param("rot_dim"))
        self.vdim = int(spec.param("vdim"))
        q_rank = spec.param("q_rank")
        self.q_rank = int(q_rank) if q_rank is not None else None
        self.rank = int(spec.param("kv_rank"))
        self.layout = spec.param("rotation_layout", "interleaved")
        self.has_gate = bool(spec.param("head_gate", False))
        self.ring = bool(spec.param("ring", True))
        if self.layout not in ("interleaved", "half"):
            raise invalid_argument("a rotation pairs neighbours ('interleaved') or halves ('half')")
        self.scale = float(spec.param("scale"))
        self.eps = float(spec.param("eps"))
        self.window = spec.param("window", None)
        self.owns_latent = bool(spec.param("owns_latent", True))
        if min(self.hidden, self.heads, self.vdim, self.q_rank if self.q_rank is not None else 1, self.rank,
               self.rot_dim) <= 0 or self.dim < 0:
            raise invalid_argument("invalid latent attention dimensions")
        if self.rank + self.rot_dim > 640:
            raise unsupported(f"a cached row of {self.rank + self.rot_dim} values exceeds 640, the widest the kernels take")
        if self.window is not None and int(self.window) <= 0:
            raise invalid_argument("an attention window must be positive")
        name = spec.param("position", None)
        self.position = env.positions[name] if name is not None else None
        if self.position is None:
            raise invalid_argument("the rotated key part needs a position encoding")
        if self.position.head_dim != self.rot_dim:
            raise invalid_argument("the rotary encoding was built for another width of the rotated part")
        self.names = {key: spec.param(key + "_name", default) for key, default in NAMES.items()}
        if self.q_rank is None and not self.owns_latent:
            raise unsupported("a layer without a query latent makes its own key/value latent")
        self.dq = self.uq = self.dkv = self.out = self.fused = None
        self.dq_norm = self.dkv_norm = self.uk_folded = self.uv = None

    def parameter_specs(self) -> List[ParamSpec]:
        n, head_q = self.names, self.dim + self.rot_dim
        specs = [
            ParamSpec(n["uk"], (self.heads * self.dim, self.rank), init=("normal", 0.1)),
            ParamSpec(n["uv"], (self.heads * self.vdim, self.rank), init=("normal", 0.1)),
            ParamSpec(n["o"], (self.hidden, self.heads * self.vdim)),
        ]
        if self.q_rank is not None:
            specs += [ParamSpec(n["dq"], (self.q_rank, self.hidden)),
                      ParamSpec(n["dq_norm"], (self.q_rank,), init=("one_plus_normal", 0.1)),
                      ParamSpec(n["uq"], (self.heads * head_q, self.q_rank), init=("normal", 0.1))]
        else:
            specs.append(ParamSpec(n["q"], (self.heads * head_q, self.hidden)))
        if self.owns_latent:
            specs.append(ParamSpec(n["dkv"], (self.rank + self.rot_dim, self.hidden)))
            specs.append(ParamSpec(n["dkv_norm"], (self.rank,), init=("one_plus_normal", 0.1)))
        if self.has_gate:
            specs.append(ParamSpec(n["gate"], (self.heads, self.hidden)))
        return specs

    def bind(self, tensors) -> None:
        n, head_q = self.names, self.dim + self.rot_dim
        q_map = tensors[n["uq"] if self.q_rank is not None else n["q"]]
        dkv = tensors[n["dkv"]] if self.owns_latent else None
        if self.layout == "half":
            # Queries' and keys' rotated parts reordered alike (see the module's text): pairs become neighbours.
            order = neighbour_order(self.rot_dim, self.position.rotary_dim).to(q_map.device)
            rows = (torch.arange(self.heads, device=q_map.device)[:, None] * head_q
                    + torch.cat([torch.arange(self.dim, device=q_map.device), self.dim + order])[None, :]).reshape(-1)
            q_map = q_map[rows].contiguous()
            if dkv is not None:
                dkv = torch.cat([dkv[:self.rank], dkv[self.rank:][order]], dim=0).contiguous()
        self.out = Linear(tensors[n["o"]])
        if self.q_rank is not None:
            self.dq, self.uq = Linear(tensors[n["dq"]]), Linear(q_map)
            self.dq_norm = tensors[n["dq_norm"]].float().contiguous()
            if self.owns_latent:
                self.dkv = Linear(dkv)
            self.gate = Linear(tensors[n["gate"]]) if self.has_gate else None
        else:
            # One product for everything that reads h: [q | latent and shared key part | gate], each piece starting
            # on a multiple of eight rows (zero rows between), so that the pieces of a result row are 16-byte aligned.
            pieces, self.offsets, at = [], {}, 0
            for name, matrix in (("q", q_map), ("kv", dkv), ("gate", tensors[n["gate"]] if self.has_gate else None)):
                if matrix is None:
                    continue
                self.offsets[name] = (at, matrix.shape[0])
                pieces.append(matrix)
                at += matrix.shape[0]
                if at % 8:
                    pieces.append(torch.zeros((8 - at % 8, self.hidden), dtype=matrix.dtype, device=matrix.device))
                    at += 8 - at % 8
            self.fused = Linear(torch.cat(pieces, dim=0).contiguous())
        # W_uk per head, transposed: [heads, rank, dim], so that q_lat = q_plain @ W_uk[h] is a product with a
        # weight stored [out, in] like every other.
        self.uk_folded = tensors[n["uk"]].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors[n["uv"]].view(self.heads, self.vdim, self.rank).contiguous()
        if self.owns_latent:
            self.dkv_norm = tensors[n["dkv_norm"]].float().contiguous()
        self._uk, self._uv, self._o = tensors[n["uk"]], tensors[n["uv"]], tensors[n["o"]]
        self._unfold = None      # (Linear of [W_uk; W_uv], Linear of W_o with padded columns), made at first use

    def _projections(self, x):
        """(q, kv or None, gate logits or None) of the rows x: views of one product's result where there is no
        query latent."""
        if self.fused is not None:
            both = self.fused.forward(x)
            piece = lambda name: both[:, self.offsets[name][0]:self.offsets[name][0] + self.offsets[name][1]] \
                if name in self.offsets else None
            return piece("q"), piece("kv"), piece("gate")
        q = self.uq.forward(ops.rms_rows(self.dq.forward(x), self.q_rank, self.dq_norm, self.eps))
        return q, (self.dkv.forward(x) if self.owns_latent else None), \
            (self.gate.forward(x) if self.gate is not None else None)

    def _unfolded_maps(self):
        if self._unfold is None:
            width = self.dim + self.rot_dim
            out = self._o
            if self.vdim < width:     # the attention kernel's result has `width` values a head, the last ones zero
                out = torch.zeros((self.hidden, self.heads, width), dtype=out.dtype, device=out.device)
                out[:, :, :self.vdim] = self._o.view(self.hidden, self.heads, self.vdim)
                out = out.view(self.hidden, self.heads * width)
            self._unfold = (Linear(torch.cat([self._uk, self._uv], dim=0).contiguous()), Linear(out))
        return self._unfold

    def _unfolds(self, x, ctx, view) -> bool:
        """Whether this step takes the unfolded form: bfloat16 prompts that all start at position 0, with head
        widths the tensor-core prompt kernels take."""
        plan, width = ctx.plan, self.dim + self.rot_dim
        return (x.dtype == torch.bfloat16 and not plan.is_decode and int(plan.seq_start.max()) == 0
                and self.vdim <= width
                and attention_kernels.fast_fits(x.dtype, self.heads, self.heads, width, False)
                and (view is None or view.page_size == 64))

    def cache_requests(self) -> list:
        # One row [c | rotated key part] per token and no values of their own: the values are maps of c.
        window = int(self.window) if self.window is not None and self.ring else None
        return [KVRequest(1, self.rank + self.rot_dim, window, value_dim=0)]

    def launch_signature(self, rows: int, longest: int) -> tuple:
        """What a captured decode step freezes: into how many shares the tensor-core kernel cuts a sequence's
        pages (the general kernel, which the 32-bit engine runs, has no such choice)."""
        if (self.window is not None and self.ring) or not latent_kernels.tensor_core_fits(
                self.env.dtype, self.rank, self.rot_dim, self.window, None):
            return ()
        return (latent_kernels.decode_splits(rows, self.heads, longest, self.env.device, self.window),)

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        x = plain_rows(x)
        view = views[0]
        if owns_cache != self.owns_latent:
            raise invalid_argument("a latent attention layer either owns its latent and its cache, or neither")
        if view.ring_pages > 0 and not ctx.plan.is_decode:
            raise unsupported("latent attention over a windowed (ring) cache takes one token per step")
        rows = x.shape[0]
        heads, rank, rot_dim = self.heads, self.rank, self.rot_dim
        q, kv, gate = self._projections(x)
        if self._unfolds(x, ctx, view):
            return self._forward_unfolded(q, kv, gate, ctx, view)
        folded = torch.empty((rows, heads * (rank + rot_dim)), dtype=q.dtype, device=q.device)
        position = self.position
        latent_kernels.prepare(q, folded, kv, self.dkv_norm, heads=heads, dim=self.dim, rot_dim=rot_dim, rank=rank,
                               rotary_dims=position.rotary_dim,
                               cos=position.cos, sin=position.sin, eps=self.eps, tables=ctx.tables, kv_view=view)
        if self.dim:
            ops.gemm_heads(q.view(rows, heads, self.dim + rot_dim)[:, :, :self.dim], self.uk_folded,
                           folded.view(rows, heads, rank + rot_dim)[:, :, :rank])
        else:
            folded.view(rows, heads, rank + rot_dim)[:, :, :rank].zero_()
        summed = torch.empty((rows, heads * rank), dtype=q.dtype, device=q.device)
        if latent_kernels.tensor_core_fits(q.dtype, rank, rot_dim, self.window, view):
            latent_kernels.attention_tensor_core(ctx, folded, summed, heads=heads, rank=rank, rot_dim=rot_dim,
                                                 scale=self.scale, kv_view=view, window=self.window)
        else:
            latent_kernels.attention(folded, summed, heads=heads, rank=rank, rot_dim=rot_dim, scale=self.scale,
                                     window=self.window, tables=ctx.tables, kv_view=view)
        attended = torch.empty((rows, heads * self.vdim), dtype=q.dtype, device=q.device)
        ops.gemm_heads(summed.view(rows, heads, rank), self.uv, attended.view(rows, heads, self.vdim))
        if gate is not None:
            ops.head_gate(attended, gate, heads, self.vdim)
        return self.out.forward(attended)

    def _forward_unfolded(self, q, kv, gate, ctx, view) -> torch.Tensor:
        rows, heads, width = q.shape[0], self.heads, self.dim + self.rot_dim
        position = self.position
        rotation = dict(rotary_dims=position.rotary_dim, cos=position.cos, sin=position.sin)
        if self.owns_latent:
            latent_kernels.prepare(q, None, kv, self.dkv_norm, heads=heads, dim=self.dim, rot_dim=self.rot_dim,
                                   rank=self.rank, eps=self.eps, tables=ctx.tables, kv_view=view, write_back=True,
                                   **rotation)
        else:
            kv = latent_kernels.gather(view, rows, self.rank + self.rot_dim, ctx.tables)
        unfold, out = self._unfolded_maps()
        unfolded = unfold.forward(kv[:, :self.rank])
        packed = latent_kernels.pack(q, kv, unfolded, heads=heads, dim=self.dim, rot_dim=self.rot_dim, rank=self.rank,
                                     vdim=self.vdim, tables=ctx.tables, **rotation)
        attended = torch.empty((rows, heads * width), dtype=q.dtype, device=q.device)
        attention_kernels.run(ctx, packed, attended, heads=heads, kv_heads=heads, head_dim=width, scale=self.scale,
                              window=self.window, kv_view=None, keys_in_step=True, gate=gate)
        return out.forward(attended)
