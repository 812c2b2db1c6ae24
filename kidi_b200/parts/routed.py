"""A feed-forward of many small gated experts, of which each token uses a few.

    z = W_router h                       router logits, 32-bit
    s = sigmoid(z)                       scores; the `top` experts with the largest scores are taken
    w = s of the chosen experts          (divided by their sum when `renormalise` is set)
    y = sum over the chosen experts of expert_e(w_e h)           `weight_on` = "input"
      or sum of w_e expert_e(h)                                   `weight_on` = "output"
    expert(x) = W_down (silu(W_gate x) * (W_up x))

Parameters (`spec.params`): hidden_size, expert_size, experts, top, score ("sigmoid"), renormalise (false),
weight_on ("input"), router_name ("router"), expert_name ("e{index}."), gate_name, up_name, down_name. A file
holds each expert's three matrices under `<prefix><expert_name><gate|up|down>`; they are bound as two stacked
tensors, [experts, 2 * expert_size, hidden] (gate rows, then up rows) and [experts, hidden, expert_size].

Variants, all parameters: score "softmax" (s = softmax(z) over all experts); renormalise_eps (added to the sum
that the chosen scores are divided by); groups and keep_groups: the experts form `groups` equal runs of
neighbours, a group's score is its largest, and only experts of the `keep_groups` best groups can be chosen;
expert_form "plain": an expert has no gate, expert(x) = W_down gelu(W_up x) with the exact (erf) gelu, and the
first stacked tensor is [experts, expert_size, hidden]; shared_size and shared_name ("shared."): one more expert
of the same form and that width, under `<prefix><shared_name><gate|up|down>`, that every token passes and whose
result is added with weight 1.

Steps of few rows, steps inside a captured decode graph, and every step of the 32-bit engine read the
chosen experts' weights through the choice on the device (no host round trip). Prompts of the bfloat16
engine sort the (row, choice) pairs by expert on the host and gather the rows; every expert's rows, up to twice
the mean count, are then padded to one count and run through two batched products of the vendor library, and
what an expert has beyond that (or everything, where the widths are no multiples of 8) through the ordinary
products, with one activation kernel for all of them.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..errors import invalid_argument, unsupported
from ..kernels import ops, routed, skinny
from .base import Part, plain_rows
from .linear import Linear
from .registry import register_part
from .spec import ParamSpec

# Up to this many (row, choice) pairs a step reads the experts through the choice; above, a bfloat16 prompt
# sorts them by expert.
SLOT_PATH_MAX = 128


@register_part("feed_forward", "routed_experts")
class RoutedExperts(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.inter = int(spec.param("expert_size"))
        self.experts = int(spec.param("experts"))
        self.top = int(spec.param("top"))
        self.renormalise = bool(spec.param("renormalise", False))
        self.weight_on_input = spec.param("weight_on", "input") == "input"
        if spec.param("weight_on", "input") not in ("input", "output"):
            raise invalid_argument("routed experts weigh an expert's input or its output")
        self.score = spec.param("score", "sigmoid")
        if self.score not in ("sigmoid", "softmax"):
            raise unsupported(f"router score '{self.score}' is not built (sigmoid and softmax are)")
        self.renormalise_eps = float(spec.param("renormalise_eps", 0.0))
        self.groups = int(spec.param("groups", 1))
        self.keep_groups = int(spec.param("keep_groups", self.groups))
        self.gated = spec.param("expert_form", "gated") == "gated"
        if spec.param("expert_form", "gated") not in ("gated", "plain"):
            raise invalid_argument("an expert is 'gated' (SiLU gate times up) or 'plain' (gelu of up)")
        shared = spec.param("shared_size", None)
        self.shared_size = int(shared) if shared is not None else None
        self.shared_name = spec.param("shared_name", "shared.")
        if min(self.hidden, self.inter, self.experts, self.top) <= 0 or self.top > self.experts:
            raise invalid_argument("invalid routed feed-forward dimensions")
        if self.experts > 1024 or self.top > 32:
            raise unsupported("the router takes up to 1,024 experts and 32 choices a token")
        if self.groups < 1 or self.experts % self.groups or not 1 <= self.keep_groups <= self.groups \
                or self.keep_groups * (self.experts // self.groups) < self.top:
            raise invalid_argument("the experts split into equal groups, and the kept groups hold at least `top` experts")
        if self.shared_size is not None and self.shared_size <= 0:
            raise invalid_argument("a shared expert has a positive width")
        self.router_name = spec.param("router_name", "router")
        self.expert_name = spec.param("expert_name", "e{index}.")
        self.gate_name, self.up_name, self.down_name = (spec.param(key + "_name", key) for key in ("gate", "up", "down"))
        self.router: Optional[torch.Tensor] = None
        self.gate_up: Optional[torch.Tensor] = None
        self.down: Optional[torch.Tensor] = None

    def parameter_specs(self) -> List[ParamSpec]:
        names = [self.expert_name.format(index=index) for index in range(self.experts)]
        first, down = [], []
        for name in names:
            if self.gated:
                first.append((name + self.gate_name, (self.inter, self.hidden)))
            first.append((name + self.up_name, (self.inter, self.hidden)))
            down.append((name + self.down_name, (self.hidden, self.inter)))
        per = (2 if self.gated else 1) * self.inter
        specs = [ParamSpec(self.router_name, (self.experts, self.hidden)),
                 ParamSpec("experts.gate_up", (self.experts * per, self.hidden), sources=tuple(first)),
                 ParamSpec("experts.down", (self.experts * self.hidden, self.inter), sources=tuple(down))]
        if self.shared_size is not None:
            name = self.shared_name
            if self.gated:
                specs.append(ParamSpec(name + "gate_up", (2 * self.shared_size, self.hidden), sources=(
                    (name + self.gate_name, (self.shared_size, self.hidden)),
                    (name + self.up_name, (self.shared_size, self.hidden)))))
            else:
                specs.append(ParamSpec(name + self.up_name, (self.shared_size, self.hidden)))
            specs.append(ParamSpec(name + self.down_name, (self.hidden, self.shared_size)))
        return specs

    def bind(self, tensors) -> None:
        per = (2 if self.gated else 1) * self.inter
        self.router = tensors[self.router_name]
        self.gate_up = tensors["experts.gate_up"].view(self.experts, per, self.hidden)
        self.down = tensors["experts.down"].view(self.experts, self.hidden, self.inter)
        self._gate_up = [Linear(self.gate_up[index]) for index in range(self.experts)]
        self._down = [Linear(self.down[index]) for index in range(self.experts)]
        self._shared = None
        if self.shared_size is not None:
            name = self.shared_name
            self._shared = (Linear(tensors[name + ("gate_up" if self.gated else self.up_name)]),
                            Linear(tensors[name + self.down_name]))

    def _activate(self, first: torch.Tensor) -> torch.Tensor:
        """The experts' activation on the first product's result (in place where it can be)."""
        return ops.silu_gate(first) if self.gated else ops.gelu(first, out=first)

    def forward(self, x, ctx) -> torch.Tensor:
        x = plain_rows(x)
        shared = None
        if self._shared is not None:
            # The shared expert's result joins the routed sum in the kernel that forms it (a 32-bit sum).
            up, down = self._shared
            if not self.gated and up.bias is None and skinny.fits(x, up.weight):
                mid = skinny.gemm(x, up.weight, x.dtype, activation="gelu")       # few rows: the gelu in the epilogue
            else:
                mid = self._activate(up.forward(x))
            shared = down.forward(mid)
        return self._forward_routed(x, ctx, shared)

    def _forward_routed(self, x, ctx, addend=None) -> torch.Tensor:
        rows = x.shape[0]
        chosen, weight = routed.route(x, self.router, self.top, self.renormalise, self.score, self.groups,
                                      self.keep_groups, self.renormalise_eps)
        slots = rows * self.top
        if x.dtype == torch.float32 or self.gate_up.dtype == torch.float32 or ctx.plan.is_decode \
                or slots <= SLOT_PATH_MAX:
            return routed.expert_slots(x, self.gate_up, self.down, chosen, weight, self.weight_on_input, self.gated, addend)
        # Many rows: (row, choice) pairs in the order of their experts (a stable sort, so a row's place among
        # its expert's rows follows its place in the step), one host round trip for the counts.
        picked = chosen.reshape(-1).cpu().numpy()
        order = np.argsort(picked, kind="stable").astype(np.int32)
        counts = np.bincount(picked, minlength=self.experts)
        # Every expert's first `cap` rows stand in one padded batch [experts, cap] (two batched products of the
        # vendor library for all experts); the rows that an expert has beyond `cap` follow the batch, expert by
        # expert, and run through the ordinary products. `cap` is the largest count, but at most twice the mean, so
        # that the padding stays below the rows themselves however uneven the choice is. Widths that are no
        # multiples of 8 take the ordinary products only (cap 0).
        cap = 0
        if self.hidden % 8 == 0 and self.inter % 8 == 0:
            cap = int(-(-min(int(counts.max()), -(-2 * slots // self.experts)) // 8) * 8)
        begins = np.concatenate([[0], np.cumsum(counts)[:-1]])
        experts_sorted = picked[order]
        within = np.arange(slots) - begins[experts_sorted]
        over = within >= cap
        extra = np.maximum(counts - cap, 0)
        extra_begins = self.experts * cap + np.concatenate([[0], np.cumsum(extra)[:-1]])
        at = np.where(over, extra_begins[experts_sorted] + within - cap, experts_sorted * cap + within).astype(np.int32)
        total = self.experts * cap + int(extra.sum())
        source = np.full(total, -1, dtype=np.int32)
        source[at] = order
        place = np.empty(slots, dtype=np.int32)
        place[order] = at
        tables = torch.from_numpy(np.concatenate([source, place])).to(x.device)
        gathered = routed.gather_slots(x, tables[:total], weight, self.top, self.weight_on_input)
        first = torch.empty((total, self.gate_up.shape[1]), dtype=x.dtype, device=x.device)
        result = torch.empty((total, self.hidden), dtype=x.dtype, device=x.device)
        batch = self.experts * cap
        spans = [(index, int(begin), int(begin + count)) for index, (begin, count) in enumerate(zip(extra_begins, extra))
                 if count]
        if cap:
            torch.bmm(gathered[:batch].view(self.experts, cap, self.hidden), self.gate_up.transpose(1, 2),
                      out=first[:batch].view(self.experts, cap, first.shape[1]))
            ops.note("library_bmm")
        for index, begin, end in spans:
            self._gate_up[index].forward(gathered[begin:end], out=first[begin:end])
        mid = self._activate(first)                  # one activation kernel for the rows of all experts
        if cap:
            torch.bmm(mid[:batch].view(self.experts, cap, self.inter), self.down.transpose(1, 2),
                      out=result[:batch].view(self.experts, cap, self.hidden))
            ops.note("library_bmm")
        for index, begin, end in spans:
            self._down[index].forward(mid[begin:end], out=result[begin:end])
        return routed.combine_slots(result, tables[total:], weight, rows, self.top, self.weight_on_input, addend)
