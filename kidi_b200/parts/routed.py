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
engine sort the (row, choice) pairs by expert on the host and gather the scaled rows; every expert's rows are
then padded to one count and run through two batched products of the vendor library, or, where one expert has
far more rows than the others or the widths are no multiples of 8, each expert's rows through the ordinary
products.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..errors import invalid_argument, unsupported
from ..kernels import ops, routed
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
            shared = down.forward(self._activate(up.forward(x)))
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
        place = np.empty(slots, dtype=np.int32)
        most = int(-(-int(counts.max()) // 8) * 8)
        if self.hidden % 8 == 0 and self.inter % 8 == 0 and self.experts * most <= 3 * slots:
            # Every expert's rows padded to one count: two batched products of the vendor library and one gate
            # for all experts (taken unless one expert has far more rows than the others).
            begins = np.concatenate([[0], np.cumsum(counts)[:-1]])
            experts_sorted = picked[order]
            at = (experts_sorted * most + (np.arange(slots) - begins[experts_sorted])).astype(np.int32)
            padded = np.full(self.experts * most, -1, dtype=np.int32)
            padded[at] = order
            place[order] = at
            both_tables = torch.from_numpy(np.concatenate([padded, place])).to(x.device)
            gathered = routed.gather_slots(x, both_tables[:padded.size], weight, self.top, self.weight_on_input)
            both = torch.bmm(gathered.view(self.experts, most, self.hidden), self.gate_up.transpose(1, 2))
            ops.note("library_bmm")
            mid = self._activate(both.view(self.experts * most, both.shape[-1]))
            result = torch.bmm(mid.view(self.experts, most, self.inter), self.down.transpose(1, 2))
            ops.note("library_bmm")
            return routed.combine_slots(result.view(self.experts * most, self.hidden), both_tables[padded.size:], weight,
                                        rows, self.top, self.weight_on_input, addend)
        place[order] = np.arange(slots, dtype=np.int32)
        both = torch.from_numpy(np.concatenate([order, place])).to(x.device)
        gathered = routed.gather_slots(x, both[:slots], weight, self.top, self.weight_on_input)
        result = torch.empty((slots, self.hidden), dtype=x.dtype, device=x.device)
        begin = 0
        for index, count in enumerate(counts.tolist()):
            if count:
                mid = self._activate(self._gate_up[index].forward(gathered[begin:begin + count]))
                self._down[index].forward(mid, out=result[begin:begin + count])
                begin += count
        return routed.combine_slots(result, both[slots:], weight, rows, self.top, self.weight_on_input, addend)
