"""Two mixers side by side as one mixer: both read the same input, each result is divided by its root mean
square over the model width and multiplied by a weight of its own, and the mixer's result is a weighted sum of
the two (half of each by default).

    y = share_left * left(h) / rms(left(h)) * w_left + share_right * right(h) / rms(right(h)) * w_right

The norms and the sum are 32-bit and the result is handed on in 32-bit. Each child keeps what it needs of the
cache; the requests of the left child come first.

Parameters (`spec.params`): hidden_size, eps, left and right (the `PartSpec`s of two mixers), left_norm_name and
right_norm_name (the norm weights' tensor names under this part's prefix), share_left and share_right (default 0.5).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..errors import invalid_argument
from ..kernels import ops
from . import registry as part_registry
from .base import Part, plain_rows
from .registry import register_part
from .spec import ParamSpec


@register_part("mixer", "parallel_mixers")
class ParallelMixers(Part):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.param("hidden_size"))
        self.eps = float(spec.param("eps"))
        self.left = part_registry.build_part("mixer", spec.param("left"), env)
        self.right = part_registry.build_part("mixer", spec.param("right"), env)
        self.left_norm_name = spec.param("left_norm_name", "left.out")
        self.right_norm_name = spec.param("right_norm_name", "right.out")
        self.share_left = float(spec.param("share_left", 0.5))
        self.share_right = float(spec.param("share_right", 0.5))
        if self.hidden <= 0:
            raise invalid_argument("invalid width of parallel mixers")
        self._split = len(self.left.cache_requests())
        self.left_norm = self.right_norm = None

    def children(self):
        return (self.left, self.right)

    def parameter_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.left_norm_name, (self.hidden,), init=("one_plus_normal", 0.1)),
                ParamSpec(self.right_norm_name, (self.hidden,), init=("one_plus_normal", 0.1))]

    def bind(self, tensors) -> None:
        self.left_norm = tensors[self.left_norm_name].float().contiguous()
        self.right_norm = tensors[self.right_norm_name].float().contiguous()

    def cache_requests(self) -> list:
        return list(self.left.cache_requests()) + list(self.right.cache_requests())

    def forward(self, x, ctx, views, owns_cache: bool, sink=None) -> Optional[torch.Tensor]:
        x = plain_rows(x)
        left = self.left.forward(x, ctx, views[:self._split], owns_cache)
        right = self.right.forward(x, ctx, views[self._split:], owns_cache)
        return ops.normed_pair_sum(left, right, self.left_norm, self.right_norm, self.eps, self.share_left,
                                   self.share_right, out_dtype=torch.float32)
