"""Python face of the routed-experts kernels (csrc/routed.cu), compiled when a model with such a
feed-forward first runs."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument
from . import ops
from .ops import _check, c_float, c_int, c_void_p, dtype_code

_library = None


def library():
    global _library
    if _library is None:
        lib = load_library("routed")
        lib.kidi_route.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_int, c_int, c_float, c_void_p]
        lib.kidi_expert_slots.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
        lib.kidi_gather_slots.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_void_p]
        lib.kidi_combine_slots.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                           c_void_p, c_void_p]
        for name in ("kidi_route", "kidi_expert_slots", "kidi_gather_slots", "kidi_combine_slots"):
            getattr(lib, name).restype = c_int
        _library = lib
    return _library


def _check_addend(addend, like: torch.Tensor, rows: int, hidden: int) -> None:
    if addend is not None and (addend.shape != (rows, hidden) or addend.dtype != like.dtype or not addend.is_contiguous()
                               or not addend.is_cuda):
        raise invalid_argument("the addend has the result's shape and type")


def route(x: torch.Tensor, router: torch.Tensor, top: int, renormalise: bool, score: str = "sigmoid", groups: int = 1,
          keep: int = 1, renormalise_eps: float = 0.0):
    """(chosen int32 [rows, top], weight float32 [rows, top]) for rows x [rows, hidden] and a router
    [experts, hidden]: logits in 32-bit, scores (a sigmoid of each logit, or with `score` "softmax" a softmax over
    all experts), the `top` largest (ties: the lower index), their scores as weights (with `renormalise` divided by
    their sum plus `renormalise_eps`). With `groups` > 1 the experts form that many equal runs of neighbours and
    only experts of the `keep` groups with the largest best score can be chosen."""
    ops._need_cuda(x, router)
    if x.dim() != 2 or not x.is_contiguous() or router.dim() != 2 or not router.is_contiguous() \
            or router.shape[1] != x.shape[1]:
        raise invalid_argument("the router takes contiguous rows and a contiguous [experts, hidden] matrix")
    rows, hidden = x.shape
    chosen = torch.empty((rows, top), dtype=torch.int32, device=x.device)
    weight = torch.empty((rows, top), dtype=torch.float32, device=x.device)
    _check(library().kidi_route(x.data_ptr(), dtype_code(x.dtype), router.data_ptr(), dtype_code(router.dtype),
                                chosen.data_ptr(), weight.data_ptr(), rows, hidden, router.shape[0], top,
                                1 if renormalise else 0, 1 if score == "softmax" else 0, int(groups), int(keep),
                                float(renormalise_eps), ops._stream()), "route")
    return chosen, weight


def expert_slots(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, chosen: torch.Tensor,
                 weight: torch.Tensor, weight_on_input: bool, gated: bool = True,
                 addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Every row through its chosen experts, the experts' weights read through the choice: x [rows, hidden],
    gate_up [experts, 2 * inter, hidden] (without a gate: the up rows only, [experts, inter, hidden], and the
    exact gelu as activation), down [experts, hidden, inter] -> [rows, hidden]. `addend` [rows, hidden], if given, is
    added to the result (in 32-bit, before it is rounded)."""
    ops._need_cuda(x, gate_up, down, chosen, weight)
    rows, hidden = x.shape
    experts, first_rows, _ = gate_up.shape
    inter, top = first_rows // (2 if gated else 1), chosen.shape[1]
    if (not x.is_contiguous() or gate_up.shape != (experts, (2 if gated else 1) * inter, hidden) or down.shape != (experts, hidden, inter)
            or not gate_up.is_contiguous() or not down.is_contiguous() or gate_up.dtype != down.dtype):
        raise invalid_argument("expert_slots: the experts' weights do not fit the rows")
    _check_addend(addend, x, rows, hidden)
    mid = torch.empty((rows * top, inter), dtype=x.dtype, device=x.device)
    out = torch.empty((rows, hidden), dtype=x.dtype, device=x.device)
    _check(library().kidi_expert_slots(x.data_ptr(), dtype_code(x.dtype), gate_up.data_ptr(), down.data_ptr(),
                                       dtype_code(gate_up.dtype), chosen.data_ptr(), weight.data_ptr(), mid.data_ptr(),
                                       out.data_ptr(), rows, top, hidden, inter, 1 if weight_on_input else 0,
                                       1 if gated else 0, addend.data_ptr() if addend is not None else 0,
                                       ops._stream()), "expert_slots", 2)
    return out


def gather_slots(x: torch.Tensor, order: torch.Tensor, weight: torch.Tensor, top: int, weight_on_input: bool) -> torch.Tensor:
    """Row i of the result is x[order[i] // top] (times weight[order[i]] when the weight is on the input); zeros
    where order[i] is negative."""
    slots, hidden = order.shape[0], x.shape[1]
    out = torch.empty((slots, hidden), dtype=x.dtype, device=x.device)
    _check(library().kidi_gather_slots(x.data_ptr(), dtype_code(x.dtype), order.data_ptr(), weight.data_ptr(),
                                       out.data_ptr(), slots, top, hidden, 1 if weight_on_input else 0, ops._stream()),
           "gather_slots")
    return out


def combine_slots(y: torch.Tensor, place: torch.Tensor, weight: torch.Tensor, rows: int, top: int,
                  weight_on_input: bool, addend: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = sum over k of y[place[r * top + k]] (times weight[r, k] when the weight is on the output), plus
    addend[r] if given."""
    hidden = y.shape[1]
    _check_addend(addend, y, rows, hidden)
    out = torch.empty((rows, hidden), dtype=y.dtype, device=y.device)
    _check(library().kidi_combine_slots(y.data_ptr(), dtype_code(y.dtype), place.data_ptr(), weight.data_ptr(),
                                        out.data_ptr(), rows, top, hidden, 1 if weight_on_input else 0,
                                        addend.data_ptr() if addend is not None else 0, ops._stream()),
           "combine_slots")
    return out
