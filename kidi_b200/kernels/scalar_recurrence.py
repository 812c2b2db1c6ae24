"""Python faces of the recurrences with one decay per head and token (csrc/scalar_recurrence.cu), of the
gate and finishing kernels of the two mixers that use them, and of the short causal convolution with carried
inputs. The library is compiled when a model with such a layer first runs."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument
from . import ops
from .ops import _check, _ptr, c_float, c_int, c_longlong, c_void_p, dtype_code

MAX_TAPS = 32
MAX_DIM = 256


class ScalarRecurrenceArgs(ctypes.Structure):
    _fields_ = [("k", c_void_p), ("ldk", c_longlong), ("q", c_void_p), ("ldq", c_longlong), ("v", c_void_p),
                ("ldv", c_longlong), ("coef", c_void_p), ("state", c_void_p), ("out", c_void_p), ("row_seq", c_void_p),
                ("seq_slot", c_void_p), ("seq_row0", c_void_p), ("seq_len", c_void_p), ("seqs", c_int), ("heads", c_int),
                ("k_heads", c_int), ("q_heads", c_int), ("dim", c_int), ("vdim", c_int), ("extra", c_int),
                ("coef_width", c_int), ("q_scale", c_float)]


class ShortConvArgs(ctypes.Structure):
    _fields_ = [("x", c_void_p), ("ldx", c_longlong), ("weight", c_void_p), ("bias", c_void_p), ("state", c_void_p),
                ("out", c_void_p), ("ldo", c_longlong), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("seq_start", c_void_p), ("seq_row0", c_void_p), ("seq_len", c_void_p),
                ("rows", c_int), ("seqs", c_int), ("channels", c_int), ("taps", c_int), ("silu", c_int)]


_library = None


def library():
    global _library
    if _library is None:
        lib = load_library("scalar_recurrence")
        lib.kidi_scalar_recurrence.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_short_conv.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_short_conv_state.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_short_conv_step.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_state_space_gates.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                               c_void_p]
        lib.kidi_state_space_finish.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p,
                                                c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_float,
                                                c_void_p]
        lib.kidi_matrix_memory_gates.argtypes = [c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
                                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
        lib.kidi_matrix_memory_finish.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p,
                                                  c_longlong, c_int, c_int, c_int, c_float, c_void_p]
        for name in ("kidi_scalar_recurrence", "kidi_short_conv", "kidi_short_conv_state", "kidi_short_conv_step",
                     "kidi_state_space_gates", "kidi_state_space_finish", "kidi_matrix_memory_gates",
                     "kidi_matrix_memory_finish"):
            getattr(lib, name).restype = c_int
        _library = lib
    return _library


def _rows_view(x: torch.Tensor, what: str) -> None:
    if x.dim() != 2 or x.stride(1) != 1:
        raise invalid_argument(f"{what}: a matrix whose rows are contiguous is needed")


def _float_tensor(x: torch.Tensor, shape, what: str) -> None:
    if x.dtype != torch.float32 or tuple(x.shape) != tuple(shape) or not x.is_contiguous():
        raise invalid_argument(f"{what} must be a contiguous float32 tensor of shape {tuple(shape)}")


def scalar_recurrence(k: torch.Tensor, q: torch.Tensor, v: torch.Tensor, coef: torch.Tensor, state: torch.Tensor, *,
                      heads: int, k_heads: int, q_heads: int, dim: int, vdim: int, extra: int = 0,
                      q_scale: float = 1.0, tables, seqs: int) -> torch.Tensor:
    """S_t = a_t S_(t-1) + b_t k_t (v_t, 1 if `extra`)^T and o_t = S_t^T (q_scale q_t) for every sequence's rows of
    the step, from and into `state` [slots + 1, heads, dim, vdim + extra] (float32). k [rows, k_heads * dim],
    q [rows, q_heads * dim], v [rows, heads * vdim] are views of the step's element type (head h reads key head
    h // (heads / k_heads), likewise q); coef float32 [rows, heads, >= 2] holds (a_t, b_t). Returns the read-out,
    float32 [rows, heads * (vdim + extra)]."""
    ops._need_cuda(k, q, v, coef, state)
    rows = v.shape[0]
    for tensor, width, what in ((k, k_heads * dim, "keys"), (q, q_heads * dim, "queries"), (v, heads * vdim, "values")):
        _rows_view(tensor, "scalar recurrence")
        if tensor.shape != (rows, width) or tensor.dtype != v.dtype:
            raise invalid_argument(f"scalar recurrence: the {what} have the wrong shape or type")
    if coef.dtype != torch.float32 or coef.dim() != 3 or coef.shape[:2] != (rows, heads) or coef.shape[2] < 2 \
            or not coef.is_contiguous():
        raise invalid_argument("scalar recurrence: the coefficients are float32 [rows, heads, >= 2]")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (heads, dim, vdim + extra) or not state.is_contiguous():
        raise invalid_argument("scalar recurrence: the state is float32 [slots, heads, dim, vdim (+ 1)]")
    if dim > MAX_DIM:
        raise invalid_argument(f"scalar recurrence: the kernel takes up to {MAX_DIM} state rows a head")
    out = torch.empty((rows, heads * (vdim + extra)), dtype=torch.float32, device=v.device)
    args = ScalarRecurrenceArgs(k.data_ptr(), k.stride(0), q.data_ptr(), q.stride(0), v.data_ptr(), v.stride(0),
                                coef.data_ptr(), state.data_ptr(), out.data_ptr(), tables.row_seq.data_ptr(),
                                tables.seq_slot.data_ptr(), tables.seq_row0.data_ptr(), tables.seq_len.data_ptr(),
                                seqs, heads, k_heads, q_heads, dim, vdim, extra, coef.shape[2], float(q_scale))
    _check(library().kidi_scalar_recurrence(ctypes.byref(args), dtype_code(v.dtype), ops._stream()), "scalar_recurrence")
    return out


def short_conv(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: Optional[torch.Tensor], *,
               silu: bool, tables, seqs: int, one_token: bool = False) -> torch.Tensor:
    """A causal convolution over time on every channel of x [rows, channels] (a view of the step's element type):
    y_t = bias + sum_j weight[c, j] x_(t - taps + 1 + j), then SiLU if asked; inputs of earlier steps come from
    `state` [slots + 1, taps - 1, channels] (the step's element type), which then takes the sequence's last
    taps - 1 inputs. weight float32 [channels, taps], bias float32 [channels] or None. `one_token`: every sequence
    of the step brings one token (decoding): result and state in one kernel."""
    ops._need_cuda(x, weight, bias, state)
    _rows_view(x, "short convolution")
    rows, channels = x.shape
    taps = weight.shape[1] if weight.dim() == 2 else 0
    _float_tensor(weight, (channels, taps), "the convolution's weight")
    if bias is not None:
        _float_tensor(bias, (channels,), "the convolution's bias")
    if not 1 <= taps <= MAX_TAPS:
        raise invalid_argument(f"the short convolution takes 1 to {MAX_TAPS} taps")
    if taps > 1 and (state is None or state.dtype != x.dtype or tuple(state.shape[1:]) != (taps - 1, channels)
                     or not state.is_contiguous()):
        raise invalid_argument("short convolution: the state is [slots, taps - 1, channels] of the step's type")
    out = torch.empty((rows, channels), dtype=x.dtype, device=x.device)
    args = ShortConvArgs(x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), _ptr(state if taps > 1 else None),
                         out.data_ptr(), out.stride(0), tables.row_seq.data_ptr(), tables.row_pos.data_ptr(),
                         tables.seq_slot.data_ptr(), tables.seq_start.data_ptr(), tables.seq_row0.data_ptr(),
                         tables.seq_len.data_ptr(), rows, seqs, channels, taps, 1 if silu else 0)
    lib = library()
    if one_token and taps > 1:
        _check(lib.kidi_short_conv_step(ctypes.byref(args), dtype_code(x.dtype), ops._stream()), "short_conv[one token]")
        return out
    _check(lib.kidi_short_conv(ctypes.byref(args), dtype_code(x.dtype), ops._stream()), "short_conv")
    if taps > 1:
        _check(lib.kidi_short_conv_state(ctypes.byref(args), dtype_code(x.dtype), ops._stream()), "short_conv_state")
    return out


def state_space_gates(dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor) -> torch.Tensor:
    """coef[row, head] = (exp(-exp(a_log) * step), step) with step = softplus(dt + dt_bias), float32 [rows, heads, 2]."""
    ops._need_cuda(dt, dt_bias, a_log)
    _rows_view(dt, "state-space gates")
    rows, heads = dt.shape
    _float_tensor(dt_bias, (heads,), "the step bias")
    _float_tensor(a_log, (heads,), "the log decay rate")
    coef = torch.empty((rows, heads, 2), dtype=torch.float32, device=dt.device)
    _check(library().kidi_state_space_gates(dt.data_ptr(), dt.stride(0), dtype_code(dt.dtype), dt_bias.data_ptr(),
                                            a_log.data_ptr(), coef.data_ptr(), rows, heads, ops._stream()),
           "state_space_gates")
    return coef


def state_space_finish(read: torch.Tensor, x: torch.Tensor, z: torch.Tensor, skip: torch.Tensor, weight: torch.Tensor, *,
                       heads: int, vdim: int, parts: int, eps: float) -> torch.Tensor:
    """y = (read + skip[head] * x) * silu(z), each of `parts` equal parts of a row divided by its root mean square,
    times weight. read float32 [rows, heads * vdim]; x, z views of the step's element type; the result has that type."""
    ops._need_cuda(read, x, z, skip, weight)
    rows, inner = x.shape[0], heads * vdim
    _rows_view(x, "state-space finish")
    _rows_view(z, "state-space finish")
    if x.shape != (rows, inner) or z.shape != (rows, inner) or x.dtype != z.dtype:
        raise invalid_argument("state-space finish: x and z have the wrong shape or type")
    _float_tensor(read, (rows, inner), "the read-out")
    _float_tensor(skip, (heads,), "the skip weights")
    _float_tensor(weight, (inner,), "the norm weight")
    if parts <= 0 or inner % parts:
        raise invalid_argument("state-space finish: the row splits into equal parts")
    out = torch.empty((rows, inner), dtype=x.dtype, device=x.device)
    _check(library().kidi_state_space_finish(read.data_ptr(), x.data_ptr(), x.stride(0), z.data_ptr(), z.stride(0),
                                             dtype_code(x.dtype), skip.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                             out.stride(0), rows, heads, vdim, parts, float(eps), ops._stream()),
           "state_space_finish")
    return out


def matrix_memory_gates(projected: torch.Tensor, offset_i: int, offset_f: int, cap: float, maximum: torch.Tensor, *,
                        heads: int, tables, seqs: int) -> torch.Tensor:
    """The log gates i = cap tanh(i~ / cap), f = logsigmoid(cap tanh(f~ / cap)) from columns offset_i + head and
    offset_f + head of `projected`, the running maximum m_t = max(f_t + m_(t-1), i_t) from and into `maximum`
    [slots + 1, heads] (float32), and coef[row, head] = (exp(f + m_(t-1) - m_t), exp(i - m_t), exp(-m_t))."""
    ops._need_cuda(projected, maximum)
    _rows_view(projected, "matrix-memory gates")
    rows = projected.shape[0]
    if max(offset_i, offset_f) + heads > projected.shape[1] or min(offset_i, offset_f) < 0:
        raise invalid_argument("matrix-memory gates: the gate columns lie outside the projection")
    if maximum.dtype != torch.float32 or tuple(maximum.shape[1:]) != (heads,) or not maximum.is_contiguous():
        raise invalid_argument("matrix-memory gates: the running maximum is float32 [slots, heads]")
    coef = torch.empty((rows, heads, 3), dtype=torch.float32, device=projected.device)
    _check(library().kidi_matrix_memory_gates(projected.data_ptr(), projected.stride(0), int(offset_i), int(offset_f),
                                              dtype_code(projected.dtype), float(cap), coef.data_ptr(),
                                              maximum.data_ptr(), tables.row_seq.data_ptr(), tables.seq_slot.data_ptr(),
                                              tables.seq_row0.data_ptr(), tables.seq_len.data_ptr(), seqs, heads,
                                              ops._stream()), "matrix_memory_gates")
    return coef


def matrix_memory_finish(read: torch.Tensor, coef: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, *, heads: int,
                         vdim: int, eps: float) -> torch.Tensor:
    """Per head: o / (max(|n . q|, exp(-m)) + 1e-6) with n . q the head's last column of `read` [rows, heads *
    (vdim + 1)], divided by its root mean square over vdim, times weight [heads * vdim], times sigmoid(gate)."""
    ops._need_cuda(read, coef, weight, gate)
    _rows_view(gate, "matrix-memory finish")
    rows = gate.shape[0]
    _float_tensor(read, (rows, heads * (vdim + 1)), "the read-out")
    _float_tensor(coef, (rows, heads, 3), "the gate coefficients")
    _float_tensor(weight, (heads * vdim,), "the norm weight")
    if gate.shape != (rows, heads * vdim):
        raise invalid_argument("matrix-memory finish: the gate has the wrong shape")
    out = torch.empty((rows, heads * vdim), dtype=gate.dtype, device=gate.device)
    _check(library().kidi_matrix_memory_finish(read.data_ptr(), coef.data_ptr(), weight.data_ptr(), gate.data_ptr(),
                                               gate.stride(0), dtype_code(gate.dtype), out.data_ptr(), out.stride(0),
                                               rows, heads, vdim, float(eps), ops._stream()), "matrix_memory_finish")
    return out
