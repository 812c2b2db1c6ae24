"""Python faces of the CUDA kernels.

Each function checks shapes, element types and contiguity on the host, hands raw
device pointers and the current stream to the compiled launcher, and raises if the
launcher refuses the arguments or the launch fails. There is no CPU path: a tensor
that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument, runtime_error, unsupported

F32, BF16, NONE = 0, 1, -1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

c_void_p, c_int, c_float, c_longlong, c_ulonglong = (
    ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong)


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise unsupported(f"the kernels take float32 and bfloat16, not {dtype}") from None


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(tensor.data_ptr() if tensor is not None else 0)


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise runtime_error("the kernels run on a CUDA device only (there is no CPU path)")


launch_count = 0  # kernels of this package launched (or captured into a graph) so far
_launch_log: Optional[list] = None


class record_launches:
    """Collects, while it is open, the name of every kernel this package launches and of every
    product handed to the vendor library (`library_mm`), in order: `with record_launches() as
    names: ...`. Names carry the form a launcher chose, e.g. `attention_decode[ring]`, so that a
    test can assert which branch of a dispatch ran."""

    def __enter__(self) -> list:
        global _launch_log
        self._outer, _launch_log = _launch_log, []
        return _launch_log

    def __exit__(self, *exc) -> None:
        global _launch_log
        inner, _launch_log = _launch_log, self._outer
        if self._outer is not None:
            self._outer.extend(inner)


def note(what: str) -> None:
    """Records work that is not one of this package's kernels (a vendor-library product), after it was queued."""
    if _launch_log is not None:
        _launch_log.append(what)
    if _timed is not None:
        _timed.mark(what)


_timed = None


class time_launches:
    """Times the kernels of the launches made while it is open, one by one, on the device: a CUDA event is recorded
    behind every launch, and a launch's time is the span since the event before it. So that the spans hold no idle
    time of a device waiting for the host, the stream is first kept busy for `head_start_ms` (a spin kernel of the
    tensor library) while the host queues the launches behind it. `with time_launches() as timed: ...` then
    `timed.spans()` -> [(name, microseconds)] in launch order (it synchronises)."""

    def __init__(self, head_start_ms: float = 20.0):
        self.head_start_ms = head_start_ms
        self.names, self.events = [], []

    def mark(self, what: str) -> None:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        self.names.append(what)
        self.events.append(event)

    def __enter__(self) -> "time_launches":
        global _timed
        self._outer, _timed = _timed, self
        torch.cuda.synchronize()
        if self.head_start_ms > 0:
            torch.cuda._sleep(int(self.head_start_ms * 1.5e6))     # cycles; the clock is between 1 and 2 GHz
        self.mark("(start)")
        return self

    def __exit__(self, *exc) -> None:
        global _timed
        _timed = self._outer

    def spans(self) -> list:
        torch.cuda.synchronize()
        return [(name, 1e3 * before.elapsed_time(after))
                for name, before, after in zip(self.names[1:], self.events[:-1], self.events[1:])]


def _check(status: int, what: str, launches: int = 1) -> None:
    global launch_count
    if status == 0:
        launch_count += launches
        if _launch_log is not None:
            _launch_log.append(what)
        if _timed is not None:
            _timed.mark(what)
        return
    if status == -2:
        raise unsupported(f"{what}: this combination of element types is not compiled")
    if status == -3:
        raise unsupported(f"{what}: a size lies outside what the kernel takes")
    if status < 0:
        raise unsupported(f"{what}: refused ({status})")
    raise runtime_error(f"{what}: CUDA error {status} at launch")


_core = None


def core():
    """The core kernel library, compiled at the first call."""
    global _core
    if _core is None:
        lib = load_library("core")
        lib.kidi_embedding.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
        lib.kidi_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                         c_int, c_int, c_float, c_int, c_void_p]
        lib.kidi_silu_gate.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.kidi_gemm_simt.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                       c_longlong, c_longlong, c_longlong, c_void_p, c_void_p]
        lib.kidi_add_bias.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_longlong, c_void_p]
        lib.kidi_apply_row_factors.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_float, c_void_p,
                                               c_int, c_int, c_void_p]
        lib.kidi_rope_store.argtypes = [c_void_p, c_int, c_int, c_void_p]
        lib.kidi_attention_generic.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_argmax.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
        lib.kidi_sample.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_ulonglong, c_void_p, c_void_p,
                                    c_void_p, c_void_p]
        lib.kidi_argmax_slices.argtypes = [c_int]
        lib.kidi_argmax_slices.restype = c_int
        lib.kidi_advance_decode.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_void_p]
        lib.kidi_add_layernorm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                           c_int, c_int, c_float, c_int, c_void_p, c_float, c_void_p]
        lib.kidi_head_gate.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p]
        lib.kidi_gelu.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p]
        lib.kidi_add_vector.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.kidi_scale.argtypes = [c_void_p, c_longlong, c_float, c_void_p]
        for name in ("kidi_head_gate", "kidi_gelu", "kidi_add_vector", "kidi_scale"):
            getattr(lib, name).restype = c_int
        lib.kidi_rms_rows.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_int, c_int, c_int,
                                      c_float, c_void_p]
        lib.kidi_poly_norm.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p]
        lib.kidi_token_gate.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_longlong, c_int, c_void_p, c_int,
                                        c_int, c_int, c_void_p]
        lib.kidi_add_normed_mix.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p,
                                            c_longlong, c_void_p, c_int, c_void_p, c_void_p]
        lib.kidi_add_cast.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p]
        lib.kidi_gemm_simt_batched.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                               c_longlong, c_longlong, c_longlong, c_int, c_longlong, c_longlong,
                                               c_longlong, c_void_p]
        lib.kidi_gemm_rows_batched.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                                               c_longlong, c_longlong, c_int, c_longlong, c_longlong, c_longlong,
                                               c_void_p]
        lib.kidi_gemm_rows_batched.restype = c_int
        lib.kidi_add_table_rows.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
        lib.kidi_bounded_gate.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p]
        lib.kidi_tanh_cap.argtypes = [c_void_p, c_longlong, c_float, c_void_p]
        for name in ("kidi_add_table_rows", "kidi_bounded_gate", "kidi_tanh_cap"):
            getattr(lib, name).restype = c_int
        lib.kidi_lanes_rmsnorm.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                           c_void_p, c_int, c_int, c_float, c_void_p]
        lib.kidi_lanes_mix.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p,
                                       c_int, c_longlong, c_void_p]
        lib.kidi_lanes_mix_rmsnorm.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
                                               c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                               c_int, c_int, c_float, c_void_p]
        lib.kidi_lanes_mix_rmsnorm.restype = c_int
        lib.kidi_normed_pair_sum.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p,
                                             c_int, c_int, c_int, c_float, c_void_p]
        lib.kidi_sigmoid_gate.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_void_p]
        lib.kidi_relu_squared.argtypes = [c_void_p, c_void_p, c_int, c_longlong, c_void_p]
        for name in ("kidi_lanes_rmsnorm", "kidi_lanes_mix", "kidi_normed_pair_sum", "kidi_sigmoid_gate",
                     "kidi_relu_squared"):
            getattr(lib, name).restype = c_int
        for name in ("kidi_add_layernorm", "kidi_rms_rows", "kidi_poly_norm", "kidi_token_gate", "kidi_add_normed_mix",
                     "kidi_add_cast", "kidi_gemm_simt_batched"):
            getattr(lib, name).restype = c_int
        for name in ("kidi_embedding", "kidi_add_rmsnorm", "kidi_silu_gate", "kidi_gemm_simt", "kidi_add_bias",
                     "kidi_apply_row_factors", "kidi_rope_store",
                     "kidi_attention_generic", "kidi_argmax", "kidi_sample", "kidi_advance_decode"):
            getattr(lib, name).restype = c_int
        _core = lib
    return _core


# ----------------------------------------------------------------- structures
class CacheGeometry(ctypes.Structure):
    _fields_ = [("table", c_void_p), ("pages_per_seq", c_int), ("page_shift", c_int), ("ring_pages", c_int),
                ("kv_heads", c_int), ("head_dim", c_int)]


class RopeStoreArgs(ctypes.Structure):
    _fields_ = [("qkv", c_void_p), ("ld", c_longlong), ("q_norm", c_void_p), ("k_norm", c_void_p),
                ("cos_table", c_void_p), ("sin_table", c_void_p), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("seq_start", c_void_p), ("seq_len", c_void_p), ("k_cache", c_void_p),
                ("v_cache", c_void_p), ("cache", CacheGeometry), ("rows", c_int), ("heads", c_int),
                ("kv_heads", c_int), ("head_dim", c_int), ("rotary_dim", c_int), ("eps", c_float), ("transform", c_int),
                ("value_dim", c_int), ("q_scale", c_void_p)]


class AttentionArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("ldq", c_longlong), ("k_step", c_void_p), ("v_step", c_void_p),
                ("ldkv", c_longlong), ("k_cache", c_void_p), ("v_cache", c_void_p), ("cache", CacheGeometry),
                ("out", c_void_p), ("ldo", c_longlong), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("seq_start", c_void_p), ("seq_row0", c_void_p), ("rows", c_int),
                ("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("window", c_int), ("scale", c_float),
                ("softcap", c_float), ("slopes", c_void_p), ("value_dim", c_int), ("sinks", c_void_p),
                ("gate", c_void_p), ("ldg", c_longlong)]


def cache_geometry(view, kv_heads: int, head_dim: int) -> CacheGeometry:
    """The geometry of a `KVView` (or an empty one when there is no cache)."""
    if view is None:
        return CacheGeometry(0, 0, 0, 0, kv_heads, head_dim)
    page_size = view.page_size
    return CacheGeometry(view.table.data_ptr(), view.table.shape[1], page_size.bit_length() - 1, view.ring_pages,
                         kv_heads, head_dim)


# -------------------------------------------------------------------- kernels
def embedding(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r, :] = table[tokens[r], :] * scale, in float32 (the residual stream)."""
    _need_cuda(tokens, table)
    if tokens.dtype != torch.int32 or tokens.dim() != 1 or not tokens.is_contiguous():
        raise invalid_argument("embedding takes a contiguous int32 vector of token ids")
    if table.dim() != 2 or not table.is_contiguous():
        raise invalid_argument("the embedding table must be a contiguous matrix")
    rows, (vocab, hidden) = tokens.shape[0], table.shape
    if out is None:
        out = torch.empty((rows, hidden), dtype=torch.float32, device=table.device)
    _check(core().kidi_embedding(_ptr(out), _ptr(table), dtype_code(table.dtype), _ptr(tokens), rows, hidden, vocab,
                                 float(scale), _stream()), "embedding")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """residual += delta (in place, float32), then y = rmsnorm(residual) * weight.
    With `row_index`, row r of the output is computed from row row_index[r] and the
    residual is left as it is."""
    _need_cuda(residual, delta, weight, row_index)
    if residual.dtype != torch.float32 or residual.dim() != 2 or not residual.is_contiguous():
        raise invalid_argument("the residual stream is a contiguous float32 matrix")
    rows_in, hidden = residual.shape
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise invalid_argument("the residual delta must match the residual stream")
    if weight.shape != (hidden,) or not weight.is_contiguous():
        raise invalid_argument(f"the norm weight must have {hidden} elements")
    if row_index is not None:
        if row_index.dtype != torch.int32 or row_index.dim() != 1:
            raise invalid_argument("row_index must be an int32 vector")
        rows = row_index.shape[0]
    else:
        rows = rows_in
    if out is None:
        out = torch.empty((rows, hidden), dtype=out_dtype, device=residual.device)
    _check(core().kidi_add_rmsnorm(
        _ptr(residual), _ptr(delta), dtype_code(delta.dtype) if delta is not None else NONE, _ptr(weight),
        dtype_code(weight.dtype), _ptr(out), dtype_code(out.dtype), _ptr(row_index), rows, hidden, float(eps),
        0 if row_index is not None else 1, _stream()), "add_rmsnorm")
    return out


def _float_vector(vector: Optional[torch.Tensor], size: int, what: str) -> None:
    if vector is not None and (vector.dtype != torch.float32 or vector.shape != (size,) or not vector.is_contiguous()):
        raise invalid_argument(f"{what} must be a contiguous float32 vector of {size} elements")


def add_layernorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: Optional[torch.Tensor],
                  bias: Optional[torch.Tensor], eps: float, out_dtype: Optional[torch.dtype],
                  row_index: Optional[torch.Tensor] = None, delta_weight: Optional[torch.Tensor] = None,
                  delta_eps: float = 0.0) -> Optional[torch.Tensor]:
    """residual += delta (in place, float32), then y = (v - mean) / sqrt(var + eps) * weight + bias over each
    row v of the residual. With `row_index`, row r of the output comes from row row_index[r] and the
    residual is left as it is. With `delta_weight` the delta passes a layer norm of its own first (weight
    `delta_weight`, no bias, `delta_eps`) and the normalised rows are what is added. With `out_dtype` None only
    the sum is formed and nothing is returned."""
    _need_cuda(residual, delta, weight, bias, row_index, delta_weight)
    if residual.dtype != torch.float32 or residual.dim() != 2 or not residual.is_contiguous():
        raise invalid_argument("the residual stream is a contiguous float32 matrix")
    hidden = residual.shape[1]
    if delta is not None and (delta.shape != residual.shape or not delta.is_contiguous()):
        raise invalid_argument("the residual delta must match the residual stream")
    _float_vector(weight, hidden, "the norm weight")
    _float_vector(bias, hidden, "the norm bias")
    _float_vector(delta_weight, hidden, "the weight of the delta's norm")
    if out_dtype is not None and weight is None:
        raise invalid_argument("a layer norm needs its weight")
    if row_index is not None and (row_index.dtype != torch.int32 or row_index.dim() != 1):
        raise invalid_argument("row_index must be an int32 vector")
    rows = row_index.shape[0] if row_index is not None else residual.shape[0]
    out = torch.empty((rows, hidden), dtype=out_dtype, device=residual.device) if out_dtype is not None else None
    _check(core().kidi_add_layernorm(
        _ptr(residual), _ptr(delta), dtype_code(delta.dtype) if delta is not None else NONE, _ptr(weight), _ptr(bias),
        _ptr(out), dtype_code(out.dtype) if out is not None else NONE, _ptr(row_index), rows, hidden, float(eps),
        0 if row_index is not None else 1, _ptr(delta_weight), float(delta_eps), _stream()), "add_layernorm")
    return out


def head_gate(x: torch.Tensor, gate: torch.Tensor, heads: int, width: int) -> torch.Tensor:
    """x[r, h, :] *= sigmoid(gate[r, h]) in place, for x [rows, heads * width] and gate logits [rows, heads] (views
    whose last axis is contiguous); sigmoid and product in 32-bit."""
    _need_cuda(x, gate)
    rows = x.shape[0]
    if x.shape != (rows, heads * width) or gate.shape != (rows, heads) or x.stride(1) != 1 or gate.stride(1) != 1 \
            or gate.dtype != x.dtype:
        raise invalid_argument("head_gate takes [rows, heads * width] and [rows, heads] of one type")
    _check(core().kidi_head_gate(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), dtype_code(x.dtype), rows, heads,
                                 width, _stream()), "head_gate")
    return x


def gelu(z: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """0.5 z (1 + erf(z / sqrt 2)) element by element (the arithmetic is 32-bit); `out` may be z itself."""
    _need_cuda(z, out)
    if not z.is_contiguous() or (out is not None and (out.shape != z.shape or out.dtype != z.dtype or not out.is_contiguous())):
        raise invalid_argument("gelu takes a contiguous tensor")
    if out is None:
        out = torch.empty_like(z)
    _check(core().kidi_gelu(_ptr(z), _ptr(out), dtype_code(z.dtype), z.numel(), _stream()), "gelu")
    return out


def scale(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (x float32, contiguous)."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise invalid_argument("scale takes a contiguous float32 tensor")
    _check(core().kidi_scale(_ptr(x), x.numel(), float(factor), _stream()), "scale")
    return x


def add_vector(x: torch.Tensor, vector: torch.Tensor) -> None:
    """x[r, :] += vector for every row of the float32 matrix x, in place."""
    _need_cuda(x, vector)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or vector.shape != (x.shape[1],) \
            or not vector.is_contiguous():
        raise invalid_argument("add_vector takes a contiguous float32 matrix and a vector of its width")
    _check(core().kidi_add_vector(_ptr(x), _ptr(vector), dtype_code(vector.dtype), x.shape[0], x.shape[1], _stream()),
           "add_vector")


def rms_rows(x: torch.Tensor, width: int, weight: Optional[torch.Tensor], eps: float,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Every group of `width` consecutive entries of a row of x (the row holds a whole number of groups)
    divided by its root mean square and multiplied by `weight` (float32 [width], shared by the groups)."""
    _need_cuda(x, weight, out)
    if x.dim() != 2 or x.stride(1) != 1 or width <= 0 or x.shape[1] % width:
        raise invalid_argument("rms_rows takes rows that hold a whole number of groups")
    _float_vector(weight, width, "the norm weight")
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    if out.shape != x.shape or out.dtype != x.dtype or out.stride(1) != 1:
        raise invalid_argument("rms_rows: the output must match the input")
    _check(core().kidi_rms_rows(_ptr(x), x.stride(0), _ptr(out), out.stride(0), dtype_code(x.dtype), _ptr(weight),
                                x.shape[0], x.shape[1] // width, width, float(eps), _stream()), "rms_rows")
    return out


def poly_norm(z: torch.Tensor, coefficients: torch.Tensor, eps: float) -> torch.Tensor:
    """a z/rms(z) + b z^2/rms(z^2) + c z^3/rms(z^3) + e over each row, (a, b, c, e) = coefficients."""
    _need_cuda(z, coefficients)
    if z.dim() != 2 or not z.is_contiguous():
        raise invalid_argument("poly_norm takes a contiguous matrix")
    _float_vector(coefficients, 4, "the PolyNorm coefficients")
    out = torch.empty_like(z)
    _check(core().kidi_poly_norm(_ptr(z), _ptr(out), dtype_code(z.dtype), _ptr(coefficients), z.shape[0], z.shape[1],
                                 float(eps), _stream()), "poly_norm")
    return out


def token_gate(gate: torch.Tensor, table: torch.Tensor, offset: int, tokens: torch.Tensor) -> torch.Tensor:
    """gelu_tanh(gate[r, c]) * table[tokens[r], offset + c]."""
    _need_cuda(gate, table, tokens)
    rows, dim = gate.shape
    if not gate.is_contiguous() or table.dim() != 2 or table.stride(1) != 1 or offset < 0 or offset + dim > table.shape[1]:
        raise invalid_argument("token_gate: the gate must be contiguous and the table hold the asked columns")
    if tokens.dtype != torch.int32 or tokens.shape[0] < rows:
        raise invalid_argument("token_gate takes int32 token ids, one per row")
    out = torch.empty_like(gate)
    _check(core().kidi_token_gate(_ptr(gate), _ptr(out), dtype_code(gate.dtype), _ptr(table), dtype_code(table.dtype),
                                  table.stride(0), int(offset), _ptr(tokens), table.shape[0], rows, dim, _stream()),
           "token_gate")
    return out


def add_normed_mix(x: torch.Tensor, y: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                   kept: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                   mixed: Optional[torch.Tensor] = None) -> None:
    """x += y / rms(y) * weight (x float32 in place; y optional), then, if `mixed` is given,
    mixed = sum_j mix[j] * kept[j] over the first len(mix) matrices of `kept` [n, rows, hidden] (float32; x is
    usually one of them)."""
    _need_cuda(x, y, weight, kept, mix, mixed)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise invalid_argument("the residual stream is a contiguous float32 matrix")
    rows, hidden = x.shape
    if y is not None:
        if y.shape != x.shape or not y.is_contiguous():
            raise invalid_argument("add_normed_mix: y must match the stream")
        _float_vector(weight, hidden, "the norm weight")
    count = 0
    if mixed is not None:
        count = mix.shape[0]
        if (kept.dtype != torch.float32 or kept.dim() != 3 or kept.shape[1:] != x.shape or not kept.is_contiguous()
                or kept.shape[0] < count or mix.dtype != torch.float32 or not mix.is_contiguous()
                or mixed.dtype != torch.float32 or mixed.shape != x.shape or not mixed.is_contiguous()):
            raise invalid_argument("add_normed_mix: kept streams, weights and result must be float32 and fit the stream")
    _check(core().kidi_add_normed_mix(_ptr(x), _ptr(y), dtype_code(y.dtype) if y is not None else NONE, _ptr(weight),
                                      rows, hidden, float(eps), _ptr(kept), rows * hidden, _ptr(mix), count,
                                      _ptr(mixed), _stream()), "add_normed_mix")


def add_cast(x: torch.Tensor, delta: Optional[torch.Tensor], copy_dtype: Optional[torch.dtype]) -> Optional[torch.Tensor]:
    """x += delta (float32, in place) and a copy of x in `copy_dtype` (None: no copy)."""
    _need_cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous() or (delta is not None and (delta.shape != x.shape or not delta.is_contiguous())):
        raise invalid_argument("add_cast takes a contiguous float32 matrix and a delta of its shape")
    copy = torch.empty(x.shape, dtype=copy_dtype, device=x.device) if copy_dtype is not None else None
    _check(core().kidi_add_cast(_ptr(x), _ptr(delta), dtype_code(delta.dtype) if delta is not None else NONE,
                                _ptr(copy), dtype_code(copy_dtype) if copy_dtype is not None else NONE, x.numel(),
                                _stream()), "add_cast")
    return copy


def gemm_heads(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """A product per head: out[r, h, :] = x[r, h, :] @ weight[h].T for x [rows, heads, K], weight [heads, N, K]
    and out [rows, heads, N] (views whose last axis is contiguous), each output one ascending-k chain of 32-bit
    multiply-adds."""
    _need_cuda(x, weight, out)
    if x.dim() != 3 or weight.dim() != 3 or out.dim() != 3 or x.stride(2) != 1 or out.stride(2) != 1 or not weight.is_contiguous():
        raise invalid_argument("gemm_heads takes [rows, heads, K], [heads, N, K] and [rows, heads, N]")
    rows, heads, K = x.shape
    N = weight.shape[1]
    if weight.shape != (heads, N, K) or out.shape != (rows, heads, N):
        raise invalid_argument("gemm_heads: the shapes do not fit")
    if rows <= 8 and x.dtype == torch.bfloat16 and weight.dtype == x.dtype and out.dtype == x.dtype:
        # few rows of the bfloat16 engine (decoding): a warp an output feature, the weights read once
        _check(core().kidi_gemm_rows_batched(_ptr(x), _ptr(weight), _ptr(out), dtype_code(x.dtype), rows, N, K,
                                             x.stride(0), K, out.stride(0), heads, x.stride(1), N * K, out.stride(1),
                                             _stream()), "gemm_heads[rows]")
        return out
    _check(core().kidi_gemm_simt_batched(_ptr(x), dtype_code(x.dtype), _ptr(weight), dtype_code(weight.dtype), _ptr(out),
                                         dtype_code(out.dtype), rows, N, K, x.stride(0), K, out.stride(0), heads,
                                         x.stride(1), N * K, out.stride(1), _stream()), "gemm_heads")
    return out


def silu_gate(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise invalid_argument("silu_gate takes a contiguous [rows, 2*I] matrix")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(core().kidi_silu_gate(_ptr(gate_up), _ptr(out), dtype_code(gate_up.dtype), rows, inter, _stream()),
           "silu_gate")
    return out


def bounded_gate(gate_up: torch.Tensor, limit: float, alpha: float, up_shift: float) -> torch.Tensor:
    """g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + up_shift) for
    gate_up [rows, 2*I] (gate columns first)."""
    _need_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise invalid_argument("bounded_gate takes a contiguous [rows, 2*I] matrix")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _check(core().kidi_bounded_gate(_ptr(gate_up), _ptr(out), dtype_code(gate_up.dtype), rows, inter, float(limit),
                                    float(alpha), float(up_shift), _stream()), "bounded_gate")
    return out


def add_table_rows(x: torch.Tensor, table: torch.Tensor, index: torch.Tensor, scale: float = 1.0) -> None:
    """x[r] += table[index[r]] * scale (x float32, in place); rows whose index lies outside the table stay."""
    _need_cuda(x, table, index)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise invalid_argument("the residual stream is a contiguous float32 matrix")
    if table.dim() != 2 or table.shape[1] != x.shape[1] or not table.is_contiguous():
        raise invalid_argument("add_table_rows: the table's rows must be as wide as the stream's")
    if index.dtype != torch.int32 or index.dim() != 1 or index.shape[0] < x.shape[0]:
        raise invalid_argument("add_table_rows takes an int32 index per row")
    _check(core().kidi_add_table_rows(_ptr(x), _ptr(table), dtype_code(table.dtype), _ptr(index), x.shape[0], x.shape[1],
                                      table.shape[0], float(scale), _stream()), "add_table_rows")


def lanes_rmsnorm(lanes: torch.Tensor, read: Optional[torch.Tensor], weight: Optional[torch.Tensor], eps: float,
                  out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u = sum_s read[s] * lanes[s] (`read` None: the plain sum), y = u / sqrt(mean(u^2) + eps) * weight (`weight`
    None: y = u). `lanes` is float32 [count, rows, hidden], each lane contiguous (an expanded view of one matrix
    will do). With `row_index`, row r of the output comes from row row_index[r]."""
    _need_cuda(lanes, read, weight, row_index)
    if lanes.dtype != torch.float32 or lanes.dim() != 3 or lanes.stride(2) != 1 or lanes.stride(1) != lanes.shape[2]:
        raise invalid_argument("lanes_rmsnorm takes float32 lanes [count, rows, hidden] with contiguous matrices")
    count, rows_in, hidden = lanes.shape
    _float_vector(read, count, "the lanes' read weights")
    if weight is not None and (weight.shape != (hidden,) or not weight.is_contiguous()):
        raise invalid_argument(f"the norm weight must have {hidden} elements")
    if row_index is not None and (row_index.dtype != torch.int32 or row_index.dim() != 1):
        raise invalid_argument("row_index must be an int32 vector")
    rows = row_index.shape[0] if row_index is not None else rows_in
    out = torch.empty((rows, hidden), dtype=out_dtype, device=lanes.device)
    _check(core().kidi_lanes_rmsnorm(_ptr(lanes), lanes.stride(0), count, _ptr(read), _ptr(weight),
                                     dtype_code(weight.dtype) if weight is not None else NONE, _ptr(out),
                                     dtype_code(out_dtype), _ptr(row_index), rows, hidden, float(eps), _stream()),
           "lanes_rmsnorm")
    return out


def lanes_mix(source: torch.Tensor, target: torch.Tensor, mix: torch.Tensor, write: torch.Tensor,
              y: torch.Tensor) -> torch.Tensor:
    """target[t] = sum_s mix[s, t] * source[s] + write[t] * y for float32 lanes [count, rows, hidden]; `source` may
    be `target` itself, or an expanded view of one matrix. mix float32 [count, count] ([from, to]), write float32
    [count], y [rows, hidden] of any element type."""
    _need_cuda(source, target, mix, write, y)
    count = target.shape[0]
    for lanes in (source, target):
        if lanes.dtype != torch.float32 or lanes.dim() != 3 or lanes.shape != target.shape or lanes.stride(2) != 1 \
                or lanes.stride(1) != lanes.shape[2]:
            raise invalid_argument("lanes_mix takes float32 lanes [count, rows, hidden] with contiguous matrices")
    if mix.dtype != torch.float32 or mix.shape != (count, count) or not mix.is_contiguous():
        raise invalid_argument("lanes_mix: the mixing matrix is float32 [count, count]")
    _float_vector(write, count, "the lanes' write weights")
    if y.shape != target.shape[1:] or not y.is_contiguous():
        raise invalid_argument("lanes_mix: y must be a contiguous matrix of a lane's shape")
    _check(core().kidi_lanes_mix(_ptr(source), source.stride(0), _ptr(target), target.stride(0), count, _ptr(mix),
                                 _ptr(write), _ptr(y), dtype_code(y.dtype), y.numel(), _stream()), "lanes_mix")
    return target


def lanes_mix_rmsnorm(source: torch.Tensor, target: torch.Tensor, mix: torch.Tensor, write: torch.Tensor,
                      y: torch.Tensor, read: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                      out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`lanes_mix` and then `lanes_rmsnorm` of the new lanes, in one kernel where the width allows (else in two): the
    lanes are updated (target[t] = sum_s mix[s, t] source[s] + write[t] y) and read at once as sum_t read[t]
    target[t], normalised. With `row_index` only those rows are produced and no lane is written (the update is then
    lost: for the last reader of a stream)."""
    _need_cuda(source, target, mix, write, y, read, weight, row_index)
    count, rows_in, hidden = target.shape
    rows = row_index.shape[0] if row_index is not None else rows_in
    fits = (hidden % 4 == 0 and weight is not None and source.dim() == 3 and source.shape == target.shape
            and all(lanes.dtype == torch.float32 and lanes.stride(2) == 1 and lanes.stride(1) == hidden
                    for lanes in (source, target)) and y.shape == (rows_in, hidden) and y.is_contiguous())
    if fits:
        _float_vector(read, count, "the lanes' read weights")
        _float_vector(write, count, "the lanes' write weights")
        if mix.dtype != torch.float32 or mix.shape != (count, count) or not mix.is_contiguous():
            raise invalid_argument("lanes_mix: the mixing matrix is float32 [count, count]")
        if weight.shape != (hidden,) or not weight.is_contiguous():
            raise invalid_argument(f"the norm weight must have {hidden} elements")
        out = torch.empty((rows, hidden), dtype=out_dtype, device=target.device)
        status = core().kidi_lanes_mix_rmsnorm(
            _ptr(source), source.stride(0), _ptr(target), target.stride(0), count, _ptr(mix), _ptr(write), _ptr(y),
            dtype_code(y.dtype), _ptr(read), _ptr(weight), dtype_code(weight.dtype), _ptr(out), dtype_code(out_dtype),
            _ptr(row_index), rows, hidden, float(eps), _stream())
        if status != -3:
            _check(status, "lanes_mix_rmsnorm")
            return out
    if row_index is not None:      # the stream stays as it is: the new lanes of the picked rows go to scratch memory
        picked = row_index.long()
        source, y = source[:, picked].contiguous(), y[picked].contiguous()
        target = torch.empty_like(source)
        row_index = None
    lanes_mix(source, target, mix, write, y)
    return lanes_rmsnorm(target, read, weight, eps, out_dtype, row_index=row_index)


def normed_pair_sum(a: torch.Tensor, b: torch.Tensor, weight_a: torch.Tensor, weight_b: torch.Tensor, eps: float,
                    share_a: float = 0.5, share_b: float = 0.5, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """share_a * a / rms(a) * weight_a + share_b * b / rms(b) * weight_b over each row (32-bit arithmetic)."""
    _need_cuda(a, b, weight_a, weight_b)
    if a.dim() != 2 or a.shape != b.shape or a.dtype != b.dtype or not a.is_contiguous() or not b.is_contiguous():
        raise invalid_argument("normed_pair_sum takes two contiguous matrices of one shape and type")
    rows, hidden = a.shape
    _float_vector(weight_a, hidden, "the first norm weight")
    _float_vector(weight_b, hidden, "the second norm weight")
    out = torch.empty((rows, hidden), dtype=out_dtype, device=a.device)
    _check(core().kidi_normed_pair_sum(_ptr(a), _ptr(b), dtype_code(a.dtype), _ptr(weight_a), _ptr(weight_b),
                                       float(share_a), float(share_b), _ptr(out), dtype_code(out_dtype), rows, hidden,
                                       float(eps), _stream()), "normed_pair_sum")
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x *= sigmoid(gate) element by element, in place; x and gate [rows, width] of one type (views whose last axis
    is contiguous); sigmoid and product in 32-bit."""
    _need_cuda(x, gate)
    if x.dim() != 2 or x.shape != gate.shape or x.dtype != gate.dtype or x.stride(1) != 1 or gate.stride(1) != 1:
        raise invalid_argument("sigmoid_gate takes two [rows, width] matrices of one type")
    _check(core().kidi_sigmoid_gate(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0), dtype_code(x.dtype), x.shape[0],
                                    x.shape[1], _stream()), "sigmoid_gate")
    return x


def relu_squared(z: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """max(z, 0)^2 element by element; `out` may be z itself."""
    _need_cuda(z, out)
    if not z.is_contiguous() or (out is not None and (out.shape != z.shape or out.dtype != z.dtype or not out.is_contiguous())):
        raise invalid_argument("relu_squared takes a contiguous tensor")
    if out is None:
        out = torch.empty_like(z)
    _check(core().kidi_relu_squared(_ptr(z), _ptr(out), dtype_code(z.dtype), z.numel(), _stream()), "relu_squared")
    return out


def tanh_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap), float32, in place."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous() or not cap > 0:
        raise invalid_argument("tanh_cap takes a contiguous float32 tensor and a positive bound")
    _check(core().kidi_tanh_cap(_ptr(x), x.numel(), float(cap), _stream()), "tanh_cap")
    return x


def check_bias(bias: Optional[torch.Tensor], features: int) -> None:
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (features,) or not bias.is_contiguous()):
        raise invalid_argument(f"a bias is a contiguous float32 vector of {features} elements")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[r, :] += bias, in place (after a product the vendor library computed)."""
    _need_cuda(y, bias)
    if y.dim() != 2 or y.stride(1) != 1:
        raise invalid_argument("add_bias takes a matrix with contiguous rows")
    check_bias(bias, y.shape[1])
    _check(core().kidi_add_bias(_ptr(y), dtype_code(y.dtype), _ptr(bias), y.shape[0], y.shape[1], y.stride(0),
                                _stream()), "add_bias")
    return y


def apply_row_factors(values: torch.Tensor, parts: torch.Tensor, width: int, eps: float) -> torch.Tensor:
    """values[r, :] / sqrt(sum(parts[r, :]) / width + eps) as a new bfloat16 matrix: rows that were stored
    without their norm's factor, made plain."""
    _need_cuda(values, parts)
    if values.dtype != torch.bfloat16 or values.dim() != 2 or values.stride(1) != 1:
        raise invalid_argument("apply_row_factors takes a bfloat16 matrix with contiguous rows")
    if parts.dtype != torch.float32 or parts.dim() != 2 or parts.shape[0] != values.shape[0] or parts.stride(1) != 1:
        raise invalid_argument("apply_row_factors takes float32 parts, one row of them per row of values")
    out = torch.empty(values.shape, dtype=torch.bfloat16, device=values.device)
    _check(core().kidi_apply_row_factors(_ptr(values), values.stride(0), _ptr(parts), parts.shape[1], parts.stride(0),
                                         int(width), float(eps), _ptr(out), values.shape[0], values.shape[1],
                                         _stream()), "apply_row_factors")
    return out


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
              out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ weight.T (+ bias) with 32-bit fused multiply-adds in ascending k."""
    _need_cuda(x, weight, bias)
    check_bias(bias, weight.shape[0])
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise invalid_argument(f"gemm: x {tuple(x.shape)} does not fit weight {tuple(weight.shape)}")
    if x.stride(1) != 1 or weight.stride(1) != 1:
        raise invalid_argument("gemm: rows must be contiguous")
    M, K = x.shape
    N = weight.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _check(core().kidi_gemm_simt(_ptr(x), dtype_code(x.dtype), _ptr(weight), dtype_code(weight.dtype), _ptr(out),
                                 dtype_code(out.dtype), M, N, K, x.stride(0), weight.stride(0), out.stride(0),
                                 _ptr(bias), _stream()), "gemm_simt")
    return out


def rope_store(qkv: torch.Tensor, *, heads: int, kv_heads: int, head_dim: int, q_norm: Optional[torch.Tensor],
               k_norm: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               rotary_dim: int, tables, kv_view, store: bool, transform: bool = True,
               value_dim: Optional[int] = None, q_scale: Optional[torch.Tensor] = None) -> None:
    """In place on qkv [rows, (heads + kv_heads) * head_dim + kv_heads * value_dim (+ columns that are left
    alone)]: per-head RMSNorm and rotation of the q and k heads; k and v heads are also written to the cache when
    `store` is set. With `transform=False` nothing is normalised or rotated: the k and v
    heads are only copied to the cache. `tables` is the step's `DeviceTables`. `value_dim` (default head_dim) is
    the width of a v head. `q_scale` (float32 [positions]): a q head at position p is multiplied by q_scale[p] after
    its norm and rotation. With `kv_heads` 0 the rows hold q heads only (a layer that reads another layer's keys
    and values) and nothing is stored."""
    _need_cuda(qkv)
    rows = qkv.shape[0]
    value_dim = head_dim if value_dim is None else int(value_dim)
    if qkv.dim() != 2 or qkv.stride(1) != 1 or qkv.shape[1] < (heads + kv_heads) * head_dim + kv_heads * value_dim:
        raise invalid_argument("rope_store: qkv has the wrong shape")
    if (q_norm is None) != (k_norm is None):
        raise invalid_argument("rope_store: q_norm and k_norm come together")
    norm_dtype = q_norm.dtype if q_norm is not None else torch.float32
    if q_norm is not None and (q_norm.shape != (head_dim,) or k_norm.shape != (head_dim,) or k_norm.dtype != norm_dtype):
        raise invalid_argument("rope_store: the head norms must have head_dim elements and one type")
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape):
        raise invalid_argument("rope_store: the rotation tables must be float32 [positions, rotary_dim/2]")
    if q_scale is not None and (q_scale.dtype != torch.float32 or q_scale.dim() != 1 or not q_scale.is_contiguous()):
        raise invalid_argument("rope_store: the query scale is a float32 vector with an entry per position")
    view = kv_view if store and kv_heads > 0 else None
    if view is not None and view.keys.dtype != qkv.dtype:
        raise invalid_argument("rope_store: the cache and the activations differ in element type")
    args = RopeStoreArgs(
        qkv.data_ptr(), qkv.stride(0), _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin),
        tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(),
        tables.seq_start.data_ptr(), tables.seq_len.data_ptr(),
        view.keys.data_ptr() if view is not None else 0, view.values.data_ptr() if view is not None else 0,
        cache_geometry(view, kv_heads, head_dim), rows, heads, kv_heads, head_dim, rotary_dim, float(eps),
        1 if transform else 0, value_dim, _ptr(q_scale))
    _check(core().kidi_rope_store(ctypes.byref(args), dtype_code(qkv.dtype), dtype_code(norm_dtype), _stream()),
           "rope_store")


def attention_generic(qkv: torch.Tensor, out: torch.Tensor, *, heads: int, kv_heads: int, head_dim: int,
                      scale: float, window: Optional[int], tables, kv_view, keys_in_step: bool,
                      softcap: float = 0.0, slopes: Optional[torch.Tensor] = None, value_dim: Optional[int] = None,
                      sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> None:
    """Causal attention of every row of the step over its sequence's keys. Keys of the
    step's own rows are read from `qkv` when `keys_in_step` is set, earlier ones (or
    all of them) from the cache. `softcap` > 0 bounds a score s to softcap * tanh(s / softcap);
    `slopes` (float32 [heads]) adds slopes[h] * (key position - query position) to head h's scores.
    `value_dim` (default head_dim): the width of a value head and of a head of `out`. `sinks` (float32
    [heads]): exp(sinks[h]) joins head h's softmax denominator. `gate` ([rows, heads], a view of the step's
    element type): head h of a row is multiplied by sigmoid(gate[row, h])."""
    value_dim = head_dim if value_dim is None else int(value_dim)
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.shape != (heads,) or not sinks.is_contiguous()
                              or sinks.device != qkv.device):
        raise invalid_argument("attention: the sinks must be a float32 vector with one entry per head")
    if gate is not None and (gate.shape != (qkv.shape[0], heads) or gate.dtype != qkv.dtype or gate.stride(1) != 1):
        raise invalid_argument("attention: the gate has one entry per row and head, in the rows' element type")
    if slopes is not None and (slopes.dtype != torch.float32 or slopes.shape != (heads,) or not slopes.is_contiguous()
                               or slopes.device != qkv.device):
        raise invalid_argument("attention: the score slopes must be a float32 vector with one entry per head")
    _need_cuda(qkv, out)
    rows = qkv.shape[0]
    if out.shape != (rows, heads * value_dim) or out.dtype != qkv.dtype or out.stride(1) != 1:
        raise invalid_argument("attention: the output has the wrong shape or type")
    if kv_view is None and not keys_in_step:
        raise invalid_argument("attention: there is neither a cache nor keys in the step")
    item = qkv.element_size()
    k_step = qkv.data_ptr() + heads * head_dim * item if keys_in_step else 0
    v_step = qkv.data_ptr() + (heads + kv_heads) * head_dim * item if keys_in_step else 0
    args = AttentionArgs(
        qkv.data_ptr(), qkv.stride(0), k_step, v_step, qkv.stride(0),
        kv_view.keys.data_ptr() if kv_view is not None else 0, kv_view.values.data_ptr() if kv_view is not None else 0,
        cache_geometry(kv_view, kv_heads, head_dim), out.data_ptr(), out.stride(0),
        tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(),
        tables.seq_start.data_ptr(), tables.seq_row0.data_ptr(), rows, heads, kv_heads, head_dim,
        int(window or 0), float(scale), float(softcap or 0.0), slopes.data_ptr() if slopes is not None else 0,
        value_dim, _ptr(sinks), _ptr(gate), gate.stride(0) if gate is not None else 0)
    _check(core().kidi_attention_generic(ctypes.byref(args), dtype_code(qkv.dtype), _stream()), "attention")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need_cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise invalid_argument("argmax takes a contiguous float32 [rows, vocab] matrix")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    scratch, launches = _argmax_scratch(rows, vocab, logits.device)
    _check(core().kidi_argmax(_ptr(logits), _ptr(out), rows, vocab, _ptr(scratch), _stream()), "argmax", launches)
    return out


def _argmax_scratch(rows: int, vocab: int, device):
    """Scratch for the two-stage argmax of a wide vocabulary (None when one stage does)."""
    slices = core().kidi_argmax_slices(vocab)
    if slices == 1:
        return None, 1
    return torch.empty(2 * rows * slices, dtype=torch.float32, device=device), 2


def sample(logits: torch.Tensor, temperature: torch.Tensor, seed: int, keys: torch.Tensor, steps: torch.Tensor,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row: argmax where temperature is 0, else a draw from
    softmax(logits / temperature) keyed by (seed, keys[r], steps[r])."""
    _need_cuda(logits, temperature, keys, steps)
    if logits.dtype != torch.float32 or logits.dim() != 2 or not logits.is_contiguous():
        raise invalid_argument("sample takes a contiguous float32 [rows, vocab] matrix")
    rows, vocab = logits.shape
    if (temperature.dtype != torch.float32 or keys.dtype != torch.int64 or steps.dtype != torch.int32
            or temperature.shape != (rows,) or keys.shape != (rows,) or steps.shape != (rows,)):
        raise invalid_argument("sample: temperature float32, keys int64 and steps int32, one per row")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    scratch, launches = _argmax_scratch(rows, vocab, logits.device)
    _check(core().kidi_sample(_ptr(logits), _ptr(out), rows, vocab, _ptr(temperature),
                              ctypes.c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _ptr(keys), _ptr(steps), _ptr(scratch),
                              _stream()), "sample", launches + 1)
    return out


def advance_decode(tokens: torch.Tensor, selected: torch.Tensor, row_seq: torch.Tensor, row_pos: torch.Tensor,
                   seq_start: torch.Tensor, steps: torch.Tensor, vocab: int) -> None:
    """After a decode step: every live row takes its selected token as its next input
    and moves one position on (tokens, positions and step counters change in place)."""
    _need_cuda(tokens, selected, row_seq, row_pos, seq_start, steps)
    rows = tokens.shape[0]
    for tensor in (tokens, selected, row_seq, row_pos, seq_start, steps):
        if tensor.dtype != torch.int32 or tensor.shape[0] < rows:
            raise invalid_argument("advance_decode takes int32 vectors of one length")
    _check(core().kidi_advance_decode(_ptr(tokens), _ptr(selected), _ptr(row_seq), _ptr(row_pos), _ptr(seq_start),
                                      _ptr(steps), rows, vocab, _stream()), "advance_decode")
