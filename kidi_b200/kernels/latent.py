"""Python faces of the latent-attention kernels (csrc/latent_attention.cu).

The library is compiled when a model with such a layer first runs. `prepare` normalises the
latent, rotates the shared key part and the queries' rotated parts and writes the cache row;
`attention` is causal softmax attention of every row of a step over its sequence's cached rows.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from ..csrc.build import load_library
from ..errors import invalid_argument
from . import ops
from .ops import CacheGeometry, _check, c_float, c_int, c_longlong, c_void_p, cache_geometry, dtype_code


class PrepareArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("ldq", c_longlong), ("folded", c_void_p), ("ldf", c_longlong), ("kv", c_void_p),
                ("ldkv", c_longlong), ("write_back", c_int), ("skip_queries", c_int), ("kv_norm", c_void_p), ("cos_table", c_void_p), ("sin_table", c_void_p),
                ("row_seq", c_void_p), ("row_pos", c_void_p), ("seq_slot", c_void_p), ("cache", c_void_p),
                ("geometry", CacheGeometry), ("rows", c_int), ("heads", c_int), ("dim", c_int), ("rot_dim", c_int),
                ("rotary_dims", c_int), ("rank", c_int), ("eps", c_float)]


class AttentionArgs(ctypes.Structure):
    _fields_ = [("folded", c_void_p), ("ldf", c_longlong), ("cache", c_void_p), ("geometry", CacheGeometry),
                ("out", c_void_p), ("ldo", c_longlong), ("row_seq", c_void_p), ("row_pos", c_void_p),
                ("seq_slot", c_void_p), ("rows", c_int), ("heads", c_int), ("rank", c_int), ("rot_dim", c_int),
                ("window", c_int), ("scale", c_float)]


_library = None
# KIDI_B200_LATENT_PAGE_BUFFERS: 1 or 2 page buffers in the tensor-core kernel whatever the sizes (default: chosen)
PAGE_BUFFERS = int(os.environ.get("KIDI_B200_LATENT_PAGE_BUFFERS", "0"))


def library():
    global _library
    if _library is None:
        lib = load_library("latent_attention")
        lib.kidi_latent_prepare.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_latent_attention.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_latent_pack.argtypes = [c_void_p, c_int, c_void_p]
        lib.kidi_latent_gather.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int,
                                           c_int, c_int, c_void_p]
        lib.kidi_latent_decode.argtypes = [c_void_p, c_void_p]
        lib.kidi_latent_decode_workspace.argtypes = [c_int, c_int, c_int, c_int]
        lib.kidi_latent_decode_workspace.restype = c_longlong
        for name in ("kidi_latent_prepare", "kidi_latent_attention", "kidi_latent_pack", "kidi_latent_gather",
                     "kidi_latent_decode"):
            getattr(lib, name).restype = c_int
        _library = lib
    return _library


def prepare(q: torch.Tensor, folded: Optional[torch.Tensor], kv: Optional[torch.Tensor], kv_norm: Optional[torch.Tensor], *,
            heads: int, dim: int, rot_dim: int, rank: int, rotary_dims: int, cos: torch.Tensor, sin: torch.Tensor,
            eps: float, tables, kv_view, write_back: bool = False) -> None:
    """Without `folded` only the cache entries are made; with `write_back` the normalised latent and the rotated
    key part also replace the rows of kv. q [rows, heads * (dim + rot_dim)]: the rotated part of every head is turned by its row's position and
    written to folded[:, head, rank:] (folded [rows, heads * (rank + rot_dim)]). kv [rows, rank + rot_dim], if
    given: its first `rank` entries, RMS-normalised with `kv_norm`, and its rotated last rot_dim entries become
    the row's cache entry."""
    ops._need_cuda(q, folded, kv, kv_norm, cos, sin)
    rows = q.shape[0]
    if q.shape != (rows, heads * (dim + rot_dim)) or q.stride(1) != 1:
        raise invalid_argument("latent prepare: the queries have the wrong shape")
    if folded is not None and (folded.shape != (rows, heads * (rank + rot_dim)) or folded.stride(1) != 1
                               or folded.dtype != q.dtype):
        raise invalid_argument("latent prepare: the folded queries have the wrong shape")
    if cos.dtype != torch.float32 or cos.dim() != 2 or cos.shape[1] != rotary_dims // 2 or sin.shape != cos.shape:
        raise invalid_argument("latent prepare: the rotation tables must be float32 [positions, rotary_dims/2]")
    if kv is not None:
        if kv.shape != (rows, rank + rot_dim) or kv.stride(1) != 1 or kv.dtype != q.dtype:
            raise invalid_argument("latent prepare: the latent rows have the wrong shape")
        if kv_norm is None or kv_norm.dtype != torch.float32 or kv_norm.shape != (rank,) or not kv_norm.is_contiguous():
            raise invalid_argument("latent prepare: the latent's norm weight is a float32 vector of `rank` entries")
        if kv_view is None or kv_view.keys.dtype != q.dtype or kv_view.keys.shape[-1] != rank + rot_dim:
            raise invalid_argument("latent prepare: the cache does not fit the latent rows")
    args = PrepareArgs(
        q.data_ptr(), q.stride(0), folded.data_ptr() if folded is not None else 0,
        folded.stride(0) if folded is not None else 0, kv.data_ptr() if kv is not None else 0,
        kv.stride(0) if kv is not None else 0, 1 if write_back else 0, 1 if folded is None else 0, kv_norm.data_ptr() if kv is not None else 0, cos.data_ptr(),
        sin.data_ptr(), tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(),
        kv_view.keys.data_ptr() if kv is not None else 0, cache_geometry(kv_view if kv is not None else None, 1,
                                                                         rank + rot_dim),
        rows, heads, dim, rot_dim, rotary_dims, rank, float(eps))
    _check(library().kidi_latent_prepare(ctypes.byref(args), dtype_code(q.dtype), ops._stream()), "latent_prepare")


def attention(folded: torch.Tensor, out: torch.Tensor, *, heads: int, rank: int, rot_dim: int, scale: float,
              window: Optional[int], tables, kv_view) -> None:
    """out[r, head, :rank] = sum_u softmax_u((folded[r, head] . entry_u) * scale) entry_u[:rank] over the cached
    entries u of the row's sequence with u <= the row's position (and u > position - window)."""
    ops._need_cuda(folded, out)
    rows = folded.shape[0]
    if folded.shape != (rows, heads * (rank + rot_dim)) or out.shape != (rows, heads * rank) or out.dtype != folded.dtype \
            or folded.stride(1) != 1 or out.stride(1) != 1:
        raise invalid_argument("latent attention: folded queries or output have the wrong shape")
    if kv_view.keys.dtype != folded.dtype or kv_view.keys.shape[-1] != rank + rot_dim:
        raise invalid_argument("latent attention: the cache does not fit the queries")
    args = AttentionArgs(folded.data_ptr(), folded.stride(0), kv_view.keys.data_ptr(),
                         cache_geometry(kv_view, 1, rank + rot_dim), out.data_ptr(), out.stride(0),
                         tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), tables.seq_slot.data_ptr(), rows, heads,
                         rank, rot_dim, int(window or 0), float(scale))
    _check(library().kidi_latent_attention(ctypes.byref(args), dtype_code(folded.dtype), ops._stream()),
           "latent_attention")


class PackArgs(ctypes.Structure):
    _fields_ = [("q", c_void_p), ("ldq", c_longlong), ("latent", c_void_p), ("ldl", c_longlong), ("unfolded", c_void_p),
                ("ldu", c_longlong), ("packed", c_void_p), ("ldp", c_longlong), ("cos_table", c_void_p),
                ("sin_table", c_void_p), ("row_seq", c_void_p), ("row_pos", c_void_p), ("rows", c_int), ("heads", c_int),
                ("dim", c_int), ("rot_dim", c_int), ("rotary_dims", c_int), ("rank", c_int), ("vdim", c_int)]


def pack(q: torch.Tensor, latent: torch.Tensor, unfolded: torch.Tensor, *, heads: int, dim: int, rot_dim: int,
         rank: int, vdim: int, rotary_dims: int, cos: torch.Tensor, sin: torch.Tensor, tables) -> torch.Tensor:
    """The matrix [rows, 3 * heads * (dim + rot_dim)] of queries (rotated here), keys and zero-padded values that
    the prompt attention kernels take, from q [rows, heads * (dim + rot_dim)], the rows' cache entries `latent`
    [rows, rank + rot_dim] and `unfolded` [rows, heads * dim + heads * vdim] (plain keys, then values)."""
    ops._need_cuda(q, latent, unfolded, cos, sin)
    rows, width = q.shape[0], dim + rot_dim
    if q.shape != (rows, heads * width) or latent.shape != (rows, rank + rot_dim) \
            or unfolded.shape != (rows, heads * (dim + vdim)) or vdim > width \
            or any(t.stride(1) != 1 or t.dtype != q.dtype for t in (q, latent, unfolded)):
        raise invalid_argument("latent pack: the shapes do not fit")
    packed = torch.empty((rows, 3 * heads * width), dtype=q.dtype, device=q.device)
    args = PackArgs(q.data_ptr(), q.stride(0), latent.data_ptr(), latent.stride(0), unfolded.data_ptr(),
                    unfolded.stride(0), packed.data_ptr(), packed.stride(0), cos.data_ptr(), sin.data_ptr(),
                    tables.row_seq.data_ptr(), tables.row_pos.data_ptr(), rows, heads, dim, rot_dim, rotary_dims, rank,
                    vdim)
    _check(library().kidi_latent_pack(ctypes.byref(args), dtype_code(q.dtype), ops._stream()), "latent_pack")
    return packed


def gather(kv_view, rows: int, width: int, tables) -> torch.Tensor:
    """The cache entries of the step's rows as a matrix [rows, width]."""
    out = torch.empty((rows, width), dtype=kv_view.keys.dtype, device=kv_view.keys.device)
    geometry = cache_geometry(kv_view, 1, width)
    _check(library().kidi_latent_gather(kv_view.keys.data_ptr(), ctypes.byref(geometry), out.data_ptr(), out.stride(0),
                                        tables.row_seq.data_ptr(), tables.row_pos.data_ptr(),
                                        tables.seq_slot.data_ptr(), rows, width, dtype_code(out.dtype), ops._stream()),
           "latent_gather")
    return out


class DecodeArgs(ctypes.Structure):
    _fields_ = [("folded", c_void_p), ("ldf", c_longlong), ("cache", c_void_p), ("table", c_void_p),
                ("pages_per_seq", c_int), ("row_seq", c_void_p), ("row_pos", c_void_p), ("seq_slot", c_void_p),
                ("part_o", c_void_p), ("part_stat", c_void_p), ("out", c_void_p), ("ldo", c_longlong), ("rows", c_int),
                ("heads", c_int), ("rank", c_int), ("rot_dim", c_int), ("splits", c_int), ("scale", c_float),
                ("splits_are_long", c_int), ("window", c_int)]


def tensor_core_fits(dtype: torch.dtype, rank: int, rot_dim: int, window, kv_view) -> bool:
    """Whether the folded form can run on the tensor cores: bfloat16, widths in multiples of 16, a latent of at
    most 512 values, a cache of 64-token pages that keeps every page (a window is then a mask)."""
    return (dtype == torch.bfloat16 and rank % 16 == 0 and rot_dim % 16 == 0 and 0 < rank <= 512
            and (kv_view is None or (kv_view.page_size == 64 and kv_view.ring_pages == 0
                                     and kv_view.keys.is_contiguous() and kv_view.table.is_contiguous())))


def decode_splits(rows: int, heads: int, longest: int, device: torch.device, window=None) -> int:
    """How many blocks share a sequence's pages: as many as fill the GPU once (every share costs a trip of its
    partial result through the workspace), at most one a page (of those a window reaches)."""
    from .attention import sm_count
    pages = max(1, -(-longest // 64))
    if window:
        pages = min(pages, (int(window) + 62) // 64 + 1)
    tiles = -(-heads // 16)
    return max(1, min(pages, sm_count(device) // max(1, rows * tiles)))


def attention_tensor_core(ctx, folded: torch.Tensor, out: torch.Tensor, *, heads: int, rank: int, rot_dim: int,
                          scale: float, kv_view, splits: Optional[int] = None, window=None) -> None:
    """The folded form on the tensor cores (see `attention`), every row of the step against its sequence's pages;
    the shares of a row's pages meet in a workspace and a second kernel merges them."""
    ops._need_cuda(folded, out)
    rows = folded.shape[0]
    if folded.shape != (rows, heads * (rank + rot_dim)) or out.shape != (rows, heads * rank) or folded.stride(1) != 1 \
            or out.stride(1) != 1 or folded.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 \
            or kv_view.keys.shape[-1] != rank + rot_dim:
        raise invalid_argument("latent attention: folded queries, output or cache have the wrong shape")
    splits = splits or decode_splits(rows, heads, ctx.plan.max_total, folded.device, window)
    reach = -(-ctx.plan.max_total // 64)
    if window:
        reach = min(reach, (int(window) + 62) // 64 + 1)
    count = int(library().kidi_latent_decode_workspace(rows, heads, rank, splits))
    workspace = ctx.workspace("latent_partial", count)
    tables = ctx.tables
    args = DecodeArgs(folded.data_ptr(), folded.stride(0), kv_view.keys.data_ptr(), kv_view.table.data_ptr(),
                      kv_view.table.shape[1], tables.row_seq.data_ptr(), tables.row_pos.data_ptr(),
                      tables.seq_slot.data_ptr(), workspace.data_ptr(),
                      workspace.data_ptr() + rows * splits * heads * rank * 4, out.data_ptr(), out.stride(0), rows,
                      heads, rank, rot_dim, splits, float(scale),
                      -1 if PAGE_BUFFERS == 1 else 1 if PAGE_BUFFERS == 2 or reach > splits else 0, int(window or 0))
    _check(library().kidi_latent_decode(ctypes.byref(args), ops._stream()), f"latent_attention[mma.sync, {splits} shares]", 2)
