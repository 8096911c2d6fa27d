"""Wrappers of `csrc/streams.cu`: a residual kept as several streams,
fp32 [tokens, streams, width] (hyper-connections)."""
from __future__ import annotations

from typing import Optional

import torch

from . import KernelError, _c_float, _c_int, _check, _code, _contig, _need_cuda, _ptr, _stream, build


def _residual(x: torch.Tensor) -> None:
    if x.dtype != torch.float32 or x.dim() != 3:
        raise KernelError("a residual of streams is float32 [tokens, streams, width]")
    _contig(x, "residual streams")


def embed_norm(table: torch.Tensor, ids: torch.Tensor, gain: torch.Tensor, eps: float,
               out: torch.Tensor, device_tokens: Optional[torch.Tensor] = None) -> None:
    """out[t, s, :] = rmsnorm(table[ids[t]]) * gain for every stream s."""
    _need_cuda(table, ids, gain, out, device_tokens)
    _residual(out)
    if ids.dtype != torch.int32 or gain.dtype != torch.float32:
        raise KernelError("embed_norm takes int32 ids and a float32 gain")
    _contig(table, "embedding table")
    lib = build.load("streams")
    _check(lib.cb_embed_norm_streams(_ptr(table), _c_int(_code(table.dtype)), _ptr(ids), _ptr(gain),
                                     _ptr(out), _c_int(ids.shape[0]), _c_int(table.shape[1]),
                                     _c_int(table.shape[0]), _c_int(out.shape[1]), _c_float(eps),
                                     _ptr(device_tokens), _stream()), "embed_norm_streams")


def read(x: torch.Tensor, weights: torch.Tensor, gain: torch.Tensor, eps: float,
         h: torch.Tensor) -> None:
    """h = rmsnorm(sum_s weights[s] x[:, s]) * gain."""
    _need_cuda(x, weights, gain, h)
    _residual(x)
    _contig(h, "normalised rows")
    lib = build.load("streams")
    _check(lib.cb_streams_read(_ptr(x), _ptr(weights), _ptr(gain), _ptr(h), _c_int(_code(h.dtype)),
                               _c_int(x.shape[0]), _c_int(x.shape[2]), _c_int(x.shape[1]),
                               _c_float(eps), _stream()), "streams_read")


def write(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, out_w: torch.Tensor, *,
          next_weights: Optional[torch.Tensor] = None, next_gain: Optional[torch.Tensor] = None,
          eps: float = 0.0, h: Optional[torch.Tensor] = None) -> None:
    """x[:, t] <- sum_s mix[s, t] x[:, s] + out_w[t] y for all t at once.  With
    `next_weights`, `next_gain` and `h`: also the read of the sublayer that follows,
    h = rmsnorm(sum_t next_weights[t] x[:, t]) * next_gain, in the same pass."""
    _need_cuda(x, y, mix, out_w, next_weights, next_gain, h)
    _residual(x)
    if y.dtype != torch.float32 or y.shape != (x.shape[0], x.shape[2]):
        raise KernelError("streams.write: y is float32 [tokens, width]")
    _contig(y, "sublayer result")
    lib = build.load("streams")
    _check(lib.cb_streams_write(_ptr(x), _ptr(y), _ptr(mix), _ptr(out_w), _c_int(x.shape[0]),
                                _c_int(x.shape[2]), _c_int(x.shape[1]), _ptr(next_weights),
                                _ptr(next_gain), _ptr(h),
                                _c_int(_code(h.dtype) if h is not None else 0), _c_float(eps),
                                _stream()), "streams_write")


def sum_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = sum_s x[rows[i], s]."""
    _need_cuda(x, rows, out)
    _residual(x)
    if out.dtype != torch.float32 or rows.dtype != torch.int32:
        raise KernelError("streams.sum_rows takes int32 rows and a float32 output")
    lib = build.load("streams")
    _check(lib.cb_streams_sum_rows(_ptr(x), _ptr(rows), _ptr(out), _c_int(out.shape[0]),
                                   _c_int(x.shape[2]), _c_int(x.shape[1]), _stream()),
           "streams_sum_rows")
