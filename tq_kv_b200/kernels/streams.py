"""Python entry points of the parallel residual streams (csrc/stream_mix.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream

MAX_STREAMS = 8
MAX_WIDTH = 12288


def streams_fill(x: torch.Tensor, n_streams: int) -> torch.Tensor:
    """[S, T, W] float32 with every stream equal to x [T, W]."""
    if x.dtype != torch.float32 or x.dim() != 2:
        raise KernelError("streams_fill: x must be float32 [T, W]")
    need_contiguous(x=x)
    xs = torch.empty((n_streams, *x.shape), dtype=torch.float32, device=x.device)
    check(core().tq_streams_fill(ptr(x), ptr(xs), n_streams, x.numel(), stream()), "streams_fill")
    return xs


def streams_step(xs: torch.Tensor, *, y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                 write: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None,
                 norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                 out_dtype: Optional[torch.dtype] = None, rows: Optional[torch.Tensor] = None):
    """One sublayer boundary of the streams xs [S, T, W] (float32, changed in place).

    With `y` [T, W]: xs_new[r] = sum_s mix[s, r] * xs[s] + write[r] * y.  With `read` [S]: returns
    u = sum_s read[s] * xs_new[s] — normed, u / sqrt(mean(u^2) + eps) * norm_weight, if a weight is given — as
    [T, W] of `out_dtype`, or of the tokens `rows` only (the streams are then left unchanged: the write is applied on the way to the result only)."""
    if xs.dtype != torch.float32 or xs.dim() != 3:
        raise KernelError("streams_step: xs must be float32 [S, T, W]")
    S, T, W = xs.shape
    if S > MAX_STREAMS or W > MAX_WIDTH:
        raise KernelError(f"streams_step: at most {MAX_STREAMS} streams of width {MAX_WIDTH} (got {S} of {W})")
    if y is not None:
        if y.dtype != torch.float32 or tuple(y.shape) != (T, W) or mix is None or write is None:
            raise KernelError("streams_step: a write needs y float32 [T, W], mix [S, S] and write [S]")
        if tuple(mix.shape) != (S, S) or tuple(write.shape) != (S,):
            raise KernelError(f"streams_step: mix {tuple(mix.shape)} / write {tuple(write.shape)} do not fit {S} streams")
    for name, t in (("mix", mix), ("write", write), ("read", read), ("norm_weight", norm_weight)):
        if t is not None and t.dtype != torch.float32:
            raise KernelError(f"streams_step: {name} must be float32")
    out = None
    if read is not None:
        if tuple(read.shape) != (S,) or (norm_weight is not None and tuple(norm_weight.shape) != (W,)):
            raise KernelError("streams_step: read must be [S] and the norm's weight [W]")
        if rows is not None and rows.dtype != torch.int32:
            raise KernelError("streams_step: rows must be int32")
        n = T if rows is None else rows.shape[0]
        out = torch.empty((n, W), dtype=out_dtype or torch.float32, device=xs.device)
    elif y is None:
        return None
    need_contiguous(xs=xs, y=y, mix=mix, write=write, read=read, norm_weight=norm_weight, rows=rows)
    n_rows = T if rows is None else rows.shape[0]
    check(core().tq_streams_step(ptr(xs), S, T, W, ptr(y), ptr(mix), ptr(write), ptr(read), ptr(norm_weight),
                                 float(eps), ptr(out), dtype_code(out) if out is not None else 0, ptr(rows), n_rows,
                                 stream()), "streams_step")
    return out
