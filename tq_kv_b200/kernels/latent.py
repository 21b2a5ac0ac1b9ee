"""Python entry points of the kernels around attention through a latent (csrc/latent_attention.cu)."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream


def _check_tables(cos, sin, rot_dims, r):
    if rot_dims % 2 or not 0 <= rot_dims <= r:
        raise KernelError(f"latent attention: {rot_dims} rotated entries must be even and within the rotated part ({r})")
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape \
            or cos.shape[1] != max(1, rot_dims // 2):
        raise KernelError("latent attention: cos/sin must be float32 [positions, rot_dims / 2]")


def latent_rows(proj: torch.Tensor, cq_out: Optional[torch.Tensor], *, off_q: int, off_kv: int, q_rank: int, kv_rank: int,
                rot_dim: int, row_width: int, q_weight: torch.Tensor, kv_weight: torch.Tensor, eps: float,
                cos: torch.Tensor, sin: torch.Tensor, rot_dims: int, paired: bool, tok_pos, tok_seq, new_lens,
                row_out: Optional[torch.Tensor] = None, pages: Optional[torch.Tensor] = None,
                block_table: Optional[torch.Tensor] = None, table_width: int = 0, page_tokens: int = 64,
                ring_pages: int = 0, out_dtype: Optional[torch.dtype] = None):
    """(q_rank 0: no query latent, cq_out and q_weight None; `out_dtype` then names the rows' type.  ring_pages > 0:
    the pages of a sequence are a ring, written at logical page (pos / page_tokens) % ring_pages.)
    From the float32 results of the down projections (proj [T, ld]: the query latent at column off_q, the
    key/value latent and the rotated key part at off_kv): cq_out [T, q_rank] = rms_norm(query latent) * q_weight;
    the cache row [rms_norm(latent) * kv_weight, rotated key part, zeros up to row_width] into row_out
    [T, row_width] and / or the sequence's page (pages [n, 1, page_tokens, row_width])."""
    T = proj.shape[0]
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or max(off_q + q_rank, off_kv + kv_rank + rot_dim) > proj.shape[1]:
        raise KernelError("latent_rows: proj must be float32 rows that hold both down projections")
    if (q_rank > 0 and (cq_out is None or tuple(cq_out.shape) != (T, q_rank))) or row_width < kv_rank + rot_dim:
        raise KernelError("latent_rows: cq_out must be [T, q_rank]; rows must hold the latent and the rotated part")
    dtype = cq_out.dtype if q_rank > 0 else (out_dtype or next(t.dtype for t in (row_out, pages) if t is not None))
    for name, t in (("row_out", row_out), ("pages", pages)):
        if t is not None and (t.dtype != dtype or t.shape[-1] != row_width):
            raise KernelError(f"latent_rows: {name} must have cq_out's dtype and rows of {row_width}")
    if pages is not None and (block_table is None or tuple(pages.shape[1:]) != (1, page_tokens, row_width)):
        raise KernelError("latent_rows: pages must be [n, 1, page_tokens, row_width] with a block table")
    if kv_weight.dtype != torch.float32 or kv_weight.shape[0] != kv_rank or (
            q_rank > 0 and (q_weight is None or q_weight.dtype != torch.float32 or q_weight.shape[0] != q_rank)):
        raise KernelError("latent_rows: the norms' weights must be float32 [q_rank] and [kv_rank]")
    _check_tables(cos, sin, rot_dims, rot_dim)
    need_contiguous(cq_out=cq_out, row_out=row_out, pages=pages, cos=cos, sin=sin, q_weight=q_weight, kv_weight=kv_weight)
    q_rank = int(q_rank)
    check(core().tq_latent_rows(ptr(proj), proj.stride(0), off_q, off_kv, q_rank, kv_rank, rot_dim, row_width,
                                ptr(q_weight), ptr(kv_weight), float(eps), ptr(cos), ptr(sin), rot_dims, int(paired),
                                ptr(tok_pos), ptr(tok_seq), ptr(new_lens), ptr(cq_out), ptr(row_out), ptr(pages),
                                ptr(block_table), table_width, page_tokens, int(ring_pages),
                                dtype_code(torch.empty(0, dtype=dtype)), T, stream()),
          "latent_rows")


def latent_query(q: torch.Tensor, up_k: torch.Tensor, out: torch.Tensor, *, heads: int, dim: int, rot_dim: int,
                 kv_rank: int, row_width: int, cos, sin, rot_dims: int, paired: bool, tok_pos):
    """out[t, h] = [up_k[h]^T q[t, h, :dim], rotate(q[t, h, dim:]), zeros] — the query carried into the latent's
    space.  q float32 [T, heads * (dim + rot_dim)]; up_k [heads * dim, kv_rank] of out's dtype; out
    [T, heads * row_width]."""
    T = q.shape[0]
    if q.dtype != torch.float32 or tuple(q.shape) != (T, heads * (dim + rot_dim)) or q.stride(1) != 1:
        raise KernelError("latent_query: q must be float32 [T, heads * (dim + rot_dim)] (may be a column slice)")
    if tuple(up_k.shape) != (heads * dim, kv_rank) or up_k.dtype != out.dtype:
        raise KernelError("latent_query: up_k must be [heads * dim, kv_rank] of out's dtype")
    if tuple(out.shape) != (T, heads * row_width) or row_width < kv_rank + rot_dim:
        raise KernelError("latent_query: out must be [T, heads * row_width]")
    _check_tables(cos, sin, rot_dims, rot_dim)
    need_contiguous(up_k=up_k, out=out, cos=cos, sin=sin)
    check(core().tq_latent_query(ptr(q), q.stride(0), heads, dim, rot_dim, kv_rank, row_width, ptr(up_k), ptr(cos), ptr(sin),
                                 rot_dims, int(paired), ptr(tok_pos), ptr(out), dtype_code(out), T, stream()),
          "latent_query")
    return out


def latent_heads(q: torch.Tensor, kfv: torch.Tensor, rows: torch.Tensor, q_out: torch.Tensor, k_out: torch.Tensor,
                 v_out: torch.Tensor, *, heads: int, dim: int, rot_dim: int, value_dim: int, kv_rank: int, cos, sin,
                 rot_dims: int, paired: bool, tok_pos):
    """Expanded heads for the ordinary attention kernels, all `hw` = q_out.shape[1] / heads wide: q_out[t, h] =
    [q[t, h, :dim], rotate(q[t, h, dim:]), zeros], k_out[t, h] = [flat key of head h, rows[t, kv_rank : kv_rank +
    rot_dim], zeros], v_out[t, h] = [value of head h, zeros].  q float32 [T, heads * (dim + rot_dim)]; kfv float32
    [T, heads * dim + heads * value_dim] (flat keys, then values, head by head); rows [T, row] of the outputs'
    dtype (the cache rows)."""
    T = q.shape[0]
    hw = q_out.shape[1] // heads
    if q.dtype != torch.float32 or tuple(q.shape) != (T, heads * (dim + rot_dim)) or q.stride(1) != 1:
        raise KernelError("latent_heads: q must be float32 [T, heads * (dim + rot_dim)] (may be a column slice)")
    if kfv.dtype != torch.float32 or tuple(kfv.shape) != (T, heads * (dim + value_dim)) or kfv.stride(1) != 1:
        raise KernelError("latent_heads: kfv must be float32 [T, heads * dim + heads * value_dim]")
    if hw < max(dim + rot_dim, value_dim) or rows.shape[0] != T or rows.shape[1] < kv_rank + rot_dim:
        raise KernelError("latent_heads: heads too narrow, or rows without the rotated part")
    for t in (q_out, k_out, v_out):
        if tuple(t.shape) != (T, heads * hw) or t.dtype != rows.dtype:
            raise KernelError("latent_heads: q_out, k_out, v_out must be [T, heads * hw] of rows' dtype")
    _check_tables(cos, sin, rot_dims, rot_dim)
    need_contiguous(rows=rows, q_out=q_out, k_out=k_out, v_out=v_out, cos=cos, sin=sin)
    check(core().tq_latent_heads(ptr(q), q.stride(0), ptr(kfv), kfv.stride(0), heads * dim, ptr(rows), rows.shape[1], kv_rank, heads,
                                 dim, rot_dim, value_dim, hw, ptr(cos), ptr(sin), rot_dims, int(paired), ptr(tok_pos),
                                 ptr(q_out), ptr(k_out), ptr(v_out), dtype_code(q_out), T, stream()), "latent_heads")


def latent_expand(lat: torch.Tensor, up_v: Optional[torch.Tensor], out: torch.Tensor, *, heads: int, kv_rank: int,
                  row_width: int, value_dim: int, gate: Optional[torch.Tensor] = None):
    """out[t, h] = up_v[h] lat[t, h, :kv_rank], times sigmoid(gate[t, h]) entry by entry.  lat [T, heads *
    row_width]; up_v [heads * value_dim, kv_rank]; gate float32 [T, heads * value_dim] (may be a column slice);
    out [T, heads * value_dim].  Without up_v (then kv_rank >= value_dim) a head's first value_dim entries pass,
    gated."""
    T = lat.shape[0]
    if tuple(lat.shape) != (T, heads * row_width) or tuple(out.shape) != (T, heads * value_dim) or lat.dtype != out.dtype:
        raise KernelError("latent_expand: lat must be [T, heads * row_width] and out [T, heads * value_dim] of one dtype")
    if up_v is None:
        if kv_rank < value_dim:
            raise KernelError("latent_expand: without a matrix the heads must hold value_dim entries")
    elif tuple(up_v.shape) != (heads * value_dim, kv_rank) or up_v.dtype != out.dtype:
        raise KernelError("latent_expand: up_v must be [heads * value_dim, kv_rank] of out's dtype")
    ldg = 0
    if gate is not None:
        if gate.dtype != torch.float32 or tuple(gate.shape) != (T, heads * value_dim) or gate.stride(1) != 1:
            raise KernelError("latent_expand: gate must be float32 [T, heads * value_dim]")
        ldg = gate.stride(0)
    need_contiguous(lat=lat, up_v=up_v, out=out)        # (need_contiguous passes None)
    check(core().tq_latent_expand(ptr(lat), heads, kv_rank, row_width, value_dim, ptr(up_v), ptr(gate), ldg, ptr(out),
                                  dtype_code(out), T, stream()), "latent_expand")
    return out
