"""Python entry points of the kernels around the matrix memory with exponential gates (csrc/mlstm.cu)."""
from __future__ import annotations

import torch

from ._lib import KernelError, check, core, dtype_code, need_contiguous, ptr, stream


def mlstm_gates(in_raw: torch.Tensor, forget_raw: torch.Tensor, cap: float, state_m: torch.Tensor,
                cu_seqlens: torch.Tensor, slots: torch.Tensor, n_seqs: int) -> torch.Tensor:
    """From the raw gate values (projection plus bias; float32 [T, H] column slices of one buffer) to the scan's
    scalars, float32 [T, H, 4] = (a, b, m, 0): with i = cap tanh(in / cap), f = logsigmoid(cap tanh(forget / cap))
    and the running maximum m_t = max(f + m_{t-1}, i):  a = exp(f + m_{t-1} - m_t), b = exp(i - m_t).  `state_m`
    float32 [slots, H] (a column slice of the per-sequence state) holds each sequence's m before the step and after."""
    T, H = in_raw.shape
    for t in (in_raw, forget_raw):
        if t.dtype != torch.float32 or tuple(t.shape) != (T, H) or t.stride(1) != 1 or t.stride(0) != in_raw.stride(0):
            raise KernelError("mlstm_gates: both gates float32 [T, H], column slices of one buffer")
    if state_m.dtype != torch.float32 or state_m.dim() != 2 or state_m.shape[1] != H or state_m.stride(1) != 1:
        raise KernelError("mlstm_gates: state_m must be float32 [slots, H]")
    need_contiguous(cu_seqlens=cu_seqlens, slots=slots)
    scal = torch.empty((T, H, 4), dtype=torch.float32, device=in_raw.device)
    check(core().tq_mlstm_gates(ptr(in_raw), ptr(forget_raw), in_raw.stride(0), float(cap), ptr(cu_seqlens), ptr(slots),
                                ptr(state_m), state_m.stride(0), H, ptr(scal), int(n_seqs), stream()), "mlstm_gates")
    return scal


def mlstm_read(o: torch.Tensor, scalars: torch.Tensor, gate: torch.Tensor, norm_weight: torch.Tensor, out: torch.Tensor,
               *, heads: int, value_dim: int, q_scale: float, floor: float, eps: float) -> torch.Tensor:
    """The memory's read after the scan.  o float32 [T, heads * ea]: per head the value_dim columns of S^T q, then
    n . q, then padding (ea = o.shape[1] / heads); scalars as `mlstm_gates` left them (m in entry 2).
    out[t, h] = rms(o_h q_scale / (max(|n . q| q_scale, exp(-m)) + floor)) * norm_weight_h * sigmoid(gate[t, h]),
    rms(x) = x / sqrt(mean(x^2) + eps) per head.  gate float32 [T, heads * value_dim] (may be a column slice)."""
    T = o.shape[0]
    ea = o.shape[1] // heads
    e = int(value_dim)
    if o.dtype != torch.float32 or not o.is_contiguous() or o.shape[1] != heads * ea or ea <= e:
        raise KernelError("mlstm_read: o must be contiguous float32 [T, heads * (more than value_dim)]")
    if scalars.dtype != torch.float32 or tuple(scalars.shape) != (T, heads, 4) or not scalars.is_contiguous():
        raise KernelError("mlstm_read: scalars must be float32 [T, heads, 4]")
    if gate.dtype != torch.float32 or tuple(gate.shape) != (T, heads * e) or gate.stride(1) != 1:
        raise KernelError("mlstm_read: gate must be float32 [T, heads * value_dim]")
    if norm_weight.dtype != torch.float32 or norm_weight.shape[0] != heads * e or tuple(out.shape) != (T, heads * e):
        raise KernelError("mlstm_read: norm_weight float32 [heads * value_dim], out [T, heads * value_dim]")
    need_contiguous(norm_weight=norm_weight, out=out)
    check(core().tq_mlstm_read(ptr(o), ea, e, ptr(scalars), ptr(gate), gate.stride(0), ptr(norm_weight), float(q_scale),
                               float(floor), float(eps), heads, ptr(out), dtype_code(out), T, stream()), "mlstm_read")
    return out
