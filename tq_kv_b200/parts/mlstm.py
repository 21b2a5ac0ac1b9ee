"""A mixer with a matrix of memory per head and exponential gates (the mLSTM of xLSTM):

    q = W_q x / sqrt(d),  k = W_k x  (heads x d),   v = W_v x  (heads x e)
    i = cap tanh((W_i x + b_i) / cap)                   log of the input gate, one per head
    f = logsigmoid(cap tanh((W_f x + b_f) / cap))       log of the forget gate
    m_t = max(f + m_{t-1}, i)                           a running maximum, m_0 = 0 (not minus infinity)
    S_t = exp(f + m_{t-1} - m_t) S_{t-1} + exp(i - m_t) k v^T,     n_t likewise with k alone
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + read_floor)
    out = W_o ((each head's o over its root mean square) * w_norm * sigmoid(W_g x))

S, n and m start at zero, are float32 and live in the cache's per-sequence state, so a prompt and a decoded
token run the same kernels.  n rides in S as one more value column: the value projection carries, per head, a
row of zeros whose bias is 1 (and zero rows up to a multiple of four columns), which makes the update the scan
with one decay per head and token of csrc/linear_scan.cu, its scalars made by csrc/mlstm.cu.  The queries go
into the scan unscaled; the read applies 1 / sqrt(d) to both S^T q and n . q.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateRequest
from ..kernels.scan import MAX_KEY_WIDTH
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector


class MatrixMemoryMixer(Mixer):
    graph_capturable = True             # slots and lengths are read on the device
    can_store_result = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.key_dim, self.value_dim = int(p["heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.gate_cap = float(p["gate_cap"])
        self.eps = float(p["eps"])
        self.read_floor = float(p.get("read_floor", 1e-6))
        self.names = dict(p["names"])
        if self.key_dim > MAX_KEY_WIDTH:
            raise kernels.KernelError(f"matrix memory: keys of {self.key_dim} exceed the scan's {MAX_KEY_WIDTH}")
        self.value_cols = -(-(self.value_dim + 1) // 4) * 4         # e values, n . q, zeros up to a multiple of four
        H, d, e, ea = self.heads, self.key_dim, self.value_dim, self.value_cols
        self.off_k = H * d
        self.off_v = 2 * H * d
        self.off_g = self.off_v + H * ea
        self.off_i = self.off_g + H * e
        self.off_f = self.off_i + H
        self.state_floats = H * d * ea
        self.w_in = self.bias = self.norm_w = self.w_o = None

    def _n(self, which: str) -> str:
        return self.prefix + self.names[which]

    def weight_specs(self):
        H, d, e, W = self.heads, self.key_dim, self.value_dim, self.hidden
        return [WeightSpec(self._n("q"), (H * d, W), "matrix"), WeightSpec(self._n("k"), (H * d, W), "matrix"),
                WeightSpec(self._n("v"), (H * e, W), "matrix"), WeightSpec(self._n("gate"), (H * e, W), "matrix"),
                WeightSpec(self._n("input"), (H, W), "matrix"), WeightSpec(self._n("input_bias"), (H,), "bias"),
                WeightSpec(self._n("forget"), (H, W), "matrix"), WeightSpec(self._n("forget_bias"), (H,), "bias"),
                WeightSpec(self._n("norm"), (H * e,), "norm_scale"), WeightSpec(self._n("out"), (W, H * e), "matrix")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        H, e, ea, W = self.heads, self.value_dim, self.value_cols, self.hidden
        ws = [tensors[self._n(x)] for x in ("q", "k", "v", "gate", "input", "forget")]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        v = ws[2].new_zeros((H, ea, W))                     # per head: the value rows, then zero rows
        v[:, :e] = ws[2].reshape(H, e, W)
        self.w_in = torch.cat([ws[0], ws[1], v.reshape(H * ea, W), ws[3], ws[4], ws[5]], dim=0).contiguous()
        bias = torch.zeros(self.w_in.shape[0], dtype=torch.float32, device=self.w_in.device)
        bias[self.off_v:self.off_g].reshape(H, ea)[:, e] = 1.0      # the column that accumulates n
        bias[self.off_i:self.off_i + H] = float32_vector(tensors[self._n("input_bias")])
        bias[self.off_f:self.off_f + H] = float32_vector(tensors[self._n("forget_bias")])
        self.bias = bias
        self.norm_w = float32_vector(tensors[self._n("norm")])
        self.w_o = tensors[self._n("out")].contiguous()

    def state_request(self):
        return StateRequest((self.state_floats + self.heads,), torch.float32)       # [S with n | m]

    def forward(self, x, ctx: StepContext, residual):
        b, dev = ctx.batch, residual.device
        H, d, e, ea = self.heads, self.key_dim, self.value_dim, self.value_cols
        proj = kernels.linear(x, self.w_in, bias=self.bias, out_dtype=torch.float32)
        kernels.mark("qkv")
        T = proj.shape[0]
        scal = kernels.mlstm_gates(proj[:, self.off_i:self.off_i + H], proj[:, self.off_f:self.off_f + H], self.gate_cap,
                                   ctx.state[:, self.state_floats:], b.cu_seqlens, b.slots, b.n_seqs)
        kernels.mark("conv")
        o = torch.empty((T, H * ea), dtype=torch.float32, device=dev)
        kernels.gated_scan(proj[:, :self.off_k], proj[:, self.off_k:self.off_v], proj[:, self.off_v:self.off_g], scal,
                           ctx.state[:, :self.state_floats], b.cu_seqlens, b.slots, o, n_seqs=b.n_seqs, heads=H,
                           qk_heads=H, key_dim=d, value_dim=ea, delta=False, single_tokens=b.single_tokens)
        kernels.mark("scan")
        y = torch.empty((T, H * e), dtype=ctx.runtime.act_dtype, device=dev)
        kernels.mlstm_read(o, scal, proj[:, self.off_g:self.off_i], self.norm_w, y, heads=H, value_dim=e,
                           q_scale=d ** -0.5, floor=self.read_floor, eps=self.eps)
        kernels.mark("norms")
        kernels.linear(y, self.w_o, out=residual, accumulate=not ctx.store_result)
        kernels.mark("o")
