"""Softmax attention whose keys and values come from a small latent per token.

With H heads, per head `dim` unrotated and `rot_dim` rotated query/key entries
and values of `value_dim`, and a latent of `kv_rank`:

    c_q = rms_norm(W_dq x) * w_q            q[h] = (W_uq c_q)[h] = [q_flat[h] (dim), q_rot[h] (rot_dim)]
    [c' , k_r'] = W_dkv x                   c = rms_norm(c') * w_kv,  k_r = rotate(k_r')   (shared by the heads)
    key[h] = [U_k[h] c, k_r]                value[h] = U_v[h] c
    score = (q_flat[h] . U_k[h] c + rotate(q_rot[h]) . k_r) * scale,   softmax over the keys j <= i
    out = W_o ((heads side by side) * sigmoid(W_g x))            (the gate is optional)

Without a query latent (`q_rank` absent) the queries are projected directly, q = W_q x.  With `window` the query at
position i reads the keys j with 0 <= i - j < window, and the cache is a ring of the window's rows.

Only c and k_r are cached: one row of kv_rank + rot_dim values per token (one key/value "head" whose value rows
are not used).  The attention itself runs in the latent's space: the query is carried there,
q~[h] = [U_k[h]^T q_flat[h], rotate(q_rot[h])], the attention kernels see one shared key/value head whose value
is the cached row itself, and the weighted mean of latents is expanded afterwards, U_v[h] mean(c)
(csrc/latent_attention.cu).  That is how everything that reads the pages runs (decoding, portions of prompts, a
prompt beside decoding rows).  Prompts from position 0 bring all their keys along: there the keys and values of all
heads are expanded once, by two matrix products, and the ordinary attention kernels run with this mixer's heads
(fewer operations per score, and the tensor-core prompt kernels take the heads' widths).  Rows are padded with
zeros to a multiple of 16 values (what the attention kernels take).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache import PAGE_TOKENS, KVRequest, ring_pages_for
from ..config import ConfigError
from ..kernels.attention import MAX_HEAD_DIM
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector
from .registry import make_part

MAX_ROW = MAX_HEAD_DIM          # widest cached row (latent + rotated part) the attention kernels take


class LatentAttention(Mixer):
    padded_rows_ok = True               # causal, and rows past a sequence's new length are not cached
    can_store_result = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.dim, self.rot_dim = int(p["heads"]), int(p["dim"]), int(p["rot_dim"])
        self.value_dim = int(p["value_dim"])
        self.q_rank, self.kv_rank = int(p.get("q_rank") or 0), int(p["kv_rank"])      # q_rank 0: q = W_q x directly
        self.window = int(p["window"]) if p.get("window") else None
        self.window_chunk = 1
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.output_gate = bool(p.get("output_gate", False))
        self.names = dict(p["names"])
        self.position = make_part(p["position"])
        self.row = -(-(self.kv_rank + self.rot_dim) // 16) * 16
        if self.row > MAX_ROW:
            raise ConfigError(f"latent attention: a cached row of {self.kv_rank} + {self.rot_dim} values exceeds the "
                              f"attention kernels' {MAX_ROW}")
        if self.position.rotary_dim > self.rot_dim:
            raise ConfigError("latent attention: more rotated entries than the rotated part holds")
        self.w_in = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.q_norm_w = self.kv_norm_w = None

    def _n(self, which: str) -> str:
        return self.prefix + self.names[which]

    def weight_specs(self):
        h, H = self.hidden, self.heads
        if self.q_rank:
            specs = [WeightSpec(self._n("q_down"), (self.q_rank, h), "matrix"),
                     WeightSpec(self._n("q_norm"), (self.q_rank,), "norm_scale"),
                     WeightSpec(self._n("q_up"), (H * (self.dim + self.rot_dim), self.q_rank), "matrix")]
        else:
            specs = [WeightSpec(self._n("q"), (H * (self.dim + self.rot_dim), h), "matrix")]
        specs += [WeightSpec(self._n("kv_down"), (self.kv_rank + self.rot_dim, h), "matrix"),
                  WeightSpec(self._n("kv_norm"), (self.kv_rank,), "norm_scale"),
                  WeightSpec(self._n("k_up"), (H * self.dim, self.kv_rank), "matrix"),
                  WeightSpec(self._n("v_up"), (H * self.value_dim, self.kv_rank), "matrix"),
                  WeightSpec(self._n("out"), (h, H * self.value_dim), "matrix")]
        if self.output_gate:
            specs.append(WeightSpec(self._n("gate"), (H * self.value_dim, h), "matrix"))
        return specs

    def bind(self, tensors, runtime: Runtime, shared=None):
        ws = [tensors[self._n("q_down" if self.q_rank else "q")], tensors[self._n("kv_down")]]
        self.q_cols = self.q_rank or self.heads * (self.dim + self.rot_dim)      # columns of the first projection
        if self.output_gate:
            ws.append(tensors[self._n("gate")])
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()          # query latent | key/value latent, rotated part | gate
        self.w_uq = tensors[self._n("q_up")].contiguous() if self.q_rank else None
        self.window_chunk = runtime.window_chunk
        act = runtime.act_dtype                                 # the per-head products read these in the activations' dtype
        self.w_uk = tensors[self._n("k_up")].to(act).contiguous()
        self.w_uv = tensors[self._n("v_up")].to(act).contiguous()
        self.w_ukv = torch.cat([self.w_uk, self.w_uv], dim=0).contiguous()     # prompts expand keys and values at once
        self.head_width = -(-max(self.dim + self.rot_dim, self.value_dim) // 16) * 16
        self.w_o = tensors[self._n("out")].contiguous()
        self.q_norm_w = float32_vector(tensors[self._n("q_norm")]) if self.q_rank else None
        self.kv_norm_w = float32_vector(tensors[self._n("kv_norm")])
        self.position.bind(tensors, runtime, shared)
        self.position.prepare(runtime, shared)

    def cache_request(self):
        return KVRequest(1, self.row, self.window, 1)

    def check_step(self, start_pos, step_lens, owns_cache):
        if self.window is None or self._use_packed(start_pos, step_lens, owns_cache):
            return
        ring_tokens = ring_pages_for(self.window, self.window_chunk - 1) * PAGE_TOKENS
        longest = max(step_lens)
        if longest > ring_tokens - self.window + 1:
            raise kernels.KernelError(
                f"a layer with a window of {self.window} keeps {ring_tokens} rows per sequence and cannot continue "
                f"a sequence by {longest} tokens in one step (at most {ring_tokens - self.window + 1}; the engine's "
                f"window_chunk option sets this)")

    @staticmethod
    def _use_packed(start_pos, step_lens, owns_cache) -> bool:
        return owns_cache and all(s == 0 for s in start_pos) and any(n > 1 for n in step_lens)

    def forward(self, x, ctx: StepContext, residual):
        b, kv, dev = ctx.batch, ctx.kv, residual.device
        act = ctx.runtime.act_dtype
        H, row, pos = self.heads, self.row, self.position
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)
        kernels.mark("qkv")
        T = proj.shape[0]
        owns = kv is not None and kv.writes
        packed = self._use_packed(b.host_start, b.host_lens, owns)
        cq = torch.empty((T, self.q_rank), dtype=act, device=dev) if self.q_rank else None
        rows = torch.empty((T, row), dtype=act, device=dev) if packed else None
        rot = dict(cos=pos.cos, sin=pos.sin, rot_dims=pos.rotary_dim, paired=pos.paired, tok_pos=b.tok_pos)
        kernels.latent_rows(proj, cq, off_q=0, off_kv=self.q_cols, q_rank=self.q_rank, kv_rank=self.kv_rank,
                            rot_dim=self.rot_dim, row_width=row, q_weight=self.q_norm_w, kv_weight=self.kv_norm_w,
                            eps=self.eps, tok_seq=b.tok_seq, new_lens=b.new_lens, row_out=rows,
                            pages=kv.k_pages if owns else None, block_table=kv.block_table if owns else None,
                            table_width=kv.table_width if owns else 0,
                            page_tokens=kv.page_tokens if kv is not None else 64,
                            ring_pages=kv.ring_pages if owns else 0, out_dtype=act, **rot)
        kernels.mark("rotary")
        if self.q_rank:
            q = kernels.linear(cq, self.w_uq, out_dtype=torch.float32)
            kernels.mark("qkv")
        else:
            q = proj[:, :self.q_cols]
        gate = proj[:, self.q_cols + self.kv_rank + self.rot_dim:] if self.output_gate else None
        y = torch.empty((T, H * self.value_dim), dtype=act, device=dev)
        if packed:
            # A prompt from position 0 brings all its keys along: they are expanded once (two matrix products for
            # all heads) and the ordinary attention kernels run with this mixer's heads as they are.
            hw = self.head_width
            kfv = kernels.linear(rows[:, :self.kv_rank], self.w_ukv, out_dtype=torch.float32)
            kernels.mark("qkv")
            qh, kh, vh = (torch.empty((T, H * hw), dtype=act, device=dev) for _ in range(3))
            kernels.latent_heads(q, kfv, rows, qh, kh, vh, heads=H, dim=self.dim, rot_dim=self.rot_dim,
                                 value_dim=self.value_dim, kv_rank=self.kv_rank, **rot)
            kernels.mark("rotary")
            oh = torch.empty_like(qh)
            kernels.attention(qh, oh, k_packed=kh, v_packed=vh, n_heads=H, n_kv_heads=H, head_dim=hw, tok_pos=b.tok_pos,
                              tok_seq=b.tok_seq, cu_seqlens=b.cu_seqlens, start_pos=b.start_pos, window=self.window,
                              scale=self.scale)
            kernels.mark("attention")
            kernels.latent_expand(oh, None, y, heads=H, kv_rank=hw, row_width=hw, value_dim=self.value_dim, gate=gate)
            kernels.mark("rotary")
            kernels.linear(y, self.w_o, out=residual, accumulate=not ctx.store_result)
            kernels.mark("o")
            return
        qa = torch.empty((T, H * row), dtype=act, device=dev)
        kernels.latent_query(q, self.w_uk, qa, heads=H, dim=self.dim, rot_dim=self.rot_dim, kv_rank=self.kv_rank,
                             row_width=row, **rot)
        kernels.mark("rotary")
        lat = torch.empty_like(qa)
        max_keys = b.max_new_len if self.window is None else min(b.max_new_len, self.window)
        n_splits = kernels.plan_splits(T, 1, max_keys, ctx.runtime.sm_count)
        scratch = None
        if n_splits > 1:
            scratch = torch.empty(kernels.split_scratch_floats(T, H, row, n_splits), dtype=torch.float32, device=dev)
        kernels.attention(qa, lat, n_heads=H, n_kv_heads=1, head_dim=row, tok_pos=b.tok_pos, tok_seq=b.tok_seq,
                          cu_seqlens=b.cu_seqlens, start_pos=b.start_pos, window=self.window, scale=self.scale,
                          k_pages=kv.k_pages, v_pages=kv.k_pages, block_table=kv.block_table,
                          table_width=kv.table_width, ring_pages=kv.ring_pages, page_tokens=kv.page_tokens,
                          n_splits=n_splits, scratch=scratch)
        kernels.mark("attention")
        kernels.latent_expand(lat, self.w_uv, y, heads=H, kv_rank=self.kv_rank, row_width=row,
                              value_dim=self.value_dim, gate=gate)
        kernels.mark("rotary")
        kernels.linear(y, self.w_o, out=residual, accumulate=not ctx.store_result)
        kernels.mark("o")
