"""Grouped-query softmax attention with options, every one a parameter:

  values            "projected": v = W_v x;  "keys": there is no W_v, the values are
                    the keys as projected, before any rotation
  position          a `rotary_tables` part: q and k are rotated over their first
                    rotary_dim entries, entry i with i + rotary_dim/2 (layout "halves") or
                    entry 2i with 2i + 1 (layout "pairs"); None: no rotation
  row_norm_eps      q and k are RMS-normed over their WHOLE projections (all heads of a
                    token at once, x / sqrt(mean(x^2) + eps) * weight, weights `q_norm` and
                    `k_norm` of the projections' sizes) before the heads are split and rotated
  sink              the softmax's denominator counts one more key of score 0 that has no
                    value: p_j = exp(s_j) / (1 + sum exp(s))
  shared_kv         the layer has no key/value tensors: it reads the cache of the schedule
                    entry it is given (whose keys are stored normed and rotated) with its own
                    queries, window and everything else
  cache_window      the window the cache keeps (default: `window`; wider where other layers
                    with wider windows read this layer's cache; None: all keys)
  shares_packed     a prompt's packed keys and values are left in the step's shared dict for
                    the layers that read this layer's cache
  qk_norm_eps       q and k are divided per head by their root mean square,
                    x / sqrt(mean(x^2) + eps), without a weight
  scale             s = q . k * scale
  softcap           s <- softcap * tanh(s / softcap)
  slope_exponent    a bias that grows with the distance: s <- s - m_h * (i - j),
                    m_h = 2^(-slope_exponent * (h + 1) / heads) for head h = 0 ..
  window            the query at position i sees key j <= i if i - j < window
  keep_first        ... or if j < keep_first (the first tokens stay visible; they keep
                    their true positions)
  output_gate       the heads side by side are multiplied entry by entry with
                    sigmoid(W_g x) before the output projection
Query head h reads key/value head h // (heads / kv_heads).  Key rows and value rows
may differ in width; widths that are no multiple of 8 are padded with zeros inside.
No biases.

All projections are one product with the concatenated weight (float32 result); one
kernel encodes q and k, splits the heads and appends k and v to the cache
(csrc/head_encode.cu).  Prompts from position 0 attend over the step's own keys;
everything else reads the paged cache: a ring for a plain window, all keys where
first tokens are kept (the kernels skip what lies between the kept tokens and the
window).  Scores, softmax and the bias are float32.  bfloat16 steps whose keys and
values have one width run the tensor-core kernels (`kernels.attention_ext`), which
also apply the output gate where they can.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..cache import PAGE_TOKENS, KVRequest, ring_pages_for
from ..config import ConfigError
from .base import Mixer, Runtime, StepContext, WeightSpec, float32_vector
from .registry import make_part


class SoftmaxAttention(Mixer):
    padded_rows_ok = True               # causal: no row sees a later one; rows past a sequence's length are not cached
    can_store_result = True

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["num_heads"])
        self.n_kv_heads = int(p["num_kv_heads"])
        # The kernels take rows of whole 16-byte pieces: heads of other widths (`key_dim_given`, `value_dim_given`)
        # are padded to the next multiple of 8 with zero rows of W_q, W_k, W_v, W_g and zero columns of W_o, which
        # changes no score and no result (a mean over a head's entries is corrected below).
        self.key_dim_given = int(p["key_dim"])
        self.values = p.get("values", "projected")
        if self.values not in ("projected", "keys"):
            raise ConfigError(f"softmax attention: values '{self.values}' (projected or keys)")
        self.value_dim_given = int(p.get("value_dim") or self.key_dim_given)
        if self.values == "keys" and self.value_dim_given != self.key_dim_given:
            raise ConfigError(f"softmax attention: values that are the keys have the keys' width "
                              f"{self.key_dim_given}, not {self.value_dim_given}")
        if self.key_dim_given < 1 or self.value_dim_given < 1:
            raise ConfigError("softmax attention: heads need at least one entry")
        self.key_dim = -(-self.key_dim_given // 8) * 8
        self.value_dim = -(-self.value_dim_given // 8) * 8
        self.scale = float(p["scale"])
        self.softcap = float(p["softcap"]) if p.get("softcap") else None
        self.slope_exponent = float(p["slope_exponent"]) if p.get("slope_exponent") else None
        self.qk_norm_eps = float(p["qk_norm_eps"]) if p.get("qk_norm_eps") else 0.0
        if self.qk_norm_eps and self.key_dim != self.key_dim_given:
            # the kernel's mean runs over d' = key_dim entries of which d = key_dim_given are not zero:
            # x / sqrt(sum / d + eps) = sqrt(d / d') * x / sqrt(sum / d' + eps * d / d'), for q and for k
            ratio = self.key_dim_given / self.key_dim
            self.qk_norm_eps *= ratio
            self.scale *= ratio
        self.window: Optional[int] = int(p["window"]) if p.get("window") else None
        self.cache_window: Optional[int] = self.window
        if "cache_window" in p:
            self.cache_window = int(p["cache_window"]) if p.get("cache_window") else None
        if self.window is None and self.cache_window is not None:
            raise ConfigError("softmax attention: a layer without a window needs a cache of all keys")
        if self.window is not None and self.cache_window is not None and self.cache_window < self.window:
            raise ConfigError(f"softmax attention: a cache of {self.cache_window} keys is too small for a window of {self.window}")
        self.row_norm_eps = float(p["row_norm_eps"]) if p.get("row_norm_eps") else 0.0
        self.sink = bool(p.get("sink", False))
        self.shared_kv = bool(p.get("shared_kv", False))
        self.shares_packed = bool(p.get("shares_packed", False))
        if self.shared_kv and self.values != "projected":
            raise ConfigError("softmax attention: a layer that reads another's cache has no keys to take its values from")
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.output_gate = bool(p.get("output_gate", False))
        self.names = dict(p.get("names", {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}))
        kernels.check_row_widths(self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim)
        self.position = make_part(p["position"]) if p.get("position") is not None else None
        if self.position is not None:
            if getattr(self.position, "layout", None) not in ("halves", "pairs"):
                raise ConfigError("softmax attention rotates by a rotary_tables part (layout halves or pairs)")
            if self.position.rotary_dim > self.key_dim_given:
                raise ConfigError(f"softmax attention: {self.position.rotary_dim} rotated entries in heads of "
                                  f"{self.key_dim_given}")
            if self.qk_norm_eps:
                raise ConfigError("softmax attention: either a rotation or unit-size q and k, not both")
        if self.qk_norm_eps and self.row_norm_eps:
            raise ConfigError("softmax attention: q and k are normed per head or over the whole row, not both")
        self.q_width = self.n_heads * self.key_dim
        self.k_width = 0 if self.shared_kv else self.n_kv_heads * self.key_dim
        self.v_width = self.n_kv_heads * self.value_dim if self.values == "projected" and not self.shared_kv else 0
        self.o_width = self.n_heads * self.value_dim
        self.w_in = self.w_o = self.slopes = None
        self.window_chunk = 1

    # ---- weights ----------------------------------------------------------
    def _n(self, which: str) -> str:
        return f"{self.prefix}{self.names[which]}"

    def weight_specs(self):
        d, e, H, G = self.key_dim_given, self.value_dim_given, self.n_heads, self.n_kv_heads
        specs = [WeightSpec(self._n("q"), (H * d, self.hidden), "matrix")]
        if not self.shared_kv:
            specs.append(WeightSpec(self._n("k"), (G * d, self.hidden), "matrix"))
            if self.values == "projected":
                specs.append(WeightSpec(self._n("v"), (G * e, self.hidden), "matrix"))
        if self.row_norm_eps:
            specs.append(WeightSpec(self._n("q_norm"), (H * d,), "norm_scale"))
            if not self.shared_kv:
                specs.append(WeightSpec(self._n("k_norm"), (G * d,), "norm_scale"))
        if self.output_gate:
            specs.append(WeightSpec(self._n("gate"), (H * e, self.hidden), "matrix"))
        specs.append(WeightSpec(self._n("out"), (self.hidden, H * e), "matrix"))
        return specs

    @staticmethod
    def _pad_heads(w: torch.Tensor, heads: int, given: int, padded: int) -> torch.Tensor:
        """[heads * given, W] -> [heads * padded, W] with zero rows behind every head's own."""
        if given == padded:
            return w
        out = w.new_zeros((heads, padded, w.shape[1]))
        out[:, :given] = w.reshape(heads, given, w.shape[1])
        return out.reshape(heads * padded, w.shape[1])

    def bind(self, tensors, runtime: Runtime, shared: Optional[dict] = None):
        which = ["q"] + ([] if self.shared_kv else ["k"] + (["v"] if self.values == "projected" else [])) \
            + (["gate"] if self.output_gate else [])
        heads = {"q": (self.n_heads, self.key_dim_given, self.key_dim),
                 "k": (self.n_kv_heads, self.key_dim_given, self.key_dim),
                 "v": (self.n_kv_heads, self.value_dim_given, self.value_dim),
                 "gate": (self.n_heads, self.value_dim_given, self.value_dim)}
        ws = [self._pad_heads(tensors[self._n(x)], *heads[x]) for x in which]
        if len({w.dtype for w in ws}) != 1:
            ws = [w.to(torch.float32) for w in ws]
        self.w_in = torch.cat(ws, dim=0).contiguous()        # one product: [q | k | (v) | (gate)]
        w_o = tensors[self._n("out")]
        if self.value_dim != self.value_dim_given:           # zero columns where the heads were padded
            w_o = self._pad_heads(w_o.t(), self.n_heads, self.value_dim_given, self.value_dim).t()
        self.w_o = w_o.contiguous()
        self.k_col = 0 if self.shared_kv else self.q_width
        self.v_col = self.q_width + self.k_width if self.values == "projected" and not self.shared_kv else -1
        self.q_norm_w = self.k_norm_w = None
        if self.row_norm_eps:                               # weights over the whole rows, padded like the heads
            def padded(name, heads):
                w = float32_vector(tensors[self._n(name)]).reshape(heads, self.key_dim_given)
                out = w.new_zeros((heads, self.key_dim))
                out[:, :self.key_dim_given] = w
                return out.reshape(-1).contiguous()
            self.q_norm_w = padded("q_norm", self.n_heads)
            if not self.shared_kv:
                self.k_norm_w = padded("k_norm", self.n_kv_heads)
        self.g_col = self.q_width + self.k_width + self.v_width
        if self.slope_exponent is not None:
            h = torch.arange(1, self.n_heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(torch.tensor(2.0, dtype=torch.float64),
                                    -self.slope_exponent * h / self.n_heads).to(torch.float32).to(runtime.device)
        self.window_chunk = runtime.window_chunk
        if self.position is not None:
            self.position.bind(tensors, runtime, shared)
            self.position.prepare(runtime, shared)

    # ---- cache ------------------------------------------------------------
    @property
    def _ring(self) -> bool:
        return self.cache_window is not None and self.keep_first == 0

    def cache_request(self):
        if self.shared_kv:
            return None
        return KVRequest(self.n_kv_heads, self.key_dim, self.cache_window if self._ring else None,
                         self.value_dim if self.value_dim != self.key_dim else None)

    def _use_packed(self, start_pos, step_lens, owns_cache) -> bool:
        """Prompts that start at position 0 attend over the step's own keys: their own, or (a layer that reads
        another's cache) the ones that layer left in the step's shared dict."""
        return (owns_cache or self.shared_kv) and all(s == 0 for s in start_pos) and any(n > 1 for n in step_lens)

    def check_step(self, start_pos, step_lens, owns_cache):
        if self.shared_kv and owns_cache:
            raise kernels.KernelError("a layer without keys and values of its own must be given another entry's cache")
        if not self._ring or self._use_packed(start_pos, step_lens, owns_cache):
            return
        ring_tokens = ring_pages_for(self.cache_window, self.window_chunk - 1) * PAGE_TOKENS
        longest = max(step_lens)
        if longest > ring_tokens - self.window + 1:
            raise kernels.KernelError(
                f"a layer with a window of {self.cache_window} keeps {ring_tokens} keys per sequence and cannot continue "
                f"a sequence by {longest} tokens in one step (at most {ring_tokens - self.window + 1}; the engine's "
                f"window_chunk option sets this)")

    # ---- one step -----------------------------------------------------------
    def forward(self, x, ctx: StepContext, residual):
        b, kv, dev = ctx.batch, ctx.kv, x.device
        T = x.shape[0]
        act = ctx.runtime.act_dtype
        owns = kv is not None and kv.writes and not self.shared_kv
        packed = self._use_packed(b.host_start, b.host_lens, owns)
        proj = kernels.linear(x, self.w_in, out_dtype=torch.float32)
        kernels.mark("qkv")
        q = torch.empty((T, self.q_width), dtype=act, device=dev)
        k = v = None
        if packed and self.shared_kv:
            k, v = ctx.step_shared[("packed_kv", ctx.cache_entry)]
        elif packed:
            k = torch.empty((T, self.k_width), dtype=act, device=dev)
            v = torch.empty((T, self.n_kv_heads * self.value_dim), dtype=act, device=dev)
            if self.shares_packed and ctx.step_shared is not None:
                ctx.step_shared[("packed_kv", ctx.entry)] = (k, v)
        pos = self.position
        row_inv = None
        if self.row_norm_eps:
            row_inv = kernels.row_inv_rms(proj, q_col=0, q_width=self.q_width, q_count=self.n_heads * self.key_dim_given,
                                          k_col=self.k_col, k_width=self.k_width,
                                          k_count=self.n_kv_heads * self.key_dim_given, eps=self.row_norm_eps)
        kernels.head_encode(
            proj, (b.tok_pos, b.tok_seq, b.new_lens), q, q_col=0, k_col=self.k_col, v_col=self.v_col,
            n_heads=self.n_heads, n_kv_heads=0 if self.shared_kv else self.n_kv_heads, key_dim=self.key_dim,
            value_dim=self.value_dim, row_inv=row_inv, q_weight=self.q_norm_w, k_weight=self.k_norm_w,
            paired=pos is not None and pos.paired,
            cos=pos.cos if pos is not None else None, sin=pos.sin if pos is not None else None,
            rotary_dim=pos.rotary_dim if pos is not None else 0, norm_eps=self.qk_norm_eps,
            k_out=None if self.shared_kv else k, v_out=None if self.shared_kv else v,
            k_pages=kv.k_pages if owns else None, v_pages=kv.v_pages if owns else None,
            block_table=kv.block_table if owns else None, table_width=kv.table_width if owns else 0,
            ring_pages=kv.ring_pages if owns else 0, page_tokens=kv.page_tokens if kv is not None else PAGE_TOKENS)
        kernels.mark("rotary")
        out = torch.empty((T, self.o_width), dtype=act, device=dev)
        common = dict(n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, key_dim=self.key_dim,
                      value_dim=self.value_dim, tok_pos=b.tok_pos, tok_seq=b.tok_seq, cu_seqlens=b.cu_seqlens,
                      start_pos=b.start_pos, scale=self.scale, window=self.window, keep_first=self.keep_first,
                      softcap=self.softcap, slopes=self.slopes, sink=self.sink,
                      gate=proj[:, self.g_col:self.g_col + self.o_width] if self.output_gate else None)
        if packed:
            kernels.attention_ext(q, out, k_packed=k, v_packed=v, **common)
        else:
            max_keys = b.max_new_len if self.window is None else min(b.max_new_len, self.window + self.keep_first)
            n_splits = kernels.plan_splits(T, self.n_kv_heads, max_keys, ctx.runtime.sm_count)
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(kernels.split_scratch_floats(T, self.n_heads, self.value_dim, n_splits),
                                      dtype=torch.float32, device=dev)
            kernels.attention_ext(q, out, k_pages=kv.k_pages, v_pages=kv.v_pages, block_table=kv.block_table,
                                  table_width=kv.table_width, ring_pages=kv.ring_pages, page_tokens=kv.page_tokens,
                                  n_splits=n_splits, scratch=scratch, **common)
        kernels.mark("attention")
        kernels.linear(out, self.w_o, out=residual, accumulate=not ctx.store_result)
        kernels.mark("o")
