"""Rotary position encoding, rotate-half layout.

Reference: tables — src/models/turbo_generic.rs:1654-1670: inv[j] =
1 / theta^(2j / rotary_dim) in float32, angle[p, j] = float32(p) * inv[j],
cos and sin of the angles, [positions, rotary_dim / 2] float32; application —
:417-427 (first half / second half) at rows `index_pos .. index_pos + s`
(:746-768).  Keys are cached after the rotation (:832-833, :1606-1618).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import PositionEncoding, Runtime, StepContext


class RotaryHalved(PositionEncoding):
    padded_rows_ok = True               # rows at or past their sequence's new length are not cached

    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(self.params["head_dim"])
        self.rotary_dim = int(self.params["rotary_dim"])
        self.theta = float(self.params["theta"])
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def table_key(self):
        return ("rotary_halved", self.rotary_dim, self.theta)

    def prepare(self, runtime: Runtime, shared: Optional[dict] = None) -> None:
        """Tables are computed once per (rotary_dim, theta) and shared by the
        layers of a model through `shared`.  They are built on the host in
        float32, as the reference builds them, then copied to the device."""
        key = (self.table_key(), runtime.max_context, str(runtime.device))
        if shared is not None and key in shared:
            self.cos, self.sin = shared[key]
            return
        theta = torch.tensor(self.theta, dtype=torch.float32)
        expo = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / float(self.rotary_dim)
        inv = 1.0 / torch.pow(theta, expo)
        pos = torch.arange(runtime.max_context, dtype=torch.float32).reshape(-1, 1)
        ang = pos * inv.reshape(1, -1)
        self.cos = torch.cos(ang).contiguous().to(runtime.device)
        self.sin = torch.sin(ang).contiguous().to(runtime.device)
        if shared is not None:
            shared[key] = (self.cos, self.sin)

    clears_input = True          # encode_and_store(..., clear_input=True) leaves zeros in qkv

    def encode_and_store(self, qkv, bias, ctx: StepContext, *, n_heads, n_kv_heads, head_dim, q_out, k_out, v_out,
                         clear_input=False):
        b = ctx.batch
        kv = ctx.kv
        write = kv is not None and kv.writes
        table, width = (kv.block_table, kv.table_width) if write else (None, 0)
        kernels.qkv_rope_cache(
            qkv, bias, self.cos, self.sin, b.tok_pos, b.tok_seq, b.new_lens, q_out,
            n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, rotary_dim=self.rotary_dim,
            k_out=k_out, v_out=v_out,
            k_pages=kv.k_pages if write else None, v_pages=kv.v_pages if write else None,
            block_table=table, table_width=width, ring_pages=kv.ring_pages if write else 0,
            page_tokens=kv.page_tokens if kv is not None else 64, clear_input=clear_input)


class RotaryTables(PositionEncoding):
    """Cosines and sines of the angles pos * rate_i, i < rotary_dim / 2, for mixers whose own kernels turn their
    vectors (`layout` says how the mixer pairs entries: "pairs" turns entry 2i with 2i + 1, "halves" entry i with
    i + rotary_dim / 2).  The angles are formed in float64 on the host and their cosines and sines rounded once
    to float32, so that the tables carry no error that grows with the position.

    Plain rates are theta^(-2i / rotary_dim).  With `scaling` = {factor F, original L, fast, slow} the slow
    pairs are stretched for contexts longer than the L positions the rates were made for: a pair that makes t
    turns over L positions has index n(t) = rotary_dim * ln(L / (2 pi t)) / (2 ln theta); with
    lo = max(floor(n(fast)), 0) and hi = min(ceil(n(slow)), rotary_dim - 1), pair i takes the share
    r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) of the rate divided by F and 1 - r_i of its own rate,
    and cosines and sines are multiplied by 0.1 ln F + 1 (the tables carry that factor)."""
    padded_rows_ok = True

    def __init__(self, spec):
        super().__init__(spec)
        self.rotary_dim = int(self.params["rotary_dim"])
        self.theta = float(self.params["theta"])
        self.layout = self.params.get("layout", "pairs")
        if self.layout not in ("pairs", "halves") or self.rotary_dim % 2:
            raise ValueError(f"rotary tables: layout '{self.layout}' (pairs or halves), an even rotary_dim")
        sc = self.params.get("scaling")
        self.scaling = None
        if sc:
            self.scaling = (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
            if min(self.scaling) <= 0.0:
                raise ValueError(f"rotary tables: scaling needs positive factor, original, fast and slow, not {sc}")
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    @property
    def paired(self) -> bool:
        return self.layout == "pairs"

    def rates(self) -> tuple[torch.Tensor, float]:
        """The float64 rates of the pairs and the factor on cosine and sine."""
        half = max(1, self.rotary_dim // 2)
        i = torch.arange(half, dtype=torch.float64)
        rate = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / max(2, self.rotary_dim))
        if self.scaling is None:
            return rate, 1.0
        import math
        F, L, fast, slow = self.scaling

        def index_of(turns: float) -> float:
            return self.rotary_dim * math.log(L / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(index_of(fast)), 0)
        hi = min(math.ceil(index_of(slow)), self.rotary_dim - 1)
        share = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        return rate / F * share + rate * (1.0 - share), 0.1 * math.log(F) + 1.0

    def prepare(self, runtime: Runtime, shared: Optional[dict] = None) -> None:
        key = (("rotary_tables", self.rotary_dim, self.theta, self.scaling), runtime.max_context, str(runtime.device))
        if shared is not None and key in shared:
            self.cos, self.sin = shared[key]
            return
        rate, factor = self.rates()
        ang = torch.arange(runtime.max_context, dtype=torch.float64).reshape(-1, 1) * rate.reshape(1, -1)
        self.cos = (torch.cos(ang) * factor).to(torch.float32).contiguous().to(runtime.device)
        self.sin = (torch.sin(ang) * factor).to(torch.float32).contiguous().to(runtime.device)
        if shared is not None:
            shared[key] = (self.cos, self.sin)

    def encode_and_store(self, *args, **kwargs):
        raise NotImplementedError("rotary tables are applied by the mixer's own kernels")
