"""A feed-forward of `experts` small SwiGLU layers of which each token uses `top`.

Expert e is  W_down[e] (silu(W_gate[e] x) * (W_up[e] x)),  no biases.  Which experts a
token uses is `routing`:
  "table"   there is no router: a table [vocab, top] of expert indices (the
            entries of a row differ) names them by the token's id; each has the
            weight 1 / top.
  "router"  scores s = sigmoid(W_router x), computed in float32; the `top` experts
            with the largest scores are chosen (the lowest index first among equals);
            their weights are  router_scale * s / (sum of the chosen s + weight_sum_floor).
The result is the weighted sum of the chosen experts' results.  With `shared_size` > 0
a shared expert of that inner width (same form, tensors under `names["shared"]`) runs
for every token and is added.

The experts' weights are stacked at bind time ([E, 2F, W] gate rows then up rows,
and [E, W, F]).  Few rows (decoding) and the float32 path run every (token, expert)
pair as a row-times-matrix product of its own (csrc/routed_experts.cu); bfloat16
steps with many rows, or with at least two pairs per expert, are sorted by expert
and run as tiles of one matrix product per projection
(`kernels.routed_experts_tiles`): each expert's matrices are then read once.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config import ConfigError
from .base import FeedForward, Runtime, StepContext, WeightSpec


class TableExperts(FeedForward):
    padded_rows_ok = True               # row by row
    can_store_result = True
    TILE_MIN_ROWS = 65                  # from this many rows on, bfloat16 steps run the sorted tiles
    # ... and from this many (token, expert) pairs per expert on: the row form reads an expert's matrices once per
    # pair, the tiles once per expert, so decode batches whose tokens share experts run the tiles too (measured at
    # 8 experts of 4,096 x 5,504, 2 per token: 8 rows 1.14 -> 1.09 ms a step, 64 rows 5.79 -> 1.33; 4 rows 0.83 -> 0.97)
    TILE_MIN_PAIRS_PER_EXPERT = 2

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.n_experts = int(p["experts"])
        self.top = int(p["top"])
        self.routing = p.get("routing", "table")
        if self.routing not in ("table", "router"):
            raise ConfigError(f"routed experts: unknown routing '{self.routing}' (known: table, router)")
        self.vocab = int(p["vocab_size"]) if self.routing == "table" else 0
        self.router_scale = float(p.get("router_scale", 1.0))
        self.weight_sum_floor = float(p.get("weight_sum_floor", 0.0))
        self.shared_size = int(p.get("shared_size") or 0)
        if not 1 <= self.top <= self.n_experts:
            raise ConfigError(f"routed experts: a token cannot use {self.top} of {self.n_experts} experts")
        self.names = dict(p.get("names", {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "table": "table"}))
        self.names.setdefault("router", "router")
        self.names.setdefault("shared", "shared.")
        self.w_gate_up = self.w_down = self.table = self.w_router = self.w_shared_gate_up = self.w_shared_down = None

    def _e(self, e: int, which: str) -> str:
        return f"{self.prefix}{self.names['expert'].format(e)}{self.names[which]}"

    def weight_specs(self):
        specs = []
        for e in range(self.n_experts):
            specs += [WeightSpec(self._e(e, "gate"), (self.inter, self.hidden), "matrix"),
                      WeightSpec(self._e(e, "up"), (self.inter, self.hidden), "matrix"),
                      WeightSpec(self._e(e, "down"), (self.hidden, self.inter), "matrix")]
        if self.routing == "table":
            specs.append(WeightSpec(self.prefix + self.names["table"], (self.vocab, self.top),
                                    f"choice_table:{self.n_experts}"))
        else:
            specs.append(WeightSpec(self.prefix + self.names["router"], (self.n_experts, self.hidden), "matrix"))
        if self.shared_size:
            sp = self.prefix + self.names["shared"]
            specs += [WeightSpec(sp + self.names["gate"], (self.shared_size, self.hidden), "matrix"),
                      WeightSpec(sp + self.names["up"], (self.shared_size, self.hidden), "matrix"),
                      WeightSpec(sp + self.names["down"], (self.hidden, self.shared_size), "matrix")]
        return specs

    def bind(self, tensors, runtime: Runtime, shared=None):
        mats = [tensors[self._e(e, w)] for e in range(self.n_experts) for w in ("gate", "up", "down")]
        if len({m.dtype for m in mats}) != 1:
            mats = [m.to(torch.float32) for m in mats]
        gu = [torch.cat([mats[3 * e], mats[3 * e + 1]], dim=0) for e in range(self.n_experts)]
        self.w_gate_up = torch.stack(gu).contiguous()                                       # [E, 2F, W]
        self.w_down = torch.stack([mats[3 * e + 2] for e in range(self.n_experts)]).contiguous()   # [E, W, F]
        if self.shared_size:
            sp = self.prefix + self.names["shared"]
            g, u = tensors[sp + self.names["gate"]], tensors[sp + self.names["up"]]
            if g.dtype != u.dtype:
                g, u = g.to(torch.float32), u.to(torch.float32)
            self.w_shared_gate_up = torch.cat([g, u], dim=0).contiguous()
            self.w_shared_down = tensors[sp + self.names["down"]].contiguous()
        if self.routing == "router":
            self.w_router = tensors[self.prefix + self.names["router"]].contiguous()
            return
        table = tensors[self.prefix + self.names["table"]]
        if table.dtype != torch.int32:
            raise ConfigError(f"routed experts: the table {self.prefix + self.names['table']} must hold integers")
        lo, hi = int(table.min()), int(table.max())
        if lo < 0 or hi >= self.n_experts:
            raise ConfigError(f"routed experts: the table names experts {lo} .. {hi}; there are {self.n_experts}")
        self.table = table.contiguous()

    def forward(self, x, ctx: StepContext, residual):
        weights = None
        if self.routing == "table":
            choice = kernels.table_choice(ctx.batch.tokens, self.table, self.n_experts)
        else:
            logits = kernels.linear(x, self.w_router, out_dtype=torch.float32)
            choice, weights = kernels.router_choice(logits, self.top, self.router_scale, self.weight_sum_floor)
        T = x.shape[0]
        if ((T >= self.TILE_MIN_ROWS or T * self.top >= self.TILE_MIN_PAIRS_PER_EXPERT * self.n_experts)
                and x.dtype == torch.bfloat16 and kernels.routed_tiles_ok(x, self.w_gate_up, self.w_down)):
            kernels.routed_experts_tiles(x, self.w_gate_up, self.w_down, choice, residual,
                                         accumulate=not ctx.store_result, weights=weights)
        else:
            kernels.routed_experts_rows(x, self.w_gate_up, self.w_down, choice, residual,
                                        accumulate=not ctx.store_result, weights=weights)
        kernels.mark("experts")
        if self.shared_size:
            act = kernels.linear(x, self.w_shared_gate_up, swiglu=True, out_dtype=ctx.runtime.act_dtype)
            kernels.linear(act, self.w_shared_down, out=residual, accumulate=True)
            kernels.mark("shared_expert")
