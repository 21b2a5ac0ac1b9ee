"""Token embedding and LM head.

Reference: src/models/turbo_generic.rs:1958 — embedding is a row gather
without scaling; :1983-1986 — final norm, then logits = n · W^T without bias
or scaling, for the wanted rows only; :2079-2084 — the head uses
`lm_head.weight` if the checkpoint has it and the embedding matrix otherwise
(here the configuration decides which).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Part, Runtime, WeightSpec


class TokenEmbedding(Part):
    padded_rows_ok = True               # row by row

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.width = int(self.params["width"])
        self.weight_name = self.params.get("weight_name") or self.prefix + "weight"
        # sinusoidal positions added to the rows: column 2i gets sin(p * base^(-2i / width)), column 2i+1 its cosine
        self.sinusoid_base = self.params.get("sinusoid_base")
        self.wants_positions = self.sinusoid_base is not None
        self.scale = float(self.params.get("scale", 1.0))      # the rows are multiplied by it
        self.table = None
        self.rate = None
        self.status = None

    def weight_specs(self):
        return [WeightSpec(self.weight_name, (self.vocab, self.width), "embedding")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.table = tensors[self.weight_name].contiguous()
        self.status = torch.zeros(1, dtype=torch.int32, device=runtime.device)
        if self.wants_positions:
            i = torch.arange((self.width + 1) // 2, dtype=torch.float64)
            rate = torch.pow(torch.tensor(float(self.sinusoid_base), dtype=torch.float64), -2.0 * i / self.width)
            self.rate = rate.to(torch.float32).to(runtime.device)

    def forward(self, tokens: torch.Tensor, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The float32 residual stream [T, width] of the step's tokens (`positions`: each token's place in its
        sequence, for an embedding that adds positions)."""
        out = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        if self.wants_positions:
            if positions is None:
                raise kernels.KernelError("this embedding adds positions and was given none")
            if self.scale != 1.0:
                raise kernels.KernelError("an embedding that adds positions has no scale")
            return kernels.embed_sinusoid(tokens, positions, self.table, self.rate, out, self.status)
        return kernels.embed(tokens, self.table, out, self.status, self.scale)


class LMHead(Part):
    padded_rows_ok = True               # row by row

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.width = int(self.params["width"])
        self.tied_to = self.params.get("tied_to")
        self.weight_name = self.params.get("weight_name") or self.prefix + "weight"
        self.logit_scale = float(self.params.get("logit_scale", 1.0))     # the logits are multiplied by it
        cap = self.params.get("logit_softcap")                            # then capped: cap * tanh(logits / cap)
        self.logit_softcap = float(cap) if cap else None
        self.weight = None

    def weight_specs(self):
        if self.tied_to:
            return [WeightSpec(self.tied_to, (self.vocab, self.width), "embedding")]
        return [WeightSpec(self.weight_name, (self.vocab, self.width), "matrix")]

    def ignored_weights(self):
        return [self.weight_name] if self.tied_to else []

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.weight = tensors[self.tied_to or self.weight_name].contiguous()

    def forward(self, normed_rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [rows, vocab] of already normed rows."""
        logits = kernels.linear(normed_rows, self.weight, out_dtype=torch.float32)
        if self.logit_scale != 1.0:
            kernels.scale_inplace(logits, self.logit_scale)
        if self.logit_softcap is not None:
            kernels.tanh_cap(logits, self.logit_softcap)
        return logits
