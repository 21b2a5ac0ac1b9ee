"""A residual stream kept as several parallel streams (hyper-connections), and the layer arrangement that
works on them.

Instead of one x there are S copies x_1 .. x_S, all equal to the embedding at the start.  Sublayer q of a layer
(1: the mixer, 2: the feed-forward) has three small tensors, `<layer>hc<q>.in` [S], `.out` [S] and `.mix`
[S, S] (indexed [from, to]):

    u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_r <- sum_s mix[s, r] x_s + out[r] y   (all r at once).

At the end the model reads the sum of the streams.  The streams are float32 and every sum is float32.

`ResidualStreams` holds the streams [S, T, W] and what the last sublayer still has to write.  The write is put off
until the next reader comes, so that one kernel per sublayer boundary does the write, the next read and the
norm on it (csrc/stream_mix.cu): a layer of two sublayers costs two launches, as many as the two norms of a
plain pre-norm layer.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config import ConfigError, LayerSpec
from .base import Part, Runtime, StepContext, WeightSpec, float32_vector
from .registry import make_part


class ResidualStreams:
    def __init__(self, x: torch.Tensor, n_streams: int):
        self.xs = kernels.streams_fill(x, n_streams)
        self.n_streams = n_streams
        self._pending = None                          # (y, mix, write) of the sublayer that ran last
        self._ones: Optional[torch.Tensor] = None

    def write_later(self, y: torch.Tensor, mix: torch.Tensor, write: torch.Tensor) -> None:
        if self._pending is not None:
            self.flush()
        self._pending = (y, mix, write)

    def read(self, coefs: torch.Tensor, norm_weight: Optional[torch.Tensor], eps: float, out_dtype,
             rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """sum_s coefs[s] x_s (after the write that is still due), normed if a weight is given; `rows`: of these
        tokens only — the streams are then left without the due write (it is applied on the way to the result
        only), so nothing may read them afterwards."""
        y, mix, write = self._pending or (None, None, None)
        self._pending = None
        return kernels.streams_step(self.xs, y=y, mix=mix, write=write, read=coefs, norm_weight=norm_weight, eps=eps,
                                    out_dtype=out_dtype, rows=rows)

    def read_sum(self, norm_weight, eps, out_dtype, rows=None) -> torch.Tensor:
        if self._ones is None:
            self._ones = torch.ones(self.n_streams, dtype=torch.float32, device=self.xs.device)
        return self.read(self._ones, norm_weight, eps, out_dtype, rows)

    def flush(self) -> None:
        if self._pending is not None:
            y, mix, write = self._pending
            self._pending = None
            kernels.streams_step(self.xs, y=y, mix=mix, write=write)

    def total(self) -> torch.Tensor:
        """The sum of the streams, float32 [T, W] (for whoever wants to look at the residual stream)."""
        return self.read_sum(None, 0.0, torch.float32)


class StreamConnection(Part):
    """The three tensors of one sublayer's connection to the streams."""
    padded_rows_ok = True

    def __init__(self, spec):
        super().__init__(spec)
        self.n_streams = int(self.params["streams"])
        if not 1 <= self.n_streams <= kernels.streams.MAX_STREAMS:
            raise ConfigError(f"a residual of {self.n_streams} streams (1 to {kernels.streams.MAX_STREAMS})")
        self.names = dict(self.params.get("names", {"read": "in", "write": "out", "mix": "mix"}))
        self.read = self.write = self.mix = None

    def weight_specs(self):
        S = self.n_streams
        return [WeightSpec(self.prefix + self.names["read"], (S,), "stream_read"),
                WeightSpec(self.prefix + self.names["write"], (S,), "stream_write"),
                WeightSpec(self.prefix + self.names["mix"], (S, S), "stream_mix")]

    def bind(self, tensors, runtime: Runtime, shared=None):
        self.read = float32_vector(tensors[self.prefix + self.names["read"]])
        self.write = float32_vector(tensors[self.prefix + self.names["write"]])
        self.mix = tensors[self.prefix + self.names["mix"]].to(torch.float32).contiguous()


class StreamsBlock:
    """Pre-norm layer on parallel residual streams (kind `residual_streams`): the mixer's sublayer, then — unless
    the layer has none — the feed-forward's, each with a connection of its own (parts `mixer_streams`,
    `feed_forward_streams`).  The norms must be plain RMS norms (their weight and eps go into the streams'
    kernel)."""
    padded_rows_ok = True               # as far as its parts are

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.mixer_norm = make_part(spec.part("mixer_norm"))
        self.mixer = make_part(spec.part("mixer"))
        self.mixer_streams = make_part(spec.part("mixer_streams"))
        self.feed_forward = self.feed_forward_norm = self.feed_forward_streams = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = make_part(spec.part("feed_forward_norm"))
            self.feed_forward = make_part(spec.part("feed_forward"))
            self.feed_forward_streams = make_part(spec.part("feed_forward_streams"))
        for n in (self.mixer_norm, self.feed_forward_norm):
            if n is not None and (getattr(n, "groups", 1) != 1 or not hasattr(n, "eps")):
                raise ConfigError("a layer on residual streams takes plain RMS norms")

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_streams, self.feed_forward_norm,
                            self.feed_forward, self.feed_forward_streams) if p is not None]

    def forward(self, h: ResidualStreams, ctx: StepContext) -> None:
        if not isinstance(h, ResidualStreams):
            raise kernels.KernelError("a layer of kind 'residual_streams' runs in a model that keeps streams")
        self._sublayer(h, ctx, self.mixer_norm, self.mixer, self.mixer_streams)
        if self.feed_forward is not None:
            self._sublayer(h, ctx, self.feed_forward_norm, self.feed_forward, self.feed_forward_streams)

    @staticmethod
    def _sublayer(h: ResidualStreams, ctx: StepContext, norm, part, conn) -> None:
        x = h.read(conn.read, norm.weight, norm.eps, ctx.runtime.act_dtype)
        kernels.mark("norms")
        store = bool(getattr(part, "can_store_result", False))
        y = (torch.empty if store else torch.zeros)(h.xs.shape[1:], dtype=torch.float32, device=h.xs.device)
        ctx.store_result = store
        try:
            part.forward(x, ctx, y)
        finally:
            ctx.store_result = False
        h.write_later(y, conn.mix, conn.write)
