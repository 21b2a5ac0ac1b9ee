"""Typed configuration of the Pavisun decoder and the builder that turns it
into a `ModelSpec` of parts.

A Pavisun config.json names its architecture with the key `architecture`, its
sizes with `vocab` and `width`, the norm's `eps` under `norm`, and lists its
layers one by one: every layer gives its `type` (which mixer it has), the
mixer's sizes and constants under `mixer`, and its feed-forward under `mlp`
(null: the layer has only the mixer).  Layers of different types may follow one
another in any order.

  streams         S > 0: the residual stream is S parallel streams and every
                  sublayer reads and writes them through three small tensors
                  (parts/residual_streams.py); absent: the plain pre-norm sums
  loop            {start, stop, times}: layers start .. stop-1 run `times` times in
                  a row with the same weights (each run has a cache of its own), then
                  the rest follow
  logit_softcap   c: logits <- c * tanh(logits / c)

Mixers (both are parts/softmax_attention.py with other options):
  attention     q and k rotated over their first rot.dims entries (halves layout,
                rates optionally stretched: rot.scaling), the values are the keys as
                projected, scores capped by `softcap`, a sliding window mask.size
  attention_2   q, k and v projected, q and k divided per head by their root mean
                square (the layer's eps), a bias slope_h * (i - j) taken off the
                scores, slope_h = 2^(-8 (h + 1) / heads), a sliding window that also
                keeps the first mask.keep_first tokens, a sigmoid gate on the heads
Feed-forward (parts/routed_experts.py): `router.experts` small SwiGLU layers of
inner width `expert.ff`; a table indexed by the token id names the `router.top`
experts of a token, each weighted 1 / top.

The head is a matrix of its own (`head`).  Positions have no limit by design;
`max_positions` (optional, default 32,768) bounds the cache an engine plans for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .model_spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .zodosun import _need, _optional_int, _positive

ARCHITECTURE = "Pavisun"
MODEL_TYPE = "pavisun"
DEFAULT_MAX_POSITIONS = 32768
SLOPE_EXPONENT = 8.0             # fixed by the design: head h's slope is 2^(-8 (h + 1) / heads)


def _optional_count(d: dict, key: str, where: str) -> int:
    """An integer >= 0; absent counts as 0."""
    if d.get(key) is None:
        return 0
    v = _need(d, key, int, where)
    if v < 0:
        raise ConfigError(f"config.json: {where}: '{key}' must not be negative, found {v}")
    return v


def _optional_float(d: dict, key: str, where: str) -> Optional[float]:
    if d.get(key) is None:
        return None
    v = _need(d, key, float, where)
    _positive(where, **{key: v})
    return v


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: Optional[tuple[float, float, float, float]] = None     # factor, original, fast, slow

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "RotationConfig":
        sc = d.get("scaling")
        scaling = None
        if sc is not None:
            w = where + ".scaling"
            scaling = (_need(sc, "factor", float, w), _need(sc, "original", float, w), _need(sc, "fast", float, w),
                       _need(sc, "slow", float, w))
            _positive(w, factor=scaling[0], original=scaling[1], fast=scaling[2], slow=scaling[3])
        c = cls(base=_need(d, "base", float, where), dims=_need(d, "dims", int, where), scaling=scaling)
        _positive(where, base=c.base, dims=c.dims)
        if c.dims % 2:
            raise ConfigError(f"config.json: {where}: dims {c.dims} must be even")
        if not c.base > 1.0:
            raise ConfigError(f"config.json: {where}: base {c.base} must be above 1")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            f, o, fast, slow = self.scaling
            d["scaling"] = {"factor": f, "fast": fast, "original": int(o) if float(o).is_integer() else o,
                            "slow": slow}
        return d


@dataclass(frozen=True)
class AttentionConfig:
    """Sizes and constants of either mixer; `kind` is the layer's type."""
    kind: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    keep_first: int = 0
    softcap: Optional[float] = None
    rot: Optional[RotationConfig] = None

    @classmethod
    def from_dict(cls, d: dict, where: str, kind: str) -> "AttentionConfig":
        mask = d.get("mask") or {}
        rot = None
        softcap = None
        keep_first = 0
        if kind == "attention":
            rot = RotationConfig.from_dict(_need(d, "rot", dict, where), where + ".rot")
            softcap = _optional_float(d, "softcap", where)
        else:
            keep_first = _optional_count(mask, "keep_first", where + ".mask")
        c = cls(kind=kind, heads=_need(d, "heads", int, where), kv_heads=_need(d, "kv_heads", int, where),
                dim=_need(d, "dim", int, where), vdim=_need(d, "vdim", int, where),
                scale=_need(d, "scale", float, where), window=_optional_int(mask, "size", where + ".mask"),
                keep_first=keep_first, softcap=softcap, rot=rot)
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads cannot share {c.kv_heads} key/value heads")
        if kind == "attention" and c.vdim != c.dim:
            raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {c.vdim} must equal dim {c.dim}")
        if rot is not None and rot.dims > c.dim:
            raise ConfigError(f"config.json: {where}: rot.dims {rot.dims} exceeds the head's {c.dim} entries")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
                             "vdim": self.vdim}
        mask: dict[str, Any] = {}
        if self.window is not None:
            mask["size"] = self.window
        if self.keep_first:
            mask["keep_first"] = self.keep_first
        if mask:
            d["mask"] = mask
        if self.softcap is not None:
            d["softcap"] = self.softcap
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


_MIXERS = ("attention", "attention_2")


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "ExpertsConfig":
        kind = _need(d, "kind", str, where)
        if kind != "moe":
            raise ConfigError(f"config.json: {where}: unknown kind '{kind}' (known: moe)")
        router = _need(d, "router", dict, where)
        c = cls(ff=_need(_need(d, "expert", dict, where), "ff", int, where + ".expert"),
                experts=_need(router, "experts", int, where + ".router"),
                top=_need(router, "top", int, where + ".router"))
        _positive(where, ff=c.ff, experts=c.experts, top=c.top)
        if c.top > c.experts:
            raise ConfigError(f"config.json: {where}: a token cannot use {c.top} of {c.experts} experts")
        return c

    def to_dict(self) -> dict:
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class PavisunLayer:
    type: str
    mixer: AttentionConfig
    mlp: Optional[ExpertsConfig]

    @classmethod
    def from_dict(cls, d: dict, index: int) -> "PavisunLayer":
        where = f"layers[{index}]"
        typ = _need(d, "type", str, where)
        if typ not in _MIXERS:
            raise ConfigError(f"config.json: {where}: unknown layer type '{typ}' (known: {sorted(_MIXERS)})")
        mixer = AttentionConfig.from_dict(_need(d, "mixer", dict, where), where + ".mixer", typ)
        mlp = d.get("mlp")
        return cls(typ, mixer, None if mlp is None else ExpertsConfig.from_dict(mlp, where + ".mlp"))

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class PavisunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[PavisunLayer, ...]
    streams: int = 0
    loop: Optional[tuple[int, int, int]] = None          # start, stop, times
    logit_softcap: Optional[float] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    torch_dtype: str = "bfloat16"
    stop_token_ids: tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "PavisunConfig":
        top = "the top level"
        norm = _need(d, "norm", dict, top)
        layers = _need(d, "layers", list, top)
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        loop = None
        if d.get("loop") is not None:
            lp = _need(d, "loop", dict, top)
            loop = (_need(lp, "start", int, "loop"), _need(lp, "stop", int, "loop"), _need(lp, "times", int, "loop"))
            if not (0 <= loop[0] <= loop[1] <= len(layers)) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {lp} does not fit {len(layers)} layers (0 <= start <= stop <= "
                                  f"layers, times >= 1)")
        cfg = cls(
            vocab=_need(d, "vocab", int, top),
            width=_need(d, "width", int, top),
            norm_eps=_need(norm, "eps", float, "norm"),
            layers=tuple(PavisunLayer.from_dict(l, i) for i, l in enumerate(layers)),
            streams=_optional_count(d, "streams", top),
            loop=loop,
            logit_softcap=_optional_float(d, "logit_softcap", top),
            max_positions=_optional_int(d, "max_positions", top) or DEFAULT_MAX_POSITIONS,
            torch_dtype=d.get("torch_dtype") or "bfloat16",
            stop_token_ids=tuple(int(t) for t in (d.get("stop_token_ids") or ())),
        )
        _positive(top, vocab=cfg.vocab, width=cfg.width)
        if not cfg.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cfg

    def order(self) -> list[int]:
        """The layers in the order they run (a looped layer is named once per run)."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "layers": [l.to_dict() for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }
        if self.streams:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.stop_token_ids:
            d["stop_token_ids"] = list(self.stop_token_ids)
        return d


_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}


def _mixer(cfg: PavisunConfig, m: AttentionConfig, prefix: str) -> PartSpec:
    params: dict[str, Any] = {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim,
        "value_dim": m.vdim, "scale": m.scale, "window": m.window, "keep_first": m.keep_first, "names": dict(_NAMES),
    }
    if m.kind == "attention":
        params.update(values="keys", softcap=m.softcap)
        if m.rot is not None:
            rot: dict[str, Any] = {"rotary_dim": m.rot.dims, "theta": m.rot.base, "layout": "halves"}
            if m.rot.scaling is not None:
                f, o, fast, slow = m.rot.scaling
                rot["scaling"] = {"factor": f, "original": o, "fast": fast, "slow": slow}
            params["position"] = PartSpec("rotary_tables", rot)
    else:
        params.update(values="projected", qk_norm_eps=cfg.norm_eps, slope_exponent=SLOPE_EXPONENT, output_gate=True)
    return PartSpec("softmax_attention", params, prefix)


def build_pavisun_spec(cfg: PavisunConfig) -> ModelSpec:
    """Pavisun as parts: token embedding; per layer a block on residual streams (or, without streams, the plain
    pre-norm block) of {RMS norm, softmax attention with the layer's options, RMS norm, experts named by a
    table}; the schedule repeats the looped layers, every run with a cache of its own; RMS norm; a head of its
    own with capped logits."""
    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", {"width": cfg.width, "eps": cfg.norm_eps, "weight_name": name})

    def connection(prefix: str) -> PartSpec:
        return PartSpec("stream_connection", {"streams": cfg.streams,
                                              "names": {"read": "in", "write": "out", "mix": "mix"}}, prefix)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ffn = ffn_norm = None
        extra: dict[str, PartSpec] = {}
        if layer.mlp is not None:
            ffn = PartSpec("table_experts", {
                "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "experts": layer.mlp.experts,
                "top": layer.mlp.top, "vocab_size": cfg.vocab, "routing": "table",
                "names": {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "table": "table"}}, p + "mlp.")
            ffn_norm = norm(p + "norm2")
        if cfg.streams:
            extra["mixer_streams"] = connection(p + "hc1.")
            if ffn is not None:
                extra["feed_forward_streams"] = connection(p + "hc2.")
        layers.append(LayerSpec(block="residual_streams" if cfg.streams else "prenorm_residual",
                                mixer=_mixer(cfg, layer.mixer, p + "mix."), feed_forward=ffn,
                                mixer_norm=norm(p + "norm1"), feed_forward_norm=ffn_norm, extra_parts=extra))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "width": cfg.width, "weight_name": "embed"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in cfg.order()),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "width": cfg.width, "weight_name": "head",
                                  "logit_softcap": cfg.logit_softcap}),
        stop_token_ids=cfg.stop_token_ids,
        residual_streams=cfg.streams,
    )
    spec.validate()
    return spec
