"""Typed configuration of the Furesun decoder and the builder that turns it
into a `ModelSpec` of parts.

A Furesun config.json names its architecture with the key `architecture`, its
sizes with `vocab` and `width`, the norm's `eps` under `norm`, an optional
`logit_softcap`, and lists its layers one by one: every layer gives its `type`
(which mixer it has), the mixer's sizes and constants under `mixer`, and its
feed-forward under `mlp` (null: the layer has only the mixer).  Layers of
different types may follow one another in any order.

A layer norms what its sublayers give, not what they read:
    x <- x + norm1(mixer(x));   x <- x + norm2(ff(x))          (block kind `postnorm_residual`)

Mixers:
  latent_attention   parts/latent_attention.py: queries projected directly, keys and values
                     from one cached latent per token with a rotated key part shared by the
                     heads (halves layout, rates optionally stretched), a sliding window
  mlstm              parts/mlstm.py: a matrix memory per head with exponential input and
                     forget gates, a running maximum that keeps the exponentials in range
  attention          parts/softmax_attention.py: grouped heads; q and k RMS-normed over
                     their whole projections (weights `q.norm`, `k.norm`), rotated in
                     neighbouring pairs; capped scores; a sliding window; a softmax with a
                     sink (one added to the denominator).  With `kv_from: j` the layer has
                     no key/value tensors and reads what layer j cached.
Feed-forward:
  dense              W_down (gelu_tanh(W_gate x) * (W_up x))
  moe                parts/routed_experts.py with `routing: "router"`: scores
                     sigmoid(W_router x), the `top` largest chosen, their scores over their
                     sum times `router.scale` as weights; SwiGLU experts; a shared expert
                     (`shared.ff`) added for every token.

The head is a matrix of its own (`head`).  Positions have no limit by design;
`max_positions` (optional, default 32,768) bounds the cache an engine plans for.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from .model_spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .pavisun import RotationConfig, _optional_float
from .zodosun import _need, _optional_int, _positive

ARCHITECTURE = "Furesun"
MODEL_TYPE = "furesun"
DEFAULT_MAX_POSITIONS = 32768
WEIGHT_SUM_FLOOR = 1e-20         # fixed by the design: a token's expert weights are its scores over (their sum + this)
MEMORY_READ_FLOOR = 1e-6         # fixed by the design: added to the divisor of the matrix memory's read

_MIXERS = ("latent_attention", "mlstm", "attention")


def _window(d: dict, where: str) -> Optional[int]:
    return _optional_int(d.get("mask") or {}, "size", where + ".mask")


@dataclass(frozen=True)
class LatentConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotationConfig
    window: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "LatentConfig":
        c = cls(heads=_need(d, "heads", int, where), dim=_need(d, "dim", int, where),
                rot_dim=_need(d, "rot_dim", int, where), vdim=_need(d, "vdim", int, where),
                kv_rank=_need(d, "kv_rank", int, where), scale=_need(d, "scale", float, where),
                rot=RotationConfig.from_dict(_need(d, "rot", dict, where), where + ".rot"), window=_window(d, where))
        _positive(where, heads=c.heads, dim=c.dim, rot_dim=c.rot_dim, vdim=c.vdim, kv_rank=c.kv_rank)
        if c.rot.dims > c.rot_dim:
            raise ConfigError(f"config.json: {where}: rot.dims {c.rot.dims} exceeds the rotated part's {c.rot_dim} entries")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "rot": self.rot.to_dict(),
                             "rot_dim": self.rot_dim, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class MemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "MemoryConfig":
        c = cls(heads=_need(d, "heads", int, where), dim=_need(d, "dim", int, where), vdim=_need(d, "vdim", int, where),
                gate_cap=_need(d, "gate_cap", float, where))
        _positive(where, heads=c.heads, dim=c.dim, vdim=c.vdim, gate_cap=c.gate_cap)
        return c

    def to_dict(self) -> dict:
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: RotationConfig
    softcap: Optional[float] = None
    window: Optional[int] = None
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "AttentionConfig":
        c = cls(heads=_need(d, "heads", int, where), kv_heads=_need(d, "kv_heads", int, where),
                dim=_need(d, "dim", int, where), vdim=_need(d, "vdim", int, where),
                scale=_need(d, "scale", float, where),
                rot=RotationConfig.from_dict(_need(d, "rot", dict, where), where + ".rot"),
                softcap=_optional_float(d, "softcap", where), window=_window(d, where),
                kv_from=None if d.get("kv_from") is None else _need(d, "kv_from", int, where))
        _positive(where, heads=c.heads, kv_heads=c.kv_heads, dim=c.dim, vdim=c.vdim)
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}: {c.heads} heads cannot share {c.kv_heads} key/value heads")
        if c.rot.dims > c.dim:
            raise ConfigError(f"config.json: {where}: rot.dims {c.rot.dims} exceeds the head's {c.dim} entries")
        return c

    def to_dict(self) -> dict:
        d: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "rot": self.rot.to_dict(),
                             "scale": self.scale, "vdim": self.vdim}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.softcap is not None:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class FeedForwardConfig:
    """`kind` dense: `ff`.  `kind` moe: `ff` is an expert's inner width, with `experts`, `top`, `scale` and the
    shared expert's inner width `shared_ff` (0: none)."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    scale: float = 1.0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, d: dict, where: str) -> "FeedForwardConfig":
        kind = _need(d, "kind", str, where)
        if kind == "dense":
            c = cls(kind, _need(d, "ff", int, where))
            _positive(where, ff=c.ff)
            return c
        if kind != "moe":
            raise ConfigError(f"config.json: {where}: unknown kind '{kind}' (known: dense, moe)")
        router = _need(d, "router", dict, where)
        shared = d.get("shared")
        c = cls(kind, _need(_need(d, "expert", dict, where), "ff", int, where + ".expert"),
                experts=_need(router, "experts", int, where + ".router"), top=_need(router, "top", int, where + ".router"),
                scale=_need(router, "scale", float, where + ".router"),
                shared_ff=0 if shared is None else _need(shared, "ff", int, where + ".shared"))
        _positive(where, ff=c.ff, experts=c.experts, top=c.top)
        if c.top > c.experts:
            raise ConfigError(f"config.json: {where}: a token cannot use {c.top} of {c.experts} experts")
        if shared is not None:
            _positive(where + ".shared", ff=c.shared_ff)
        return c

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        d: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe",
                             "router": {"experts": self.experts, "scale": self.scale, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


_MIXER_CONFIGS = {"latent_attention": LatentConfig, "mlstm": MemoryConfig, "attention": AttentionConfig}


@dataclass(frozen=True)
class FuresunLayer:
    type: str
    mixer: Any
    mlp: Optional[FeedForwardConfig]

    @classmethod
    def from_dict(cls, d: dict, index: int) -> "FuresunLayer":
        where = f"layers[{index}]"
        typ = _need(d, "type", str, where)
        if typ not in _MIXERS:
            raise ConfigError(f"config.json: {where}: unknown layer type '{typ}' (known: {sorted(_MIXERS)})")
        mixer = _MIXER_CONFIGS[typ].from_dict(_need(d, "mixer", dict, where), where + ".mixer")
        mlp = d.get("mlp")
        return cls(typ, mixer, None if mlp is None else FeedForwardConfig.from_dict(mlp, where + ".mlp"))

    def to_dict(self) -> dict:
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class FuresunConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[FuresunLayer, ...]
    logit_softcap: Optional[float] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    torch_dtype: str = "bfloat16"
    stop_token_ids: tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "FuresunConfig":
        top = "the top level"
        norm = _need(d, "norm", dict, top)
        layers = _need(d, "layers", list, top)
        if not layers:
            raise ConfigError("config.json: 'layers' is empty")
        cfg = cls(
            vocab=_need(d, "vocab", int, top),
            width=_need(d, "width", int, top),
            norm_eps=_need(norm, "eps", float, "norm"),
            layers=tuple(FuresunLayer.from_dict(l, i) for i, l in enumerate(layers)),
            logit_softcap=_optional_float(d, "logit_softcap", top),
            max_positions=_optional_int(d, "max_positions", top) or DEFAULT_MAX_POSITIONS,
            torch_dtype=d.get("torch_dtype") or "bfloat16",
            stop_token_ids=tuple(int(t) for t in (d.get("stop_token_ids") or ())),
        )
        _positive(top, vocab=cfg.vocab, width=cfg.width)
        if not cfg.norm_eps > 0.0:
            raise ConfigError("config.json: norm.eps must be positive")
        for i, layer in enumerate(cfg.layers):
            if layer.type != "attention" or layer.mixer.kv_from is None:
                continue
            m, j = layer.mixer, layer.mixer.kv_from
            where = f"layers[{i}].mixer"
            if not 0 <= j < i or cfg.layers[j].type != "attention" or cfg.layers[j].mixer.kv_from is not None:
                raise ConfigError(f"config.json: {where}: kv_from {j} must name an earlier attention layer with keys "
                                  f"and values of its own")
            o = cfg.layers[j].mixer
            if (o.kv_heads, o.dim, o.vdim, o.rot) != (m.kv_heads, m.dim, m.vdim, m.rot):
                raise ConfigError(f"config.json: {where}: the keys and values of layer {j} ({o.kv_heads} heads of "
                                  f"{o.dim} / {o.vdim}, rot {o.rot.to_dict()}) do not fit this layer's")
        return cfg

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architecture": ARCHITECTURE,
            "layers": [l.to_dict() for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
            "torch_dtype": self.torch_dtype,
        }
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.stop_token_ids:
            d["stop_token_ids"] = list(self.stop_token_ids)
        return d


def _rotation(rot: RotationConfig, layout: str) -> PartSpec:
    params: dict[str, Any] = {"rotary_dim": rot.dims, "theta": rot.base, "layout": layout}
    if rot.scaling is not None:
        f, o, fast, slow = rot.scaling
        params["scaling"] = {"factor": f, "original": o, "fast": fast, "slow": slow}
    return PartSpec("rotary_tables", params)


def _mixer(cfg: FuresunConfig, index: int, prefix: str) -> PartSpec:
    layer = cfg.layers[index]
    m = layer.mixer
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": cfg.width, "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
            "q_rank": None, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "window": m.window,
            "position": _rotation(m.rot, "halves"),
            "names": {"q": "q", "kv_down": "dkv", "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "out": "o"}}, prefix)
    if layer.type == "mlstm":
        return PartSpec("mlstm_mixer", {
            "hidden_size": cfg.width, "heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "gate_cap": m.gate_cap,
            "eps": cfg.norm_eps, "read_floor": MEMORY_READ_FLOOR,
            "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "input": "i", "input_bias": "i.b", "forget": "f",
                      "forget_bias": "f.b", "norm": "norm", "out": "o"}}, prefix)
    # The cache of a layer whose keys other layers read keeps the widest window among them (all keys if one has none).
    windows = [m.window] + [l.mixer.window for l in cfg.layers
                            if l.type == "attention" and l.mixer.kv_from == index]
    cache_window = None if any(w is None for w in windows) else max(windows)
    return PartSpec("softmax_attention", {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim,
        "value_dim": m.vdim, "scale": m.scale, "softcap": m.softcap, "window": m.window, "cache_window": cache_window,
        "values": "projected", "row_norm_eps": cfg.norm_eps, "sink": True, "shared_kv": m.kv_from is not None,
        "shares_packed": len(windows) > 1,
        "position": _rotation(m.rot, "pairs"),
        "names": {"q": "q", "k": "k", "v": "v", "out": "o", "q_norm": "q.norm", "k_norm": "k.norm"}}, prefix)


def _feed_forward(cfg: FuresunConfig, f: FeedForwardConfig, prefix: str) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": f.ff, "activation": "gelu_tanh",
                                   "names": {"gate": "gate", "up": "up", "down": "down"}, "weight_suffix": ""}, prefix)
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "intermediate_size": f.ff, "experts": f.experts, "top": f.top, "routing": "router",
        "router_scale": f.scale, "weight_sum_floor": WEIGHT_SUM_FLOOR, "shared_size": f.shared_ff,
        "names": {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "router": "router",
                  "shared": "shared."}}, prefix)


def build_furesun_spec(cfg: FuresunConfig) -> ModelSpec:
    """Furesun as parts: token embedding; per layer a block that norms its sublayers' results (mixer, RMS norm,
    feed-forward, RMS norm); a layer with `kv_from` reads the cache of the schedule entry of the layer it names;
    RMS norm; a head of its own with capped logits."""
    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", {"width": cfg.width, "eps": cfg.norm_eps, "weight_name": name})

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = _feed_forward(cfg, layer.mlp, p + "mlp.")
            ffn_norm = norm(p + "norm2")
        layers.append(LayerSpec(block="postnorm_residual", mixer=_mixer(cfg, i, p + "mix."), feed_forward=ffn,
                                mixer_norm=norm(p + "norm1"), feed_forward_norm=ffn_norm))
        schedule.append(ScheduleEntry(i, layer.mixer.kv_from if layer.type == "attention" else None))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "width": cfg.width, "weight_name": "embed"}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "width": cfg.width, "weight_name": "head",
                                  "logit_softcap": cfg.logit_softcap}),
        stop_token_ids=cfg.stop_token_ids,
    )
    spec.validate()
    return spec
