"""Plain, slow implementation of the Pavisun decoder: whole sequences, no
cache, one function per mechanism.  Nothing is imported from the product
package.  All math is done in the dtype asked for (float64 by default: the
anchor the product's float32 and bfloat16 paths are measured against).

Notation: T tokens, W model width, S residual streams, H query heads, G
key/value heads, d key width per head, e value width per head, sigma(z) =
1 / (1 + exp(-z)).  Position i may read position j <= i.
"""
from __future__ import annotations

import math

import torch

from plain_zodosun import read_folder, write_folder  # noqa: F401  (the file format is the same)


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def tanh_cap(z, cap):
    """cap * tanh(z / cap): close to z for small |z|, never beyond +-cap."""
    return cap * torch.tanh(z / cap)


def stretched_rates(dims: int, base: float, scaling) -> tuple[torch.Tensor, float]:
    """The rotation rates of the dims/2 pairs and the factor on cosine and sine.  Without `scaling` the rates
    are base^(-2i/dims) and the factor is 1.  With scaling (factor F, original length L, turn counts `fast` and
    `slow`): a pair that turns t times over L positions has index n(t) = dims ln(L / (2 pi t)) / (2 ln base);
    pairs below lo = max(floor(n(fast)), 0) keep their rate, pairs above hi = min(ceil(n(slow)), dims - 1) are
    slowed by F, and between them the share r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) of the slowed rate
    is mixed in; cosine and sine grow by 0.1 ln F + 1."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    F, L = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(L / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / F * r + f * (1.0 - r), 0.1 * math.log(F) + 1.0


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, scaling=None) -> torch.Tensor:
    """x [T, heads, n]: entry i < dims/2 of a head is paired with entry i + dims/2; the pair (a, b) at position p
    becomes m (a cos t - b sin t, b cos t + a sin t), t = p * rate_i; entries from `dims` on pass."""
    half = dims // 2
    rate, m = stretched_rates(dims, base, scaling)
    ang = positions.to(torch.float64).reshape(-1, 1, 1) * rate
    c, s = (torch.cos(ang) * m).to(x.dtype), (torch.sin(ang) * m).to(x.dtype)
    out = x.clone()
    a, b = x[..., :half], x[..., half:dims]
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def visible(T: int, window, keep_first: int = 0) -> torch.Tensor:
    """[T, T] bool: i reads j iff j <= i and (i - j < window or j < keep_first); no window: every j <= i."""
    i = torch.arange(T).reshape(-1, 1)
    j = torch.arange(T).reshape(1, -1)
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def head_slopes(H: int, dtype) -> torch.Tensor:
    """2^(-8 (h + 1) / H) for h = 0 .. H-1."""
    return torch.pow(torch.tensor(2.0, dtype=dtype), -8.0 * (torch.arange(H, dtype=dtype) + 1.0) / H)


_round = lambda t: t          # set by decoder(rounding=...) for its own run: what a 16-bit engine rounds


def softmax_heads(q, k, v, scale, mask, *, cap=None, slopes=None) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H * e].  Query head h reads key head h // (H / G).
    score[i, j] = q_i . k_j * scale, then cap * tanh(score / cap) if a cap is given, then minus
    slopes[h] * (i - j) if slopes are given; softmax over the visible j."""
    T, H, _ = q.shape
    G = k.shape[1]
    q, k, v = _round(q), _round(k), _round(v)
    out = []
    dist = (torch.arange(T).reshape(-1, 1) - torch.arange(T).reshape(1, -1)).to(q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap is not None:
            s = tanh_cap(s, cap)
        if slopes is not None:
            s = s - slopes[h] * dist
        s = s.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, g])
    return _round(torch.cat(out, dim=-1))


def rotary_attention(x, w, p, c, positions) -> torch.Tensor:
    """Mixer 'attention': q = W_q x, k = W_k x; the values are the keys as projected (before the rotation);
    q and k are rotated; scores are scaled, capped, masked by a sliding window; softmax; W_o."""
    H, G, d = c["heads"], c["kv_heads"], c["dim"]
    T = x.shape[0]
    q = (x @ w[p + "q"].T).reshape(T, H, d)
    k = (x @ w[p + "k"].T).reshape(T, G, d)
    v = k
    rot = c.get("rot")
    if rot:
        q = rotate_halves(q, positions, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_halves(k, positions, rot["dims"], rot["base"], rot.get("scaling"))
    m = c.get("mask") or {}
    o = softmax_heads(q, k, v, c["scale"], visible(T, m.get("size"), 0), cap=c.get("softcap"))
    return o @ w[p + "o"].T


def normed_attention(x, w, p, c, eps) -> torch.Tensor:
    """Mixer 'attention_2': q, k, v projected; q and k divided per head by their root mean square; score = q.k *
    scale - slope_h * (i - j); a sliding window that also keeps the first tokens; softmax; the heads side by
    side times sigma(W_g x); W_o."""
    H, G, d, e = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = x.shape[0]
    q = rms((x @ w[p + "q"].T).reshape(T, H, d), eps)
    k = rms((x @ w[p + "k"].T).reshape(T, G, d), eps)
    v = (x @ w[p + "v"].T).reshape(T, G, e)
    m = c.get("mask") or {}
    o = softmax_heads(q, k, v, c["scale"], visible(T, m.get("size"), int(m.get("keep_first", 0))),
                      slopes=head_slopes(H, x.dtype))
    o = _round(o * torch.sigmoid(x @ w[p + "g"].T))
    return o @ w[p + "o"].T


def expert(x, w, p):
    """W_down (silu(W_gate x) * (W_up x))."""
    return _round(silu(x @ w[p + "gate"].T) * (x @ w[p + "up"].T)) @ w[p + "down"].T


def table_experts(x, tokens, w, p, c) -> torch.Tensor:
    """Each token id names its experts in a table [vocab, top]; their outputs are averaged."""
    top = c["router"]["top"]
    table = w[p + "table"].to(torch.int64)
    out = torch.zeros_like(x)
    for t, tok in enumerate(tokens):
        for e in table[tok].tolist():
            out[t] += expert(x[t:t + 1], w, f"{p}e{e}.")[0] / top
    return out


def stream_read(xs, w, p):
    """xs [S, T, W] -> sum_s in[s] xs[s]."""
    return torch.einsum("s,stw->tw", w[p + "in"], xs)


def stream_write(xs, y, w, p):
    """new[t] = sum_s mix[s, t] xs[s] + out[t] y, all streams from the old ones."""
    return torch.einsum("sr,stw->rtw", w[p + "mix"], xs) + w[p + "out"].reshape(-1, 1, 1) * y.unsqueeze(0)


# --------------------------------------------------------------------------
# the decoder
# --------------------------------------------------------------------------
def schedule(cfg) -> list[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def decoder(cfg: dict, weights: dict, tokens: list[int], dtype=torch.float64, layers_out=None, rounding=None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence.  `layers_out`: a list that receives the residual stream (the sum of
    the streams) after every layer run.  `rounding`: a function applied to what an engine with 16-bit activations
    rounds (every sublayer's normed input; q, k and v as the cache holds them; the heads before the output
    projection; an expert's inner activation; the final norm's result): the difference to the exact logits is
    the size of error that such rounding alone causes at each position."""
    global _round
    _round = rounding or (lambda t: t)
    try:
        return _decoder(cfg, weights, tokens, dtype, layers_out)
    finally:
        _round = lambda t: t


def _decoder(cfg, weights, tokens, dtype, layers_out):
    w = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.tensor(tokens)]
    S = cfg.get("streams")
    xs = torch.stack([x] * S) if S else None

    def sublayer(fn, norm_w, hc):
        nonlocal x, xs
        if S:
            y = fn(_round(rms_norm(stream_read(xs, w, hc), norm_w, eps)))
            xs = stream_write(xs, y, w, hc)
        else:
            x = x + fn(_round(rms_norm(x, norm_w, eps)))

    for li in schedule(cfg):
        L = cfg["layers"][li]
        p = f"l{li}."
        c = L["mixer"]
        if L["type"] == "attention":
            sublayer(lambda n: rotary_attention(n, w, p + "mix.", c, positions), w[p + "norm1"], p + "hc1.")
        elif L["type"] == "attention_2":
            sublayer(lambda n: normed_attention(n, w, p + "mix.", c, eps), w[p + "norm1"], p + "hc1.")
        else:
            raise ValueError(f"unknown layer type {L['type']}")
        if L.get("mlp"):
            sublayer(lambda n: table_experts(n, tokens, w, p + "mlp.", L["mlp"]), w[p + "norm2"], p + "hc2.")
        if layers_out is not None:
            layers_out.append((xs.sum(dim=0) if S else x).clone())
    if S:
        x = xs.sum(dim=0)
    logits = _round(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return tanh_cap(logits, cap) if cap else logits


def greedy(cfg: dict, weights: dict, prompt: list[int], n: int, dtype=torch.float64) -> list[int]:
    """n greedy tokens after `prompt`, every step a whole forward pass (ties go to the lowest id)."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(decoder(cfg, weights, toks, dtype)[-1])))
    return toks[len(prompt):]
