"""Plain, slow implementation of the Furesun decoder: whole sequences, no
cache, one function per mechanism.  Nothing is imported from the product
package.  All math is done in the dtype asked for (float64 by default: the
anchor the product's float32 and bfloat16 paths are measured against).

Notation: T tokens, W model width, H query heads, G key/value heads, d key
width per head, e value width per head, sigma(z) = 1 / (1 + exp(-z)).
Position i may read position j <= i with i - j < window.

A layer is  x <- x + norm1(mixer(x));  x <- x + norm2(ff(x)):  the sublayers
read the stream itself, the norm comes after them.
"""
from __future__ import annotations

import math

import torch

from plain_zodosun import read_folder, write_folder  # noqa: F401  (the file format is the same)


# With a rounding function set (decoder(..., rounding=f)) the values that a 16-bit engine rounds are rounded here
# too: what a sublayer reads, q, k and v as the attention takes them, and what goes into an output or down product.
_rounding = [None]
_margins = [None]        # a list while decoder(..., margins_out=list) runs: per routed layer, each token's router margin


def _r(x):
    return x if _rounding[0] is None else _rounding[0](x)


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def tanh_cap(z, cap):
    return cap * torch.tanh(z / cap)


def rates(dims: int, base: float, scaling=None):
    """The dims/2 rotation rates and the factor on cosine and sine.  Plain: base^(-2i/dims), factor 1.  Stretched
    (factor F, original length L, turn counts fast and slow): n(t) = dims ln(L / (2 pi t)) / (2 ln base),
    lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), dims - 1), r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
    rate_i = f_i / F * r_i + f_i (1 - r_i); the factor is 0.1 ln F + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    F, L = float(scaling["factor"]), float(scaling["original"])

    def n(t):
        return dims * math.log(L / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(n(float(scaling["fast"]))), 0)
    hi = min(math.ceil(n(float(scaling["slow"]))), dims - 1)
    r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / F * r + f * (1.0 - r), 0.1 * math.log(F) + 1.0


def rotate(x, positions, dims: int, base: float, layout: str, scaling=None):
    """x [T, heads, n]: the first `dims` entries of every head are turned, pair (a, b) at position p into
    m (a cos t - b sin t, b cos t + a sin t), t = p * rate_i.  layout "halves": entry i with i + dims/2;
    "pairs": entry 2i with 2i + 1.  Entries from `dims` on pass."""
    half = dims // 2
    rate, m = rates(dims, base, scaling)
    ang = positions.to(torch.float64).reshape(-1, 1, 1) * rate
    c, s = (torch.cos(ang) * m).to(x.dtype), (torch.sin(ang) * m).to(x.dtype)
    out = x.clone()
    if layout == "halves":
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    else:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


def visible(T: int, window):
    """[T, T] bool: i reads j iff 0 <= i - j < window (no window: every j <= i)."""
    i = torch.arange(T).reshape(-1, 1)
    j = torch.arange(T).reshape(1, -1)
    ok = j <= i
    if window:
        ok = ok & (i - j < window)
    return ok


def softmax_heads(q, k, v, scale, mask, *, cap=None, sink=False):
    """q [T, H, d], k [T, G, d], v [T, G, e] -> [T, H, e].  Scores q . k * scale, capped if asked; weights
    exp(s_j) / (sum exp(s) [+ 1 with a sink: a key of score 0 that has no value])."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = tanh_cap(s, cap)
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink:
            m = torch.clamp(m, min=0.0)
        p = torch.exp(s - m)
        den = p.sum(dim=-1, keepdim=True)
        if sink:
            den = den + torch.exp(-m)
        out[:, h] = (p / den) @ v[:, g]
    return out


def latent_attention(x, w, p, c, positions, eps):
    """Keys and values from a small latent: q = W_q x, head by head [d plain | r turned]; [c' | k_r] = W_dkv x;
    c = rms_norm(c'); key_h = [U_k[h] c, turn(k_r)], value_h = U_v[h] c; a window; softmax; W_o."""
    T = x.shape[0]
    H, d, r, e, n = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    rot = c["rot"]
    q = (x @ w[p + "q"].T).reshape(T, H, d + r)
    dkv = x @ w[p + "dkv"].T
    lat = rms_norm(dkv[:, :n], w[p + "dkv.norm"], eps)
    k_r = rotate(dkv[:, n:].reshape(T, 1, r), positions, rot["dims"], rot["base"], "halves", rot.get("scaling"))
    q_r = rotate(q[..., d:], positions, rot["dims"], rot["base"], "halves", rot.get("scaling"))
    k_flat = (lat @ w[p + "uk"].T).reshape(T, H, d)
    val = (lat @ w[p + "uv"].T).reshape(T, H, e)
    qq = torch.cat([q[..., :d], q_r], dim=-1)
    kk = torch.cat([k_flat, k_r.expand(T, H, r)], dim=-1)
    o = softmax_heads(_r(qq), _r(kk), _r(val), c["scale"], visible(T, (c.get("mask") or {}).get("size")))
    return _r(o.reshape(T, H * e)) @ w[p + "o"].T


def mlstm(x, w, p, c, eps):
    """Matrix memory with exponential gates, token by token.  Per head: q = W_q x / sqrt(d), k, v; log gates
    i = cap tanh((W_i x + b_i) / cap), f = logsigmoid(cap tanh((W_f x + b_f) / cap)); with m_0 = 0, S_0 = 0, n_0 = 0:
    m_t = max(f + m, i); S = exp(f + m - m_t) S + exp(i - m_t) k v^T; n likewise with k; o = S^T q / (max(|n . q|,
    exp(-m_t)) + 1e-6).  Each head's o over its root mean square, times the norm's weight, times sigma(W_g x), W_o."""
    T = x.shape[0]
    H, d, e, cap = c["heads"], c["dim"], c["vdim"], float(c["gate_cap"])
    q = (x @ w[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (x @ w[p + "k"].T).reshape(T, H, d)
    v = (x @ w[p + "v"].T).reshape(T, H, e)
    ig = tanh_cap(x @ w[p + "i"].T + w[p + "i.b"], cap)
    fg = torch.nn.functional.logsigmoid(tanh_cap(x @ w[p + "f"].T + w[p + "f.b"], cap))
    S = torch.zeros((H, d, e), dtype=x.dtype)
    n = torch.zeros((H, d), dtype=x.dtype)
    m = torch.zeros((H,), dtype=x.dtype)
    out = torch.zeros((T, H, e), dtype=x.dtype)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a = torch.exp(fg[t] + m - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a.reshape(H, 1, 1) * S + b.reshape(H, 1, 1) * k[t].reshape(H, d, 1) * v[t].reshape(H, 1, e)
        n = a.reshape(H, 1) * n + b.reshape(H, 1) * k[t]
        m = m_new
        num = torch.einsum("hde,hd->he", S, q[t])
        den = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den.reshape(H, 1)
    y = rms(out, eps).reshape(T, H * e) * w[p + "norm"] * torch.sigmoid(x @ w[p + "g"].T)
    return _r(y) @ w[p + "o"].T


def attention_keys(x, w, p, c, positions, eps):
    """The keys (normed over the whole projection, then turned in neighbouring pairs) and values a layer caches."""
    T = x.shape[0]
    G, d, e = c["kv_heads"], c["dim"], c["vdim"]
    rot = c["rot"]
    k = rms_norm(x @ w[p + "k"].T, w[p + "k.norm"], eps).reshape(T, G, d)
    k = rotate(k, positions, rot["dims"], rot["base"], "pairs", rot.get("scaling"))
    v = (x @ w[p + "v"].T).reshape(T, G, e)
    return _r(k), _r(v)


def attention(x, w, p, c, positions, eps, kv=None):
    """Grouped softmax attention: q and k normed over their whole projections (with weights), turned in
    neighbouring pairs; scores capped; a window; a sink in the softmax; W_o.  `kv`: another layer's keys and
    values stand in for this layer's."""
    T = x.shape[0]
    H, d, e = c["heads"], c["dim"], c["vdim"]
    rot = c["rot"]
    q = rms_norm(x @ w[p + "q"].T, w[p + "q.norm"], eps).reshape(T, H, d)
    q = rotate(q, positions, rot["dims"], rot["base"], "pairs", rot.get("scaling"))
    k, v = kv if kv is not None else attention_keys(x, w, p, c, positions, eps)
    o = softmax_heads(_r(q), k, v, c["scale"], visible(T, (c.get("mask") or {}).get("size")), cap=c.get("softcap"), sink=True)
    return _r(o.reshape(T, H * e)) @ w[p + "o"].T


def gated_ff(x, w, p, act):
    return _r(act(x @ w[p + "gate"].T) * (x @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(x, w, p, c):
    """Scores sigma(W_router x); the `top` largest are chosen; their scores over their sum (+ 1e-20) times
    router.scale weigh the chosen experts' results; a shared expert is added for every token."""
    r = c["router"]
    z = x @ w[p + "router"].T
    s = torch.sigmoid(z)
    val, idx = torch.topk(z, r["top"], dim=-1)              # (the logits' order is the scores' order)
    val = torch.sigmoid(val)
    if _margins[0] is not None:
        # how far the last chosen logit lies above the first one left out, relative to the logits' root mean square
        zs = torch.sort(z, dim=-1, descending=True).values
        gap = zs[:, r["top"] - 1] - zs[:, r["top"]] if r["top"] < z.shape[1] else torch.full_like(zs[:, 0], math.inf)
        _margins[0].append(gap / (torch.sqrt((z * z).mean(dim=-1)) + 1e-9))
    wts = val / (val.sum(dim=-1, keepdim=True) + 1e-20) * r["scale"]
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(r["top"]):
            out[t] += wts[t, j] * gated_ff(x[t:t + 1], w, f"{p}e{int(idx[t, j])}.", silu)[0]
    if c.get("shared"):
        out = out + gated_ff(x, w, p + "shared.", silu)
    return out


def feed_forward(x, w, p, c):
    if c["kind"] == "dense":
        return gated_ff(x, w, p, gelu_tanh)
    return routed_ff(x, w, p, c)


# --------------------------------------------------------------------------
# the decoder
# --------------------------------------------------------------------------
def decoder(cfg: dict, weights: dict, tokens: list[int], dtype=torch.float64, layers_out=None, rounding=None,
            margins_out=None):
    """Logits [T, vocab] of a whole sequence.  `layers_out` (a list) receives the stream after every layer.
    `rounding`: a function applied where a 16-bit engine rounds its activations.  `margins_out` (a list) receives,
    per routed feed-forward, each token's router margin: the gap between the last chosen logit and the first one
    left out over the root mean square of the token's logits; a small margin is a choice that rounding can turn."""
    _rounding[0], _margins[0] = rounding, margins_out
    try:
        return _decoder(cfg, weights, tokens, dtype, layers_out)
    finally:
        _rounding[0] = _margins[0] = None


def _decoder(cfg, weights, tokens, dtype, layers_out):
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    kept: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        p, c = f"l{i}.mix.", layer["mixer"]
        xr = _r(x)                                            # what the sublayer reads
        if layer["type"] == "latent_attention":
            y = latent_attention(xr, w, p, c, positions, eps)
        elif layer["type"] == "mlstm":
            y = mlstm(xr, w, p, c, eps)
        elif layer["type"] == "attention":
            if c.get("kv_from") is not None:
                y = attention(xr, w, p, c, positions, eps, kv=kept[int(c["kv_from"])])
            else:
                kept[i] = attention_keys(xr, w, p, c, positions, eps)
                y = attention(xr, w, p, c, positions, eps, kv=kept[i])
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + rms_norm(y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(feed_forward(_r(x), w, f"l{i}.mlp.", layer["mlp"]), w[f"l{i}.norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = _r(rms_norm(x, w["final.norm"], eps)) @ w["head"].T
    if cfg.get("logit_softcap"):
        logits = tanh_cap(logits, float(cfg["logit_softcap"]))
    return logits


def greedy(cfg: dict, weights: dict, prompt: list[int], n: int, dtype=torch.float64) -> list[int]:
    """n tokens after the prompt, each the arg-max (lowest id on a tie) of the logits of all tokens before it."""
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(decoder(cfg, weights, toks, dtype)[-1])))
    return toks[len(prompt):]
