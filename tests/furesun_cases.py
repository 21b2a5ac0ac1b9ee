"""Small Furesun configurations, weights with a spread that lets every
mechanism matter, and the plain implementation as oracle (cached)."""
from __future__ import annotations

import math
import os

import torch

import plain_furesun as pf


def _rot(dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def latent(heads, dim, rot_dim, vdim, rank, window, scale, base=10000.0, scaling=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": _rot(rot_dim, base, scaling)}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def memory(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def attn(heads, kv, dim, vdim, window, scale, cap=None, dims=None, base=10000.0, scaling=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": _rot(dim if dims is None else dims, base, scaling)}
    if window:
        m["mask"] = {"size": window}
    if cap:
        m["softcap"] = cap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, scale, shared=None):
    d = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def model(vocab, width, eps, layers, cap=None):
    d = {"architecture": "Furesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if cap:
        d["logit_softcap"] = cap
    return d


# A: the memory first, then an attention whose keys a later layer reads with a WIDER window (the cache keeps the
#    wider one), a latent attention between them; head widths that are no multiples of 8 (padded inside); rotation
#    over part of the heads; experts with and without a shared one, a dense feed-forward, a layer without any.
F_A = model(300, 96, 1e-6, [
    {**memory(3, 24, 20, 10.0), "mlp": moe(40, 6, 2, 1.5, shared=56)},
    {**attn(6, 2, 20, 12, 33, 0.3, cap=15.0, dims=10, base=5000.0), "mlp": dense(136)},
    {**latent(4, 24, 8, 40, 48, 50, 0.2, scaling=(4.0, 64, 16.0, 2.0)), "mlp": None},
    {**attn(6, 2, 20, 12, 70, 0.25, cap=9.0, dims=10, base=5000.0, kv_from=1), "mlp": moe(32, 4, 3, 1.0)},
], cap=25.0)
# B: heads the tensor-core kernels take (64 and 128, values as wide as keys), windows of whole pages and around
#    them, two readers of one layer's keys (one with a narrower window), stretched rotation in an attention layer,
#    a latent whose expanded heads are 128 wide, memories of 64 x 64 and 128 x 128.
F_B = model(384, 160, 1e-6, [
    {**attn(4, 2, 64, 64, 128, 0.125, cap=20.0, scaling=(8.0, 256, 32.0, 1.0)), "mlp": moe(96, 4, 2, 2.0, shared=64)},
    {**memory(2, 64, 64, 15.0), "mlp": None},
    {**attn(4, 2, 64, 64, 65, 0.11, cap=30.0, scaling=(8.0, 256, 32.0, 1.0), kv_from=0), "mlp": dense(256)},
    {**latent(2, 96, 32, 128, 96, 200, 0.09, base=50000.0), "mlp": moe(64, 8, 1, 1.0, shared=32)},
    {**attn(4, 2, 64, 64, 128, 0.125, scaling=(8.0, 256, 32.0, 1.0), kv_from=0), "mlp": None},
    {**attn(2, 1, 128, 128, 130, 0.09, cap=50.0, base=50000.0), "mlp": dense(96)},
    {**memory(1, 128, 128, 20.0), "mlp": dense(64)},
])
# C: a width that is no multiple of 8, windows of 1 and 2 (a token sees itself only, or itself and one more), no
#    window at all, one expert in all and as many per token as there are, key heads == heads, one head, no cap on
#    scores or logits, a router scale of 1.
F_C = model(130, 84, 1e-5, [
    {**latent(1, 16, 4, 24, 10, 2, 0.4), "mlp": moe(50, 1, 1, 1.0)},
    {**attn(2, 2, 40, 24, 1, 0.25, dims=20), "mlp": moe(36, 3, 3, 1.0, shared=20)},
    {**memory(1, 12, 36, 6.0), "mlp": dense(50)},
    {**attn(3, 1, 16, 8, None, 0.5, cap=8.0), "mlp": None},
    {**latent(3, 8, 8, 8, 20, None, 0.3, scaling=(16.0, 32, 8.0, 0.5)), "mlp": dense(44)},
])
# S: softmaxes that are sharp (a large scale on large keys): a single key, far back or at a window's edge, decides
#    a row's result; the memory's gates swing over their whole range.
F_S = model(150, 64, 1e-5, [
    {**attn(2, 1, 32, 32, 90, 1.5, cap=60.0), "mlp": None},
    {**latent(2, 16, 16, 16, 24, 300, 2.0), "mlp": None},
    {**memory(2, 16, 16, 30.0), "mlp": None},
    {**attn(2, 1, 32, 32, 40, 1.5, cap=60.0, kv_from=0), "mlp": None},
])
CASES = {"a": F_A, "b": F_B, "c": F_C, "s": F_S}


def make_weights(cfg: dict, seed: int, sharp: bool | None = None, alike_experts: bool = False) -> dict:
    """bfloat16 tensors by name: matrices N(0, 1/fan_in) times a gain; norm weights around 1; gate biases with a
    spread, so that input and forget gates take turns.  `alike_experts`: the experts of a layer differ from one
    another by a twentieth of their size only, so that a router's choice that rounding turns moves a row by less
    than rounding itself does (the weights the bfloat16 runs through the engine use: with experts that differ
    wholly, one turned choice moves its row, and through a memory every row after it, by the size of the logits
    in any 16-bit implementation; float32 runs and the kernels' own bfloat16 tests use experts that differ wholly)."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    def matrix(out, inp, gain=1.0):
        return normal(out, inp, std=gain / inp ** 0.5)

    W, V = cfg["width"], cfg["vocab"]
    sharp = cfg is F_S if sharp is None else sharp
    w = {"embed": normal(V, W), "final.norm": normal(W, std=0.2, mean=1.0), "head": matrix(V, W, 2.0)}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = normal(W, std=0.2, mean=1.0)
        m, q = layer["mixer"], p + "mix."
        gain = 4.0 if sharp else 1.5
        if layer["type"] == "latent_attention":
            H, d, r, e, n = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[q + "q"], w[q + "dkv"] = matrix(H * (d + r), W, gain), matrix(n + r, W, gain)
            w[q + "dkv.norm"] = normal(n, std=0.2, mean=1.0)
            w[q + "uk"], w[q + "uv"] = matrix(H * d, n, gain), matrix(H * e, n, 1.5)
            w[q + "o"] = matrix(W, H * e)
        elif layer["type"] == "mlstm":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = matrix(H * d, W, 1.5), matrix(H * d, W, 1.5), matrix(H * e, W, 1.5)
            w[q + "g"], w[q + "o"] = matrix(H * e, W, 2.0), matrix(W, H * e)
            w[q + "norm"] = normal(H * e, std=0.2, mean=1.0)
            w[q + "i"], w[q + "f"] = matrix(H, W, 6.0 if sharp else 2.0), matrix(H, W, 6.0 if sharp else 2.0)
            w[q + "i.b"], w[q + "f.b"] = normal(H, std=1.0, mean=-1.0), normal(H, std=1.0, mean=2.0)
        else:
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"] = matrix(H * d, W, gain)
            w[q + "q.norm"] = normal(H * d, std=0.3, mean=1.0 if not sharp else 2.0)
            if m.get("kv_from") is None:
                w[q + "k"], w[q + "v"] = matrix(G * d, W, gain), matrix(G * e, W, 1.5)
                w[q + "k.norm"] = normal(G * d, std=0.3, mean=1.0 if not sharp else 2.0)
            w[q + "o"] = matrix(W, H * e)
        f = layer["mlp"]
        if f is None:
            continue
        w[p + "norm2"] = normal(W, std=0.2, mean=1.0)
        q = p + "mlp."
        if f["kind"] == "dense":
            w[q + "gate"], w[q + "up"], w[q + "down"] = matrix(f["ff"], W, 1.5), matrix(f["ff"], W, 1.5), matrix(W, f["ff"], 1.5)
            continue
        n = f["expert"]["ff"]
        base = (matrix(n, W, 1.5).float(), matrix(n, W, 1.5).float(), matrix(W, n, 1.5).float())
        for x in range(f["router"]["experts"]):
            own = (matrix(n, W, 1.5), matrix(n, W, 1.5), matrix(W, n, 1.5))
            if alike_experts:
                own = tuple((b + 0.05 * o.float()).to(torch.bfloat16) for b, o in zip(base, own))
            w[f"{q}e{x}.gate"], w[f"{q}e{x}.up"], w[f"{q}e{x}.down"] = own
        w[q + "router"] = matrix(f["router"]["experts"], W, 3.0)        # scores well apart: no choice hangs on rounding
        if f.get("shared"):
            n = f["shared"]["ff"]
            w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"] = matrix(n, W, 1.5), matrix(n, W, 1.5), matrix(W, n, 1.5)
    return w


_folders: dict = {}
_wants: dict = {}
CLOSE_CALL = 0.05         # router margin (see plain_furesun.decoder) below which bfloat16 rounding may turn the choice


def folder(tmp_root, name: str, seed: int = 5, cfg: dict | None = None, alike_experts: bool = False) -> str:
    key = (name, seed, alike_experts)
    if key not in _folders:
        c = CASES[name] if cfg is None else cfg
        _folders[key] = pf.write_folder(os.path.join(str(tmp_root), f"furesun_{name}_{seed}_{int(alike_experts)}"), c,
                                        make_weights(c, seed, alike_experts=alike_experts))
    return _folders[key]


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


class Want:
    """Rows of the oracle's logits with, for each row, the largest change that rounding the activations to
    bfloat16 causes in the oracle itself (`noise`, absolute).  Small models have rows where a norm divides by a
    small number, a softmax hangs between two keys or a router between two experts: there 8 bits of mantissa move
    the logits by a tenth of their size, in any implementation; elsewhere by a hundredth.  A bound that scales with
    the row's own noise stays tight on the ordinary rows."""

    def __init__(self, logits: torch.Tensor, noise: torch.Tensor, margin: torch.Tensor, routed: bool = False):
        self.logits, self.noise, self.margin, self.routed = logits, noise, margin, routed

    def __getitem__(self, rows) -> "Want":
        if isinstance(rows, int):
            rows = slice(rows, rows + 1)
        return Want(self.logits[rows], self.noise[rows], self.margin[rows], self.routed)

    def __len__(self) -> int:
        return self.logits.shape[0]

    @staticmethod
    def cat(parts) -> "Want":
        return Want(torch.cat([p.logits for p in parts]), torch.cat([p.noise for p in parts]),
                    torch.cat([p.margin for p in parts]), any(p.routed for p in parts))


def oracle(path: str, tokens: list[int]) -> Want:
    """The oracle's logits at every position and the noise of each row (cached)."""
    key = (path, tuple(tokens))
    if key not in _wants:
        cfg, w = pf.read_folder(path)
        margins: list = []
        exact = pf.decoder(cfg, w, tokens, torch.float64, margins_out=margins)
        rounded = pf.decoder(cfg, w, tokens, torch.float64, rounding=_bf16)
        margin = torch.stack(margins).amin(dim=0) if margins else torch.full((len(tokens),), math.inf, dtype=torch.float64)
        _wants[key] = Want(exact, (rounded - exact).abs().amax(dim=1), margin, bool(margins))
    return _wants[key]


def check_rows(got: torch.Tensor, want: Want, dtype: str, what: str, tol: float) -> None:
    """float32: max |difference| within `tol` of the oracle's largest logit.  bfloat16: row by row within `tol`
    of the largest logit plus three times the row's own noise (one row in fifty may pass that bound, by less than
    three times); a row whose router margin is below CLOSE_CALL hangs on
    a choice between two experts that 8 bits of mantissa can turn, in any implementation: such rows (a few in a
    hundred with random weights) are left out, and must stay few."""
    from helpers import assert_close
    if dtype != "bfloat16":
        assert_close(got, want.logits.float(), dtype, what, tol=tol)
        return
    got = got.detach().to("cpu", torch.float64)
    assert got.shape == want.logits.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.logits.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(want.logits.abs().max())
    err = (got - want.logits).abs().amax(dim=1)
    bound = tol * scale + 3.0 * want.noise
    clear = want.margin >= CLOSE_CALL
    assert len(err) < 20 or int(clear.sum()) >= 0.4 * len(err), f"{what}: too many rows hang on close router calls"
    # One realisation of the rounding bounds another only roughly: one row in fifty (or two of twenty and more) may
    # pass its bound, one of them by more than three times (a memory's read divides by |n . q|, which rounding can
    # bring near zero for a token).  A lost key, a window one place off or a lost state moves rows by the size of
    # the logits, and more than one of them.
    allowed = max(2 if len(err) >= 20 else 1, len(err) // 50)
    far = torch.nonzero((err > 3.0 * bound) & clear).flatten().tolist()
    assert len(far) <= (1 if len(err) >= 20 else 0), (f"{what}: row {far[0]}: |diff| {float(err[far[0]]):.3e} > 3 x {float(bound[far[0]]):.3e} "
                     f"(largest logit {scale:.3e}; bfloat16)")
    over = torch.nonzero((err > bound) & clear).flatten().tolist()
    assert len(over) <= allowed, (f"{what}: {len(over)} of {len(err)} rows over their bound, first row {over[0]}: |diff| "
                      f"{float(err[over[0]]):.3e} > {float(bound[over[0]]):.3e} (largest logit {scale:.3e}, the row's "
                      f"noise {float(want.noise[over[0]]):.3e}; bfloat16)")


def tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
