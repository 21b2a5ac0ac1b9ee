"""Small Pavisun configurations, weights with a spread that lets every
mechanism matter, and the plain implementation as oracle (cached)."""
from __future__ import annotations

import os

import torch

import plain_pavisun as pp


def _rot(heads, kv, dim, window, scale, cap=None, base=10000.0, dims=None, scaling=None):
    rot = {"base": base, "dims": dim if dims is None else dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}
    if window:
        m["mask"] = {"size": window}
    if cap:
        m["softcap"] = cap
    return {"type": "attention", "mixer": m}


def _unit(heads, kv, dim, vdim, window, keep, scale):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep:
            m["mask"]["keep_first"] = keep
    return {"type": "attention_2", "mixer": m}


def _moe(ff, experts, top):
    return None if ff is None else {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _model(vocab, width, eps, layers, streams=None, loop=None, cap=None):
    d = {"architecture": "Pavisun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        d["streams"] = streams
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    if cap:
        d["logit_softcap"] = cap
    return d


# A: both mixers, two experts per token, four streams, the first two layers run three times; heads of 32 and 48
#    (value rows of 16 beside keys of 32); windows of 40 and 64 (a page), five kept tokens; stretched rotation over
#    part of the head.
P_A = _model(300, 96, 1e-6, [
    {**_unit(4, 2, 32, 16, 40, 5, 0.9), "mlp": _moe(40, 6, 2)},
    {**_rot(6, 2, 48, 64, 0.2, cap=15.0, base=5000.0, dims=32, scaling=(4.0, 64, 16.0, 2.0)), "mlp": _moe(72, 4, 3)},
    {**_rot(2, 2, 64, 33, 0.15, cap=None, scaling=(16.0, 128, 32.0, 1.0)), "mlp": None},
], streams=4, loop=(0, 2, 3), cap=25.0)
# B: no streams (the plain residual sums), no loop, no cap on the logits, one expert per token; three query heads on
#    one key head; a window that keeps more first tokens than a page holds; layers without a window at all; no
#    stretching; as many experts per token as there are.
P_B = _model(1000, 128, 1e-5, [
    {**_rot(3, 1, 64, None, 0.125, cap=30.0, base=1e6), "mlp": _moe(96, 5, 1)},
    {**_unit(3, 1, 64, 64, 70, 70, 1.3), "mlp": _moe(64, 2, 2)},
    {**_unit(2, 2, 128, 128, None, 0, 0.7), "mlp": None},
    {**_rot(4, 4, 32, 100, 0.3), "mlp": _moe(32, 3, 1)},
])
# C: one stream, a loop of one run over everything, a width that is no multiple of 8, heads of 24 and 40, windows of
#    1 and 2 (a token sees itself only, or itself and one more), one kept token, one expert in all.
P_C = _model(130, 84, 1e-5, [
    {**_unit(2, 1, 24, 40, 2, 1, 1.1), "mlp": _moe(50, 1, 1)},
    {**_rot(2, 2, 40, 1, 0.25, cap=8.0, dims=20), "mlp": _moe(36, 7, 4)},
    {**_unit(1, 1, 16, 8, 3, 0, 2.0), "mlp": _moe(20, 3, 2)},
], streams=1, loop=(0, 3, 1), cap=12.0)
# D: heads the tensor-core kernels take (64 and 128, values as wide as keys), two streams, the last layer run twice,
#    windows of 128 and 200 with 3 and 64 kept tokens.
P_D = _model(384, 160, 1e-6, [
    {**_unit(4, 2, 64, 64, 128, 3, 1.0), "mlp": _moe(96, 4, 2)},
    {**_rot(2, 1, 128, 200, 0.09, cap=20.0, scaling=(8.0, 256, 32.0, 1.0)), "mlp": None},
    {**_unit(2, 2, 128, 128, 65, 64, 0.8), "mlp": _moe(64, 8, 1)},
    {**_rot(8, 4, 64, 130, 0.125, cap=50.0, base=50000.0), "mlp": _moe(48, 3, 3)},
], streams=2, loop=(3, 4, 2))
# S: attention whose softmax is sharp (a large scale on large keys), one layer of each mixer: a single key, far back,
#    at a window's edge or among the kept first tokens, decides a row's result.
P_S = _model(150, 64, 1e-5, [
    {**_rot(2, 1, 32, 300, 1.5, cap=60.0), "mlp": None},
    {**_unit(2, 2, 32, 32, 90, 4, 14.0), "mlp": None},
], streams=3)
CASES = {"a": P_A, "b": P_B, "c": P_C, "d": P_D, "s": P_S}


def make_weights(cfg: dict, seed: int) -> dict:
    """bfloat16 tensors by name (the tables int32): matrices N(0, 1/fan_in) times a gain; norm weights around 1;
    stream tensors near (1/S, 1, identity) with a spread; every table row holds distinct experts."""
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    def matrix(out, inp, gain=1.0):
        return normal(out, inp, std=gain / inp ** 0.5)

    W, V, S = cfg["width"], cfg["vocab"], cfg.get("streams") or 0
    sharp = cfg is P_S
    w = {"embed": normal(V, W), "final.norm": normal(W, std=0.2, mean=1.0), "head": matrix(V, W, 2.0)}

    def connection(p):
        w[p + "in"] = normal(S, std=0.3, mean=1.0 / S)
        w[p + "out"] = normal(S, std=0.3, mean=1.0)
        w[p + "mix"] = (torch.eye(S) + torch.randn(S, S, generator=g) * 0.2).to(torch.bfloat16)

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        w[p + "norm1"] = normal(W, std=0.2, mean=1.0)
        m, q = layer["mixer"], p + "mix."
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        gain = 4.0 if sharp else 1.5
        w[q + "q"], w[q + "k"] = matrix(H * d, W, gain), matrix(G * d, W, gain)
        if layer["type"] == "attention_2":
            w[q + "v"], w[q + "g"] = matrix(G * e, W, 1.5), matrix(H * e, W, 2.0)
        w[q + "o"] = matrix(W, H * e)
        if S:
            connection(p + "hc1.")
        if layer["mlp"] is not None:
            f, E, top = layer["mlp"]["expert"]["ff"], layer["mlp"]["router"]["experts"], layer["mlp"]["router"]["top"]
            w[p + "norm2"] = normal(W, std=0.2, mean=1.0)
            for x in range(E):
                w[f"{p}mlp.e{x}.gate"], w[f"{p}mlp.e{x}.up"] = matrix(f, W, 1.5), matrix(f, W, 1.5)
                w[f"{p}mlp.e{x}.down"] = matrix(W, f, 1.5)
            w[p + "mlp.table"] = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
            if S:
                connection(p + "hc2.")
    return w


_folders: dict = {}
_oracle: dict = {}


def folder(tmp_root, name: str, seed: int = 5) -> str:
    key = (name, seed)
    if key not in _folders:
        _folders[key] = pp.write_folder(os.path.join(str(tmp_root), f"pavisun_{name}_{seed}"), CASES[name],
                                        make_weights(CASES[name], seed))
    return _folders[key]


def oracle_logits(path: str, tokens: list[int]) -> torch.Tensor:
    """float64 logits of the plain implementation at every position."""
    key = (path, tuple(tokens))
    if key not in _oracle:
        cfg, w = pp.read_folder(path)
        _oracle[key] = pp.decoder(cfg, w, tokens, torch.float64)
    return _oracle[key]


def _bf16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


class Want:
    """Rows of the oracle's logits with, for each row, the largest change that rounding the activations to
    bfloat16 causes in the oracle itself (`noise`, absolute).  Small models have rows where a norm divides by a
    small number or a softmax hangs between two keys: there 8 bits of mantissa move the logits by a tenth of their
    size, in any implementation; elsewhere by a hundredth.  A bound that scales with the row's own noise stays
    tight on the ordinary rows."""

    def __init__(self, logits: torch.Tensor, noise: torch.Tensor):
        self.logits, self.noise = logits, noise

    def __getitem__(self, rows) -> "Want":
        if isinstance(rows, int):
            rows = slice(rows, rows + 1)
        return Want(self.logits[rows], self.noise[rows])

    def __len__(self) -> int:
        return self.logits.shape[0]

    @staticmethod
    def cat(parts) -> "Want":
        return Want(torch.cat([p.logits for p in parts]), torch.cat([p.noise for p in parts]))


_wants: dict = {}


def oracle(path: str, tokens: list[int]) -> Want:
    """The oracle's logits at every position and the noise of each row (cached)."""
    key = (path, tuple(tokens))
    if key not in _wants:
        cfg, w = pp.read_folder(path)
        exact = oracle_logits(path, tokens)
        rounded = pp.decoder(cfg, w, tokens, torch.float64, rounding=_bf16)
        _wants[key] = Want(exact, (rounded - exact).abs().amax(dim=1))
    return _wants[key]


def check_rows(got: torch.Tensor, want: Want, dtype: str, what: str, tol: float) -> None:
    """float32: max |difference| within `tol` of the oracle's largest logit.  bfloat16: row by row within `tol`
    of the largest logit plus three times the row's own noise."""
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
    over = torch.nonzero(err > bound).flatten().tolist()
    assert not over, (f"{what}: {len(over)} of {len(err)} rows over their bound, first row {over[0]}: |diff| "
                      f"{float(err[over[0]]):.3e} > {float(bound[over[0]]):.3e} (largest logit {scale:.3e}, the row's "
                      f"noise {float(want.noise[over[0]]):.3e}; bfloat16)")


def tokens(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
