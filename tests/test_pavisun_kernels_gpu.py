"""The mechanisms Pavisun adds, each kernel alone against the plain implementation's function of the same mechanism
(GPU): head encoding (stretched rotation, unit-size heads, values that are the keys, cache writes), softmax
attention with options on every kernel that serves it, residual streams, experts named by a table, caps and gates."""
import pytest
import torch

import plain_pavisun as pp

pytestmark = pytest.mark.gpu
DEV = "cuda"
I32 = dict(dtype=torch.int32, device=DEV)


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, tol, what=""):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), what
    err = float((got - want).abs().max())
    assert err <= tol * max(1.0, float(want.abs().max())), f"{what}: {err:.3e}"


def ints(x):
    return torch.tensor(x, **I32)


# ---- head encoding ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,kd,vd,rot,scaling,eps,own_v", [
    (4, 2, 32, 32, 32, (8.0, 64.0, 16.0, 1.0), 0.0, False),     # rotated, stretched, the values are the keys
    (6, 3, 48, 48, 16, None, 0.0, False),                       # part of the head rotated
    (3, 1, 40, 24, 0, None, 1e-5, True),                        # unit-size heads, values of their own width
    (2, 2, 16, 16, 0, None, 0.0, True),                         # nothing done to q and k
    (5, 5, 72, 8, 72, (2.0, 16.0, 4.0, 2.0), 0.0, True),        # rotated, values of their own
])
def test_head_encode_against_the_plain_functions(dtype, nh, nkv, kd, vd, rot, scaling, eps, own_v):
    from tq_kv_b200 import kernels
    from tq_kv_b200.config import PartSpec
    from tq_kv_b200.parts import Runtime, make_part
    lens, starts = [70, 1, 9], [0, 130, 60]                   # three rows: a prompt, a decoded token, a portion
    T = sum(lens)
    tok_pos = ints([s + i for s, n in zip(starts, lens) for i in range(n)])
    tok_seq = ints([b for b, n in enumerate(lens) for _ in range(n)])
    new_lens = ints([s + n for s, n in zip(starts, lens)])
    new_lens[2] -= 2                                           # the last two rows of the portion are padding
    extra = 12                                                 # columns behind the heads (a gate's, say)
    ld = nh * kd + nkv * kd + (nkv * vd if own_v else 0) + extra
    proj = rnd(T, ld, seed=3)
    k_col, v_col = nh * kd, (nh * kd + nkv * kd if own_v else -1)
    cos = sin = None
    if rot:
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        part = make_part(PartSpec("rotary_tables", {"rotary_dim": rot, "theta": 5000.0, "layout": "halves",
                                                    **({"scaling": sc} if sc else {})}))
        part.prepare(Runtime(torch.device(DEV), dtype, 256))
        cos, sin = part.cos, part.sin
    P, table = 64, ints([[4, 1, 7], [0, 5, 2], [3, 6, 8]])
    kp = torch.full((9, nkv, P, kd), 77.0, dtype=dtype, device=DEV)
    vp = torch.full((9, nkv, P, vd), 77.0, dtype=dtype, device=DEV)
    q = torch.empty(T, nh * kd, dtype=dtype, device=DEV)
    k = torch.empty(T, nkv * kd, dtype=dtype, device=DEV)
    v = torch.empty(T, nkv * vd, dtype=dtype, device=DEV)
    kernels.head_encode(proj, (tok_pos, tok_seq, new_lens), q, q_col=0, k_col=k_col, v_col=v_col, n_heads=nh,
                        n_kv_heads=nkv, key_dim=kd, value_dim=vd, cos=cos, sin=sin, rotary_dim=rot, norm_eps=eps, k_out=k,
                        v_out=v, k_pages=kp, v_pages=vp, block_table=table, table_width=3, ring_pages=0, page_tokens=P)
    x = proj.double().cpu()
    pos = tok_pos.cpu().long()
    wq = x[:, :nh * kd].reshape(T, nh, kd)
    wk = x[:, k_col:k_col + nkv * kd].reshape(T, nkv, kd)
    wv = x[:, v_col:v_col + nkv * vd].reshape(T, nkv, vd) if own_v else wk
    if eps:
        wq, wk = pp.rms(wq, eps), pp.rms(wk, eps)
    if rot:
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
        wq, wk = pp.rotate_halves(wq, pos, rot, 5000.0, sc), pp.rotate_halves(wk, pos, rot, 5000.0, sc)
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    close(q, wq.reshape(T, -1), tol, "q")
    close(k, wk.reshape(T, -1), tol, "k")
    close(v, wv.reshape(T, -1), tol, "v")
    # the cache holds the same rows at (page of position, row of position); padded rows are not written
    t = 0
    for b, (s, n) in enumerate(zip(starts, lens)):
        for i in range(n):
            p = s + i
            got_k, got_v = kp[table[b, p // P], :, p % P], vp[table[b, p // P], :, p % P]
            if p < int(new_lens[b]):
                assert torch.equal(got_k, k[t].reshape(nkv, kd)) and torch.equal(got_v, v[t].reshape(nkv, vd))
            else:
                assert float(got_k.float().min()) == 77.0 and float(got_v.float().min()) == 77.0
            t += 1


def test_stretched_rates_in_their_edge_cases():
    """The rotary tables against the plain rates: no stretching; a ramp that covers all pairs, none, and a single
    index (hi == lo: the ramp's width is the small constant)."""
    from tq_kv_b200.config import PartSpec
    from tq_kv_b200.parts import make_part
    for dims, base, sc in ((32, 10000.0, None), (64, 50000.0, (8.0, 512.0, 32.0, 1.0)), (16, 100.0, (4.0, 8.0, 64.0, 32.0)),
                           (24, 1e6, (2.0, 1e6, 1.0, 0.5)), (8, 10.0, (3.0, 40.0, 2.0, 2.0))):
        d = dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None
        part = make_part(PartSpec("rotary_tables", {"rotary_dim": dims, "theta": base, "layout": "halves",
                                                    **({"scaling": d} if d else {})}))
        rate, factor = part.rates()
        want_rate, want_factor = pp.stretched_rates(dims, base, d)
        assert torch.allclose(rate, want_rate, rtol=1e-14, atol=0) and abs(factor - want_factor) < 1e-15


# ---- attention with options -------------------------------------------------------------------------------------
def plain_rows(q, k, v, nh, nkv, kd, vd, scale, window, keep, cap, slopes, q_pos):
    """Rows at positions q_pos of one sequence whose keys 0 .. are k, v: the plain function on the whole square,
    of which the rows asked for are kept (q holds those rows only)."""
    Tk = k.shape[0]
    full_q = torch.zeros(Tk, nh, kd, dtype=torch.float64)
    full_q[q_pos] = q.double().cpu().reshape(-1, nh, kd)
    o = pp.softmax_heads(full_q, k.double().cpu().reshape(Tk, nkv, kd), v.double().cpu().reshape(Tk, nkv, vd), scale,
                         pp.visible(Tk, window, keep), cap=cap,
                         slopes=None if slopes is None else slopes.double().cpu())
    return o[q_pos]


def _paged(k, v, nkv, kd, vd, table_row, P=64):
    n_pages = max(table_row) + 2
    kp = torch.full((n_pages, nkv, P, kd), 1e4, dtype=k.dtype, device=DEV)     # unwritten rows hold junk, not zeros
    vp = torch.full((n_pages, nkv, P, vd), 1e4, dtype=k.dtype, device=DEV)
    for j in range(k.shape[0]):
        kp[table_row[j // P], :, j % P] = k[j].reshape(nkv, kd)
        vp[table_row[j // P], :, j % P] = v[j].reshape(nkv, vd)
    return kp, vp


OPTIONS = [
    # nh, nkv, kd, vd, window, keep, cap, slopes
    (4, 2, 64, 64, 72, 6, None, True),          # tensor-core heads, kept tokens and slopes
    (4, 2, 128, 128, 100, 0, 20.0, False),      # capped scores, a plain window
    (6, 2, 96, 96, 72, 0, 20.0, False),         # heads of 96: the mma kernel
    (3, 1, 32, 32, 130, 70, 5.0, True),         # more kept tokens than a page holds; everything at once
    (2, 2, 64, 64, None, 0, 30.0, True),        # no window at all
    (4, 4, 48, 16, 40, 5, None, True),          # value rows narrower than the keys: the general kernel
    (2, 1, 24, 40, 33, 1, 9.0, False),          # and wider
    (5, 5, 64, 64, 1, 3, None, True),           # a window of one: a token sees itself and the kept tokens
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("opts", OPTIONS)
@pytest.mark.parametrize("fast", [True, False])
def test_attention_with_options_over_packed_prompts(dtype, opts, fast):
    from tq_kv_b200 import kernels
    nh, nkv, kd, vd, window, keep, cap, sl = opts
    lens = [300, 1, 65, 130]
    T = sum(lens)
    q, k, v = rnd(T, nh * kd, dtype=dtype, seed=1), rnd(T, nkv * kd, dtype=dtype, seed=2), rnd(T, nkv * vd, dtype=dtype, seed=3)
    slopes = pp.head_slopes(nh, torch.float64).float().to(DEV) if sl else None
    gate = rnd(T, nh * vd + 8, seed=4)[:, 4:4 + nh * vd]                       # a slice of wider rows
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    out = torch.empty(T, nh * vd, dtype=dtype, device=DEV)
    kernels.attention_ext(q, out, n_heads=nh, n_kv_heads=nkv, key_dim=kd, value_dim=vd,
                          tok_pos=ints([i for n in lens for i in range(n)]),
                          tok_seq=ints([b for b, n in enumerate(lens) for _ in range(n)]), cu_seqlens=ints(cu),
                          start_pos=ints([0] * len(lens)), scale=0.3, window=window, keep_first=keep, softcap=cap,
                          slopes=slopes, k_packed=k, v_packed=v, gate=gate, use_fast=fast)
    want = torch.cat([plain_rows(q[a:b], k[a:b], v[a:b], nh, nkv, kd, vd, 0.3, window, keep, cap, slopes,
                                 list(range(b - a))) for a, b in zip(cu, cu[1:])])
    want = want * torch.sigmoid(gate.double().cpu())
    close(out, want, 3e-6 if dtype == torch.float32 else 1.2e-2, "packed")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("opts", OPTIONS)
@pytest.mark.parametrize("n_splits", [1, 3])
@pytest.mark.parametrize("fast", [True, False])
def test_attention_with_options_over_the_paged_cache(dtype, opts, n_splits, fast):
    """Single tokens of four sequences that share pages, and a portion of 70 tokens that continues a sequence."""
    from tq_kv_b200 import kernels
    nh, nkv, kd, vd, window, keep, cap, sl = opts
    Tk = 700
    k, v = rnd(Tk, nkv * kd, dtype=dtype, seed=1), rnd(Tk, nkv * vd, dtype=dtype, seed=2)
    table_row = [9, 3, 0, 11, 5, 7, 2, 10, 1, 6, 4]
    kp, vp = _paged(k, v, nkv, kd, vd, table_row)
    slopes = pp.head_slopes(nh, torch.float64).float().to(DEV) if sl else None
    for q_pos, seqs, cu, start in (([699, 64, 0, 511], [0, 1, 2, 3], [0, 1, 2, 3, 4], [699, 64, 0, 511]),
                                   (list(range(600, 670)), [0] * 70, [0, 70], [600])):
        B, R = len(start), len(q_pos)
        q = rnd(R, nh * kd, dtype=dtype)
        table = ints([table_row] * B)
        scratch = torch.empty(kernels.split_scratch_floats(R, nh, vd, n_splits), device=DEV) if n_splits > 1 else None
        out = torch.empty(R, nh * vd, dtype=dtype, device=DEV)
        kernels.attention_ext(q, out, n_heads=nh, n_kv_heads=nkv, key_dim=kd, value_dim=vd, tok_pos=ints(q_pos),
                              tok_seq=ints(seqs), cu_seqlens=ints(cu), start_pos=ints(start), scale=0.3, window=window,
                              keep_first=keep, softcap=cap, slopes=slopes, k_pages=kp, v_pages=vp, block_table=table,
                              table_width=len(table_row), n_splits=n_splits, scratch=scratch, use_fast=fast)
        want = plain_rows(q, k, v, nh, nkv, kd, vd, 0.3, window, keep, cap, slopes, q_pos)
        close(out, want, 3e-6 if dtype == torch.float32 else 1.2e-2, f"paged {R} rows")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("fast", [True, False])
@pytest.mark.parametrize("kd", [64, 96])
def test_single_keys_at_the_edges_of_the_window_and_of_the_kept_tokens(dtype, fast, kd):
    """Random scores are nearly flat, so a key that is wrongly seen or lost would hardly show.  Here one key matches
    every query strongly and its value is distinct: a row's result is that value iff the row sees the key.  The key
    is put far back, on both sides of the window's edge, on both sides of the kept tokens' edge and at page edges;
    prompts and single tokens over the cache must agree with the rule."""
    from tq_kv_b200 import kernels
    nh, nkv, Tk, window, keep = 4, 2, 400, 72, 6
    table_row = [5, 2, 6, 0, 3, 1, 4]
    for key in (0, 5, 6, 7, 63, 64, 127, 128, 250, 327, 328, 329):
        k, v = rnd(Tk, nkv * kd, scale=0.1, seed=1, dtype=dtype), rnd(Tk, nkv * kd, scale=0.1, seed=2, dtype=dtype)
        q = torch.full((Tk, nh * kd), 1.0, dtype=dtype, device=DEV)
        k[key] = 1.0
        v[key] = 5.0
        sees = lambda i: key <= i and (i - key < window or key < keep)        # noqa: E731
        common = dict(n_heads=nh, n_kv_heads=nkv, key_dim=kd, value_dim=kd, scale=0.5, window=window,
                      keep_first=keep, use_fast=fast)
        out = torch.empty_like(q)
        kernels.attention_ext(q, out, tok_pos=ints(list(range(Tk))), tok_seq=ints([0] * Tk), cu_seqlens=ints([0, Tk]),
                              start_pos=ints([0]), k_packed=k, v_packed=v, **common)
        rows = [i for i in (key, key + 1, key + window - 1, key + window, key + window + 1, Tk - 1) if i < Tk]
        kp, vp = _paged(k, v, nkv, kd, kd, table_row)
        dec = torch.empty(len(rows), nh * kd, dtype=dtype, device=DEV)
        kernels.attention_ext(q[:len(rows)], dec, tok_pos=ints(rows), tok_seq=ints(list(range(len(rows)))),
                              cu_seqlens=ints(list(range(len(rows) + 1))), start_pos=ints(rows), k_pages=kp, v_pages=vp,
                              block_table=ints([table_row] * len(rows)), table_width=len(table_row), **common)
        for n, i in enumerate(rows):
            for got, how in ((out[i], "prompt"), (dec[n], "decoded")):
                if sees(i):
                    assert float((got.float() - 5.0).abs().max()) < 2e-2, f"key {key} row {i} {how}: lost"
                else:
                    assert float(got.float().abs().max()) < 1.0, f"key {key} row {i} {how}: seen"


# ---- residual streams ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S,T,W", [(1, 5, 64), (3, 70, 256), (4, 9, 84), (8, 3, 1030), (2, 200, 4096)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_streams_write_read_and_norm(S, T, W, out_dtype):
    from tq_kv_b200 import kernels
    x = rnd(T, W, seed=1)
    xs = kernels.streams_fill(x, S)
    assert all(torch.equal(xs[s], x) for s in range(S))
    xs = rnd(S, T, W, seed=2)
    w = {"in": rnd(S, seed=3), "out": rnd(S, seed=4), "mix": rnd(S, S, seed=5)}
    y, nw = rnd(T, W, seed=6), rnd(W, seed=7)
    ref = xs.double().cpu()
    wd = {k: t.double().cpu() for k, t in w.items()}
    new = pp.stream_write(ref, y.double().cpu(), wd, "")
    want = pp.rms_norm(pp.stream_read(new, wd, ""), nw.double().cpu(), 1e-5)
    tol = 3e-6 if out_dtype == torch.float32 else 8e-3
    # some rows only: the streams stay as they were
    rows = ints([T - 1, 0])
    mine = xs.clone()
    got = kernels.streams_step(mine, y=y, mix=w["mix"], write=w["out"], read=w["in"], norm_weight=nw, eps=1e-5,
                               out_dtype=out_dtype, rows=rows)
    close(got, want[[T - 1, 0]], tol, "rows")
    assert torch.equal(mine, xs)
    # write, read and norm in one launch
    got = kernels.streams_step(mine, y=y, mix=w["mix"], write=w["out"], read=w["in"], norm_weight=nw, eps=1e-5,
                               out_dtype=out_dtype)
    close(got, want, tol, "normed")
    close(mine, new, 3e-6, "streams")
    # a write alone, then a read alone without a norm
    mine = xs.clone()
    kernels.streams_step(mine, y=y, mix=w["mix"], write=w["out"])
    close(mine, new, 3e-6, "write alone")
    close(kernels.streams_step(mine, read=w["in"]), pp.stream_read(new, wd, ""), 3e-6, "read alone")


# ---- experts named by a table ------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,F,E,top", [(1, 64, 40, 6, 2), (7, 84, 50, 1, 1), (33, 256, 96, 8, 1), (300, 128, 72, 4, 3),
                                         (700, 96, 200, 5, 5), (130, 160, 64, 16, 4)])
def test_experts_named_by_a_table(dtype, T, W, F, E, top):
    """Rows one by one and (bfloat16, widths in multiples of 8) sorted tiles, against the plain expert."""
    from tq_kv_b200 import kernels
    V = 50
    g = torch.Generator().manual_seed(T)
    table = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32).to(DEV)
    tokens = torch.randint(0, V, (T,), generator=g).to(torch.int32).to(DEV)
    w = {f"e{e}.{n}": rnd(*s, dtype=dtype, seed=10 * e + i, scale=s[1] ** -0.5)
         for e in range(E) for i, (n, s) in enumerate((("gate", (F, W)), ("up", (F, W)), ("down", (W, F))))}
    x = rnd(T, W, dtype=dtype, seed=99)
    choice = kernels.table_choice(tokens, table, E)
    assert torch.equal(choice, table[tokens.long()])
    wd = {k: t.double().cpu() for k, t in w.items()}
    wd["table"] = table.cpu()
    want = pp.table_experts(x.double().cpu(), tokens.tolist(), wd, "", {"router": {"top": top}})
    w_gu = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]).contiguous()
    w_down = torch.stack([w[f"e{e}.down"] for e in range(E)]).contiguous()
    tol = 3e-6 if dtype == torch.float32 else 1.5e-2
    y0 = rnd(T, W, seed=5)
    for accumulate in (False, True):
        y = y0.clone()
        kernels.routed_experts_rows(x, w_gu, w_down, choice, y, accumulate)
        close(y, want + (y0.double().cpu() if accumulate else 0), tol, "rows")
        if kernels.routed_tiles_ok(x, w_gu, w_down):
            y = y0.clone()
            kernels.routed_experts_tiles(x, w_gu, w_down, choice, y, accumulate)
            close(y, want + (y0.double().cpu() if accumulate else 0), tol, "tiles")


# ---- caps and gates ---------------------------------------------------------------------------------------------------
def test_tanh_cap_and_sigmoid_gate():
    from tq_kv_b200 import kernels
    x = rnd(37, 450, seed=1, scale=40.0)
    want = pp.tanh_cap(x.double().cpu(), 30.0)
    close(kernels.tanh_cap(x.clone(), 30.0), want, 2e-6, "cap")
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        o = rnd(9, 96, dtype=dtype, seed=2)
        gate = rnd(9, 200, seed=3, scale=3.0)[:, 50:146]
        want = o.double().cpu() * torch.sigmoid(gate.double().cpu())
        close(kernels.sigmoid_gate(o.clone(), gate), want, tol, "gate")
