"""The kernels that the Furesun decoder brought, each alone against float64 computations at other sizes: the gates and
the read of the matrix memory around the scan, the whole-row norm with the paired rotation, the sink in every
attention kernel (with single keys planted at the window's edges and at page borders), the router's choice and
weights, the experts' weighted forms, the gelu gate, the norm-and-add with its rounded copy, the latent rows in a ring
(GPU)."""
import math

import pytest
import torch

import plain_furesun as pf

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, tol, what=""):
    got, want = got.detach().double().cpu(), want.double().cpu()
    err = float((got - want).abs().max())
    scale = float(want.abs().max()) or 1.0
    assert err <= tol * scale, f"{what}: {err:.3e} of {scale:.3e}"


def _ints(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ---- the matrix memory ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H,d,e,lens", [(3, 24, 20, (1, 37, 2, 70)), (2, 64, 64, (130,)), (1, 12, 36, (5, 5)),
                                        (4, 128, 127, (33, 1)), (2, 8, 3, (64, 65))])
def test_the_memory_s_gates_scan_and_read_against_the_recurrence(H, d, e, lens):
    """A ragged batch with shuffled slots and states that are not zero, then the same sequences continued token by
    token with the one-token kernels."""
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(H * 100 + d)
    ea = -(-(e + 1) // 4) * 4
    cap, eps, floor = 9.0, 1e-5, 1e-6
    n_seqs, T = len(lens), sum(lens)
    slots = [5, 2, 7, 0][:n_seqs]
    state = torch.zeros((8, H * d * ea + H), dtype=torch.float64)
    state[:, :H * d * ea] = torch.randn(8, H * d * ea, generator=g, dtype=torch.float64) * 0.3
    state[:, H * d * ea:] = torch.randn(8, H, generator=g, dtype=torch.float64)
    state_dev = state.float().to(DEV)
    state = state_dev.double().cpu()                          # the float32 values are the truth both sides start from
    ld = 2 * H * d + H * ea + H * e + 2 * H
    proj = torch.randn(T + 4, ld, generator=g, dtype=torch.float64)
    proj[:, -2 * H:] *= 4.0                                    # gates over their whole range
    off_v, off_g, off_i, off_f = 2 * H * d, 2 * H * d + H * ea, ld - 2 * H, ld - H
    vv = proj[:, off_v:off_g].reshape(-1, H, ea)
    vv[:, :, e] = 1.0
    vv[:, :, e + 1:] = 0.0
    proj = proj.float().double()
    norm_w = torch.randn(H * e, generator=g, dtype=torch.float64).float().double()

    def reference(rows, S, n, m):
        out = torch.zeros(len(rows), H, e, dtype=torch.float64)
        for r, t in enumerate(rows):
            q = proj[t, :H * d].reshape(H, d) * d ** -0.5
            k = proj[t, H * d:2 * H * d].reshape(H, d)
            v = proj[t, off_v:off_g].reshape(H, ea)[:, :e]
            ig = cap * torch.tanh(proj[t, off_i:off_i + H] / cap)
            fg = torch.nn.functional.logsigmoid(cap * torch.tanh(proj[t, off_f:off_f + H] / cap))
            m_new = torch.maximum(fg + m, ig)
            a, b = torch.exp(fg + m - m_new), torch.exp(ig - m_new)
            S = a.reshape(H, 1, 1) * S + b.reshape(H, 1, 1) * k.reshape(H, d, 1) * v.reshape(H, 1, e)
            n = a.reshape(H, 1) * n + b.reshape(H, 1) * k
            m = m_new
            den = torch.maximum((n * q).sum(-1).abs(), torch.exp(-m)) + floor
            o = torch.einsum("hde,hd->he", S, q) / den.reshape(H, 1)
            o = pf.rms(o, eps)
            out[r] = o * norm_w.reshape(H, e) * torch.sigmoid(proj[t, off_g:off_i].reshape(H, e))
        return out.reshape(len(rows), H * e), S, n, m

    def run(rows_of_seq, single):
        cu = [0]
        for rows in rows_of_seq:
            cu.append(cu[-1] + len(rows))
        order = [t for rows in rows_of_seq for t in rows]
        p = proj[order].float().to(DEV).contiguous()
        Tn = len(order)
        scal = kernels.mlstm_gates(p[:, off_i:off_i + H], p[:, off_f:off_f + H], cap, state_dev[:, H * d * ea:],
                                   _ints(cu), _ints(slots), n_seqs)
        o = torch.empty((Tn, H * ea), dtype=torch.float32, device=DEV)
        kernels.gated_scan(p[:, :H * d], p[:, H * d:2 * H * d], p[:, off_v:off_g], scal, state_dev[:, :H * d * ea], _ints(cu),
                           _ints(slots), o, n_seqs=n_seqs, heads=H, qk_heads=H, key_dim=d, value_dim=ea, delta=False,
                           single_tokens=single)
        y = torch.empty((Tn, H * e), dtype=torch.float32, device=DEV)
        kernels.mlstm_read(o, scal, p[:, off_g:off_i], norm_w.float().to(DEV), y, heads=H, value_dim=e, q_scale=d ** -0.5,
                           floor=floor, eps=eps)
        return y

    starts = [sum(lens[:i]) for i in range(n_seqs)]
    held = []
    for b in range(n_seqs):
        st = state[slots[b]]
        Sn = st[:H * d * ea].reshape(H, d, ea)
        held.append((Sn[:, :, :e].clone(), Sn[:, :, e].clone(), st[H * d * ea:].clone()))
    got = run([list(range(s, s + n)) for s, n in zip(starts, lens)], False)
    for b in range(n_seqs):
        want, *held[b] = reference(range(starts[b], starts[b] + lens[b]), *held[b])
        _close(got[starts[b]:starts[b] + lens[b]], want, 3e-5, f"sequence {b}")
    for step in range(4):                                    # four more tokens each, one at a time
        got = run([[T + step]] * n_seqs, True)
        for b in range(n_seqs):
            want, *held[b] = reference([T + step], *held[b])
            _close(got[b:b + 1], want, 3e-5, f"step {step} sequence {b}")
    for b in range(n_seqs):                                  # what the slots hold afterwards
        st = state_dev[slots[b]].double().cpu()
        _close(st[:H * d * ea].reshape(H, d, ea)[:, :, :e], held[b][0], 3e-5, "S")
        _close(st[:H * d * ea].reshape(H, d, ea)[:, :, e], held[b][1], 3e-5, "n")
        _close(st[H * d * ea:], held[b][2], 1e-6, "m")


def test_a_value_written_long_ago_is_still_read_and_large_gates_do_not_overflow():
    """600 tokens whose forget gates stay open and whose input gates are shut after the first: the first token's
    value comes back; then gates at +-cap for cap = 80 (exp(80) does not fit float32 sums without the maximum)."""
    from tq_kv_b200 import kernels
    H, d, e, ea, T = 1, 8, 4, 8, 600
    cap = 80.0
    ld = 2 * d + ea + e + 2
    p = torch.zeros((T, ld), dtype=torch.float32)
    p[:, :d] = 1.0                                            # q
    p[0, d:2 * d] = 1.0                                       # only the first token writes a key
    p[0, 2 * d:2 * d + e] = torch.tensor([1.0, -2.0, 3.0, 0.5])
    p[:, 2 * d + e] = 1.0
    p[:, ld - 2] = -1000.0                                    # input gates shut (log gate -cap) ...
    p[0, ld - 2] = 1000.0                                     # ... but the first (+cap)
    p[:, ld - 1] = 1000.0                                     # forget gates open: logsigmoid(cap) = -0
    p = p.to(DEV)
    state = torch.zeros((1, d * ea + 1), dtype=torch.float32, device=DEV)
    scal = kernels.mlstm_gates(p[:, ld - 2:ld - 1], p[:, ld - 1:], cap, state[:, d * ea:], _ints([0, T]), _ints([0]), 1)
    assert torch.isfinite(scal).all()
    o = torch.empty((T, ea), dtype=torch.float32, device=DEV)
    kernels.gated_scan(p[:, :d], p[:, d:2 * d], p[:, 2 * d:2 * d + ea], scal, state[:, :d * ea], _ints([0, T]), _ints([0]), o,
                       n_seqs=1, heads=1, qk_heads=1, key_dim=d, value_dim=ea, delta=False)
    y = torch.empty((T, e), dtype=torch.float32, device=DEV)
    kernels.mlstm_read(o, scal, torch.full((T, e), 50.0, device=DEV), torch.ones(e, device=DEV), y, heads=1, value_dim=e,
                       q_scale=1.0, floor=1e-6, eps=1e-6)
    want = pf.rms(torch.tensor([[1.0, -2.0, 3.0, 0.5]], dtype=torch.float64), 1e-6)
    _close(y[-1:], want, 1e-4, "the first value after 600 tokens")
    _close(y[:1], want, 1e-4, "the first value at once")


# ---- the whole-row norm, the paired rotation and the cache ------------------------------------------------------
@pytest.mark.parametrize("H,G,d,e,rot,paired", [(6, 2, 24, 16, 10, True), (4, 4, 64, 64, 64, True), (3, 1, 40, 8, 0, True),
                                                (2, 1, 32, 32, 16, False), (5, 0, 16, 16, 8, True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_row_norm_and_paired_rotation_into_pages(H, G, d, e, rot, paired, dtype):
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(H + d)
    T, eps, page = 9, 1e-5, 64
    pos = [0, 1, 63, 64, 65, 127, 128, 300, 301]
    ld = H * d + G * d + G * e + 5
    proj = torch.randn(T, ld, generator=g).to(DEV)
    qw, kw = torch.randn(H * d, generator=g).to(DEV), torch.randn(max(G, 1) * d, generator=g).to(DEV)
    rate = torch.pow(torch.tensor(1e4, dtype=torch.float64), -2.0 * torch.arange(max(rot // 2, 1), dtype=torch.float64) / max(rot, 2))
    ang = torch.arange(400, dtype=torch.float64).reshape(-1, 1) * rate
    cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    inv = kernels.row_inv_rms(proj, q_col=0, q_width=H * d, q_count=H * d, k_col=H * d, k_width=G * d, k_count=G * d, eps=eps)
    q = torch.empty((T, H * d), dtype=dtype, device=DEV)
    k = torch.empty((T, G * d), dtype=dtype, device=DEV) if G else None
    v = torch.empty((T, G * e), dtype=dtype, device=DEV) if G else None
    k_pages = torch.zeros((8, max(G, 1), page, d), dtype=dtype, device=DEV)
    v_pages = torch.zeros((8, max(G, 1), page, e), dtype=dtype, device=DEV)
    table = _ints([[3, 6, 1, 7, 0]])
    kernels.head_encode(proj, (_ints(pos), _ints([0] * T), _ints([400])), q, q_col=0, k_col=H * d if G else 0,
                        v_col=H * d + G * d if G else -1, n_heads=H, n_kv_heads=G, key_dim=d, value_dim=e, cos=cos if rot else None,
                        sin=sin if rot else None, rotary_dim=rot, k_out=k, v_out=v, k_pages=k_pages if G else None,
                        v_pages=v_pages if G else None, block_table=table if G else None, table_width=5, paired=paired,
                        row_inv=inv, q_weight=qw, k_weight=kw if G else None)
    P = proj.double().cpu()
    layout = "pairs" if paired else "halves"
    want_q = pf.rms_norm(P[:, :H * d], qw.double().cpu(), eps).reshape(T, H, d)
    want_q = pf.rotate(want_q, torch.tensor(pos), rot, 1e4, layout) if rot else want_q
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    _close(q.reshape(T, H, d), want_q, tol, "q")
    if not G:
        return
    want_k = pf.rms_norm(P[:, H * d:H * d + G * d], kw.double().cpu(), eps).reshape(T, G, d)
    want_k = pf.rotate(want_k, torch.tensor(pos), rot, 1e4, layout) if rot else want_k
    _close(k.reshape(T, G, d), want_k, tol, "k")
    _close(v, P[:, H * d + G * d:H * d + G * d + G * e], tol, "v")
    pages = [3, 6, 1, 7, 0]
    for t, p in enumerate(pos):
        assert torch.equal(k_pages[pages[p // page], :, p % page], k[t].reshape(G, d)), p
        assert torch.equal(v_pages[pages[p // page], :, p % page], v[t].reshape(G, e)), p


# ---- the sink, on every attention kernel -------------------------------------------------------------------------
def _attention_reference(q, k, v, pos_q, scale, window, cap, sink):
    """q [Tq, H, d] at positions pos_q over keys k, v [Tk, G, .] at positions 0 .. Tk-1."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(Tq, H, v.shape[2], dtype=torch.float64)
    j = torch.arange(k.shape[0])
    for t in range(Tq):
        ok = (j <= pos_q[t]) & ((pos_q[t] - j < window) if window else torch.ones_like(j, dtype=torch.bool))
        for h in range(H):
            s = (k[:, h // (H // G)] @ q[t, h]) * scale
            if cap:
                s = cap * torch.tanh(s / cap)
            w = torch.exp(s[ok])
            out[t, h] = (w / (w.sum() + (1.0 if sink else 0.0))) @ v[ok, h // (H // G)]
    return out


@pytest.mark.parametrize("H,G,d,e", [(4, 2, 64, 64), (2, 1, 128, 128), (6, 2, 32, 32), (4, 1, 40, 24), (8, 4, 96, 96)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,cap", [(None, None), (70, 20.0), (64, None)])
def test_the_sink_in_prompts_over_pages_and_in_splits(H, G, d, e, dtype, window, cap):
    """The same rows through the packed prompt kernels, the paged prompt kernels, single tokens over the cache with
    one and with several splits (the merge step then adds the sink once), and the general kernel."""
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(d + H)
    T, scale = 300, 0.8 / math.sqrt(d)
    q = torch.randn(T, H, d, generator=g).to(dtype)
    k = torch.randn(T, G, d, generator=g).to(dtype)
    v = torch.randn(T, G, e, generator=g).to(dtype)
    q[200] *= 6.0                                            # rows whose scores are large and negative or positive:
    q[201] *= -6.0                                           # the sink then takes nearly nothing, or nearly all
    want = _attention_reference(q.double(), k.double(), v.double(), list(range(T)), scale, window, cap, True)
    no_sink = _attention_reference(q.double(), k.double(), v.double(), list(range(T)), scale, window, cap, False)
    assert float((want - no_sink).abs().max()) > 0.05        # the sink matters
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    qd, kd, vd = q.reshape(T, -1).to(DEV), k.reshape(T, -1).to(DEV), v.reshape(T, -1).to(DEV)
    pos, seq, cu, start = _ints(list(range(T))), _ints([0] * T), _ints([0, T]), _ints([0])
    common = dict(n_heads=H, n_kv_heads=G, key_dim=d, value_dim=e, scale=scale, window=window, softcap=cap, sink=True)
    for fast in (True, False):
        out = torch.empty((T, H * e), dtype=dtype, device=DEV)
        kernels.attention_ext(qd, out, k_packed=kd, v_packed=vd, tok_pos=pos, tok_seq=seq, cu_seqlens=cu, start_pos=start,
                              use_fast=fast, **common)
        _close(out.reshape(T, H, e), want, tol, f"packed fast={fast}")
    # the cache: shuffled pages
    pages = [4, 0, 3, 1, 2]
    k_pages = torch.zeros((5, G, 64, d), dtype=dtype, device=DEV)
    v_pages = torch.zeros((5, G, 64, e), dtype=dtype, device=DEV)
    for p in range(T):
        k_pages[pages[p // 64], :, p % 64] = k[p].to(DEV)
        v_pages[pages[p // 64], :, p % 64] = v[p].to(DEV)
    table = _ints([pages])
    paged = dict(k_pages=k_pages, v_pages=v_pages, block_table=table, table_width=5, page_tokens=64)
    out = torch.empty((T - 100, H * e), dtype=dtype, device=DEV)           # a portion: rows 100 .. over the pages
    kernels.attention_ext(qd[100:], out, tok_pos=pos[100:], tok_seq=seq[100:], cu_seqlens=_ints([0, T - 100]),
                          start_pos=_ints([100]), **paged, **common)
    _close(out.reshape(T - 100, H, e), want[100:], tol, "a portion over pages")
    rows = [0, 1, 63, 64, 65, 199, 200, 201, 299]                          # single tokens, each a sequence of its own
    for n_splits in (1, 3):
        for fast in (True, False):
            qs = qd[rows].contiguous()
            out = torch.empty((len(rows), H * e), dtype=dtype, device=DEV)
            scratch = torch.empty(kernels.split_scratch_floats(len(rows), H, e, n_splits), dtype=torch.float32, device=DEV) \
                if n_splits > 1 else None
            kernels.attention_ext(qs, out, tok_pos=_ints(rows), tok_seq=_ints(list(range(len(rows)))),
                                  cu_seqlens=_ints(list(range(len(rows) + 1))), start_pos=_ints(rows),
                                  k_pages=k_pages, v_pages=v_pages, block_table=_ints([pages] * len(rows)), table_width=5,
                                  page_tokens=64, n_splits=n_splits, scratch=scratch, use_fast=fast, **common)
            _close(out.reshape(len(rows), H, e), want[rows], tol, f"single tokens, {n_splits} splits, fast={fast}")


@pytest.mark.parametrize("d", [32, 64, 128])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_single_keys_at_the_window_s_edges_and_page_borders(d, dtype):
    """One key is made to stand out by e^12 against the query; the value it carries reaches the result wholly when
    the key is inside the window and not at all when it is one place outside, in prompts and for single tokens."""
    from tq_kv_b200 import kernels
    H = G = 2
    T, window = 420, 130
    g = torch.Generator().manual_seed(d)
    for key_at in (0, 63, 64, 127, 128, 200, 270):
        k = torch.randn(T, G, d, generator=g) * 0.1
        v = torch.randn(T, G, d, generator=g) * 0.1
        qv = torch.randn(d, generator=g)
        qv = qv / qv.norm()
        k[key_at] = qv * 12.0
        v[key_at] = 5.0
        q = qv.expand(T, H, d).clone()
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        want = _attention_reference(q.double(), k.double(), v.double(), list(range(T)), 1.0, window, None, True)
        inside, outside = key_at + window - 1, key_at + window
        assert float(want[inside].min()) > 4.0 and float(want[outside].abs().max()) < 1.0
        qd, kd, vd = q.reshape(T, -1).to(DEV), k.reshape(T, -1).to(DEV), v.reshape(T, -1).to(DEV)
        common = dict(n_heads=H, n_kv_heads=G, key_dim=d, value_dim=d, scale=1.0, window=window, sink=True)
        out = torch.empty((T, H * d), dtype=dtype, device=DEV)
        kernels.attention_ext(qd, out, k_packed=kd, v_packed=vd, tok_pos=_ints(list(range(T))), tok_seq=_ints([0] * T),
                              cu_seqlens=_ints([0, T]), start_pos=_ints([0]), **common)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        _close(out.reshape(T, H, d), want, tol, f"prompt, key at {key_at}")
        pages = [6, 2, 5, 0, 3, 1, 4]
        k_pages = torch.zeros((7, G, 64, d), dtype=dtype, device=DEV)
        v_pages = torch.zeros((7, G, 64, d), dtype=dtype, device=DEV)
        for p in range(T):
            k_pages[pages[p // 64], :, p % 64] = k[p].to(DEV)
            v_pages[pages[p // 64], :, p % 64] = v[p].to(DEV)
        rows = [r for r in (key_at, inside - 1, inside, outside, outside + 1) if r < T]
        for n_splits in (1, 2):
            out = torch.empty((len(rows), H * d), dtype=dtype, device=DEV)
            scratch = torch.empty(kernels.split_scratch_floats(len(rows), H, d, n_splits), dtype=torch.float32, device=DEV) \
                if n_splits > 1 else None
            kernels.attention_ext(qd[rows].contiguous(), out, tok_pos=_ints(rows), tok_seq=_ints(list(range(len(rows)))),
                                  cu_seqlens=_ints(list(range(len(rows) + 1))), start_pos=_ints(rows), k_pages=k_pages,
                                  v_pages=v_pages, block_table=_ints([pages] * len(rows)), table_width=7, page_tokens=64,
                                  n_splits=n_splits, scratch=scratch, **common)
            _close(out.reshape(len(rows), H, d), want[rows], tol, f"single tokens, key at {key_at}, {n_splits} splits")


# ---- the feed-forwards ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("E,top", [(16, 4), (5, 5), (1, 1), (40, 3), (8, 1)])
def test_the_router_s_choice_and_weights(E, top):
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(E)
    z = (torch.randn(50, E + 3, generator=g) * 2.0).to(DEV)[:, :E]      # a column slice
    choice, weights = kernels.router_choice(z, top, 1.7, 1e-20)
    val, idx = torch.topk(z.double().cpu(), top, dim=-1)
    val = torch.sigmoid(val)
    assert torch.equal(choice.cpu().long(), idx)
    _close(weights, val / (val.sum(-1, keepdim=True) + 1e-20) * 1.7, 1e-6, "weights")
    big = (z * 20.0).contiguous()                                       # logits whose sigmoids are all 1 in float32
    assert torch.equal(kernels.router_choice(big, top, 1.0, 0.0)[0].cpu().long(), torch.topk(big.double().cpu(), top, dim=-1)[1])
    ties = torch.zeros((2, E), device=DEV)                              # equal scores: the lowest indices, in order
    c, w = kernels.router_choice(ties, top, 1.0, 0.0)
    assert c.cpu().tolist() == [list(range(top))] * 2 and torch.allclose(w.cpu(), torch.full((2, top), 1.0 / top))


@pytest.mark.parametrize("T,W,F,E,top", [(5, 96, 40, 6, 2), (200, 128, 64, 8, 3), (70, 84, 36, 3, 3), (3, 64, 16, 1, 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_weighted_by_the_router_in_rows_and_in_tiles(T, W, F, E, top, dtype):
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(T + W)
    x = (torch.randn(T, W, generator=g)).to(dtype)
    gu = (torch.randn(E, 2 * F, W, generator=g) / W ** 0.5).to(dtype)
    dn = (torch.randn(E, W, F, generator=g) / F ** 0.5).to(dtype)
    z = torch.randn(T, E, generator=g).to(DEV)
    choice, weights = kernels.router_choice(z, top, 2.0, 1e-20)
    xd, gd, dd = x.double(), gu.double(), dn.double()
    want = torch.zeros(T, W, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            e_ = int(choice[t, j])
            a = pf.silu(gd[e_, :F] @ xd[t]) * (gd[e_, F:] @ xd[t])
            if dtype == torch.bfloat16:
                a = a.to(torch.bfloat16).double()
            want[t] += float(weights[t, j]) * (dd[e_] @ a)
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    base = torch.randn(T, W, generator=g).to(DEV)
    y = base.clone()
    kernels.routed_experts_rows(x.to(DEV), gu.to(DEV), dn.to(DEV), choice, y, accumulate=True, weights=weights)
    _close(y - base, want, tol, "rows, accumulated")
    if dtype == torch.bfloat16 and kernels.routed_tiles_ok(x.to(DEV), gu.to(DEV), dn.to(DEV)):
        y = torch.empty((T, W), dtype=torch.float32, device=DEV)
        kernels.routed_experts_tiles(x.to(DEV), gu.to(DEV), dn.to(DEV), choice, y, accumulate=False, weights=weights)
        _close(y, want, tol, "tiles, stored")


@pytest.mark.parametrize("M,K,N", [(1, 96, 40), (8, 256, 128), (40, 128, 64), (300, 192, 320), (16, 84, 50)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_gelu_gate_in_every_product(M, K, N, dtype):
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(M + K)
    x = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(2 * N, K, generator=g) / K ** 0.5 * 2.0).to(dtype)
    want = pf.gelu_tanh(x.double() @ w[:N].double().T) * (x.double() @ w[N:].double().T)
    for out_dtype in {dtype, torch.float32}:
        got = kernels.linear(x.to(DEV), w.to(DEV), swiglu=True, activation=kernels.ACT_GELU_TANH, out_dtype=out_dtype)
        _close(got, want, 2e-5 if dtype == torch.float32 else 1.5e-2, f"gelu gate, out {out_dtype}")
    silu = pf.silu(x.double() @ w[:N].double().T) * (x.double() @ w[N:].double().T)
    got = kernels.linear(x.to(DEV), w.to(DEV), swiglu=True, out_dtype=torch.float32)
    _close(got, silu, 2e-5 if dtype == torch.float32 else 1.5e-2, "the silu gate is the default")


@pytest.mark.parametrize("T,W", [(1, 84), (7, 192), (130, 2048), (3, 5)])
def test_the_norm_and_add_with_its_rounded_copy(T, W):
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(W)
    acc, y, w = torch.randn(T, W, generator=g).to(DEV), torch.randn(T, W, generator=g).to(DEV) * 3.0, torch.randn(W, generator=g).to(DEV)
    want = acc.double().cpu() + pf.rms_norm(y.double().cpu(), w.double().cpu(), 1e-5)
    copy = torch.empty((T, W), dtype=torch.bfloat16, device=DEV)
    kernels.add_normed_copy(acc, y, w, 1e-5, copy)
    _close(acc, want, 1e-6, "sum")
    assert torch.equal(copy, acc.to(torch.bfloat16)) and torch.equal(kernels.round_rows(acc), copy)
    kernels.add_normed_copy(acc, y, w, 1e-5, None)
    _close(acc, want + pf.rms_norm(y.double().cpu(), w.double().cpu(), 1e-5), 1e-6, "sum without a copy")


# ---- the latent's rows in a ring, queries projected directly -----------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_rows_without_a_query_latent_into_a_ring(dtype):
    from tq_kv_b200 import kernels
    g = torch.Generator().manual_seed(8)
    n, r, row, ring = 20, 8, 32, 2
    pos = list(range(100, 140))                              # a portion; a ring of two pages holds positions 12 .. 139
    T = len(pos)
    proj = torch.randn(T, 50 + n + r, generator=g).to(DEV)   # 50 columns of queries come first
    wkv = torch.randn(n, generator=g).to(DEV)
    rate, f = pf.rates(r, 1e4, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0})
    ang = torch.arange(200, dtype=torch.float64).reshape(-1, 1) * rate
    cos, sin = (torch.cos(ang) * f).float().to(DEV), (torch.sin(ang) * f).float().to(DEV)
    pages = torch.zeros((4, 1, 64, row), dtype=dtype, device=DEV)
    rows = torch.empty((T, row), dtype=dtype, device=DEV)
    kernels.latent_rows(proj, None, off_q=0, off_kv=50, q_rank=0, kv_rank=n, rot_dim=r, row_width=row, q_weight=None,
                        kv_weight=wkv, eps=1e-5, cos=cos, sin=sin, rot_dims=r, paired=False, tok_pos=_ints(pos),
                        tok_seq=_ints([0] * T), new_lens=_ints([140]), row_out=rows, pages=pages, block_table=_ints([[3, 1]]),
                        table_width=2, page_tokens=64, ring_pages=ring, out_dtype=dtype)
    P = proj.double().cpu()
    want = torch.zeros(T, row, dtype=torch.float64)
    want[:, :n] = pf.rms_norm(P[:, 50:50 + n], wkv.double().cpu(), 1e-5)
    want[:, n:n + r] = pf.rotate(P[:, 50 + n:].reshape(T, 1, r), torch.tensor(pos), r, 1e4, "halves",
                                 {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}).reshape(T, r)
    _close(rows, want, 1e-5 if dtype == torch.float32 else 1e-2, "rows")
    for t, p in enumerate(pos):
        assert torch.equal(pages[[3, 1][(p // 64) % ring], 0, p % 64], rows[t]), p
