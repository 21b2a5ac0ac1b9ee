"""Pavisun through the engine against the plain implementation: whole prompts, token-by-token decoding, prompts in
portions, unequal batches, slots and pages used again, long decoding past every window, rows that hang on one planted
key (far back, at page edges, just inside and just outside a window, among the kept first tokens and right after
them), generation through the entry points (GPU)."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_pavisun as pp
from pavisun_cases import CASES, Want, _model, _rot, _unit, check_rows, folder, make_weights, oracle, oracle_logits, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
# max |difference| relative to the oracle's largest logit: in float32 twice the largest error seen; in bfloat16 the
# package's bound, and on top three times the change that rounding the oracle's own activations to bfloat16 causes
# in that row (pavisun_cases.Want): rows that hang on a small norm or on two nearly equal scores move by a tenth of
# the logits' size under such rounding, in the oracle as in the engine, while a lost or a wrongly seen key moves the
# planted rows by all of it; float32 keeps the tight bound everywhere.
TOL = {"float32": 6e-5, "bfloat16": 3e-2}
# The sharp model's scores reach some hundreds (unit-size q and k times a large scale): rounding q and k to bfloat16
# moves a score by about one, differently for every order of summation, so one realisation of the rounding does not
# bound another; its bfloat16 rows get a tenth of the largest logit, its float32 rows the tight bound.
SHARP_BF16 = 0.1


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("pavisun")


def _engine(path, dtype, **kw):
    from tq_kv_b200.engine import Engine
    kw.setdefault("max_tokens", 2048)
    return Engine.from_folder(path, dtype=dtype, **kw)


def _check(got, want: Want, dtype, what, sharp=False):
    tol = SHARP_BF16 if dtype == "bfloat16" and what.startswith("s ") else TOL[dtype]
    check_rows(got, want, dtype, "pavisun " + what, tol)


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_decoding_token_by_token(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name)
    eng = _engine(path, dtype)
    V = CASES[name]["vocab"]
    for n in (1, 2, 3, 70, 260):                             # the first tokens alone; over two and five pages
        toks = tokens(n, V, 10 + n)
        want = oracle(path, toks)
        s = eng.new_sequence()
        _check(eng.step([StepRow(s, toks, list(range(n)))]), want, dtype, f"{name} whole {n}")
        eng.release(s)
    toks = tokens(260, V, 210)
    want = oracle(path, toks)
    s = eng.new_sequence()
    got = [eng.step([StepRow(s, toks[:150], [149])])]
    for t in range(150, 260):                                # replayed graphs from the second step on
        got.append(eng.step([StepRow(s, [toks[t]], [0])]))
    _check(torch.cat(got), want[149:], dtype, f"{name} decode")
    eng.release(s)
    s = eng.new_sequence()                                   # from the very first token on, one by one
    got = [eng.step([StepRow(s, [t], [0])]) for t in toks[:12]]
    _check(torch.cat(got), want[:12], dtype, f"{name} decode from the first token")
    eng.release(s)
    assert eng.cache.free_slots == eng.cache.max_slots
    eng.cache.book.check()


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_in_portions(tmp_root, name, dtype):
    """Portions down to one and two tokens, across page edges and across every window of the cases.  A layer with
    a window keeps a ring of window + window_chunk - 1 keys: with the default of 64 every continuing portion has at
    most 64 tokens and the rings wrap early; an engine made for portions of 288 takes the larger ones."""
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name)
    toks = tokens(280, CASES[name]["vocab"], 77)
    want = oracle(path, toks)
    plans = [({}, ((200, 2, 2, 2, 64, 10), (2, 2, 60, 1, 63, 52, 36, 64), (1, 1, 1, 2, 64, 64, 64, 64, 19),
                   (127, 2, 51, 36, 64))),
             ({"window_chunk": 288, "max_tokens": 4096}, ((2, 2, 60, 1, 63, 52, 100), (64, 64, 64, 88), (1, 1, 1, 2, 275),
                                                          (3, 61, 216)))]
    for options, all_cuts in plans:
        eng = _engine(path, dtype, **options)
        for cuts in all_cuts:
            assert sum(cuts) == 280
            s, at, got = eng.new_sequence(), 0, []
            for n in cuts:
                got.append(eng.step([StepRow(s, toks[at:at + n], list(range(n)))]))
                at += n
            _check(torch.cat(got), want, dtype, f"{name} portions {cuts}")
            eng.release(s)
        del eng


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_against_each_alone_and_slots_used_again(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name)
    eng = _engine(path, dtype, max_tokens=900, max_slots=4)
    V = CASES[name]["vocab"]
    for round_ in range(3):                                  # the same slots and pages serve three batches
        lens = [(1, 130, 66), (64, 2, 210), (129, 65, 1)][round_]
        extra = [12, 45, 20]                                 # tokens decoded after the prompt; rows end at different steps
        reqs = [tokens(n + m, V, 100 * round_ + n) for n, m in zip(lens, extra)]
        wants = [oracle(path, r) for r in reqs]
        slots = [eng.new_sequence() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step([StepRow(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, lens)])
        for i in range(3):
            got[i].append(out[i:i + 1])
        live = [0, 1, 2]
        for step in range(max(extra)):
            live = [i for i in live if step < extra[i]]
            out = eng.step([StepRow(slots[i], [reqs[i][lens[i] + step]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            for i in list(live):
                if step + 1 == extra[i]:
                    eng.release(slots[i])                    # its slot and pages go back while the others go on
        for i in range(3):
            _check(torch.cat(got[i]), wants[i][lens[i] - 1:], dtype, f"{name} batch round {round_} row {i}")
        assert eng.cache.free_slots == 4
        eng.cache.book.check()


@pytest.mark.parametrize("name", ["a", "d"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_new_prompt_beside_decoding_rows_and_a_long_decode(tmp_root, name, dtype):
    """A prompt joins rows that decode (through the paged path), and 400 tokens are decoded one by one: every
    window passes over decoded tokens several times and the rings of keys wrap."""
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name)
    V = CASES[name]["vocab"]
    eng = _engine(path, dtype, window_chunk=128, max_tokens=4096)      # a prompt of 70 tokens beside a decoding row
    a, b = tokens(430, V, 1), tokens(90, V, 2)
    wa, wb = oracle(path, a), oracle(path, b)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    got_a = [eng.step([StepRow(sa, a[:30], [29])])]
    out = eng.step([StepRow(sa, [a[30]], [0]), StepRow(sb, b[:70], [0, 69])])
    got_a.append(out[:1])
    got_b = [out[1:]]
    for t in range(31, 430):
        rows = [StepRow(sa, [a[t]], [0])]
        if 70 + (t - 31) < 90:
            rows.append(StepRow(sb, [b[70 + t - 31]], [0]))
        out = eng.step(rows)
        got_a.append(out[:1])
        if len(rows) == 2:
            got_b.append(out[1:])
    _check(torch.cat(got_a), wa[29:], dtype, f"{name} long decode")
    _check(torch.cat(got_b), Want.cat([wb[:1], wb[69:]]), dtype, f"{name} prompt beside decoding rows")


# ---- rows that hang on one planted key ------------------------------------------------------------------------------
# Two models whose first layer is the mixer under test (so that its input is a function of the token id alone).  For a
# pair of token ids (a, b) the embedding of b is made so that b's key in one head points along a's query in that head
# (for the rotating mixer: along a's query turned by a chosen distance D, so that the score peaks when a stands D
# tokens after b).  In a sequence of other tokens with one b and a few a's, an a that sees b gives it nearly all its
# weight, and an a that does not see it spreads its weight: a window or a count of kept tokens that is off by one, a
# lost page or a lost far key changes such a row by the size of the logits.
ROT_WINDOW, UNIT_WINDOW, UNIT_KEEP = 520, 100, 5
PLANT_ROT = _model(160, 64, 1e-5, [
    {**_rot(2, 1, 32, ROT_WINDOW, 0.3, cap=40.0), "mlp": None},
    {**_unit(2, 2, 16, 16, 50, 2, 1.0), "mlp": None},
], streams=2)
PLANT_UNIT = _model(160, 64, 1e-5, [
    {**_unit(2, 2, 32, 32, UNIT_WINDOW, UNIT_KEEP, 1.3), "mlp": None},
    {**_rot(2, 1, 16, 30, 0.25), "mlp": None},
], streams=2)
# (key position, distances of the queries behind it, D for the rotating mixer)
ROT_PROBES = [(0, (399, 400, 401), 400), (63, (518, 519, 520, 521), 519), (64, (518, 519, 520, 521), 519),
              (5, (58, 59, 60), 59), (130, (1, 2, 3), 2)]
UNIT_PROBES = [(4, (99, 100, 101, 300, 600), 0), (5, (98, 99, 100, 101, 300), 0), (0, (1, 99, 100, 640), 0),
               (63, (1, 98, 99, 100, 101), 0), (64, (64, 99, 100), 0), (200, (99, 100), 0)]


def _plant(cfg, w, pairs):
    """embed[b] for every (a, b, D) of `pairs`, in place: b's key in the last head along a's (turned) query."""
    c, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    H, G, d = c["heads"], c["kv_heads"], c["dim"]
    f = {n: t.double() for n, t in w.items() if t.is_floating_point()}
    read = float(f["l0.hc1.in"].sum()) if cfg.get("streams") else 1.0
    wq, wk = f["l0.mix.q"][(H - 1) * d:], f["l0.mix.k"][(G - 1) * d:]
    for a, b, D in pairs:
        h = pp.rms_norm(read * f["embed"][a], f["l0.norm1"], eps)
        q = wq @ h
        if cfg["layers"][0]["type"] == "attention":
            rot = c["rot"]
            q = pp.rotate_halves(q.reshape(1, 1, d), torch.tensor([D]), rot["dims"], rot["base"], rot.get("scaling"))[0, 0]
        h_b = torch.linalg.pinv(wk) @ q
        w["embed"][b] = (h_b / f["l0.norm1"] / read * (8.0 / h_b.abs().max())).to(torch.bfloat16)


def _planted(tmp_root, which):
    cfg, probes = (PLANT_ROT, ROT_PROBES) if which == "rot" else (PLANT_UNIT, UNIT_PROBES)
    w = make_weights(cfg, 11)
    pairs = [(10 + 2 * i, 11 + 2 * i, D) for i, (_, _, D) in enumerate(probes)]
    _plant(cfg, w, pairs)
    path = pp.write_folder(os.path.join(str(tmp_root), "planted_" + which), cfg, w)
    seqs = []
    for i, ((j, dists, _), (a, b, _)) in enumerate(zip(probes, pairs)):
        g = torch.Generator().manual_seed(50 + i)
        toks = torch.randint(40, cfg["vocab"], (j + max(dists) + 3,), generator=g).tolist()   # ids 10 .. 39 are planted
        toks[j] = b
        for dist in dists:
            toks[j + dist] = a
        seqs.append((toks, [j + dist for dist in dists]))
    return cfg, path, seqs


def _with_mask(cfg, **change):
    new = json.loads(json.dumps(cfg))
    new["layers"][0]["mixer"]["mask"].update(change)
    return new


@pytest.mark.parametrize("which", ["rot", "unit"])
def test_the_planted_keys_decide_their_rows(tmp_root, which):
    """The test's own premise, on the plain implementation (no GPU work): a window one token wider or narrower, one
    kept token more or fewer, or a window that loses the far key changes the probed rows by much of the logits' size,
    and rounding to bfloat16 changes them by far less."""
    cfg, path, seqs = _planted(tmp_root, which)
    w = pp.read_folder(path)[1]
    faults = [dict(size=ROT_WINDOW + 1), dict(size=ROT_WINDOW - 1), dict(size=300)] if which == "rot" else \
        [dict(size=UNIT_WINDOW + 1), dict(size=UNIT_WINDOW - 1), dict(keep_first=UNIT_KEEP + 1), dict(keep_first=UNIT_KEEP - 1),
         dict(keep_first=0)]
    seen, allowed = [0.0] * len(faults), 0.0
    for toks, rows in seqs:
        full = oracle(path, toks)
        want, scale = full.logits[rows], float(full.logits.abs().max())
        allowed = max(allowed, TOL["bfloat16"] + 3.0 * float(full.noise[rows].max()) / scale)
        for n, fault in enumerate(faults):
            other = pp.decoder(_with_mask(cfg, **fault), w, toks)[rows]
            seen[n] = max(seen[n], float((other - want).abs().max() / scale))
    assert min(seen) > 0.3, (faults, seen)
    assert allowed < 0.1, allowed          # what the bfloat16 bound lets pass on the probed rows is a third of a fault


@pytest.mark.parametrize("which", ["rot", "unit"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rows_that_hang_on_planted_keys_in_prompts_portions_and_decoding(tmp_root, which, dtype):
    from tq_kv_b200.engine import StepRow
    cfg, path, seqs = _planted(tmp_root, which)
    eng = _engine(path, dtype)
    wide = _engine(path, dtype, window_chunk=1024, max_tokens=8192)    # takes portions of up to 1,024 tokens
    for n, (toks, rows) in enumerate(seqs):
        T, first = len(toks), rows[0]
        want = oracle(path, toks)
        s = eng.new_sequence()
        _check(eng.step([StepRow(s, toks, list(range(T)))]), want, dtype, f"planted {which} {n} whole", sharp=True)
        eng.release(s)
        cuts = [c for c in (1, 64, first - 1, first, first + 1, first + 3, T) if 0 < c <= T]
        cuts = sorted(set(cuts))
        s, at, got = wide.new_sequence(), 0, []
        for c in cuts:                                       # portions that begin at and around the probed rows
            got.append(wide.step([StepRow(s, toks[at:c], list(range(c - at)))]))
            at = c
        _check(torch.cat(got), want, dtype, f"planted {which} {n} portions {cuts}", sharp=True)
        wide.release(s)
        s = eng.new_sequence()
        start = max(1, first - 3)
        got = [eng.step([StepRow(s, toks[:start], [start - 1])])]
        got += [eng.step([StepRow(s, [t], [0])]) for t in toks[start:]]
        _check(torch.cat(got), want[start - 1:], dtype, f"planted {which} {n} decoded", sharp=True)
        eng.release(s)
    # all probes as one unequal batch, then decoded together from before their first probed rows
    starts = [max(1, rows[0] - 2) for _, rows in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    eng.step([StepRow(s, toks[:st], []) for s, (toks, _), st in zip(slots, seqs, starts)])
    got = [[] for _ in seqs]
    for step in range(max(len(t) - st for (t, _), st in zip(seqs, starts))):
        live = [i for i, ((t, _), st) in enumerate(zip(seqs, starts)) if st + step < len(t)]
        out = eng.step([StepRow(slots[i], [seqs[i][0][starts[i] + step]], [0]) for i in live])
        for k, i in enumerate(live):
            got[i].append(out[k:k + 1])
            if starts[i] + step + 1 == len(seqs[i][0]):
                eng.release(slots[i])
    for i, (toks, _) in enumerate(seqs):
        _check(torch.cat(got[i]), oracle(path, toks)[starts[i]:], dtype, f"planted {which} {i} in a batch", sharp=True)
    assert eng.cache.free_slots == eng.cache.max_slots


# Heads whose widths are no multiples of 8 (the kernels' rows are then padded inside): keys of 20 with 10 rotated
# entries, unit-size keys of 12 beside values of 20 and of 4, one layer run twice.
P_ODD = _model(200, 72, 1e-5, [
    {**_rot(3, 1, 20, 50, 0.3, cap=10.0, dims=10, scaling=(4.0, 32, 8.0, 1.0)), "mlp": None},
    {**_unit(2, 2, 12, 20, 40, 3, 1.2), "mlp": None},
    {**_unit(4, 2, 36, 4, None, 0, 0.9), "mlp": None},
], streams=2, loop=(1, 2, 2), cap=15.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_widths_that_are_no_multiple_of_8(tmp_root, dtype):
    from tq_kv_b200.engine import StepRow
    path = pp.write_folder(os.path.join(str(tmp_root), "odd_heads"), P_ODD, make_weights(P_ODD, 21))
    eng = _engine(path, dtype)
    a, b = tokens(150, 200, 31), tokens(70, 200, 32)
    wa, wb = oracle(path, a), oracle(path, b)
    s = eng.new_sequence()
    _check(eng.step([StepRow(s, a, list(range(150)))]), wa, dtype, "odd heads whole")
    eng.release(s)
    sa, sb = eng.new_sequence(), eng.new_sequence()
    out = eng.step([StepRow(sa, a[:100], [99]), StepRow(sb, b[:20], [19])])
    got_a, got_b = [out[:1]], [out[1:]]
    for t in range(50):
        out = eng.step([StepRow(sa, [a[100 + t]], [0]), StepRow(sb, [b[20 + t]], [0])])
        got_a.append(out[:1])
        got_b.append(out[1:])
    _check(torch.cat(got_a), wa[99:], dtype, "odd heads batch row 0")
    _check(torch.cat(got_b), wb[19:], dtype, "odd heads batch row 1")


# ---- the entry points -------------------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point_and_the_command_line(tmp_root):
    import tq_kv_b200 as tq
    path = folder(tmp_root, "c")
    cfg, w = pp.read_folder(path)
    prompts = [tokens(n, cfg["vocab"], 300 + n) for n in (3, 20, 9)]
    want = [pp.greedy(cfg, w, p, 10) for p in prompts]
    eng = tq.load(path, dtype="float32", max_batch=2, max_context=128)      # three requests, two slots
    res = eng.generate(prompts, tq.GenerationParams.greedy(10, stop_token_ids=()))
    assert [r.tokens for r in res] == want and all(r.finish_reason == "length" for r in res)
    assert eng.cache.free_slots == 2
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "tq"), "run", path, "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, prompts[1])), "-n", "10", "--temperature", "0",
                        "--repeat-penalty", "1.0", "--max-context", "128"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.strip().splitlines()[-1].split(",")] == want[1]


def test_greedy_generation_past_the_windows_with_requests_that_wait_for_a_slot(tmp_root):
    """Five requests on two slots in bfloat16 and float32: each generates far past the windows of the model; the
    scheduler gives freed slots and pages to the waiting ones."""
    import tq_kv_b200 as tq
    path = folder(tmp_root, "a")
    cfg, w = pp.read_folder(path)
    prompts = [tokens(n, cfg["vocab"], 400 + n) for n in (2, 70, 31, 5, 66)]
    want = [pp.greedy(cfg, w, p, 60, torch.float32) for p in prompts]
    eng = tq.load(path, dtype="float32", max_batch=2, max_context=192)
    res = eng.generate(prompts, tq.GenerationParams.greedy(60, stop_token_ids=()))
    for r, wt, p in zip(res, want, prompts):
        # two logits may tie within float32 rounding: compare up to the first difference and make sure that it is a tie
        n = next((i for i, (x, y) in enumerate(zip(r.tokens, wt)) if x != y), 60)
        if n < 60:
            row = pp.decoder(cfg, w, p + wt[:n])[-1]
            assert abs(float(row[r.tokens[n]] - row[wt[n]])) < 1e-4 * float(row.abs().max()), (n, r.tokens, wt)
    assert eng.cache.free_slots == 2
    eng.cache.book.check()


def test_trace_replay_as_a_program(tmp_root, tmp_path):
    import numpy as np
    path = folder(tmp_root, "b")
    V = CASES["b"]["vocab"]
    a, b = tokens(100, V, 5), tokens(40, V, 6)
    wa, wb = oracle(path, a), oracle(path, b)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:90], "want": [0, 89]}, {"id": "y", "tokens": b[:38], "want": [37]}],
              "end": []}]
    for i in range(10):
        e = [{"id": "x", "tokens": [a[90 + i]], "want": [0]}]
        if i < 2:
            e.append({"id": "y", "tokens": [b[38 + i]], "want": [0] if i else []})
        steps.append({"step": i + 1, "entries": e, "end": ["y"] if i == 1 else (["x"] if i == 9 else [])})
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
        first = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, V).copy())
        _check(first, Want.cat([wa[0], wa[89], wb[37]]), dtype, "trace step 0")
        last = torch.from_numpy(np.fromfile(out / "10.f32", dtype="<f4").reshape(1, V).copy())
        _check(last, wa[99:100], dtype, "trace last step")
        two = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, V).copy())
        _check(two, Want.cat([wa[91], wb[39]]), dtype, "trace step 2")


def test_random_weights_from_a_named_shape(tmp_path):
    """`pavisun-tiny` with random weights: the engine made on the device and the folder written on the host hold the
    same weights, and the oracle agrees with both."""
    from tq_kv_b200.config import named_shape
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.weights import write_model_folder
    cfg = named_shape("pavisun-tiny")
    path = write_model_folder(cfg, str(tmp_path / "m"), 3)
    toks = tokens(90, cfg["vocab"], 4)
    want = oracle(path, toks)
    for eng in (Engine.from_random(cfg, 3, dtype="float32", max_tokens=256),
                Engine.from_folder(path, dtype="float32", max_tokens=256)):
        s = eng.new_sequence()
        _check(eng.step([StepRow(s, toks, list(range(90)))]), want, "float32", "named shape, random weights")
