"""Furesun through the engine against the plain implementation: whole prompts, token-by-token decoding from a prompt
and from the very first token, prompts in portions, unequal batches against each request alone, slots, pages and
states used again, decoding far past every window, keys at the windows' edges, generation through the entry points
and trace replay (GPU)."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_furesun as pf
from furesun_cases import CASES, Want, check_rows, folder, oracle, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..")
# max |difference| relative to the oracle's largest logit; in bfloat16 three times a row's own rounding noise on top
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
# The sharp model runs in float32 only: its scores reach hundreds, its rows hang on single keys, and bfloat16 turns
# such rows from one key to another in any implementation.  Float32 rounds the same scores a hundred times less than
# its usual bound allows for: a lost key still moves a row by its whole size.
SHARP_F32 = 2e-3


CASES_BY_DTYPE = [(n, d) for n in sorted(CASES) for d in ("float32", "bfloat16") if not (n == "s" and d == "bfloat16")]


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("furesun")


def _engine(path, dtype, **kw):
    from tq_kv_b200.engine import Engine
    kw.setdefault("max_tokens", 1024)
    return Engine.from_folder(path, dtype=dtype, **kw)


def _check(got, want, dtype, what):
    tol = TOL[dtype]
    if what.startswith("s "):
        tol = SHARP_F32
    check_rows(got, want, dtype, "furesun " + what, tol)


@pytest.mark.parametrize("name,dtype", CASES_BY_DTYPE)
def test_whole_prompts_and_decoding_token_by_token(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name, alike_experts=dtype == "bfloat16")
    eng = _engine(path, dtype)
    V = CASES[name]["vocab"]
    for n in (1, 2, 3, 70, 260):                             # the first tokens alone; over one and four pages
        toks = tokens(n, V, 10 + n)
        s = eng.new_sequence()
        _check(eng.step([StepRow(s, toks, list(range(n)))]), oracle(path, toks), dtype, f"{name} whole {n}")
        eng.release(s)
    toks = tokens(260, V, 210)
    want = oracle(path, toks)
    s = eng.new_sequence()
    got = [eng.step([StepRow(s, toks[:150], [149])])]
    for t in range(150, 260):                                # replayed graphs from the second step on
        got.append(eng.step([StepRow(s, [toks[t]], [0])]))
    _check(torch.cat(got), want[149:], dtype, f"{name} decode")
    eng.release(s)
    s = eng.new_sequence()                                   # the same slot, its state zeroed: from the very first token
    got = [eng.step([StepRow(s, [toks[t]], [0])]) for t in range(12)]
    _check(torch.cat(got), want[:12], dtype, f"{name} decode from the first token")
    eng.release(s)
    assert eng.cache.free_slots == eng.cache.max_slots
    eng.cache.book.check()


@pytest.mark.parametrize("name,dtype", CASES_BY_DTYPE)
def test_prompts_in_portions(tmp_root, name, dtype):
    """Portions down to one and two tokens, across page edges and window edges; the memory's state and running
    maximum are handed from portion to portion."""
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name, alike_experts=dtype == "bfloat16")
    eng = _engine(path, dtype)
    toks = tokens(180, CASES[name]["vocab"], 77)
    want = oracle(path, toks)
    for cuts in ((2, 2, 60, 1, 63, 52), (64, 64, 52), (1, 1, 1, 2, 64, 64, 47), (127, 2, 51), (3, 61, 64, 52)):
        assert sum(cuts) == 180
        s, at, got = eng.new_sequence(), 0, []
        for n in cuts:
            got.append(eng.step([StepRow(s, toks[at:at + n], list(range(n)))]))
            at += n
        _check(torch.cat(got), want, dtype, f"{name} portions {cuts}")
        eng.release(s)


@pytest.mark.parametrize("name,dtype", CASES_BY_DTYPE)
def test_unequal_batches_against_each_alone_and_slots_used_again(tmp_root, name, dtype):
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name, alike_experts=dtype == "bfloat16")
    eng = _engine(path, dtype, max_tokens=896, max_slots=4)
    V = CASES[name]["vocab"]
    for round_ in range(3):                                  # the same slots, pages and states serve three batches
        lens = [(1, 130, 66), (64, 2, 200), (129, 65, 1)][round_]
        extra = [12, 30, 20]                                 # tokens decoded after the prompt; rows end at different steps
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
                    eng.release(slots[i])                    # its slot, pages and state go back while the others go on
        for i in range(3):
            _check(torch.cat(got[i]), wants[i][lens[i] - 1:], dtype, f"{name} batch round {round_} row {i}")
        assert eng.cache.free_slots == 4
        eng.cache.book.check()


@pytest.mark.parametrize("name,dtype", [x for x in CASES_BY_DTYPE if x[0] != "c"])
def test_a_new_prompt_beside_decoding_rows_and_a_long_decode(tmp_root, name, dtype):
    """A prompt joins a row that decodes (through the paged path), and 400 tokens are decoded one by one: every
    window passes over decoded tokens and every ring wraps."""
    from tq_kv_b200.engine import StepRow
    path = folder(tmp_root, name, alike_experts=dtype == "bfloat16")
    eng = _engine(path, dtype)
    V = CASES[name]["vocab"]
    a, b = tokens(440, V, 41), tokens(50, V, 42)
    wa, wb = oracle(path, a), oracle(path, b)
    sa = eng.new_sequence()
    got_a = [eng.step([StepRow(sa, a[:40], [39])])]
    sb = eng.new_sequence()
    out = eng.step([StepRow(sa, [a[40]], [0]), StepRow(sb, b[:50], [0, 49])])      # a prompt beside a decoding row
    got_a.append(out[:1])
    _check(out[1:], Want.cat([wb[0], wb[49]]), dtype, f"{name} the prompt beside a decoding row")
    eng.release(sb)
    for t in range(41, 440):
        got_a.append(eng.step([StepRow(sa, [a[t]], [0])]))
    _check(torch.cat(got_a), wa[39:], dtype, f"{name} long decode")
    eng.release(sa)


# ---- keys at the windows' edges ----------------------------------------------------------------------------------
def _window_cfg():
    """One attention layer whose keys a second layer reads with a narrower window, and a latent attention, without
    feed-forwards: few keys carry a row, so that the key that enters or leaves a window moves it."""
    from furesun_cases import attn, latent, model
    return model(120, 64, 1e-5, [
        {**attn(2, 1, 32, 32, 70, 1.0, cap=80.0), "mlp": None},
        {**attn(2, 1, 32, 32, 64, 1.0, cap=80.0, kv_from=0), "mlp": None},
        {**latent(2, 16, 16, 16, 24, 65, 1.0), "mlp": None},
    ])


def test_a_window_one_key_off_moves_the_probed_rows():
    """The oracle itself: with any window one key wider or narrower the rows that the edge tests read move by a
    fifth of the largest logit or more: thousands of times the float32 bound, and several times what an ordinary
    row's bfloat16 bound allows."""
    import copy
    from furesun_cases import make_weights
    cfg = _window_cfg()
    w = make_weights(cfg, 9)
    toks = tokens(200, cfg["vocab"], 13)
    base = pf.decoder(cfg, w, toks)
    scale = float(base.abs().max())
    for delta in (-1, 1):
        for layer in range(3):
            c2 = copy.deepcopy(cfg)
            c2["layers"][layer]["mixer"]["mask"]["size"] += delta
            moved = float((pf.decoder(c2, w, toks)[100:] - base[100:]).abs().max()) / scale
            assert moved > 0.2, (layer, delta, moved)
    noise = (pf.decoder(cfg, w, toks, rounding=lambda t: t.to(torch.bfloat16).to(t.dtype)) - base).abs().amax(dim=1) / scale
    assert float(noise.median()) < 0.03


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_just_inside_and_outside_the_windows(tmp_root, dtype):
    """Prompts cut so that steps begin at, one before and one after the places where position 0, a page's first
    key and a window's oldest key leave the windows of 64, 65 and 70; then the same places decoded one by one."""
    from tq_kv_b200.engine import StepRow
    from furesun_cases import make_weights
    cfg = _window_cfg()
    path = pf.write_folder(os.path.join(str(tmp_root), "windows"), cfg, make_weights(cfg, 9))
    eng = _engine(path, dtype)
    toks = tokens(200, cfg["vocab"], 13)
    want = oracle(path, toks)

    def check(got, w, what):
        check_rows(got, w, dtype, "furesun windows " + what, TOL[dtype])

    s = eng.new_sequence()
    check(eng.step([StepRow(s, toks, list(range(200)))]), want, "whole")
    eng.release(s)
    for cuts in ((63, 1, 1, 1, 4, 58, 1, 1, 1, 64, 5), (64, 6, 58, 6, 64, 2), (65, 64, 5, 1, 63, 2), (69, 1, 64, 64, 2)):
        assert sum(cuts) == 200
        s, at, got = eng.new_sequence(), 0, []
        for n in cuts:
            got.append(eng.step([StepRow(s, toks[at:at + n], list(range(n)))]))
            at += n
        check(torch.cat(got), want, f"portions {cuts}")
        eng.release(s)
    s = eng.new_sequence()
    got = [eng.step([StepRow(s, toks[:60], [59])])]
    for t in range(60, 200):                                 # positions 63 .. 70 and 127 .. 134 are decoded alone
        got.append(eng.step([StepRow(s, [toks[t]], [0])]))
    check(torch.cat(got), want[59:], "decoded across the edges")
    eng.release(s)


# ---- the entry points -------------------------------------------------------------------------------------------
def test_greedy_generation_through_the_entry_point_and_the_command_line(tmp_root):
    import tq_kv_b200 as tq
    path = folder(tmp_root, "c")
    cfg, w = pf.read_folder(path)
    prompts = [tokens(n, cfg["vocab"], 300 + n) for n in (3, 20, 9)]
    want = [pf.greedy(cfg, w, p, 10) for p in prompts]
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


def test_greedy_generation_of_a_model_without_a_memory(tmp_root):
    """Without a mixer that keeps state the engine pads whole prompts to the sizes of captured graphs: the padded
    rows must reach neither a cache, nor the keys a later layer borrows, nor a real row's result."""
    import tq_kv_b200 as tq
    from furesun_cases import attn, dense, latent, make_weights, model, moe
    cfg = model(210, 96, 1e-6, [
        {**attn(4, 2, 24, 16, 40, 0.2, cap=20.0, dims=12), "mlp": moe(48, 4, 2, 1.5, shared=40)},
        {**latent(2, 16, 8, 24, 40, 50, 0.2, scaling=(4.0, 64, 16.0, 2.0)), "mlp": dense(120)},
        {**attn(4, 2, 24, 16, 70, 0.2, cap=20.0, dims=12, kv_from=0), "mlp": None},
    ], cap=20.0)
    path = pf.write_folder(os.path.join(str(tmp_root), "no_memory"), cfg, make_weights(cfg, 31))
    c, w = pf.read_folder(path)
    prompts = [tokens(n, cfg["vocab"], 500 + n) for n in (1, 5, 63, 64, 65, 130)]
    want = [pf.greedy(c, w, p, 12) for p in prompts]
    eng = tq.load(path, dtype="float32", max_batch=3, max_context=256)
    assert eng.model.padded_rows_ok
    for group in (prompts[:3], prompts[3:], prompts[5:]):                 # batches of three, and a prompt alone
        res = eng.generate(group, tq.GenerationParams.greedy(12, stop_token_ids=()))
        for r, p in zip(res, group):
            wt = want[prompts.index(p)]
            n = next((i for i, (x, y) in enumerate(zip(r.tokens, wt)) if x != y), 12)
            if n < 12:                                                      # a tie within float32 rounding, or a fault
                row = pf.decoder(c, w, p + wt[:n])[-1]
                assert abs(float(row[r.tokens[n]] - row[wt[n]])) < 1e-4 * float(row.abs().max()), (len(p), n, r.tokens, wt)
    assert eng.cache.free_slots == 3


def test_greedy_generation_past_the_windows_with_requests_that_wait_for_a_slot(tmp_root):
    """Five requests on two slots: each generates far past the windows of the model; the scheduler gives freed
    slots, pages and states to the waiting ones."""
    import tq_kv_b200 as tq
    path = folder(tmp_root, "a")
    cfg, w = pf.read_folder(path)
    prompts = [tokens(n, cfg["vocab"], 400 + n) for n in (2, 70, 31, 5, 66)]
    want = [pf.greedy(cfg, w, p, 80, torch.float32) for p in prompts]
    eng = tq.load(path, dtype="float32", max_batch=2, max_context=192)
    res = eng.generate(prompts, tq.GenerationParams.greedy(80, stop_token_ids=()))
    for r, wt, p in zip(res, want, prompts):
        # two logits may tie within float32 rounding: compare up to the first difference and make sure that it is a tie
        n = next((i for i, (x, y) in enumerate(zip(r.tokens, wt)) if x != y), 80)
        if n < 80:
            row = pf.decoder(cfg, w, p + wt[:n])[-1]
            assert abs(float(row[r.tokens[n]] - row[wt[n]])) < 1e-4 * float(row.abs().max()), (n, r.tokens, wt)
    assert eng.cache.free_slots == 2
    eng.cache.book.check()


def test_trace_replay_as_a_program(tmp_root, tmp_path):
    import numpy as np
    V = CASES["b"]["vocab"]
    a, b = tokens(100, V, 5), tokens(40, V, 6)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:90], "want": [0, 89]}, {"id": "y", "tokens": b[:38], "want": [37]}],
              "end": []}]
    for i in range(10):
        e = [{"id": "x", "tokens": [a[90 + i]], "want": [0]}]
        if i < 2:
            e.append({"id": "y", "tokens": [b[38 + i]], "want": [0] if i else []})
        steps.append({"step": i + 1, "entries": e, "end": ["y"] if i == 1 else (["x"] if i == 9 else [])})
    for dtype in ("float32", "bfloat16"):
        path = folder(tmp_root, "b", alike_experts=dtype == "bfloat16")
        wa, wb = oracle(path, a), oracle(path, b)
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
    """`furesun-tiny` with random weights: the engine made on the device and the folder written on the host hold the
    same weights, and the oracle agrees with both."""
    from tq_kv_b200.config import named_shape
    from tq_kv_b200.engine import Engine, StepRow
    from tq_kv_b200.weights import write_model_folder
    cfg = named_shape("furesun-tiny")
    path = write_model_folder(cfg, str(tmp_path / "m"), 3)
    toks = tokens(90, cfg["vocab"], 4)
    want = oracle(path, toks)
    for eng in (Engine.from_random(cfg, 3, dtype="float32", max_tokens=256),
                Engine.from_folder(path, dtype="float32", max_tokens=256)):
        s = eng.new_sequence()
        _check(eng.step([StepRow(s, toks, list(range(90)))]), want, "float32", "named shape, random weights")
