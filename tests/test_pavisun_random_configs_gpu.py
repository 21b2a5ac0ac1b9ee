"""Seeded random Pavisun configurations (sizes, head counts, layer order, windows, kept tokens, constants, streams and
loops all drawn) through the engine in both precisions against the plain implementation: a whole prompt over several
pages, its last tokens one by one, and an unequal batch that decodes together (GPU)."""
import os
import random

import pytest
import torch

import plain_pavisun as pp
from pavisun_cases import check_rows, make_weights, oracle, tokens

pytestmark = pytest.mark.gpu
# max |difference| relative to the oracle's largest logit; in bfloat16 three times a row's own rounding noise on top
TOL = {"float32": 6e-5, "bfloat16": 3e-2}


def _divisor(rng, n):
    return rng.choice([d for d in range(1, n + 1) if n % d == 0])


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    layers = []
    for _ in range(rng.randint(2, 5)):
        heads = rng.choice([1, 2, 3, 4, 6, 8])
        kv = _divisor(rng, heads)
        d = rng.choice([8, 16, 24, 32, 40, 64, 96, 128])
        window = rng.choice([None, 1, 2, 7, 33, 64, 65, 100, 128, 150, 300])
        if rng.random() < 0.5:
            dims = rng.choice([x for x in (2, 4, 8, 16, 24, 32, 64, 96, 128) if x <= d] + [d])
            rot = {"base": rng.choice([1e4, 5e4, 1e6, 300.0]), "dims": dims}
            if rng.random() < 0.6:
                rot["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0, 32.0]), "original": rng.choice([32, 64, 512, 4096]),
                                  "fast": rng.choice([8.0, 32.0, 64.0]), "slow": rng.choice([0.5, 1.0, 2.0])}
            m = {"heads": heads, "kv_heads": kv, "dim": d, "vdim": d, "rot": rot, "scale": d ** -0.5 * rng.choice([0.6, 1.0, 2.0])}
            if rng.random() < 0.7:
                m["softcap"] = rng.choice([5.0, 20.0, 50.0])
            if window:
                m["mask"] = {"size": window}
            kind = "attention"
        else:
            m = {"heads": heads, "kv_heads": kv, "dim": d, "vdim": rng.choice([8, 16, 32, 48, 64, 128]),
                 "scale": d ** -0.5 * rng.choice([1.0, 4.0, 9.0])}
            if window:
                m["mask"] = {"size": window}
                keep = rng.choice([0, 0, 1, 2, 6, 64, 70])
                if keep:
                    m["mask"]["keep_first"] = keep
            kind = "attention_2"
        mlp = None
        if rng.random() < 0.8:
            experts = rng.choice([1, 2, 3, 5, 8, 16])
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([16, 40, 64, 96, 200])},
                   "router": {"experts": experts, "top": rng.randint(1, min(4, experts))}}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Pavisun", "vocab": rng.randint(100, 700), "width": rng.choice([64, 72, 96, 136, 192, 256]),
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    streams = rng.choice([None, 1, 2, 3, 4, 5, 8])
    if streams:
        cfg["streams"] = streams
    if rng.random() < 0.6:
        a = rng.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": a, "stop": rng.randint(a + 1, len(layers)), "times": rng.randint(1, 3)}
    if rng.random() < 0.6:
        cfg["logit_softcap"] = rng.choice([10.0, 30.0, 50.0])
    return cfg


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("pavisun_random")


@pytest.mark.parametrize("seed", list(range(12)))
def test_a_random_configuration_whole_decoded_and_batched(tmp_root, seed):
    from tq_kv_b200.engine import Engine, StepRow
    cfg = random_config(seed)
    path = pp.write_folder(os.path.join(str(tmp_root), f"m{seed}"), cfg, make_weights(cfg, seed))
    V = cfg["vocab"]
    long_, short, mid = tokens(360, V, seed), tokens(40, V, seed + 100), tokens(139, V, seed + 200)
    want = {id(t): oracle(path, t) for t in (long_, short, mid)}
    for dtype in ("float32", "bfloat16"):
        eng = Engine.from_folder(path, dtype=dtype, max_tokens=1024)
        what = f"random {seed} {[l['type'] for l in cfg['layers']]} {dtype}"
        s = eng.new_sequence()
        got = [eng.step([StepRow(s, long_[:290], list(range(290)))])]
        got += [eng.step([StepRow(s, [t], [0])]) for t in long_[290:]]
        check_rows(torch.cat(got), want[id(long_)], dtype, what + " whole and decoded", TOL[dtype])
        eng.release(s)
        reqs, cut = [short, mid, long_[:200]], [30, 129, 190]
        slots = [eng.new_sequence() for _ in reqs]
        out = eng.step([StepRow(sl, r[:c], [c - 1]) for sl, r, c in zip(slots, reqs, cut)])
        got = [[out[i:i + 1]] for i in range(3)]
        for step in range(10):
            out = eng.step([StepRow(sl, [r[c + step]], [0]) for sl, r, c in zip(slots, reqs, cut)])
            for i in range(3):
                got[i].append(out[i:i + 1])
        for i, (r, c) in enumerate(zip(reqs, cut)):
            ref = want[id(long_)] if r is not short and r is not mid else want[id(r)]
            check_rows(torch.cat(got[i]), ref[c - 1:c + 10], dtype, what + f" batch row {i}", TOL[dtype])
        for sl in slots:
            eng.release(sl)
        assert eng.cache.free_slots == eng.cache.max_slots
        eng.cache.book.check()
