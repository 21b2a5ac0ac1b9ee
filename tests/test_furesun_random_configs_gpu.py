"""Seeded random Furesun configurations (sizes, head counts, layer order, windows, constants, who reads whose keys all
drawn) through the engine in both precisions against the plain implementation: a whole prompt over several pages, its
last tokens one by one, and an unequal batch that decodes together (GPU)."""
import os
import random

import pytest
import torch

import plain_furesun as pf
from furesun_cases import attn, check_rows, dense, latent, make_weights, memory, model, moe, oracle, tokens

pytestmark = pytest.mark.gpu
# max |difference| relative to the oracle's largest logit; in bfloat16 three times a row's own rounding noise on top
TOL = {"float32": 2e-4, "bfloat16": 3e-2}


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    layers = []
    for i in range(rng.randint(2, 6)):
        window = rng.choice([None, 1, 2, 7, 33, 64, 65, 100, 128, 150, 300])
        kind = rng.choice(["latent_attention", "mlstm", "attention", "attention"])
        scaling = rng.choice([None, (rng.choice([2.0, 8.0, 32.0]), rng.choice([32, 512, 4096]), rng.choice([8.0, 32.0]),
                                     rng.choice([0.5, 1.0, 2.0]))])
        if kind == "latent_attention":
            d, r = rng.choice([8, 16, 20, 32, 64, 96]), rng.choice([2, 8, 16, 32, 64])
            layer = latent(rng.choice([1, 2, 3, 4, 8]), d, r, rng.choice([8, 16, 24, 64, 128]), rng.choice([10, 16, 48, 64, 200]),
                           window, (d + r) ** -0.5 * rng.choice([0.6, 1.0, 2.0]), rng.choice([1e4, 5e4, 300.0]), scaling)
        elif kind == "mlstm":
            layer = memory(rng.choice([1, 2, 3, 4]), rng.choice([4, 12, 16, 32, 64, 128]), rng.choice([3, 8, 16, 20, 48, 64, 128]),
                           rng.choice([5.0, 15.0, 30.0]))
        else:
            owners = [j for j, l in enumerate(layers) if l["type"] == "attention" and l["mixer"].get("kv_from") is None]
            if owners and rng.random() < 0.5:
                j = rng.choice(owners)
                o = layers[j]["mixer"]
                layer = attn(rng.choice([h for h in (1, 2, 3, 4, 6, 8, 12) if h % o["kv_heads"] == 0]), o["kv_heads"], o["dim"],
                             o["vdim"], window, o["dim"] ** -0.5 * rng.choice([0.6, 1.0, 2.0]), rng.choice([None, 5.0, 20.0, 50.0]),
                             kv_from=j)
                layer["mixer"]["rot"] = dict(o["rot"])
            else:
                heads = rng.choice([1, 2, 3, 4, 6, 8])
                kv = rng.choice([g for g in range(1, heads + 1) if heads % g == 0])
                d = rng.choice([8, 16, 20, 32, 40, 64, 96, 128])
                e = rng.choice([d, d, 8, 16, 48, 64])
                dims = rng.choice([x for x in (2, 4, 8, 16, 32, 64, 128) if x <= d] + [d - d % 2])
                layer = attn(heads, kv, d, e, window, d ** -0.5 * rng.choice([0.6, 1.0, 2.0]), rng.choice([None, 5.0, 20.0, 50.0]),
                             dims, rng.choice([1e4, 5e4, 1e6, 300.0]), scaling)
        f = rng.random()
        if f < 0.2:
            layer["mlp"] = None
        elif f < 0.5:
            layer["mlp"] = dense(rng.choice([16, 40, 64, 96, 200]))
        else:
            experts = rng.choice([1, 2, 3, 5, 8, 16])
            layer["mlp"] = moe(rng.choice([16, 40, 64, 96]), experts, rng.randint(1, min(4, experts)), rng.choice([1.0, 2.0, 2.5]),
                               rng.choice([None, 24, 64, 128]))
        layers.append(layer)
    return model(rng.randint(100, 700), rng.choice([64, 72, 96, 136, 192, 256]), rng.choice([1e-5, 1e-6]), layers,
                 rng.choice([None, 15.0, 30.0]))


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return tmp_path_factory.mktemp("furesun_random")


@pytest.mark.parametrize("seed", list(range(12)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_random_configuration_whole_decoded_and_batched(tmp_root, seed, dtype):
    from tq_kv_b200.engine import Engine, StepRow
    cfg = random_config(seed)
    path = os.path.join(str(tmp_root), f"r{seed}_{dtype}")
    pf.write_folder(path, cfg, make_weights(cfg, 1000 + seed, alike_experts=dtype == "bfloat16"))
    eng = Engine.from_folder(path, dtype=dtype, max_tokens=1536, max_slots=4)
    V = cfg["vocab"]
    toks = tokens(290, V, seed)
    want = oracle(path, toks)
    s = eng.new_sequence()
    check_rows(eng.step([StepRow(s, toks, list(range(290)))]), want, dtype, f"random {seed} whole", TOL[dtype])
    eng.release(s)
    s = eng.new_sequence()
    got = [eng.step([StepRow(s, toks[:220], [219])])]
    for t in range(220, 290):
        got.append(eng.step([StepRow(s, [toks[t]], [0])]))
    check_rows(torch.cat(got), want[219:], dtype, f"random {seed} decode", TOL[dtype])
    eng.release(s)
    reqs = [tokens(n + 25, V, 50 + seed + n) for n in (3, 140, 65)]
    wants = [oracle(path, r) for r in reqs]
    slots = [eng.new_sequence() for _ in reqs]
    out = eng.step([StepRow(sl, r[:len(r) - 25], [len(r) - 26]) for sl, r in zip(slots, reqs)])
    got = [[out[i:i + 1]] for i in range(3)]
    for step in range(25):
        out = eng.step([StepRow(sl, [r[len(r) - 25 + step]], [0]) for sl, r in zip(slots, reqs)])
        for i in range(3):
            got[i].append(out[i:i + 1])
    for i in range(3):
        check_rows(torch.cat(got[i]), wants[i][len(reqs[i]) - 26:], dtype, f"random {seed} batch row {i}", TOL[dtype])
    for sl in slots:
        eng.release(sl)
    eng.cache.book.check()
