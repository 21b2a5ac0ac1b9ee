"""Furesun: configuration, registry, tensor list, schedule and caches, and the plain implementation's mechanisms
against closed forms (all on the CPU)."""
import copy
import math

import pytest
import torch

import plain_furesun as pf
from furesun_cases import CASES, make_weights, tokens


def _spec(cfg):
    from tq_kv_b200.config import spec_from_config_dict
    return spec_from_config_dict(cfg)


def test_the_architecture_is_registered_and_a_configuration_round_trips():
    from tq_kv_b200.config import registered_architectures
    assert "Furesun" in registered_architectures()
    kinds = {"latent_attention": "latent_attention", "mlstm": "mlstm_mixer", "attention": "softmax_attention"}
    for name, cfg in CASES.items():
        arch, typed, spec = _spec(cfg)
        back = typed.to_dict()
        assert arch.name == "Furesun" and back["layers"] == cfg["layers"], name
        assert all(back.get(k) == cfg.get(k) for k in ("logit_softcap", "vocab", "width", "norm")), name
        assert all(l.block == "postnorm_residual" for l in spec.layers)
        assert [l.mixer.kind for l in spec.layers] == [kinds[x["type"]] for x in cfg["layers"]]
        assert [l.feed_forward is None for l in spec.layers] == [x["mlp"] is None for x in cfg["layers"]]
        assert [e.layer for e in spec.schedule] == list(range(len(cfg["layers"])))
        assert [e.cache_of for e in spec.schedule] == [x["mixer"].get("kv_from") for x in cfg["layers"]]
        assert spec.head.params.get("logit_softcap") == cfg.get("logit_softcap")


@pytest.mark.parametrize("path,key", [((), "vocab"), ((), "width"), ((), "layers"), (("norm",), "eps"),
                                      (("layers", 0, "mixer"), "gate_cap"), (("layers", 0, "mixer"), "vdim"),
                                      (("layers", 1, "mixer"), "rot"), (("layers", 1, "mixer", "rot"), "base"),
                                      (("layers", 1, "mixer"), "kv_heads"), (("layers", 1, "mixer"), "scale"),
                                      (("layers", 2, "mixer"), "kv_rank"), (("layers", 2, "mixer"), "rot_dim"),
                                      (("layers", 2, "mixer", "rot", "scaling"), "fast"),
                                      (("layers", 0, "mlp", "router"), "top"), (("layers", 0, "mlp", "router"), "scale"),
                                      (("layers", 0, "mlp", "expert"), "ff"), (("layers", 0, "mlp", "shared"), "ff"),
                                      (("layers", 1, "mlp"), "ff"), (("layers", 2), "type")])
def test_a_missing_key_is_named(path, key):
    from tq_kv_b200.config import ConfigError
    cfg = copy.deepcopy(CASES["a"])
    d = cfg
    for p in path:
        d = d[p]
    del d[key]
    with pytest.raises(ConfigError, match=key):
        _spec(cfg)


def test_sizes_that_contradict_each_other_are_refused():
    from tq_kv_b200.config import ConfigError

    def broken(change):
        cfg = copy.deepcopy(CASES["a"])
        change(cfg)
        with pytest.raises(ConfigError):
            _spec(cfg)

    broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=4))                 # 6 heads on 4 key heads
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=22))             # more rotated entries than the head has
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=9))              # an odd count
    broken(lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10))             # beyond the rotated part
    broken(lambda c: c["layers"][3]["mixer"].update(kv_from=3))                  # itself
    broken(lambda c: c["layers"][3]["mixer"].update(kv_from=2))                  # not an attention layer
    broken(lambda c: c["layers"][3]["mixer"].update(dim=24))                     # other keys than layer 1 caches
    broken(lambda c: c["layers"][3]["mixer"]["rot"].update(base=10000.0))        # another rotation
    broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=7))              # 7 of 6 experts
    broken(lambda c: c["layers"][0].update(type="lstm"))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="sparse"))
    broken(lambda c: c["norm"].update(eps=0.0))
    cfg = copy.deepcopy(CASES["a"])
    cfg["layers"].insert(1, copy.deepcopy(cfg["layers"][3]))                     # reads a layer that comes later
    with pytest.raises(ConfigError):
        _spec(cfg)


def test_the_model_asks_for_exactly_the_tensors_of_the_design_and_the_caches_its_mixers_need():
    from tq_kv_b200.engine import DecoderModel
    for name, cfg in CASES.items():
        w = make_weights(cfg, 3)
        model = DecoderModel(_spec(cfg)[2])
        specs = model.weight_specs()
        assert sorted(specs) == sorted(w), name
        for n, s in specs.items():
            assert tuple(s.shape) == tuple(w[n].shape), (name, n)
        kv, state = model.cache_requests()
        types = [l["type"] for l in cfg["layers"]]
        own = [i for i, l in enumerate(cfg["layers"]) if l["type"] != "mlstm" and l["mixer"].get("kv_from") is None]
        assert sorted(kv) == own and sorted(state) == [i for i, t in enumerate(types) if t == "mlstm"], name
        for i in own:
            m = cfg["layers"][i]["mixer"]
            if types[i] == "latent_attention":
                assert kv[i].n_kv_heads == 1 and kv[i].head_dim >= m["kv_rank"] + m["rot_dim"]
                assert kv[i].window == (m.get("mask") or {}).get("size")
            else:                                           # the widest window among the layer and its readers
                ws = [(m.get("mask") or {}).get("size")] + [(l["mixer"].get("mask") or {}).get("size")
                                                            for l in cfg["layers"] if l["mixer"].get("kv_from") == i]
                assert kv[i].window == (None if None in ws else max(ws)), (name, i)
        for i in state:
            m = cfg["layers"][i]["mixer"]
            ea = -(-(m["vdim"] + 1) // 4) * 4
            assert state[i].shape == (m["heads"] * m["dim"] * ea + m["heads"],) and state[i].dtype == torch.float32


def test_random_weights_of_a_configuration_have_the_design_s_tensors(tmp_path):
    from tq_kv_b200.weights import write_model_folder
    path = write_model_folder(CASES["c"], str(tmp_path / "m"), 11)
    cfg, w = pf.read_folder(path)
    assert sorted(w) == sorted(make_weights(CASES["c"], 1))
    assert cfg["layers"] == CASES["c"]["layers"] and cfg["architecture"] == "Furesun"
    logits = pf.decoder(cfg, w, tokens(20, cfg["vocab"], 2))
    assert logits.shape == (20, cfg["vocab"]) and torch.isfinite(logits).all()


# ---- the plain implementation's mechanisms against closed forms -----------------------------------------------------
def test_rotation_keeps_lengths_up_to_its_factor_and_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 24, generator=g, dtype=torch.float64), torch.randn(1, 1, 24, generator=g, dtype=torch.float64)
    for layout in ("halves", "pairs"):
        for scaling in (None, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}):
            f = 1.0 if scaling is None else 0.1 * math.log(8.0) + 1.0
            dots = []
            for pq, pk in ((5, 2), (105, 102), (1003, 1000)):
                a = pf.rotate(q, torch.tensor([pq]), 16, 1e4, layout, scaling)
                b = pf.rotate(k, torch.tensor([pk]), 16, 1e4, layout, scaling)
                assert torch.allclose(a[..., 16:], q[..., 16:]) and abs(float(a[..., :16].norm() / q[..., :16].norm()) - f) < 1e-12
                dots.append(float((a * b).sum()))
            assert max(dots) - min(dots) < 1e-9
    # the layouts pair other entries: pairs turns (0, 1), halves turns (0, 8)
    x = torch.zeros(1, 1, 16, dtype=torch.float64)
    x[..., 0] = 1.0
    assert float(pf.rotate(x, torch.tensor([3]), 16, 1e4, "pairs")[0, 0, 1]) == pytest.approx(math.sin(3.0))
    assert float(pf.rotate(x, torch.tensor([3]), 16, 1e4, "halves")[0, 0, 8]) == pytest.approx(math.sin(3.0))


def test_the_window_and_the_sink():
    m = pf.visible(6, 3)
    assert m.tolist() == [[j <= i and i - j < 3 for j in range(6)] for i in range(6)]
    assert pf.visible(4, None).tolist() == [[j <= i for j in range(4)] for i in range(4)]
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(5, 2, 8, generator=g, dtype=torch.float64) for _ in range(3))
    plain = pf.softmax_heads(q, k, v, 0.5, pf.visible(5, None))
    sunk = pf.softmax_heads(q, k, v, 0.5, pf.visible(5, None), sink=True)
    # the sink is one more key of score 0 whose value is zero
    k0 = torch.cat([torch.zeros(1, 2, 8, dtype=torch.float64), k])
    v0 = torch.cat([torch.zeros(1, 2, 8, dtype=torch.float64), v])
    q0 = torch.cat([q[:1], q])
    with_key = pf.softmax_heads(q0, k0, v0, 0.5, torch.ones(6, 6, dtype=torch.bool).tril())[1:]
    assert torch.allclose(sunk, with_key, atol=1e-12) and not torch.allclose(sunk, plain, atol=1e-3)
    assert (sunk.abs() <= plain.abs().max() + 1e-9).all()


def test_the_matrix_memory_as_a_weighted_sum_over_the_past():
    """Without the running maximum the memory is o_t = sum_s w_ts (k_s . q) v_s / (max(|sum_s w_ts k_s . q|, 1) + floor)
    with w_ts = exp(i_s + f_{s+1} + ... + f_t): the maximum only moves both sides of the division."""
    cfg = {"heads": 2, "dim": 6, "vdim": 5, "gate_cap": 7.0}
    g = torch.Generator().manual_seed(3)
    W, T, H, d, e = 12, 9, 2, 6, 5
    w = {"q": torch.randn(H * d, W, generator=g), "k": torch.randn(H * d, W, generator=g), "v": torch.randn(H * e, W, generator=g),
         "g": torch.randn(H * e, W, generator=g), "o": torch.eye(H * e), "norm": torch.ones(H * e),
         "i": torch.randn(H, W, generator=g), "f": torch.randn(H, W, generator=g), "i.b": torch.randn(H, generator=g),
         "f.b": torch.randn(H, generator=g)}
    w = {("m." + n): t.double() for n, t in w.items()}
    x = torch.randn(T, W, generator=g, dtype=torch.float64)
    got = pf.mlstm(x, w, "m.", cfg, 1e-6).reshape(T, H, e)
    q = (x @ w["m.q"].T).reshape(T, H, d) / d ** 0.5
    k, v = (x @ w["m.k"].T).reshape(T, H, d), (x @ w["m.v"].T).reshape(T, H, e)
    ig = 7.0 * torch.tanh((x @ w["m.i"].T + w["m.i.b"]) / 7.0)
    fg = torch.nn.functional.logsigmoid(7.0 * torch.tanh((x @ w["m.f"].T + w["m.f.b"]) / 7.0))
    gate = torch.sigmoid(x @ w["m.g"].T).reshape(T, H, e)
    for t in range(T):
        for h in range(H):
            m = 0.0                                          # the maximum as the recurrence keeps it
            for s in range(t + 1):
                m = max(float(fg[s, h]) + m, float(ig[s, h]))
            lw = torch.stack([ig[s, h] + fg[s + 1:t + 1, h].sum() for s in range(t + 1)])
            kq = k[:t + 1, h] @ q[t, h]
            num = (torch.exp(lw - m) * kq) @ v[:t + 1, h]
            den = max(abs(float((torch.exp(lw - m) * kq).sum())), math.exp(-m)) + 1e-6
            o = num / den
            want = o / torch.sqrt((o * o).mean() + 1e-6) * gate[t, h]
            assert torch.allclose(got[t, h], want, atol=1e-9), (t, h)


def test_the_router_s_weights_and_the_shared_expert():
    cfg = {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 5, "top": 2, "scale": 1.7}, "shared": {"ff": 4}}
    g = torch.Generator().manual_seed(4)
    W = 8
    w = {"p.router": torch.randn(5, W, generator=g, dtype=torch.float64)}
    for n in [f"e{i}." for i in range(5)] + ["shared."]:
        f = 4 if n == "shared." else 6
        w["p." + n + "gate"], w["p." + n + "up"] = (torch.randn(f, W, generator=g, dtype=torch.float64) for _ in range(2))
        w["p." + n + "down"] = torch.randn(W, f, generator=g, dtype=torch.float64)
    x = torch.randn(3, W, generator=g, dtype=torch.float64)
    got = pf.routed_ff(x, w, "p.", cfg)
    for t in range(3):
        s = torch.sigmoid(w["p.router"] @ x[t])
        top = sorted(range(5), key=lambda i: -float(s[i]))[:2]
        want = sum(1.7 * s[i] / (s[top[0]] + s[top[1]]) * pf.gated_ff(x[t:t + 1], w, f"p.e{i}.", pf.silu)[0] for i in top)
        want = want + pf.gated_ff(x[t:t + 1], w, "p.shared.", pf.silu)[0]
        assert torch.allclose(got[t], want, atol=1e-12)
    z = torch.linspace(-4, 4, 9, dtype=torch.float64)
    assert torch.allclose(pf.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"), atol=1e-12)


def test_a_layer_norms_what_its_sublayers_give_and_shared_keys_are_the_other_layer_s():
    cfg = copy.deepcopy(CASES["a"])
    w = make_weights(cfg, 6)
    toks = tokens(40, cfg["vocab"], 7)
    layers = []
    pf.decoder(cfg, w, toks, layers_out=layers)
    wd = {k: v.double() for k, v in w.items()}
    x0 = wd["embed"][torch.tensor(toks)]
    y = pf.mlstm(x0, wd, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6)
    x1 = x0 + pf.rms_norm(y, wd["l0.norm1"], 1e-6)
    x1 = x1 + pf.rms_norm(pf.feed_forward(x1, wd, "l0.mlp.", cfg["layers"][0]["mlp"]), wd["l0.norm2"], 1e-6)
    assert torch.allclose(layers[0], x1, atol=1e-10)
    # layer 3 reads layer 1's keys (made from layer 1's input), with its own queries and window
    pos = torch.arange(40)
    kv = pf.attention_keys(layers[0], wd, "l1.mix.", cfg["layers"][1]["mixer"], pos, 1e-6)
    a = pf.attention(layers[2], wd, "l3.mix.", cfg["layers"][3]["mixer"], pos, 1e-6, kv=kv)
    x3 = layers[2] + pf.rms_norm(a, wd["l3.norm1"], 1e-6)
    x3 = x3 + pf.rms_norm(pf.feed_forward(x3, wd, "l3.mlp.", cfg["layers"][3]["mlp"]), wd["l3.norm2"], 1e-6)
    assert torch.allclose(layers[3], x3, atol=1e-10)
