"""Pavisun: configuration, registry, tensor list, schedule and caches, and the plain implementation's mechanisms
against closed forms (all on the CPU)."""
import copy
import math

import pytest
import torch

import plain_pavisun as pp
from pavisun_cases import CASES, make_weights, tokens


def _spec(cfg):
    from tq_kv_b200.config import spec_from_config_dict
    return spec_from_config_dict(cfg)


def test_the_architecture_is_registered_and_a_configuration_round_trips():
    from tq_kv_b200.config import registered_architectures
    assert "Pavisun" in registered_architectures()
    for name, cfg in CASES.items():
        arch, typed, spec = _spec(cfg)
        back = typed.to_dict()
        assert arch.name == "Pavisun" and back["layers"] == cfg["layers"], name
        assert all(back.get(k) == cfg.get(k) for k in ("streams", "loop", "logit_softcap", "vocab", "width", "norm")), name
        S = cfg.get("streams") or 0
        assert spec.residual_streams == S
        assert all(l.block == ("residual_streams" if S else "prenorm_residual") for l in spec.layers)
        assert all(l.mixer.kind == "softmax_attention" for l in spec.layers)
        assert [l.feed_forward is None for l in spec.layers] == [x["mlp"] is None for x in cfg["layers"]]
        assert [e.layer for e in spec.schedule] == pp.schedule(cfg) == typed.order()
        assert spec.head.params.get("logit_softcap") == cfg.get("logit_softcap")


def test_the_order_of_looped_layers():
    from tq_kv_b200.config import PavisunConfig
    base = copy.deepcopy(CASES["b"])                                   # four layers
    for loop, want in (((1, 3, 2), [0, 1, 2, 1, 2, 3]), ((0, 4, 2), [0, 1, 2, 3, 0, 1, 2, 3]), ((3, 4, 3), [0, 1, 2, 3, 3, 3]),
                       ((2, 2, 5), [0, 1, 2, 3]), ((0, 1, 1), [0, 1, 2, 3])):
        cfg = dict(base, loop=dict(zip(("start", "stop", "times"), loop)))
        assert PavisunConfig.from_dict(cfg).order() == want == pp.schedule(cfg)


@pytest.mark.parametrize("path,key", [((), "vocab"), ((), "width"), ((), "layers"), (("norm",), "eps"),
                                      (("layers", 0, "mixer"), "heads"), (("layers", 0, "mixer"), "scale"),
                                      (("layers", 1, "mixer"), "rot"), (("layers", 1, "mixer", "rot"), "base"),
                                      (("layers", 1, "mixer", "rot", "scaling"), "fast"),
                                      (("layers", 0, "mlp", "router"), "top"), (("layers", 0, "mlp", "expert"), "ff"),
                                      (("layers", 2), "type"), (("loop",), "times")])
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

    def bad(change):
        cfg = copy.deepcopy(CASES["a"])
        change(cfg)
        with pytest.raises(ConfigError):
            _spec(cfg)

    bad(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))                     # 4 heads on 3 key heads
    bad(lambda c: c["layers"][1]["mixer"].update(vdim=32))                        # the values are the keys
    bad(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=50))                 # more than the head holds
    bad(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7))                  # pairs
    bad(lambda c: c["layers"][0]["mlp"]["router"].update(top=7))                  # of six experts
    bad(lambda c: c["loop"].update(stop=4))                                       # of three layers
    bad(lambda c: c["layers"][0].update(type="something"))
    bad(lambda c: c["layers"][0]["mlp"].update(kind="dense"))


def test_the_model_asks_for_exactly_the_tensors_of_the_design_and_a_cache_per_run():
    from tq_kv_b200.engine.model import DecoderModel
    for name, cfg in CASES.items():
        model = DecoderModel(_spec(cfg)[2])
        want = make_weights(cfg, 1)
        specs = model.weight_specs()
        assert set(specs) == set(want), name
        assert all(tuple(specs[n].shape) == tuple(want[n].shape) for n in want), name
        kv, state = model.cache_requests()
        order = pp.schedule(cfg)
        assert sorted(kv) == list(range(len(order))) and not state, name      # every run of a layer has its own cache
        for i, li in enumerate(order):
            m = cfg["layers"][li]["mixer"]
            mask = m.get("mask") or {}
            assert kv[i].n_kv_heads == m["kv_heads"] and kv[i].head_dim == m["dim"]
            # a plain window keeps a ring of keys; kept first tokens, or no window, keep them all
            assert kv[i].window == (mask.get("size") if not mask.get("keep_first") else None), (name, i)


def test_random_weights_of_a_configuration_have_the_design_s_tensors(tmp_path):
    from tq_kv_b200.weights import write_model_folder
    cfg = CASES["a"]
    folder = write_model_folder(cfg, str(tmp_path / "m"), 3)
    want = make_weights(cfg, 1)
    cfg2, w = pp.read_folder(folder)
    assert set(w) == set(want) and all(tuple(w[n].shape) == tuple(want[n].shape) for n in want)
    table = w["l0.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 6
    assert all(len(set(r)) == len(r) for r in table.tolist())                    # the entries of a row differ
    assert torch.isfinite(pp.decoder(cfg2, w, tokens(20, cfg["vocab"], 1))).all()


# ---- the plain implementation's mechanisms ------------------------------------------------------------------
def test_rotation_keeps_lengths_up_to_its_factor_and_depends_on_the_distance_only():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 12, generator=g, dtype=torch.float64), torch.randn(1, 1, 12, generator=g, dtype=torch.float64)
    sc = {"factor": 4.0, "original": 32.0, "fast": 8.0, "slow": 1.0}

    def dot(i, j):
        return float((pp.rotate_halves(q, torch.tensor([i]), 8, 100.0, sc) * pp.rotate_halves(k, torch.tensor([j]), 8, 100.0, sc)).sum())
    assert abs(dot(7, 3) - dot(104, 100)) < 1e-9 and abs(dot(7, 3) - dot(7, 4)) > 1e-6
    r = pp.rotate_halves(q, torch.tensor([5]), 8, 100.0, sc)
    m = 0.1 * math.log(4.0) + 1.0
    assert torch.allclose(r[..., 8:], q[..., 8:])
    assert abs(float(r[..., :8].norm()) - m * float(q[..., :8].norm())) < 1e-12
    rate, _ = pp.stretched_rates(8, 100.0, sc)
    a = 5 * float(rate[1])                                      # the second pair: entries 1 and 5
    assert abs(float(r[0, 0, 1]) - m * float(q[0, 0, 1] * math.cos(a) - q[0, 0, 5] * math.sin(a))) < 1e-12
    assert abs(float(r[0, 0, 5]) - m * float(q[0, 0, 5] * math.cos(a) + q[0, 0, 1] * math.sin(a))) < 1e-12


def test_stretched_rates_by_hand():
    # dims 8, base 100, L 32: n(t) = 8 ln(32 / (2 pi t)) / (2 ln 100); fast 2 -> 0.81.., slow 0.25 -> 2.61..: lo 0, hi 3
    rate, m = pp.stretched_rates(8, 100.0, {"factor": 2.0, "original": 32.0, "fast": 2.0, "slow": 0.25})
    f = [100.0 ** (-2 * i / 8) for i in range(4)]
    share = [0.0, 1 / 3, 2 / 3, 1.0]
    assert all(abs(float(rate[i]) - (f[i] / 2 * share[i] + f[i] * (1 - share[i]))) < 1e-15 for i in range(4))
    assert abs(m - (0.1 * math.log(2.0) + 1.0)) < 1e-15
    plain, one = pp.stretched_rates(8, 100.0, None)
    assert one == 1.0 and all(abs(float(plain[i]) - f[i]) < 1e-15 for i in range(4))


def test_the_window_with_kept_first_tokens():
    v = pp.visible(10, 3, 2)
    assert v[9].tolist() == [True, True, False, False, False, False, False, True, True, True]
    assert v[2].tolist() == [True, True, True] + [False] * 7
    assert pp.visible(5, None)[4].all() and pp.visible(5, 1)[4].tolist() == [False] * 4 + [True]


def test_slopes_and_the_cap():
    s = pp.head_slopes(4, torch.float64)
    assert [float(x) for x in s] == [0.25, 0.0625, 0.015625, 0.00390625]
    assert abs(float(pp.tanh_cap(torch.tensor(1e-3, dtype=torch.float64), 20.0)) - 1e-3) < 1e-10
    assert float(pp.tanh_cap(torch.tensor(1e3, dtype=torch.float64), 20.0)) == 20.0


def test_streams_reduce_to_the_plain_residual_sum():
    """With read 1, write 1 and the identity as mix, one stream is the ordinary x <- x + y."""
    g = torch.Generator().manual_seed(0)
    xs, y = torch.randn(1, 4, 6, generator=g, dtype=torch.float64), torch.randn(4, 6, generator=g, dtype=torch.float64)
    w = {"in": torch.ones(1, dtype=torch.float64), "out": torch.ones(1, dtype=torch.float64), "mix": torch.eye(1, dtype=torch.float64)}
    assert torch.equal(pp.stream_read(xs, w, ""), xs[0]) and torch.allclose(pp.stream_write(xs, y, w, "")[0], xs[0] + y)
    xs3 = torch.randn(3, 2, 4, generator=g, dtype=torch.float64)
    w3 = {"in": torch.randn(3, generator=g, dtype=torch.float64), "out": torch.randn(3, generator=g, dtype=torch.float64),
          "mix": torch.randn(3, 3, generator=g, dtype=torch.float64)}
    new = pp.stream_write(xs3, y[:2, :4], w3, "")
    for r in range(3):                                          # mix is indexed [from, to]
        want = sum(w3["mix"][s, r] * xs3[s] for s in range(3)) + w3["out"][r] * y[:2, :4]
        assert torch.allclose(new[r], want)
