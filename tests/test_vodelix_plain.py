"""Vodelix on the host: configuration errors, the schedule of looped layers, the manifest, and the
plain implementation's own mechanisms against hand arithmetic and against each other."""
import copy
import math

import numpy as np
import pytest

import plain_vodelix as pv
import tiny_vodelix as tv
from crane_b200.config import ConfigError, resolve
from crane_b200.parts import model_manifest


def _spec(config):
    arch = resolve(config)
    return arch, arch.build_spec(arch.config_from_dict(config))


def test_registered_by_its_name():
    arch, spec = _spec(tv.VA)
    assert arch.name == "Vodelix" and spec.architecture == "Vodelix"
    assert [l.block for l in spec.layers] == ["sandwich_residual"] * 4
    assert [l.parts["mixer"].name for l in spec.layers] == ["sink_attention", "general_delta", "general_delta",
                                                            "sink_attention"]
    assert "ffn" not in spec.layers[2].parts and "norm2b" not in spec.layers[2].parts
    assert spec.layers[0].parts["ffn"].name == "routed_experts" and spec.layers[1].parts["ffn"].name == "act_mlp"


@pytest.mark.parametrize("name", ["VA", "VB", "VC", "VL"])
def test_schedule_follows_the_loop(name):
    cfg = tv.TINY[name]["config"]
    _, spec = _spec(cfg)
    runs = pv.layer_runs(cfg)
    assert [s.layer for s in spec.schedule] == [i for i, _, _ in runs]
    for s, (i, t, first) in zip(spec.schedule, runs):
        if first:
            assert s.enter == {"row": t, "add_embedding": t > 0}
        else:
            assert s.enter is None
    assert (spec.entry is not None) == ("loop" in cfg)
    assert all(s.cache_of is None for s in spec.schedule)          # every pass keeps a cache of its own


def test_schedule_by_hand():
    _, spec = _spec(tv.VC)                                          # layers 0 1, the loop is layer 1 three times
    assert [(s.layer, s.enter and s.enter["row"]) for s in spec.schedule] == [(0, None), (1, 0), (1, 1), (1, 2)]
    _, spec = _spec(tv.VA)                                          # the loop opens the stack
    assert [(s.layer, s.enter and s.enter["row"]) for s in spec.schedule] == [(0, 0), (1, None), (0, 1), (1, None),
                                                                            (2, None), (3, None)]


def test_manifest_names_and_shapes():
    _, spec = _spec(tv.VA)
    m = model_manifest(spec)
    assert m["embed"].shape == (211, 96) and m["loop.step"].shape == (2, 96) and m["side.embed"].shape == (211, 32)
    assert m["l0.mix.q"].shape == (96, 96) and m["l0.mix.k"].shape == (32, 96) and m["l0.mix.v"].shape == (48, 96)
    assert m["l0.mix.o"].shape == (96, 144) and m["l0.mix.q.norm"].shape == (96,) and m["l0.mix.k.norm"].shape == (32,)
    assert m["l1.mix.w1"].shape == (8, 96) and m["l1.mix.w2"].shape == (96, 8) and m["l1.mix.a.b"].shape == (96,)
    assert m["l0.mlp.router"].shape == (5, 96) and m["l0.mlp.e4.up"].shape == (24, 96)
    assert m["l0.mlp.shared.down"].shape == (96, 40) and "l3.mlp.shared.up" not in m
    assert "l2.norm2" not in m and "l2.mlp.up" not in m and m["l3.side.proj"].shape == (96, 8)
    assert m["final.norm"].shape == (96,)
    # without decay_rank in the configuration the inner size is read from the stored tensors
    cfg = copy.deepcopy(tv.VB)
    del cfg["layers"][0]["mixer"]["decay_rank"]
    assert model_manifest(_spec(cfg)[1])["l0.mix.w1"].shape == (-1, 80)
    assert "loop.step" not in model_manifest(_spec(tv.VB)[1]) and "side.embed" not in model_manifest(_spec(tv.VB)[1])


@pytest.mark.parametrize("change, word", [
    (lambda c: c["layers"][0].update(type="conv"), "no mixer"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "router.top"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "feed-forward kind"),
    (lambda c: c.pop("width"), "width"),
])
def test_configuration_errors(change, word):
    cfg = copy.deepcopy(tv.VA)
    change(cfg)
    with pytest.raises(ConfigError, match=word):
        resolve(cfg).config_from_dict(cfg)


# ------------------------------------------------------------------ the plain mechanisms
def test_sinusoid_by_hand():
    s = pv.sinusoid([0, 3], 6)
    assert np.allclose(s[0], [0, 1, 0, 1, 0, 1])
    f1 = 10000.0 ** (-2.0 / 6)
    assert np.allclose(s[1, :4], [math.sin(3), math.cos(3), math.sin(3 * f1), math.cos(3 * f1)])
    assert pv.sinusoid([5], 7).shape == (1, 7)                       # an odd width ends on a sine


def test_sink_softmax_by_hand():
    """One head, keys and values chosen so that the scores are 0 and ln 3: the weights are
    1 / 5 and 3 / 5, and a fifth goes to the sink."""
    d = 2
    w = {"q": np.eye(d), "k": np.eye(d), "v": np.eye(d), "o": np.eye(d), "q.norm": np.ones(d), "k.norm": np.ones(d)}
    h = np.array([[0.0, 1.0], [1.0, 0.0]])
    mixer = {"heads": 1, "dim": d, "scale": math.log(3.0) / 2.0}    # normed rows have squared length 2
    out = pv.sink_attention(h, {("p." + k): v for k, v in w.items()}, "p.", mixer, 0.0)
    assert np.allclose(out[0], np.array([0.0, 1.0]) * 3 / 4)        # alone with the sink: e^s / (1 + e^s), s = ln 3
    assert np.allclose(out[1], 0.2 * h[0] + 0.6 * h[1])


def test_delta_rule_step_by_hand():
    S = np.array([[1.0, 2.0], [3.0, 4.0]])
    unit = np.array([1.0, 0.0])
    S2, o = pv.delta_rule_step(S, r=np.array([1.0, 1.0]), k=np.array([2.0, 0.0]), v=np.array([1.0, -1.0]),
                               decay=np.array([0.5, 1.0]), rate=np.array([1.0, 0.5]), unit=unit)
    # row 0: 0.5 * [1, 2] - 1 * [1, 2] + 2 * [1, -1]; row 1: untouched by a removal along e0 and a key along e0
    assert np.allclose(S2, [[1.5, -3.0], [3.0, 4.0]]) and np.allclose(o, [4.5, 1.0])


def test_delta_rule_continues_from_its_state():
    rng = np.random.default_rng(0)
    H, d, W, R, n = 2, 6, 10, 3, 9
    w = {"p." + k: rng.standard_normal(s) * 0.5 for k, s in
         {"r": (H * d, W), "k": (H * d, W), "v": (H * d, W), "g": (H * d, W), "a": (H * d, W), "a.b": (H * d,),
          "w1": (R, W), "w2": (H * d, R), "w0": (H * d,), "norm": (H * d,), "o": (W, H * d)}.items()}
    h = rng.standard_normal((n, W))
    whole, S = pv.general_delta(h, w, "p.", {"heads": H, "dim": d}, 1e-5)
    a, Sa = pv.general_delta(h[:4], w, "p.", {"heads": H, "dim": d}, 1e-5)
    b, Sb = pv.general_delta(h[4:], w, "p.", {"heads": H, "dim": d}, 1e-5, Sa)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(S, Sb)
    dec = pv.delta_rule_inputs(h, w, "p.", H, d)[3]
    assert dec.min() > math.exp(-math.exp(-0.5)) and dec.max() < 1.0


def test_route_by_hand():
    w = {"p.router": np.array([[1.0, 0], [0, 1.0], [1.0, 1.0], [0, 0]])}
    idx, wt = pv.route(np.array([[2.0, 1.0], [0.0, 0.0]]), w, "p.", 2)
    assert idx[0].tolist() == [2, 0] and np.allclose(wt[0], [math.e / (1 + math.e), 1 / (1 + math.e)])
    assert idx[1].tolist() == [0, 1] and np.allclose(wt[1], [0.5, 0.5])        # ties go to the lower index


def test_activations():
    z = np.array([-2.0, 0.0, 0.5, 3.0])
    assert np.allclose(pv.relu_squared(z), [0, 0, 0.25, 9])
    assert np.allclose(pv.gelu_erf(z), [z_ * 0.5 * (1 + math.erf(z_ / math.sqrt(2))) for z_ in z])
    assert abs(pv.gelu_tanh(np.array([1.0]))[0] - 0.841192) < 1e-6


def test_whole_model_equals_its_own_continuation(model_folders):
    """The plain model run layer by layer over a prompt's two halves, the recurrent state carried,
    agrees with the whole prompt for the layers that have no attention (VB's first layer)."""
    cfg, w = pv.load_folder(model_folders("VB", "float32"))
    toks = list(range(3, 15))
    x = pv.embedding(w, toks, range(len(toks)), cfg["width"])
    whole, _ = pv.layer(x, toks, cfg, w, 0)
    a, S = pv.layer(x[:5], toks[:5], cfg, w, 0)
    b, _ = pv.layer(x[5:], toks[5:], cfg, w, 0, S)
    assert np.allclose(np.concatenate([a, b]), whole)
