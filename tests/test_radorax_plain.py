"""Radorax on the host: the configuration and its layout as parts, the weight manifest, and the
plain implementation's mechanisms checked against one another and against brute force."""
import copy
import math

import numpy as np
import pytest

import plain_radorax as pr
import tiny_radorax as tr
from crane_b200.config import ConfigError, resolve
from crane_b200.config.spec import PartSpec
from crane_b200.parts import model_manifest
from crane_b200.parts.position import YarnRope


def _spec(config):
    arch = resolve(config)
    return arch.build_spec(arch.config_from_dict(config))


def test_architecture_is_found_by_its_single_name():
    assert resolve(tr.RA).name == "Radorax"
    assert resolve({"model_type": "radorax"}).name == "Radorax"


def test_layout_and_manifest():
    spec = _spec(tr.RB)
    assert [s.cache_of for s in spec.schedule] == [None, 0, 0, None]
    assert all(layer.block == "parallel_depth_average" for layer in spec.layers)
    m = {k: tuple(v.shape) for k, v in model_manifest(spec).items()}
    assert m["embed"] == (333, 160) and m["bigram"] == (102, 160)
    assert m["l0.mix.q"] == (5 * 28, 160) and m["l0.mix.dkv"] == (76, 160) and m["l0.mix.dkv.norm"] == (72,)
    assert "l1.mix.dkv" not in m and "l2.mix.dkv.norm" not in m
    assert m["l2.mix.uk"] == (48, 72) and m["l2.mix.uv"] == (56, 72) and m["l2.mix.g"] == (56, 160)
    assert m["l2.mix.o"] == (160, 56) and m["l2.mlp.up"] == (72, 160) and m["l2.mlp.act"] == (2,)
    assert m["l3.dwa"] == (5,) and m["l0.dwa"] == (2,) and m["final.norm.b"] == (160,)
    # a layer without feed-forward has no second norm; a model without bigram table no state
    ma = model_manifest(_spec(tr.RA))
    assert "l2.norm2" not in ma and "l2.mlp.up" not in ma and "l2.norm1.b" in ma
    assert "bigram" not in model_manifest(_spec(tr.RC))
    # tensors that a folder may hold for parts that a layer does not have are passed over
    ignored = _spec(tr.RA).ignored_tensors
    assert "l2.norm2" in ignored and "l1.mix.dkv" in ignored and "l0.norm2" not in ignored


@pytest.mark.parametrize("change, word", [
    (lambda c: c["layers"][0].update(type="ring_attention"), "no mixer"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "cache of its own"),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=16), "must be equal"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "feed-forward kind"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
])
def test_configurations_that_cannot_be(change, word):
    c = copy.deepcopy(tr.RA)
    change(c)
    with pytest.raises(ConfigError) as e:
        _spec(c)
    assert word in str(e.value)


def test_bigram_rows():
    rows = pr.bigram_rows([5, 9, 9, 0], 37, 31, 5)
    assert rows == [37, (5 * 31 + 9 * 5) % 37, (9 * 31 + 9 * 5) % 37, (9 * 31) % 37]
    # a portion that goes on behind token 9
    assert pr.bigram_rows([9, 0], 37, 31, 5, before=9) == rows[2:]


def test_xielu():
    p, q = 0.3, -0.7
    z = np.array([-3.0, -1e-4, 0.0, 1e-4, 2.0])
    y = pr.xielu(z, p, q)
    assert y[2] == 0.0 and abs(y[1] + 5e-5) < 1e-7 and abs(y[3] - 5e-5) < 1e-7      # slope 1/2 through 0
    assert math.isclose(y[4], math.log1p(math.exp(p)) * 4 + 1)
    assert math.isclose(y[0], (0.5 + math.log1p(math.exp(q))) * (math.exp(-3) - 1 + 3) - 1.5)


def test_yarn_tables():
    rot = {"dims": 8, "base": 1000.0}
    cos, sin = pr.yarn_tables(rot, np.arange(5))
    f = 1000.0 ** (-np.arange(4) / 4.0)
    assert np.allclose(cos, np.cos(np.arange(5)[:, None] * f)) and np.allclose(sin[1], np.sin(f))
    sc = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
    cos2, _ = pr.yarn_tables(dict(rot, scaling=sc), np.array([0]))
    assert np.allclose(cos2, 0.1 * math.log(4.0) + 1)
    # by hand: dim(t) = 8 ln(32 / (2 pi t)) / (2 ln 1000)
    lo = max(math.floor(8 * math.log(32 / (2 * math.pi * 8)) / (2 * math.log(1000))), 0)
    hi = min(math.ceil(8 * math.log(32 / (2 * math.pi * 1)) / (2 * math.log(1000))), 7)
    assert (lo, hi) == (0, 1)
    ramp = np.clip((np.arange(4) - lo) / (hi - lo), 0, 1)
    want = f / 4 * ramp + f * (1 - ramp)
    part = YarnRope(PartSpec("position", "yarn_rope", {"dims": 8, "base": 1000.0, "scaling": sc,
                                                       "max_positions": 64}))
    got, mult = part.frequencies()
    assert np.allclose(got, want) and math.isclose(mult, 0.1 * math.log(4.0) + 1)
    for name in ("RA", "RB"):                   # the engine's frequencies against the plain tables
        for layer in tr.TINY[name]["config"]["layers"]:
            rot = layer["mixer"]["rot"]
            part = YarnRope(PartSpec("position", "yarn_rope", dict(rot, max_positions=64)))
            f, mult = part.frequencies()
            cos, sin = pr.yarn_tables(rot, np.array([3]))
            assert np.allclose(np.cos(3 * f) * mult, cos[0]) and np.allclose(np.sin(3 * f) * mult, sin[0])


def test_rotation_is_partial_and_interleaved():
    x = np.arange(12, dtype=np.float64).reshape(1, 2, 6)
    cos, sin = np.array([[0.0], [1.0]]), np.array([[1.0], [0.0]])       # a quarter turn, then none
    y = pr.rotate_pairs(x, cos, sin, 2)
    assert y[0, 0].tolist() == [-1.0, 0.0, 2.0, 3.0, 4.0, 5.0] and y[0, 1].tolist() == x[0, 1].tolist()


def test_depth_average_and_layer_norm():
    rs = [np.full((2, 3), 1.0), np.full((2, 3), 10.0), np.full((2, 3), 100.0)]
    assert np.allclose(pr.depth_average(rs, np.array([0.5, 0.25, 2.0])), 203.0)
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    y = pr.layer_norm(x, np.ones(4), np.zeros(4), 0.0)
    assert np.allclose(y.mean(), 0) and np.allclose((y * y).mean(), 1)


def test_decoding_from_cache_rows_equals_the_whole_prompt(model_folders):
    """The plain mixer on a prompt, and token by token from kept cache rows; and the identity
    the engine rests on: q . (U c) = (U^T q) . c, sum_j p_j (V c_j) = V sum_j p_j c_j."""
    cfg, w = pr.load_folder(model_folders("RA", "bfloat16"))
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    rng = np.random.default_rng(0)
    h = rng.standard_normal((9, cfg["width"]))
    pos = np.arange(9)
    c, kr = pr.latent_cache_rows(h, w, "l0.mix.", m, eps, pos)
    whole = pr.latent_attention(h, w, "l0.mix.", m, c, kr, pos, pos)
    for t in range(9):
        one = pr.latent_attention(h[t:t + 1], w, "l0.mix.", m, c[:t + 1], kr[:t + 1], pos[t:t + 1], pos[:t + 1])
        assert np.allclose(one[0], whole[t], atol=1e-12)
    H, d, r = m["heads"], m["dim"], m["kv_rank"]
    U = w["l0.mix.uk"].reshape(H, d, r)
    q = rng.standard_normal((H, d))
    assert np.allclose(np.einsum("hd,hdr,r->h", q, U, c[3]), np.einsum("hd,hd->h", q, (c[3] @ w["l0.mix.uk"].T).reshape(H, d)))


def test_streams_are_kept_per_layer(model_folders):
    cfg, w = pr.load_folder(model_folders("RB", "bfloat16"))
    streams = []
    lg = pr.logits_all(cfg, w, [1, 2, 3, 4], streams)
    assert len(streams) == 4 and lg.shape == (4, 333) and np.isfinite(lg).all()
    # causal: a later token changes nothing before it; the bigram table makes the change start AT it
    lg2 = pr.logits_all(cfg, w, [1, 2, 7, 4])
    assert np.allclose(lg[:2], lg2[:2]) and not np.allclose(lg[2], lg2[2])
