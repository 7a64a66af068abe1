"""The Sezopel family without a GPU: the registry, the model as data (layers that read another
layer's keys and values, cache lines and states), tensor names and shapes, defaults of absent
keys, refusals, the rotary frequencies, and the plain implementation's own consistency (a
prefix against the whole; retention's recurrence against its sum over all earlier tokens)."""
import json

import numpy as np
import pytest

from mormot2_ai_b200 import ConfigError, DecoderModel, SezopelConfig, architectures
from mormot2_ai_b200.config.registry import family_of
from tests.plain import sezopel_plain as plain
from tests.sezopel_models import SMALL, small_doc


def test_registry_and_round_trip():
    assert "Sezopel" in architectures()
    for name in SMALL:
        doc = small_doc(name)
        assert family_of(doc) is SezopelConfig
        c = SezopelConfig.from_dict(doc)
        again = SezopelConfig.from_dict(json.loads(json.dumps(c.to_dict())))
        assert again == c
        assert c.vocab_size == doc["vocab"] and c.hidden_size == doc["width"]
        assert c.num_hidden_layers == len(doc["layers"])


def test_layers_that_read_another_layers_keys_and_values():
    spec = SezopelConfig.from_dict(small_doc("P")).to_model_spec()
    assert [r.layer for r in spec.schedule] == [0, 1, 2, 3, 4]
    assert [r.cache_line for r in spec.schedule] == [0, 0, 2, 0, 4]
    assert [r.writes_cache for r in spec.schedule] == [True, False, True, False, True]
    assert all(l.block.kind == "output_norm_residual" for l in spec.layers)
    model = DecoderModel(spec)
    shapes = {t.name: t.shape for t in model.tensors()}
    assert "l1.mix.k" not in shapes and "l1.mix.v" not in shapes and "l3.mix.k" not in shapes
    assert shapes["l0.mix.q"] == (4 * 24, 80) and shapes["l0.mix.k"] == (2 * 24, 80)
    assert shapes["l0.mix.v"] == (2 * 40, 80) and shapes["l0.mix.o"] == (80, 4 * 40)
    assert shapes["l0.mix.g"] == (4, 80) and shapes["l1.mix.g"] == (4, 80)
    assert shapes["l2.mix.q"] == (3 * 20, 80) and shapes["l2.mix.v"] == (3 * 12, 80)
    assert shapes["l2.mix.g"] == (3 * 12, 80) and shapes["l2.mix.o"] == (80, 3 * 12)
    assert shapes["l0.mlp.up"] == (96, 80) and shapes["l1.mlp.down"] == (80, 72)
    assert "l3.mlp.up" not in shapes and "l3.norm2" not in shapes and "l3.norm1" in shapes
    assert shapes["side.embed"] == (211, 5 * 12)
    assert shapes["l4.side.gate"] == (12, 80) and shapes["l4.side.proj"] == (80, 12)
    assert shapes["l4.side.norm"] == (80,) and shapes["head"] == (211, 80)
    # one line of keys and values (value rows of their own size), read by three layers; a
    # state of heads x dim x vdim floats for each retention layer
    assert set(model.line_needs) == {0}
    assert model.line_needs[0].head_dim == 24 and model.line_needs[0].v_dim == 40
    assert set(model.state_needs) == {2, 4}
    assert model.state_needs[2].shape == (3 * 20 * 12,)
    assert model.state_needs[4].shape == (2 * 8 * 36,)
    # each layer's slice of the second table
    assert [l.block.params["side"]["col0"] for l in spec.layers] == [0, 12, 24, 36, 48]
    # mixers with equal rotation constants share one encoding
    assert len(spec.positions) == 3
    assert spec.head.params["softcap"] == 9.0 and spec.embedding.params["scale"] == 5.0


def test_absent_keys():
    spec = SezopelConfig.from_dict(small_doc("Q")).to_model_spec()
    assert spec.embedding.params["scale"] == 1.0 and spec.head.params["softcap"] == 0.0
    assert all("side" not in l.block.params for l in spec.layers)
    att = spec.layers[1].mixer.params
    assert att["kv_heads"] == att["heads"] == 3 and att["v_dim"] == att["head_dim"] == 10
    assert att["softcap"] == 0.0 and spec.positions[att["position"]].kind == "none"
    ret = spec.layers[3].mixer.params
    assert ret["vdim"] == 9 and ret["dim"] == 6
    names = {t.name for t in DecoderModel(spec).tensors()}
    assert "side.embed" not in names and not any(".side." in n for n in names)


@pytest.mark.parametrize("change,match", [
    (lambda d: d["layers"][0].update(type="conv"), "mixer type"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "key/value heads"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=26), "rotating"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), "rotating"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda d: d["layers"][1]["mixer"].update(kv_from=2), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda d: d["layers"][1]["mixer"].update(heads=2), "differ"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=24), "differ"),
    (lambda d: d["layers"][2]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "feed-forward kind"),
    (lambda d: d["layers"][0]["mixer"].update(softcap=-1.0), "score cap"),
    (lambda d: d.update(architecture="Other"), "architecture"),
    (lambda d: d.update(layers=[]), "layers"),
    (lambda d: d["norm"].update(kind="layer"), "norm kind"),
])
def test_refusals(change, match):
    doc = small_doc("P")
    change(doc)
    with pytest.raises(ConfigError, match=match):
        SezopelConfig.from_dict(doc).to_model_spec()


@pytest.mark.parametrize("base,dims", [(1e4, 16), (2.5e5, 64), (77.0, 6), (1e6, 128)])
def test_rotary_frequencies(base, dims):
    """theta^(-2i/dims), formed in 64 bits and rounded once."""
    from mormot2_ai_b200 import PartSpec
    from mormot2_ai_b200.parts import POSITIONS

    class Rt:
        device = "cpu"
    pos = POSITIONS.build(PartSpec("rope_half", {"theta": base, "rot_dim": dims,
                                                 "rounding": "once"}))
    pos.bind({}, Rt())
    f, n = pos.frequencies()
    want = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    assert n == dims and np.allclose(f.numpy().astype(np.float64), want, rtol=6e-8, atol=0)
    # the plain rotation turns pair (i, i + dims/2) by position * f_i and leaves the rest
    x = np.random.default_rng(dims).normal(0, 1, (3, 2, dims + 4))
    y = plain.rotate(x, [0, 5, 1000], {"base": base, "dims": dims})
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[..., dims:], x[..., dims:])
    a = 1000 * want[1]
    u, v = x[2, 1, 1], x[2, 1, 1 + dims // 2]
    assert np.isclose(y[2, 1, 1], u * np.cos(a) - v * np.sin(a))
    assert np.isclose(y[2, 1, 1 + dims // 2], v * np.cos(a) + u * np.sin(a))
    assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1))


def _weights(doc, seed, std=0.15):
    rng = np.random.default_rng(seed)
    W = {}
    for n in DecoderModel(SezopelConfig.from_dict(doc).to_model_spec()).tensors():
        W[n.name] = rng.normal(0, std, n.shape)
        if n.role == "vector":
            W[n.name] = 1 + 0.1 * W[n.name]
    return W


def test_the_plain_model_does_not_depend_on_where_a_sequence_ends():
    for name in ("P", "Q"):
        doc = small_doc(name)
        W = _weights(doc, 3)
        ids = np.random.default_rng(1).integers(0, doc["vocab"], 14).tolist()
        whole = plain.forward(doc, W, ids)
        assert whole.shape == (14, doc["vocab"])
        assert np.allclose(plain.forward(doc, W, ids[:6]), whole[:6], rtol=1e-9, atol=1e-9)
        if doc.get("logit_softcap"):
            assert np.abs(whole).max() < doc["logit_softcap"]


def test_the_plain_retention_is_a_decayed_sum_over_earlier_tokens():
    """o_t = sum_{j<=t} d^(t-j) (q_t . k_j) v_j with rotated q and k, k scaled by dim^(-1/2);
    a carried state continues the sequence."""
    rng = np.random.default_rng(7)
    m = {"heads": 2, "dim": 6, "vdim": 5, "decay": [0.9, 1.0], "rot": {"base": 50.0, "dims": 4}}
    W = {"p.mix." + s: rng.normal(0, 0.4, shape) for s, shape in
         (("q", (12, 9)), ("k", (12, 9)), ("v", (10, 9)), ("g", (10, 9)), ("o", (9, 10)))}
    h = rng.normal(0, 1, (11, 9))
    pos = np.arange(11)
    out, S = plain.retention_mixer(h, W, "p.", m, 1e-6, pos)
    q = plain.rotate((h @ W["p.mix.q"].T).reshape(11, 2, 6), pos, m["rot"])
    k = plain.rotate((h @ W["p.mix.k"].T).reshape(11, 2, 6), pos, m["rot"]) / np.sqrt(6)
    v = (h @ W["p.mix.v"].T).reshape(11, 2, 5)
    o = np.zeros((11, 2, 5))
    for t in range(11):
        for j in range(t + 1):
            for hd in range(2):
                o[t, hd] += m["decay"][hd] ** (t - j) * (q[t, hd] @ k[j, hd]) * v[j, hd]
    o = o / np.sqrt((o ** 2).mean(-1, keepdims=True) + 1e-6)
    want = (o.reshape(11, 10) * plain.silu(h @ W["p.mix.g"].T)) @ W["p.mix.o"].T
    assert np.allclose(out, want, rtol=1e-9, atol=1e-12)
    first, S1 = plain.retention_mixer(h[:4], W, "p.", m, 1e-6, pos[:4])
    rest, S2 = plain.retention_mixer(h[4:], W, "p.", m, 1e-6, pos[4:], state=S1)
    assert np.allclose(np.concatenate([first, rest]), out) and np.allclose(S2, S)


def test_the_plain_attention_caps_scores_and_gates_heads():
    rng = np.random.default_rng(11)
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 3, "scale": 40.0, "softcap": 2.0}
    W = {"p.mix." + s: rng.normal(0, 0.5, shape) for s, shape in
         (("q", (8, 7)), ("k", (4, 7)), ("v", (3, 7)), ("g", (2, 7)), ("o", (7, 6)))}
    h = rng.normal(0, 1, (6, 7))
    pos = np.arange(6)
    kv = plain.attention_keys_values(h, W, "p.", m, 1e-6, pos)
    assert np.allclose((kv[0] ** 2).mean(-1), 1.0, atol=1e-5)       # unit root mean square
    out = plain.attention_mixer(h, W, "p.", m, 1e-6, pos, kv)
    # with scores capped at 2 no softmax weight is below e^-4 of the largest: the last token's
    # output stays within the hull of the values, far from any single one
    q = plain.unit_rms((h @ W["p.mix.q"].T).reshape(6, 2, 4), 1e-6)
    s = 2.0 * np.tanh((q[5, 0] @ kv[0][:, 0].T) * 40.0 / 2.0)
    p = np.exp(s) / np.exp(s).sum()
    assert p.min() > np.exp(-4.0) / 6 * 0.99
    head0 = (p @ kv[1][:, 0]) * plain.sigmoid(h[5] @ W["p.mix.g"][0])
    o_inv = np.linalg.pinv(W["p.mix.o"].T)
    assert np.allclose((out[5] @ o_inv)[:3], head0, atol=1e-9)
