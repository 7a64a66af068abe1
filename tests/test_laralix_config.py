"""The Laralix family without a GPU: the registry, the model as data (looped layers with cache
lines of their own and what a pass adds, mixers side by side, kept first positions), tensor
names and shapes, defaults of absent keys, refusals, the order in which rotating neighbours
are laid for the rotate-half kernels, and the plain implementation's own consistency."""
import json

import numpy as np
import pytest

from mormot2_ai_b200 import ConfigError, DecoderModel, LaralixConfig, PartSpec, architectures
from mormot2_ai_b200.config.registry import family_of
from mormot2_ai_b200.parts import POSITIONS
from tests.laralix_models import SMALL, small_doc
from tests.plain import laralix_plain as plain


def test_registry_and_round_trip():
    assert "Laralix" in architectures()
    for name in SMALL:
        doc = small_doc(name)
        assert family_of(doc) is LaralixConfig
        c = LaralixConfig.from_dict(doc)
        again = LaralixConfig.from_dict(json.loads(json.dumps(c.to_dict())))
        assert again == c
        assert c.vocab_size == doc["vocab"] and c.hidden_size == doc["width"]
        assert c.num_hidden_layers == len(doc["layers"])


def test_looped_layers_have_lines_of_their_own_and_passes_add_their_inputs():
    c = LaralixConfig.from_dict(small_doc("A"))
    spec = c.to_model_spec()
    assert [r.layer for r in spec.schedule] == [0, 1, 0, 1, 2]
    assert [r.cache_line for r in spec.schedule] == [0, 1, 2, 3, 4]
    before = [r.before for r in spec.schedule]
    assert before[1] is None and before[3] is None and before[4] is None
    assert before[0].kind == "pass_input" and before[0].params["row"] == 0
    assert not before[0].params["add_embedding"]
    assert before[2].params["row"] == 1 and before[2].params["add_embedding"]
    assert c.order() == plain.layer_runs(small_doc("A"))
    c3 = LaralixConfig.from_dict(small_doc("C"))
    assert [r.layer for r in c3.to_model_spec().schedule] == [0, 1, 2, 1, 2, 1, 2]
    assert c3.order() == plain.layer_runs(small_doc("C"))
    # no loop: no entries, every layer once
    spec_b = LaralixConfig.from_dict(small_doc("B")).to_model_spec()
    assert [r.layer for r in spec_b.schedule] == [0, 1, 2]
    assert all(r.before is None for r in spec_b.schedule)
    assert not DecoderModel(spec_b).keeps_embedding and DecoderModel(spec).keeps_embedding


def test_tensor_names_shapes_lines_and_states():
    model = DecoderModel(LaralixConfig.from_dict(small_doc("A")).to_model_spec())
    shapes = {t.name: t.shape for t in model.tensors()}
    W = 72
    assert shapes["embed"] == (150, W) and shapes["head"] == (150, W)
    assert shapes["loop.step"] == (2, W) and shapes["final.norm"] == (W,)
    # parallel: attention with value rows of another size, the delta rule with its taps
    assert shapes["l0.mix.left.q"] == (4 * 18, W) and shapes["l0.mix.left.k"] == (2 * 18, W)
    assert shapes["l0.mix.left.v"] == (2 * 10, W) and shapes["l0.mix.left.o"] == (W, 4 * 10)
    assert shapes["l0.mix.left.q.norm"] == (18,) and shapes["l0.mix.left.k.norm"] == (18,)
    assert shapes["l0.mix.right.q"] == (2 * 10, W) and shapes["l0.mix.right.v"] == (4 * 14, W)
    assert shapes["l0.mix.right.q.conv"] == (2 * 10, 4) and shapes["l0.mix.right.v.conv"] == (4 * 14, 4)
    assert shapes["l0.mix.right.b"] == (4, W) and shapes["l0.mix.right.A_log"] == (4,)
    assert shapes["l0.mix.right.norm"] == (14,) and shapes["l0.mix.right.o"] == (W, 4 * 14)
    assert shapes["l0.mix.left.out"] == (W,) and shapes["l0.mix.right.out"] == (W,)
    # latent attention
    assert shapes["l1.mix.dq"] == (26, W) and shapes["l1.mix.uq"] == (3 * (10 + 8), 26)
    assert shapes["l1.mix.dkv"] == (22 + 8, W) and shapes["l1.mix.dkv.norm"] == (22,)
    assert shapes["l1.mix.uk"] == (3 * 10, 22) and shapes["l1.mix.uv"] == (3 * 14, 22)
    # parallel_2: no value projection, norms as wide as the projections, a low rank that the
    # stored tensor gives
    assert "l2.mix.left.v" not in shapes
    assert shapes["l2.mix.left.q.norm"] == (6 * 12,) and shapes["l2.mix.left.k.norm"] == (3 * 12,)
    assert shapes["l2.mix.right.a1"] == (5, W) and shapes["l2.mix.right.a2"] == (2 * 14, 5)
    doc = small_doc("A")
    del doc["layers"][2]["mixer"]["right"]["rank"]      # then only the stored tensors give it
    free = {t.name: t.shape for t in
            DecoderModel(LaralixConfig.from_dict(doc).to_model_spec()).tensors()}
    assert free["l2.mix.right.a1"] == (-1, W) and free["l2.mix.right.a2"] == (2 * 14, -1)
    assert shapes["l2.mix.right.a2.b"] == (2 * 14,) and shapes["l2.mix.right.norm"] == (6,)
    assert "l2.mix.left.out" not in shapes
    # lines: a window keeps a ring unless first positions are kept; the latent line is one plane
    needs = model.line_needs
    assert needs[0].window == 21 and needs[0].head_dim == 18 and needs[0].v_dim == 10
    assert needs[1].planes == 1 and needs[1].head_dim == 22 + 8
    assert needs[4].window == 0 and needs[4].head_dim == 12 and needs[4].kv_heads == 3
    assert needs[2] == needs[0] and needs[3] == needs[1]
    # states: the matrices and the convolutions' last inputs; the decayed matrices alone
    assert model.state_needs[0].shape == (4 * 10 * 14 + 3 * (2 * 10 + 2 * 10 + 4 * 14),)
    assert model.state_needs[4].shape == (2 * 14 * 6,)
    assert 1 not in model.state_needs


def test_absent_keys_and_a_layer_without_feed_forward():
    doc = small_doc("B")
    c = LaralixConfig.from_dict(doc)
    assert c.embedding_scale == 1.0 and c.logit_scale == 1.0 and c.loop is None
    spec = c.to_model_spec()
    left = spec.layers[1].mixer.params["branches"][0]["mixer"].params
    assert left["window"] == 0 and left["softcap"] == 0.0 and left["keep_first"] == 0
    assert left["sink_value"] == 0.0 and left["distance_exponent"] == -8.0
    assert spec.layers[1].feed_forward.kind == "none"
    shapes = {t.name: t for t in DecoderModel(spec).tensors()}
    assert "l1.mlp.up" not in shapes and shapes["l1.norm2"].optional
    first = spec.layers[0].mixer.params["branches"][0]["mixer"].params
    assert first["window"] == 9 and first["keep_first"] == 13
    assert [b["scale"] for b in spec.layers[0].mixer.params["branches"]] == [1.0, 0.5]
    assert [b["scale"] for b in spec.layers[1].mixer.params["branches"]] == [0.5, 0.5]


@pytest.mark.parametrize("change,text", [
    (lambda d: d["layers"][0].update(type="other"), "not known"),
    (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "key/value heads"),
    (lambda d: d["layers"][2]["mixer"]["left"].update(vdim=8), "values are the keys"),
    (lambda d: d["layers"][2]["mixer"]["right"].update(tau=0), "tau"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(conv=0), "conv"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=10), "rotating"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=5), "rotating"),
    (lambda d: d["loop"].update(stop=0), "stop"),
    (lambda d: d["loop"].update(stop=4), "stop"),
    (lambda d: d["layers"][0].update(mlp={"kind": "routed", "ff": 8}), "feed-forward kind"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_refusals(change, text):
    doc = small_doc("A")
    change(doc)
    with pytest.raises(ConfigError) as e:
        LaralixConfig.from_dict(doc).to_model_spec()
    assert text in str(e.value)


def test_neighbours_laid_out_for_the_rotate_half_kernels():
    """Turning neighbours (2i, 2i+1) of a vector equals turning the halves (i, i + n/2) of the
    vector laid out in ``half_order``, as far as dot products go."""
    rot = POSITIONS.build(PartSpec("rope_pairs", {"theta": 300.0, "rot_dim": 6, "rounding": "once"}))
    order = rot.half_order(9)
    assert order == [0, 2, 4, 1, 3, 5, 6, 7, 8]
    rng = np.random.default_rng(0)
    q, k = rng.normal(size=(2, 4, 9))
    pos = np.array([0, 3, 17, 400])
    want = (plain.rotate_pairs(q, pos, 6, 300.0) * plain.rotate_pairs(k, pos, 6, 300.0)).sum(-1)

    def halves(x):
        x = x[:, order]
        f = 300.0 ** (-2.0 * np.arange(3) / 6)
        a = pos[:, None] * f[None, :]
        out = x.copy()
        out[:, :3] = x[:, :3] * np.cos(a) - x[:, 3:6] * np.sin(a)
        out[:, 3:6] = x[:, 3:6] * np.cos(a) + x[:, :3] * np.sin(a)
        return out
    assert np.allclose((halves(q) * halves(k)).sum(-1), want)


def _weights(doc, seed):
    from mormot2_ai_b200.weights import random_tensors
    model = DecoderModel(LaralixConfig.from_dict(doc).to_model_spec())
    w = random_tensors(model.tensors(), seed, std=0.15, norm_std=0.2)
    return {k: v.double().numpy() for k, v in w.items()}


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_plain_implementation_is_causal_and_windows_close(name):
    """A prefix gives the logits the whole sequence gives at its positions; a token outside
    every window, prefix and state's reach does not matter where nothing reaches it."""
    doc = small_doc(name)
    w = _weights(doc, 3)
    ids = np.random.default_rng(1).integers(0, doc["vocab"], 40).tolist()
    whole = plain.forward(doc, w, ids)
    assert np.allclose(plain.forward(doc, w, ids[:17]), whole[:17], rtol=1e-9, atol=1e-9)
    assert np.isfinite(whole).all()


def test_plain_masks_and_softmax_with_one_more_term():
    m = plain.visible(8, 3, 2)
    assert m[7].tolist() == [True, True, False, False, False, True, True, True]
    assert m[2].tolist() == [True, True, True] + [False] * 5
    assert plain.visible(4, None)[3].all() and not plain.visible(4, 2)[3, 1]
    s = np.array([[0.0, np.log(3.0)]])
    p = plain.softmax_rows(s, np.array([[True, True]]), True)
    assert np.allclose(p, [[1 / 5, 3 / 5]])
    assert np.allclose(plain.softmax_rows(s, np.array([[True, True]]), False), [[1 / 4, 3 / 4]])
    assert np.allclose(plain.distance_slopes(4), [0.25, 0.0625, 2.0 ** -6, 2.0 ** -8])


def test_plain_delta_rule_replaces_what_a_key_holds():
    """With beta = 1, no decay and unit keys, writing (k, v) and then (k, v') leaves v' under
    k: what the rule is for. Checked through the plain branch with weights made for it."""
    D, V, W = 4, 3, 6
    w = {"q": np.zeros((D, W)), "k": np.zeros((D, W)), "v": np.zeros((V, W)),
         "q.conv": np.zeros((D, 2)), "k.conv": np.zeros((D, 2)), "v.conv": np.zeros((V, 2)),
         "b": np.zeros((1, W)), "a": np.zeros((1, W)), "A_log": np.array([-50.0]),
         "dt_bias": np.array([0.0]), "g": np.zeros((V, W)), "norm": np.ones(V),
         "o": np.eye(W)[:, :V]}
    for n in ("q.conv", "k.conv", "v.conv"):
        w[n][:, -1] = 1.0                           # the convolution passes the current token
    w["q"][0, 0] = w["k"][0, 0] = 50.0              # silu(50) = 50: q = k = e_0 after the norm
    w["v"][:, 1:4] = np.eye(3) * 10.0
    w["b"][0, 4] = 50.0                             # beta = 1
    w["g"][:, 5] = 50.0
    h = np.zeros((2, W))
    h[:, 0] = h[:, 4] = h[:, 5] = 1.0
    h[0, 1], h[1, 2] = 1.0, 1.0                     # v = (10, 0, 0) then (0, 10, 0)
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": V}
    out = plain.gated_delta(h, {"x." + k: v for k, v in w.items()}, "x.", m, 1e-6)
    # the second read-out sees only the second value (the first was taken back out)
    assert abs(out[1, 0]) < 1e-3 * abs(out[1, 1]) and out[1, 1] > 0
    assert out[0, 0] > 0 and abs(out[0, 1]) < 1e-9


def test_a_model_without_a_loop_may_store_the_passes_vectors():
    spec = LaralixConfig.from_dict(small_doc("B")).to_model_spec()
    needs = {t.name: t for t in DecoderModel(spec).tensors()}
    assert needs["loop.step"].optional and needs["loop.step"].shape == (-1, 40)
    looped = {t.name: t for t in DecoderModel(
        LaralixConfig.from_dict(small_doc("A")).to_model_spec()).tensors()}
    assert not looped["loop.step"].optional
