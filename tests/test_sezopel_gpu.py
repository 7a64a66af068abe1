"""The Sezopel family on a B200 against the plain implementation, in float32 and bfloat16:
each mechanism alone (with weights or inputs made so that a fault shows), then the engine on
four small models of other sizes: whole prompts with the residual after every layer, prompts
against token-by-token decoding, portions down to two tokens, unequal batches against each
request alone, slots, pages and state used again, the first tokens, long decoding across page
borders, decode graphs, and greedy generation through the entry point."""
import os

import numpy as np
import pytest
import torch

from mormot2_ai_b200 import Engine, Entry, LlmClient, PartSpec, Runtime
from mormot2_ai_b200 import kernels as K
from mormot2_ai_b200.cache.pages import PAGE, pages_for
from mormot2_ai_b200.cache.storage import CacheLine
from mormot2_ai_b200.parts import FEED_FORWARDS, MIXERS, POSITIONS
from mormot2_ai_b200.parts.block import settle
from mormot2_ai_b200.weights import random_tensors
from tests.gpu_helpers import DEV, make_step
from tests.plain import sezopel_plain as plain
from tests.sezopel_models import SMALL, SmallModel

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module", params=sorted(SMALL))
def small(request, tmp_path_factory):
    return SmallModel(request.param, str(tmp_path_factory.mktemp("sezopel_" + request.param)))


@pytest.fixture(scope="module")
def small_p(tmp_path_factory):
    return SmallModel("P", str(tmp_path_factory.mktemp("sezopel_P_only")))


# The bounds of this family's comparisons, set from what was measured and never widened to
# pass. float32: the largest difference of a logit over the largest logit. bfloat16: per
# position, the largest difference of a logit over the spread of the plain logits, bounded
# in the median, the ninth decile and the worst position of a comparison. A wrong key, state,
# page or slot fails the float32 bound by orders of magnitude; the bfloat16 runs are there for
# the kernels that only they reach. Whole models norm what a sublayer gives back, so a position
# whose sublayer output nearly cancels is moved far by rounding alone (the first tokens of a
# retention layer above all): there the bfloat16 bounds are three times what the plain
# implementation shows when it rounds what a 16-bit run rounds (``rounded``), where that is more.
F32_TOL = 5e-5
BF16_TOL = {"median": 0.06, "decile": 0.15, "worst": 0.4}


def spread_errors(got, want):
    rows = np.abs(got - want).reshape(-1, want.shape[-1]).max(axis=1) / want.std()
    return np.median(rows), np.quantile(rows, 0.9), rows.max(), len(rows)


def check(got, want, dtype, what, rounded=None):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    record = os.environ.get("MORMOT_TOL_RECORD")
    if dtype == "float32":
        err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
        if record:
            with open(record, "a") as f:
                f.write(f"float32\t{err:.3e}\t{what}\n")
        assert err <= F32_TOL, f"{what}: relative error {err:.3g} (float32)"
        return
    med, dec, worst, n = spread_errors(got, want)
    tol = dict(BF16_TOL)
    if rounded is not None:
        r = spread_errors(np.asarray(rounded, dtype=np.float64), want)
        tol = {k: max(tol[k], 3.0 * r[i]) for i, k in enumerate(("median", "decile", "worst"))}
    if record:
        with open(record, "a") as f:
            f.write(f"bfloat16\t{med:.3f}\t{dec:.3f}\t{worst:.3f}\t{n}\t{what}\t{tol}\n")
    assert worst <= tol["worst"], f"{what}: a position off by {worst:.3g} of the spread"
    if n >= 8:
        assert med <= tol["median"] and dec <= tol["decile"], \
            f"{what}: median {med:.3g}, ninth decile {dec:.3g} of the spread (bfloat16)"


def part_weights(part, seed=0, std=0.1):
    w = random_tensors(part.tensors(), seed, std=std, norm_std=0.2, dtype=torch.bfloat16)
    return w, {k: v.double().numpy() for k, v in w.items()}


def to_dev(w, dtype):
    return {k: v.to(TORCH[dtype]).to(DEV) for k, v in w.items()}


def rounded(a, dtype):
    return torch.tensor(np.asarray(a), dtype=torch.float32).to(TORCH[dtype]).double().numpy()


def line_of(n_slots, max_len, kv_heads, dim, vdim, dtype, seed=0):
    """A cache line (value rows of a size of their own where vdim differs), pages scrambled
    over the pool."""
    per = pages_for(max_len)
    n_pages = n_slots * per + 3
    ids = np.random.default_rng(seed).permutation(n_pages)[:n_slots * per]
    table = torch.tensor(ids.reshape(n_slots, per), dtype=torch.int32, device=DEV)
    k = torch.zeros((n_pages, kv_heads, PAGE, dim), dtype=dtype, device=DEV)
    v = torch.zeros((n_pages, kv_heads, PAGE, vdim), dtype=dtype, device=DEV)
    return CacheLine(k, v, table, per, 0, 0, kv_heads, dim, 0 if vdim == dim else vdim)


def run_mixer(mixer, hs, cuts, hidden, dtype, line=None, state=None, writes=True, store=False):
    """Feeds each sequence of ``hs`` (float arrays [n, hidden]) through the mixer in the
    portions that ``cuts`` names (all sequences of a step together), from slots 2, 0, 1, ...;
    returns the outputs per sequence."""
    slots = [2, 0, 1, 3][:len(hs)]
    outs = [[] for _ in hs]
    for lo, hi in cuts:
        seqs, rows = [], []
        for b, h in enumerate(hs):
            a, e = min(lo, len(h)), min(hi, len(h))
            if e > a:
                seqs.append((slots[b], a, [0] * (e - a), []))
                rows.append((b, a, e))
        if not seqs:
            continue
        step = make_step(seqs)
        h = torch.tensor(np.concatenate([hs[b][a:e] for b, a, e in rows])).to(TORCH[dtype]).to(DEV)
        base = 0.0 if store else 0.5
        x = torch.full((h.shape[0], hidden), 0.5, device=DEV)
        pending = mixer.forward(h, x, step, line, state, writes, **({"store": True} if store else {}))
        if pending is not None:                 # split sums that the next norm would add
            if store:
                x = pending.partial.sum(0) if hasattr(pending, "partial") else x
            else:
                settle(x, pending)
        got = x.cpu().double().numpy() - base
        at = 0
        for b, a, e in rows:
            outs[b].append(got[at:at + e - a])
            at += e - a
    return [np.concatenate(o) for o in outs]


def rope(rt, rot):
    pos = POSITIONS.build(PartSpec("rope_half", {"theta": rot["base"], "rot_dim": rot["dims"],
                                                 "rounding": "once"}))
    pos.bind({}, rt)
    return pos


# ---------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,parts", [(5, 50, 0), (3, 200, 3), (70, 1031, 2), (1, 8, 1)])
def test_output_norm_into_the_residual(dtype, T, H, parts):
    """x += w * y / rms(y) with y given whole or as split sums; the new x also rounded for
    the next reader."""
    rng = np.random.default_rng(H)
    x = rng.normal(0, 2, (T, H)) + 1.0
    ys = rng.normal(0, 3, (max(parts, 1), T, H))
    ys[:, 0] *= 1e-5                                  # a row so small that eps counts
    w = rounded(1 + 0.2 * rng.normal(0, 1, H), dtype)
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    xd = f32(x)
    h = torch.empty((T, H), dtype=TORCH[dtype], device=DEV)
    K.norm_add(f32(ys) if parts else f32(ys[0]), f32(w).to(TORCH[dtype]), 1e-5, xd, h)
    want = x + plain.rms_norm(ys.sum(0), w, 1e-5)
    assert np.allclose(xd.cpu().numpy(), want, rtol=2e-6, atol=2e-6)
    assert np.array_equal(h.float().cpu().numpy(), xd.to(TORCH[dtype]).float().cpu().numpy())
    assert abs(plain.rms_norm(ys.sum(0), w, 1e-5)[0]).max() < 0.2      # eps did count


@pytest.mark.parametrize("dtype", DTYPES)
def test_activations_and_the_tokens_factor(dtype):
    rng = np.random.default_rng(4)
    T, N, V, col0 = 9, 13, 31, 7
    z = rounded(rng.normal(0, 2, (T, N + 3)), dtype)
    table = rounded(rng.normal(0, 1, (V, 40)), dtype)
    ids = rng.integers(0, V, T)
    dev = lambda a: torch.tensor(a).to(TORCH[dtype]).to(DEV)
    zd = dev(z)[:, :N]                                # rows wider than what is read
    for name, fn in (("relu_squared", lambda a: np.maximum(a, 0) ** 2), ("silu", plain.silu),
                     ("gelu_tanh", plain.gelu_tanh)):
        out = torch.empty((T, N), dtype=TORCH[dtype], device=DEV)
        K.unary_act(zd, out, K.UNARY_ACTIVATIONS[name])
        tol = 1e-6 if dtype == "float32" else 1e-2
        assert np.allclose(out.float().cpu().numpy(), fn(z[:, :N]), rtol=tol, atol=tol), name
    out = torch.empty((T, N), dtype=TORCH[dtype], device=DEV)
    K.unary_act(zd, out, K.UNARY_ACTIVATIONS["gelu_tanh"], dev(table), col0,
                torch.tensor(ids, dtype=torch.int32, device=DEV))
    want = plain.gelu_tanh(z[:, :N]) * table[ids][:, col0:col0 + N]
    assert np.allclose(out.float().cpu().numpy(), want, rtol=tol, atol=tol)
    logits = torch.tensor(rng.normal(0, 30, (4, 77)), dtype=torch.float32, device=DEV)
    ref = plain.soft_cap(logits.cpu().double().numpy(), 12.5)
    K.softcap_rows(logits, 12.5)
    assert np.allclose(logits.cpu().numpy(), ref, rtol=1e-6, atol=1e-5)
    assert np.abs(ref).max() > 12.4                   # the cap was in reach


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,ff", [(40, 56), (96, 320), (50, 33)])
def test_feed_forward_alone(dtype, hidden, ff):
    rt = Runtime(TORCH[dtype])
    part = FEED_FORWARDS.build(PartSpec("mlp", {"hidden_size": hidden, "intermediate_size": ff,
                                                "activation": "relu_squared",
                                                "names": {"up": "up", "down": "down"}}), "f.")
    w, ref = part_weights(part, seed=ff, std=0.2)
    part.bind(to_dev(w, dtype), rt)
    rng = np.random.default_rng(ff)
    for T in (1, 70):
        h = rounded(rng.normal(0, 1, (T, hidden)), dtype)
        want = plain.dense_ff(h, {"p.mlp.up": ref["f.up"], "p.mlp.down": ref["f.down"]}, "p.")
        hd = torch.tensor(h).to(TORCH[dtype]).to(DEV)
        x = torch.full((T, hidden), 2.0, device=DEV)
        pending = part.forward(hd, x, make_step([(0, 0, [0] * T, [])]))
        if pending is not None:
            settle(x, pending)
        check(x.cpu().numpy() - 2.0, want, dtype, f"added, {T} tokens")
        y = torch.full((T, hidden), 9.0, device=DEV)
        pending = part.forward(hd, y, make_step([(0, 0, [0] * T, [])]), store=True)
        got = pending.partial.sum(0) if pending is not None else y
        check(got.cpu().numpy(), want, dtype, f"stored, {T} tokens")


def retention_of(hidden, heads, dim, vdim, decay, rot, rt):
    positions = {"r": rope(rt, rot)} if rot else {}
    return MIXERS.build(PartSpec("retention", {
        "hidden_size": hidden, "heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
        "eps": 1e-5, "position": "r" if rot else "",
        "names": {s: "mix." + s for s in "qkvgo"}}), "m.", positions=positions)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,hidden,rot", [
    (3, 20, 12, 40, {"base": 500.0, "dims": 20}), (2, 32, 48, 96, {"base": 2e5, "dims": 32}),
    (1, 9, 22, 50, None), (2, 128, 64, 64, {"base": 1e4, "dims": 32}),
    (1, 64, 200, 48, {"base": 1e4, "dims": 2}), (5, 6, 6, 30, {"base": 77.0, "dims": 4}),
    (1, 256, 256, 24, {"base": 1e4, "dims": 256}), (1, 512, 320, 16, None)])
def test_retention_alone(dtype, heads, dim, vdim, hidden, rot):
    """Whole sequences, then the same in portions of 1, 2 and 30 tokens with a batch mate: the
    state carries over and slots' states do not mix. Decays from fast to exactly one."""
    rt = Runtime(TORCH[dtype])
    decay = [0.9, 1.0, 0.999, 0.5, 0.99][:heads]
    mixer = retention_of(hidden, heads, dim, vdim, decay, rot, rt)
    w, ref = part_weights(mixer, seed=dim)
    mixer.bind(to_dev(w, dtype), rt)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rot}
    rng = np.random.default_rng(dim)
    hs = [rounded(rng.normal(0, 1, (n, hidden)), dtype) for n in (70, 37)]
    want = [plain.retention_mixer(h, ref, "m.", m, 1e-5, np.arange(len(h)))[0] for h in hs]
    for cuts in ([(0, 70)], [(0, 1), (1, 3), (3, 33), (33, 34), (34, 70)]):
        for store in (True, False):
            state = torch.zeros((4,) + mixer.state_need().shape, device=DEV)
            state[1].fill_(7.0)                 # a slot that no sequence of the step uses
            got = run_mixer(mixer, hs, cuts, hidden, dtype, state=state, store=store)
            for g, wnt in zip(got, want):
                check(g, wnt, dtype, f"cuts {cuts}")
            assert bool((state[1] == 7.0).all())
    # the state after the tokens is the plain one
    S = plain.retention_mixer(hs[1], ref, "m.", m, 1e-5, np.arange(37))[1]
    got = state[0].cpu().double().numpy().reshape(S.shape)
    tol = 1e-5 if dtype == "float32" else 3e-2
    assert np.abs(got - S).max() <= tol * max(1.0, np.abs(S).max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,hidden,rot", [
    (3, 20, 12, 40, {"base": 500.0, "dims": 20}), (1, 9, 22, 50, None),
    (2, 64, 128, 64, {"base": 1e4, "dims": 64}), (2, 128, 64, 64, {"base": 1e4, "dims": 32}),
    (1, 64, 200, 48, {"base": 1e4, "dims": 2}), (1, 128, 160, 32, {"base": 3e3, "dims": 64}),
    (1, 256, 256, 24, {"base": 1e4, "dims": 256})])
def test_retention_chunk_by_chunk(dtype, heads, dim, vdim, hidden, rot):
    """The walk chunk by chunk (what a long portion takes) and the walk token by token give the
    plain outputs and leave the plain state: sequences that end inside a chunk, one token
    behind a chunk's last, and a single token, in one step; then portions that take turns
    between the two forms, so that either starts from the state the other left."""
    rt = Runtime(TORCH[dtype])
    decay = [0.97, 1.0, 0.5][:heads]
    mixer = retention_of(hidden, heads, dim, vdim, decay, rot, rt)
    assert K.retention_chunk(dim, vdim) in (32, 64)
    w, ref = part_weights(mixer, seed=dim + 1)
    mixer.bind(to_dev(w, dtype), rt)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rot}
    rng = np.random.default_rng(vdim)
    hs = [rounded(rng.normal(0, 1, (n, hidden)), dtype) for n in (193, 65, 1, 150)]
    plain_runs = [plain.retention_mixer(h, ref, "m.", m, 1e-5, np.arange(len(h))) for h in hs]
    tol = 1e-5 if dtype == "float32" else 3e-2
    for form, cuts in ((True, [(0, 200)]), (False, [(0, 200)]),
                       (True, [(0, 3), (3, 67), (67, 131), (131, 200)]),
                       (None, [(0, 130), (130, 132), (132, 200)])):
        mixer.chunked = form
        state = torch.zeros((4,) + mixer.state_need().shape, device=DEV)
        got = run_mixer(mixer, hs, cuts, hidden, dtype, state=state, store=True)
        for g, (want, _) in zip(got, plain_runs):
            check(g, want, dtype, f"chunked {form}, cuts {cuts}")
        for slot, (_, S) in zip([2, 0, 1, 3], plain_runs):
            have = state[slot].cpu().double().numpy().reshape(S.shape)
            assert np.abs(have - S).max() <= tol * max(1.0, np.abs(S).max()), (form, slot)


def test_retention_heads_too_large_for_a_chunk_are_walked_token_by_token():
    assert K.retention_chunk(512, 512) == 0 and K.retention_chunk(64, 64) == 64
    assert K.retention_chunk(64, 128) == 32


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far", [2, 63, 64, 500])
def test_retention_keeps_a_token_from_far_back(dtype, far):
    """With a decay of one the first token's key is made the one that the last query meets
    (all keys between are orthogonal to it but for a faint near one): the head's output is
    then made of that token's value row, however far back it lies. With a decay below one the
    same token has faded by decay^far."""
    heads, dim, vdim, hidden = 2, 16, 8, 16
    rt = Runtime(TORCH[dtype])
    d = 0.5 ** (1.0 / 8)
    mixer = retention_of(hidden, heads, dim, vdim, [1.0, d], None, rt)
    n = far + 1
    rng = np.random.default_rng(far)
    eye = np.eye(hidden)
    W = {"m.mix.q": np.concatenate([eye, eye]), "m.mix.k": np.concatenate([eye, eye]),
         "m.mix.v": rounded(rng.normal(0, 1, (heads * vdim, hidden)), dtype),
         "m.mix.g": rounded(rng.normal(0, 1, (heads * vdim, hidden)), dtype),
         "m.mix.o": np.eye(hidden, heads * vdim)}
    mixer.bind({k: torch.tensor(v).to(TORCH[dtype]).to(DEV) for k, v in W.items()}, rt)
    h = np.zeros((n, hidden))
    h[:, 2:] = rounded(rng.normal(0, 1, (n, hidden - 2)), dtype)
    h[0, :2] = [1.0, 0.0]                        # the far token: the only one along e_0
    h[-1] = 0.0
    h[-1, 0] = 1.0                               # the last query looks along e_0 only
    h[-2, 0] = 1.0 / 64                          # a near token that is faintly along e_0 too
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [1.0, d]}
    want = plain.retention_mixer(h, W, "m.", m, 1e-5, np.arange(n))[0]
    cuts = [(0, n)] if far < 500 else [(0, 300), (300, n - 1), (n - 1, n)]
    for form in (None, True, False):             # as the step's shape chooses, then either form
        mixer.chunked = form
        state = torch.zeros((4,) + mixer.state_need().shape, device=DEV)
        got = run_mixer(mixer, [h], cuts, hidden, dtype, state=state, store=True)[0]
        check(got[-1:], want[-1:], dtype, f"a token {far} back, chunked {form}")
    # head 0 in closed form: the far token, the faint near one and the last token itself
    gate = plain.silu(h[-1] @ W["m.mix.g"].T)
    Wv = W["m.mix.v"][:vdim]
    o = (h[0] + h[-2] / 64 + h[-1]) @ Wv.T
    assert np.allclose(want[-1][:vdim], plain.unit_rms(o, 1e-5 * dim) * gate[:vdim],
                       rtol=1e-9, atol=1e-9)
    assert np.abs(h[0] @ Wv.T).max() > 8 * np.abs(h[-2] @ Wv.T / 64).max()


def attention_of(hidden, heads, kv, dim, vdim, rot, softcap, scale, rt, shared=False):
    positions = {"r": rope(rt, rot)} if rot else {}
    names = {"q": "mix.q", "o": "mix.o", "g": "mix.g"}
    if not shared:
        names.update({"k": "mix.k", "v": "mix.v"})
    return MIXERS.build(PartSpec("gqa_attention", {
        "hidden_size": hidden, "heads": heads, "kv_heads": kv, "head_dim": dim, "v_dim": vdim,
        "scale": scale, "softcap": softcap, "head_norm": "unit_after_rotation",
        "head_norm_eps": 1e-5, "shared_kv": shared, "position": "r" if rot else "",
        "names": names}), "a.", positions=positions)


ATTENTION_SIZES = [
    (4, 2, 24, 40, {"base": 1e4, "dims": 16}, 7.0),     # the general kernel: value rows of 40
    (3, 3, 10, 6, None, 0.0),                           # no rotation, no cap, no grouping
    (4, 1, 64, 64, {"base": 5e5, "dims": 64}, 3.0),     # tensor-core sizes
    (2, 1, 128, 128, {"base": 1e4, "dims": 64}, 12.0),
    (6, 2, 128, 128, {"base": 1e4, "dims": 128}, 0.0),
    (1, 1, 14, 14, {"base": 77.0, "dims": 14}, 1.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,vdim,rot,softcap", ATTENTION_SIZES)
def test_attention_alone(dtype, heads, kv, dim, vdim, rot, softcap, monkeypatch):
    """Prompts over a page border in portions and decoded tokens, with a batch mate; then a
    second mixer without keys and values of its own reads what the first one kept. In
    bfloat16, heads of 64 and 128 values with value rows of the same size run on the
    tensor-core kernels, cap and gates included; everything else on the general kernel."""
    hidden, scale = 72, 2.5
    rt = Runtime(TORCH[dtype])
    general = []
    simt = K.attention_simt
    monkeypatch.setattr(K, "attention_simt", lambda *a, **k: (general.append(1), simt(*a, **k))[1])
    mixer = attention_of(hidden, heads, kv, dim, vdim, rot, softcap, scale, rt)
    need = mixer.cache_need()
    assert (need.head_dim, need.v_dim or need.head_dim) == (dim, vdim)
    w, ref = part_weights(mixer, seed=dim)
    w["a.mix.g"] = w["a.mix.g"] * 20                   # gates from nearly shut to nearly open
    ref["a.mix.g"] = w["a.mix.g"].double().numpy()
    mixer.bind(to_dev(w, dtype), rt)
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot,
         "softcap": softcap or None}
    rename = lambda r: {k.replace("a.", "p."): v for k, v in r.items()}
    rng = np.random.default_rng(vdim)
    hs = [rounded(rng.normal(0, 1, (n, hidden)), dtype) for n in (131, 9)]
    kvs = [plain.attention_keys_values(h, rename(ref), "p.", m, 1e-5, np.arange(len(h))) for h in hs]
    want = [plain.attention_mixer(h, rename(ref), "p.", m, 1e-5, np.arange(len(h)), kv_)
            for h, kv_ in zip(hs, kvs)]
    line = line_of(3, 192, kv, dim, vdim, TORCH[dtype])
    cuts = [(0, 3), (3, 65), (65, 128), (128, 129), (129, 130), (130, 131)]
    got = run_mixer(mixer, hs, cuts, hidden, dtype, line=line, store=True)
    for g, wnt in zip(got, want):
        check(g, wnt, dtype, "portions and single tokens")
    # a reader of the same line: its own queries, gates, scale and cap
    reader = attention_of(hidden, heads, kv, dim, vdim, rot, 2.0, 4.0, rt, shared=True)
    assert not any(t.name.endswith((".k", ".v")) for t in reader.tensors())
    w2, ref2 = part_weights(reader, seed=dim + 1)
    reader.bind(to_dev(w2, dtype), rt)
    m2 = dict(m, softcap=2.0, scale=4.0)
    want2 = [plain.attention_mixer(h, rename(ref2), "p.", m2, 1e-5, np.arange(len(h)), kv_)
             for h, kv_ in zip(hs, kvs)]
    got2 = run_mixer(reader, hs, [(0, 131)], hidden, dtype, line=line, writes=False, store=True)
    for g, wnt in zip(got2, want2):
        check(g, wnt, dtype, "a reader of another mixer's keys and values")
    fast = dtype == "bfloat16" and dim == vdim and dim in (64, 128)
    assert (len(general) == 0) == fast


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("past", [63, 64, 700])
@pytest.mark.parametrize("dim,vdim", [(32, 48), (64, 64), (128, 128)])
def test_attention_finds_one_far_key_under_the_cap(dtype, past, dim, vdim, monkeypatch):
    """One key far back is made loud for the last query (the first key, one at a page border,
    one in the middle): its raw score is far above the cap, so its weight is e^cap against
    e^(small) of the others, no more; the head's output is multiplied by the gate's sigmoid.
    Heads of 64 and 128 values go to the tensor-core kernels in bfloat16."""
    heads, kv, cap, scale = 2, 1, 6.0, 0.5
    rt = Runtime(TORCH[dtype])
    T = TORCH[dtype]
    general = []
    simt = K.attention_simt
    monkeypatch.setattr(K, "attention_simt", lambda *a, **k: (general.append(1), simt(*a, **k))[1])
    line = line_of(1, past + 1, kv, dim, vdim, T)
    rng = np.random.default_rng(past)
    keys = rounded(rng.normal(0, 0.1, (past + 1, dim)), dtype)
    vals = rounded(rng.normal(0, 1, (past + 1, vdim)), dtype)
    q = rounded(rng.normal(0, 1, (heads, dim)), dtype)
    gates = rounded(np.array([1.5, -0.7]), dtype)
    table = line.page_table.cpu()
    for loud in sorted({0, min(past, 64), past // 2}):
        k = keys.copy()
        k[loud] = rounded(q[0] * 200.0 / (q[0] @ q[0]), dtype)       # raw score 100 for head 0
        for pos in range(past + 1):
            page = int(table[0, pos // PAGE])
            line.k[page, 0, pos % PAGE] = torch.tensor(k[pos]).to(T).to(DEV)
            line.v[page, 0, pos % PAGE] = torch.tensor(vals[pos]).to(T).to(DEV)
        step = make_step([(0, past, [0], [])])
        out = torch.empty((1, heads * vdim), dtype=T, device=DEV)
        row = torch.tensor(np.concatenate([q.reshape(-1), gates, np.zeros(6)])[None]).to(T).to(DEV)
        rt.attention(row, row.shape[1], out, step, line, heads, kv, dim, 0, scale, vd=vdim,
                     softcap=cap, gate=row[:, heads * dim:], gate_stride=row.shape[1])
        for h in range(heads):
            s = plain.soft_cap((k @ q[h]) * scale, cap)
            e = np.exp(s - s.max())
            want = (e @ vals) / e.sum() * plain.sigmoid(gates[h])
            check(out.float().cpu().numpy()[0, h * vdim:(h + 1) * vdim], want, dtype,
                  f"head {h}, loud key {loud} of {past + 1}")
        # the cap counts: without it the loud key alone would be the output
        s0 = plain.soft_cap((k @ q[0]) * scale, cap)
        assert abs(s0[loud] - cap) < 1e-3 and np.exp(s0 - s0.max())[loud] / np.exp(s0 - s0.max()).sum() < 0.999
    assert (len(general) == 0) == (dtype == "bfloat16" and dim == vdim)


# ---------------------------------------------------------------------------- the engine
def engine_of(model, dtype, **kw):
    kw.setdefault("max_tokens", 2048)
    return Engine.from_folder(model.folder, dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_states_after_every_layer(small, dtype):
    eng = engine_of(small, dtype)
    for n in small.prompt_lens:
        ids = small.tokens(n, seed=n)
        states = []
        eng.on_state = lambda name, x: states.append((name, x.cpu().numpy().copy()))
        slot = eng.open()
        out = eng.step([Entry(slot, ids, list(range(n)))])
        eng.on_state = None
        eng.close(slot)
        want_states = []
        want = small.reference(ids, want_states)
        check(out.cpu().numpy(), want, dtype, f"{small.name}: whole prompt of {n}",
              small.rounded(ids, dtype))
        runs = [x for name, x in states if name.startswith("run")]
        assert len(runs) == len(want_states) == len(small.doc["layers"])
        moved = []                 # how far rounding alone moves each state (bfloat16)
        if dtype == "bfloat16":
            small.plain.forward(small.plain_config, small.weights, ids, moved,
                                rnd=small.plain.bfloat16)
        for i, (got, ref) in enumerate(zip(runs, want_states)):
            size = max(1.0, np.abs(ref).max())
            err = np.abs(got - ref).max(axis=1) / size
            if dtype == "float32":
                assert err.max() <= F32_TOL, (n, i, err.max())
            else:
                # a position whose scores are sharp or whose sublayer output nearly cancels is
                # moved far by rounding, and not the same way twice: bounds on the distribution
                alone = np.abs(moved[i] - ref).max(axis=1) / size
                for what, base, f in (("median", 0.02, np.median),
                                      ("decile", 0.06, lambda a: np.quantile(a, 0.9)),
                                      ("worst", BF16_TOL["worst"], np.max)):
                    assert f(err) <= max(base, 3.0 * f(alone)), (n, i, what, f(err))
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_token_by_token_decoding(small, dtype):
    """The last tokens one by one through the cache and the state, across a page border, and
    a sequence that is decoded from its second token on."""
    eng = engine_of(small, dtype)
    for n, head in ((75, 58), (12, 1), (140, 126)):
        ids = small.tokens(n, seed=100 + n)
        slot = eng.open()
        got = [eng.step([Entry(slot, ids[:head], [head - 1])]).cpu().numpy()]
        for t in range(head, n):
            got.append(eng.step([Entry(slot, [ids[t]])]).cpu().numpy().copy())
        assert eng.length(slot) == n
        eng.close(slot)
        rounded = small.rounded(ids, dtype)
        check(np.concatenate(got), small.reference(ids)[head - 1:], dtype,
              f"{n} tokens after a prompt of {head}",
              None if rounded is None else rounded[head - 1:])
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [2, 7, 64])
def test_portions_of_prompts(small, dtype, chunk):
    eng = engine_of(small, dtype, prefill_chunk=chunk)
    n = 131
    ids = small.tokens(n, seed=500 + chunk)
    ref, rounded = small.reference(ids), small.rounded(ids, dtype)
    slot = eng.open()
    want = [0, 1, 62, 63, 64, 65, n - 1]
    out = eng.step([Entry(slot, ids, want)]).cpu().numpy()
    eng.close(slot)
    check(out, ref[want], dtype, f"{n} tokens in passes of {chunk}",
          None if rounded is None else rounded[want])
    slot = eng.open()
    got = [eng.step([Entry(slot, ids[a:b], list(range(b - a)))]).cpu().numpy()
           for a, b in ((0, 3), (3, 5), (5, 66), (66, n))]
    eng.close(slot)
    check(np.concatenate(got), ref, dtype, "steps of 3, 2, 61 and 65 tokens", rounded)
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_against_each_alone_with_reuse(small, dtype):
    """Batches of unequal requests, one after another in three slots and just enough pages:
    every logit equals that of the request's own whole pass; slots, pages and the slots'
    retention state are given back and used again (a state that was not set back would show)."""
    lens = small.prompt_lens + [2, 65, 33]
    decode = [small.decode_steps, 3, 1, small.decode_steps, 5, 2, 4][:len(lens)]
    lens = lens[:len(decode)]
    pages = max(sum(-(-(n + d) // 64) for n, d in list(zip(lens, decode))[b0:b0 + 3])
                for b0 in range(0, len(lens), 3))
    eng = engine_of(small, dtype, max_tokens=64 * pages, max_slots=3)
    reqs = [small.tokens(n + d, seed=200 + i) for i, (n, d) in enumerate(zip(lens, decode))]
    for b0 in range(0, len(reqs), 3):
        idx = list(range(b0, min(b0 + 3, len(reqs))))
        slots = {i: eng.open() for i in idx}
        assert sorted(slots.values()) == list(range(len(idx)))
        got = {i: {} for i in idx}
        out = eng.step([Entry(slots[i], reqs[i][:lens[i]]) for i in idx]).cpu().numpy()
        for row, i in enumerate(idx):
            got[i][lens[i] - 1] = out[row:row + 1]
        at = {i: lens[i] for i in idx}
        live = list(idx)
        while live:
            live = [i for i in live if at[i] < len(reqs[i])]
            for i in idx:
                if i not in live and i in slots:
                    eng.close(slots.pop(i))
            if not live:
                break
            out = eng.step([Entry(slots[i], [reqs[i][at[i]]]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                got[i][at[i]] = out[row:row + 1].copy()
                at[i] += 1
        for i in idx:
            ref, rounded = small.reference(reqs[i]), small.rounded(reqs[i], dtype)
            at_t = sorted(got[i])
            check(np.concatenate([got[i][t] for t in at_t]), ref[at_t], dtype, f"request {i}",
                  None if rounded is None else rounded[at_t])
    assert all(eng.book.held_pages(g) == 0 for g in range(len(eng.plans)))
    assert eng.book.slots.free == 3
    assert eng.faults() == []
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_mates_do_not_matter(small_p, dtype):
    small = small_p
    eng = engine_of(small, dtype)
    a = small.tokens(70, seed=1)
    others = [small.tokens(n, seed=2 + n) for n in (3, 129)]
    s = eng.open()
    alone = [eng.step([Entry(s, a[:66], [0, 64, 65])]).cpu().numpy()]
    alone += [eng.step([Entry(s, [t])]).cpu().numpy().copy() for t in a[66:]]
    eng.close(s)
    slots = [eng.open() for _ in range(3)]
    out = eng.step([Entry(slots[0], others[0], []), Entry(slots[1], a[:66], [0, 64, 65]),
                    Entry(slots[2], others[1], [])]).cpu().numpy()
    tol = 1e-5 if dtype == "float32" else 3e-2
    scale = np.abs(alone[0]).max()
    assert np.abs(out - alone[0]).max() <= tol * scale
    for k, t in enumerate(a[66:]):
        out = eng.step([Entry(slots[0], [5]), Entry(slots[1], [t]), Entry(slots[2], [7])])
        assert np.abs(out.cpu().numpy()[1:2] - alone[1 + k]).max() <= tol * scale
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_the_first_token(small_p, dtype):
    small = small_p
    eng = engine_of(small, dtype, max_tokens=512)
    n = 200
    ids = small.tokens(n, seed=300)
    slot = eng.open()
    got = [eng.step([Entry(slot, [t])]).cpu().numpy().copy() for t in ids]
    eng.close(slot)
    check(np.concatenate(got), small.reference(ids), dtype, "200 tokens one by one",
          small.rounded(ids, dtype))
    eng.rt.check()


def test_other_orders_of_layers(tmp_path):
    """A model of retention layers only (no keys and values anywhere: the cache has no page
    pool at all), and one of attention layers only in which two owners of keys and values each
    have a reader, the second reader after another owner's layer."""
    import json
    from mormot2_ai_b200 import SezopelConfig, write_random_model
    from tests.plain.qwen3_plain import read_safetensors
    from tests.sezopel_models import _att, _ret
    rot = {"base": 900.0, "dims": 8}
    docs = [{"architecture": "Sezopel", "vocab": 97, "width": 40, "norm": {"eps": 1e-5},
             "token_side": {"dim": 5},
             "layers": [_ret(2, 12, [0.9, 0.999], vdim=8, rot=rot, ff=24),
                        _ret(1, 16, [0.97], rot=rot)]},
            {"architecture": "Sezopel", "vocab": 61, "width": 48, "norm": {"eps": 1e-6},
             "logit_softcap": 4.0,
             "layers": [_att(2, 16, 2.0, kv=1, vdim=24, rot=rot, softcap=5.0, ff=40),
                        _att(3, 12, 3.0, vdim=8, ff=20),
                        _att(2, 16, 1.0, kv=1, vdim=24, rot=rot, kv_from=0),
                        _att(3, 12, 5.0, vdim=8, softcap=2.0, kv_from=1, ff=28)]}]
    for k, doc in enumerate(docs):
        folder = str(tmp_path / f"m{k}")
        write_random_model(folder, SezopelConfig.from_dict(doc), 50 + k, std=0.15, norm_std=0.2)
        W = {n: np.asarray(v, dtype=np.float64)
             for n, v in read_safetensors(folder + "/model.safetensors").items()}
        with open(folder + "/config.json") as f:
            cfg = json.load(f)
        ids = np.random.default_rng(k).integers(0, doc["vocab"], 90).tolist()
        ref = plain.forward(cfg, W, ids)
        eng = Engine.from_folder(folder, dtype="float32", max_tokens=256)
        assert len(eng.plans) == (0 if k == 0 else 2)
        slot = eng.open()
        got = [eng.step([Entry(slot, ids[:70], list(range(70)))]).cpu().numpy()]
        got += [eng.step([Entry(slot, [t])]).cpu().numpy().copy() for t in ids[70:]]
        eng.close(slot)
        check(np.concatenate(got), ref, "float32", f"order {k}")
        eng.rt.check()
        client = LlmClient(folder, dtype="float32", max_batch=2, cache_tokens=256)
        prompts = [ids[:5], ids[5:40], ids[40:42]]
        for p, tokens in zip(prompts, client.generate(prompts, max_tokens=3, temperature=0.0, stop=[])):
            seq = list(p)
            for a in tokens:
                assert a == int(np.argmax(plain.forward(cfg, W, seq)[-1])), (k, seq, a)
                seq.append(a)


def test_a_step_that_fails_leaves_the_state_as_it_found_it(small_p):
    """A refused step changes nothing, and after it the sequence goes on as if it had not been."""
    small = small_p
    eng = engine_of(small, "float32", max_tokens=256)
    ids = small.tokens(40, seed=9)
    slot = eng.open()
    eng.step([Entry(slot, ids[:30], [])])
    with pytest.raises(Exception):
        eng.step([Entry(slot, [small.doc["vocab"] + 5])])
    out = eng.step([Entry(slot, ids[30:], list(range(10)))]).cpu().numpy()
    check(out, small.reference(ids)[30:], "float32", "after a refused step")


def test_decode_graphs_replay_what_was_computed(small_p):
    small = small_p
    ids = [small.tokens(40 + 3 * i, seed=600 + i) for i in range(2)]
    for dtype in DTYPES:
        outs = {}
        for graphs in (True, False):
            eng = engine_of(small, dtype, max_tokens=1024)
            assert eng.use_graphs
            eng.use_graphs = graphs
            slots = [eng.open() for _ in ids]
            eng.step([Entry(s, r[:30], []) for s, r in zip(slots, ids)])
            outs[graphs] = [eng.step([Entry(s, [r[t]]) for s, r in zip(slots, ids)]).cpu().numpy().copy()
                            for t in range(30, 40)]
            assert len(eng.graphs) == (1 if graphs else 0)
            eng.rt.check()
        for a, b in zip(outs[True], outs[False]):
            assert np.array_equal(a, b)
        if dtype == "float32":
            for row, r in enumerate(ids):
                check(np.concatenate([o[row:row + 1] for o in outs[True]]),
                      small.reference(r)[30:40], dtype, f"row {row}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_entry_point(small, dtype):
    client = LlmClient(small.folder, dtype=dtype, max_batch=3, cache_tokens=1024)
    prompts = [small.tokens(n, seed=800 + n) for n in (4, 70, 17, 1)]
    steps = small.decode_steps
    got = client.generate(prompts, max_tokens=steps, temperature=0.0, stop=[])
    for p, tokens in zip(prompts, got):
        assert len(tokens) == steps
        ids = list(p)
        for i, a in enumerate(tokens):
            logits = small.reference(ids)[-1]
            order = np.argsort(-logits, kind="stable")
            if a != int(order[0]):
                margin = float(logits[order[0]] - logits[order[1]])
                assert dtype == "bfloat16" and margin < 0.06 * logits.std(), (i, a, margin)
                break
            ids.append(a)
    assert all(client.engine.book.held_pages(g) == 0 for g in range(len(client.engine.plans)))
