"""The Laralix family on a B200 against the plain implementation, in float32 and bfloat16:
each mechanism alone (with weights or inputs made so that a fault shows), then the engine on
four small models of other sizes: whole prompts with the residual after every layer run,
prompts against token-by-token decoding, portions down to two tokens, unequal batches against
each request alone, slots, pages and state used again, the first tokens, long decoding past
windows and page borders, decode graphs, and greedy generation through the entry point."""
import os

import numpy as np
import pytest
import torch

from mormot2_ai_b200 import Engine, Entry, LaralixConfig, LlmClient, PartSpec, Runtime
from mormot2_ai_b200 import kernels as K
from mormot2_ai_b200.cache.pages import PAGE, pages_for
from mormot2_ai_b200.cache.storage import CacheLine
from mormot2_ai_b200.parts import MIXERS, POSITIONS
from mormot2_ai_b200.parts.block import settle
from mormot2_ai_b200.weights import random_tensors
from tests.gpu_helpers import DEV, make_step
from tests.laralix_models import SMALL, SmallModel, _lat, _par, _par2
from tests.plain import laralix_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module", params=sorted(SMALL))
def small(request, tmp_path_factory):
    return SmallModel(request.param, str(tmp_path_factory.mktemp("laralix_" + request.param)))


@pytest.fixture(scope="module")
def small_a(tmp_path_factory):
    return SmallModel("A", str(tmp_path_factory.mktemp("laralix_A_only")))


# The bounds of this family's comparisons, set from what was measured and never widened to
# pass. float32: the largest difference of a logit over the largest logit. bfloat16: per
# position, the largest difference of a logit over the spread of the plain logits, bounded in
# the median, the ninth decile and the worst position of a comparison, and never tighter than
# three times what the plain implementation itself moves by when it rounds what a 16-bit run
# rounds. A wrong key, state, page or slot fails the float32 bound by orders of magnitude; the
# bfloat16 runs are there for the kernels that only they reach.
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


def line_of(n_slots, max_len, need, dtype, seed=0):
    """A cache line for a mixer's ``CacheNeed`` (all pages kept), pages scrambled over the pool."""
    per = pages_for(max_len)
    n_pages = n_slots * per + 3
    ids = np.random.default_rng(seed).permutation(n_pages)[:n_slots * per]
    table = torch.tensor(ids.reshape(n_slots, per), dtype=torch.int32, device=DEV)
    vdim = need.v_dim or need.head_dim
    k = torch.zeros((n_pages, need.kv_heads, PAGE, need.head_dim), dtype=dtype, device=DEV)
    v = (torch.zeros((n_pages, need.kv_heads, PAGE, vdim), dtype=dtype, device=DEV)
         if need.planes == 2 else None)
    return CacheLine(k, v, table, per, 0, 0, need.kv_heads, need.head_dim, need.v_dim)


def run_mixer(mixer, hs, cuts, hidden, dtype, line=None, state=None):
    """Feeds each sequence of ``hs`` (float arrays [n, hidden]) through the mixer in the
    portions that ``cuts`` names (all sequences of a step together), from slots 2, 0, 1, ...;
    returns what the mixer added to the residual, per sequence."""
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
        x = torch.full((h.shape[0], hidden), 0.5, device=DEV)
        pending = mixer.forward(h, x, step, line, state, True)
        if pending is not None:                 # split sums that the next norm would add
            settle(x, pending)
        got = x.cpu().double().numpy() - 0.5
        at = 0
        for b, a, e in rows:
            outs[b].append(got[at:at + e - a])
            at += e - a
    return [np.concatenate(o) for o in outs]


def mixer_of(layer, hidden, rt, eps=1e-5):
    """The library's mixer for a layer of a configuration (as the family builds it) and the
    plain implementation's sizes for it."""
    doc = {"architecture": "Laralix", "vocab": 8, "width": hidden, "norm": {"eps": eps},
           "layers": [layer]}
    spec = LaralixConfig.from_dict(doc).to_model_spec()
    positions = {k: POSITIONS.build(v) for k, v in spec.positions.items()}
    for p in positions.values():
        p.bind({}, rt)
    return MIXERS.build(spec.layers[0].mixer, "m.", positions=positions), layer["mixer"]


PORTIONS = [(0, 1), (1, 3), (3, 33), (33, 34), (34, 64), (64, 66), (66, 200)]


# ---------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_what_a_pass_adds(dtype):
    rng = np.random.default_rng(0)
    T, H = 7, 50
    x, x0 = rng.normal(0, 1, (T, H)), rng.normal(0, 3, (T, H))
    b = rounded(rng.normal(0, 1, H), dtype)
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    bd = f32(b).to(TORCH[dtype])
    xd = f32(x)
    K.pass_input(xd, bd, f32(x0))
    assert np.allclose(xd.cpu().numpy(), x + x0 + b, rtol=1e-6, atol=1e-6)
    xd = f32(x)
    K.pass_input(xd, bd)
    assert np.allclose(xd.cpu().numpy(), x + b, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("qw,kw,copy", [(24, 12, True), (300, 50, False), (7, 5, True)])
def test_norms_over_whole_rows_of_q_and_k(dtype, qw, kw, copy):
    rng = np.random.default_rng(qw)
    T, ld = 5, qw + 2 * kw + 3
    rows = rounded(rng.normal(0, 2, (T, ld)), dtype)
    rows[0, :qw] *= 1e-4                             # a row so small that eps counts
    rows = rounded(rows, dtype)
    wq, wk = rounded(1 + 0.3 * rng.normal(size=qw), dtype), rounded(1 + 0.3 * rng.normal(size=kw), dtype)
    dev = lambda a: torch.tensor(a).to(TORCH[dtype]).to(DEV)
    d = dev(rows)
    K.wide_qk_norm(d, qw, kw, dev(wq), dev(wk), 1e-5, copy)
    got = d.float().cpu().double().numpy()
    tol = 1e-6 if dtype == "float32" else 1e-2
    assert np.allclose(got[:, :qw], plain.rms_norm(rows[:, :qw], wq, 1e-5), rtol=tol, atol=tol)
    assert np.allclose(got[:, qw:qw + kw], plain.rms_norm(rows[:, qw:qw + kw], wk, 1e-5), rtol=tol, atol=tol)
    behind = got[:, qw + kw:qw + 2 * kw]
    assert np.array_equal(behind, rows[:, qw:qw + kw] if copy else rows[:, qw + kw:qw + 2 * kw])
    assert np.array_equal(got[:, qw + 2 * kw:], rows[:, qw + 2 * kw:])


def _attention_reference(q, keys, vals, pos, nkv, scale, softcap, slopes, sink, window, keep):
    """One query position ``pos`` over keys [n, nkv, D] with the plain implementation's mask
    and softmax: [heads, vdim]."""
    H = q.shape[0]
    n = keys.shape[0]
    mask = plain.visible(n, window or None, keep)[pos:pos + 1]
    out = []
    for h in range(H):
        g = h // (H // nkv)
        s = (keys[:, g] @ q[h]) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[h] * (pos - np.arange(n))
        out.append(plain.softmax_rows(s[None, :], mask, sink)[0] @ vals[:, g])
    return np.stack(out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,vdim", [(20, 12), (64, 64), (128, 128)])
@pytest.mark.parametrize("window,keep", [(40, 0), (40, 20), (70, 3), (5, 64)])
def test_loud_keys_at_the_edges_of_the_window_and_of_the_kept_prefix(dtype, dim, vdim, window, keep):
    """One key is made loud for the query: the last one inside the window and the first one
    outside it, the last kept position and the first one that is not kept, the sequence's
    first key and one far back. Inside, its value row dominates the output; outside, it must
    not show at all. The query is a decoded token (one token in the step) or the last token of
    a prompt's portion, at positions on either side of a page border."""
    heads, nkv, scale = 4, 2, 0.5
    T = TORCH[dtype]
    rt = Runtime(T)
    rng = np.random.default_rng(window + keep)
    slopes = plain.distance_slopes(heads) if keep == 0 else None
    sink = keep == 0
    dev_slopes = (torch.tensor(slopes, dtype=torch.float32, device=DEV) if slopes is not None else None)
    dev_sink = torch.zeros(heads, device=DEV) if sink else None
    from mormot2_ai_b200.parts.base import CacheNeed
    for pos in (63, 64, 150):
        n = pos + 1
        line = line_of(1, n, CacheNeed(nkv, dim, 0, 2, 0 if vdim == dim else vdim), T, seed=pos)
        keys = rounded(rng.normal(0, 0.1, (n, nkv, dim)), dtype)
        vals = rounded(rng.normal(0, 1, (n, nkv, vdim)), dtype)
        q = rounded(rng.normal(0, 1, (heads, dim)), dtype)
        table = line.page_table.cpu()
        lo = max(0, pos + 1 - window)
        spots = {lo, lo - 1, keep - 1, keep, 0, pos // 2, pos}
        for loud in sorted(s for s in spots if 0 <= s <= pos):
            k = keys.copy()
            k[loud, 0] = rounded(q[0] * 60.0 / (q[0] @ q[0]), dtype)      # raw score 30 for head 0
            for p in range(n):
                page = int(table[0, p // PAGE])
                line.k[page, :, p % PAGE] = torch.tensor(k[p]).to(T).to(DEV)
                line.v[page, :, p % PAGE] = torch.tensor(vals[p]).to(T).to(DEV)
            want = _attention_reference(q, k, vals, pos, nkv, scale, 0.0, slopes, sink, window, keep)
            seen = loud >= lo or loud < keep
            share = np.abs(want[0] - vals[loud, 0]).max()
            if slopes is None:      # (with a distance bias a far key's score is taken down again)
                assert (share < 1e-2) == seen, (pos, loud, share)
            for new in (1, 7):      # decoded alone, or the last token of a portion
                first = pos + 1 - new
                step = make_step([(0, first, [0] * new, [])])
                rows = np.zeros((new, heads * dim + 5))
                rows[-1, :heads * dim] = q.reshape(-1)
                row = torch.tensor(rows).to(T).to(DEV)
                out = torch.empty((new, heads * vdim), dtype=T, device=DEV)
                rt.attention(row, row.shape[1], out, step, line, heads, nkv, dim, window, scale,
                             vd=vdim, sink=dev_sink, slopes=dev_slopes, keep_first=keep)
                check(out[-1].float().cpu().numpy().reshape(heads, vdim), want, dtype,
                      f"query {pos}, loud key {loud}, {new} tokens in the step")
    rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_more_term_in_the_denominator_shrinks_a_lonely_token(dtype):
    """A sequence's first token sees itself and the sink: out = v e^s / (1 + e^s)."""
    T = TORCH[dtype]
    rt = Runtime(T)
    from mormot2_ai_b200.parts.base import CacheNeed
    line = line_of(1, 4, CacheNeed(1, 8, 0, 2, 0), T)
    k, v = np.full(8, 0.5), np.arange(8.0)
    page = int(line.page_table[0, 0])
    line.k[page, 0, 0] = torch.tensor(k).to(T).to(DEV)
    line.v[page, 0, 0] = torch.tensor(v).to(T).to(DEV)
    q = torch.tensor(np.full((1, 8), 0.25)).to(T).to(DEV)
    out = torch.empty((1, 8), dtype=T, device=DEV)
    rt.attention(q, 8, out, make_step([(0, 0, [0], [])]), line, 1, 1, 8, 0, 1.0,
                 sink=torch.zeros(1, device=DEV), slopes=torch.ones(1, device=DEV))
    s = 8 * 0.5 * 0.25
    assert np.allclose(out.float().cpu().numpy()[0], v * np.exp(s) / (1 + np.exp(s)), rtol=1e-2)


# ---------------------------------------------------------------------------- mixers alone
PARALLEL = [
    _par(4, 2, 18, 10, 0.3, 21, 4, 2, 10, 14, 4, softcap=6.0),
    _par(2, 2, 12, 12, 0.35, 0, 1, 1, 16, 8, 2),
    _par(8, 2, 64, 64, 0.125, 70, 2, 1, 64, 64, 3, softcap=20.0),
    _par(3, 1, 128, 128, 0.09, 100, 2, 2, 128, 128, 3, softcap=40.0),
    _par(2, 1, 16, 24, 0.2, 3, 3, 1, 200, 40, 1),          # rows of a state over eight lanes
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", PARALLEL, ids=[str(i) for i in range(len(PARALLEL))])
def test_attention_and_delta_rule_side_by_side(dtype, layer):
    """The ``parallel`` mixer alone: whole sequences, then portions down to one token with a
    batch mate and a slot that no sequence of the step uses; the branches' states afterwards."""
    hidden = 48
    rt = Runtime(TORCH[dtype])
    mixer, m = mixer_of(layer, hidden, rt)
    w, ref = part_weights(mixer, seed=m["left"]["dim"], std=0.15)
    # decays close to one, so that tokens far back still count in the state
    w["m.mix.right.A_log"] = w["m.mix.right.A_log"] - 4.0
    ref["m.mix.right.A_log"] = w["m.mix.right.A_log"].double().numpy()
    mixer.bind(to_dev(w, dtype), rt)
    rng = np.random.default_rng(3)
    hs = [rounded(rng.normal(0, 1, (n, hidden)), dtype) for n in (200, 37)]
    want = [plain.mixer_parallel(h, ref, "m.mix.", m, 1e-5) for h in hs]
    moved = [plain.mixer_parallel(h, ref, "m.mix.", m, 1e-5, rnd=plain.bfloat16) for h in hs]
    for cuts in ([(0, 200)], PORTIONS):
        line = line_of(4, 256, mixer.cache_need(), TORCH[dtype])
        state = torch.zeros((4,) + mixer.state_need().shape, device=DEV)
        state[1].fill_(7.0)
        got = run_mixer(mixer, hs, cuts, hidden, dtype, line=line, state=state)
        for g, wnt, mv in zip(got, want, moved):
            check(g, wnt, dtype, f"cuts {cuts}", mv if dtype == "bfloat16" else None)
        assert bool((state[1] == 7.0).all())
    rt.check()


PARALLEL_2 = [
    _par2(6, 3, 12, 0.25, 19, 5, 2, 14, 6, 8.0, 0.7, 1.2),
    _par2(1, 1, 20, 0.2, 9, 13, 3, 6, 10, 3.0, 1.0, 0.5),
    _par2(4, 1, 64, 0.1, 72, 9, 2, 32, 64, 12.0, 0.9, 0.6),
    _par2(2, 2, 128, 0.08, 66, 70, 2, 128, 64, 20.0, 1.1, 0.4),
    _par2(2, 1, 8, 0.5, 4, 0, 1, 256, 12, 50.0, 0.3, 2.0, rank=3),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", PARALLEL_2, ids=[str(i) for i in range(len(PARALLEL_2))])
def test_keys_as_values_and_gated_linear_attention_side_by_side(dtype, layer):
    hidden = 56
    rt = Runtime(TORCH[dtype])
    mixer, m = mixer_of(layer, hidden, rt)
    w, ref = part_weights(mixer, seed=m["left"]["dim"], std=0.15)
    mixer.bind(to_dev(w, dtype), rt)
    rng = np.random.default_rng(4)
    hs = [rounded(rng.normal(0, 1, (n, hidden)), dtype) for n in (200, 37)]
    want = [plain.mixer_parallel_2(h, ref, "m.mix.", m, 1e-5) for h in hs]
    moved = [plain.mixer_parallel_2(h, ref, "m.mix.", m, 1e-5, rnd=plain.bfloat16) for h in hs]
    for cuts in ([(0, 200)], PORTIONS):
        line = line_of(4, 256, mixer.cache_need(), TORCH[dtype])
        state = torch.zeros((4,) + mixer.state_need().shape, device=DEV)
        state[1].fill_(7.0)
        got = run_mixer(mixer, hs, cuts, hidden, dtype, line=line, state=state)
        for g, wnt, mv in zip(got, want, moved):
            check(g, wnt, dtype, f"cuts {cuts}", mv if dtype == "bfloat16" else None)
        assert bool((state[1] == 7.0).all())
    rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["gla", "delta"])
@pytest.mark.parametrize("far", [2, 63, 64, 500])
def test_a_state_keeps_a_token_from_far_back(dtype, mode, far):
    """One token writes a key that only the last query meets, ``far`` tokens later; every
    other key is orthogonal to that query. Without decay the last output is that token's
    value row; with decay it fades by the product of the decays in between (the heads' norm
    runs with an eps of one, so that the size of the output still shows). The kernel is fed the
    projections directly."""
    T = TORCH[dtype]
    H, D, V = 2, 16, 12
    n = far + 1
    rng = np.random.default_rng(far)
    q = np.zeros((n, H, D))
    k = rng.normal(0, 1, (n, H, D))
    k[:, :, 0] = 0.0                                # nobody else writes channel 0
    k[0, :, 0] = 3.0
    if mode == "delta":
        k[0, :, 1:] = 0.0                           # a unit key along channel 0 after its norm
    q[-1, :, 0] = 1.0                               # and only the last token reads it
    eps = 1.0
    v = rng.normal(0, 1, (n, H, V))
    f32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.float32, device=DEV)
    step = make_step([(1, 0, [0] * n, [])])
    out = torch.empty((n, H * V), dtype=T, device=DEV)
    state = torch.zeros((3, H * D * V), device=DEV)
    gate = np.full((n, H * V), 30.0)                # silu(30) = 30
    normw = np.ones(V)
    qkv = f32(np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1), gate], 1))
    cols = (0, H * D, 2 * H * D)
    if mode == "gla":
        z = np.full((n, H * D), 9.0)                # a = sigmoid(9)^(1/tau)
        K.linear_state_scan("gla", qkv, cols, 1, qkv, 2 * H * D + H * V, f32(normw), eps, state,
                            step, out, H, D, V, decay_logits=f32(z), decay_bias=f32(np.zeros(H * D)),
                            inv_tau=0.5)
        fade = (1.0 / (1.0 + np.exp(-9.0))) ** (0.5 * far)
        o = 3.0 * D ** -0.5 * fade * v[0] + (k[-1] * q[-1] * D ** -0.5).sum(-1, keepdims=True) * v[-1]
    else:
        sc = np.zeros((n, 2 * H))
        sc[:, :H] = 40.0                            # beta = 1
        sc[:, H:] = 0.0
        a_log = np.log(np.array([1e-9, 0.01]))     # head 0 keeps everything, head 1 fades
        dt = np.zeros(H)
        # unit keys that are orthogonal to e_0 take nothing away from what lies under e_0
        K.linear_state_scan("delta", qkv, cols, 1, qkv, 2 * H * D + H * V, f32(normw), eps,
                            state, step, out, H, D, V, scalars=f32(sc), beta_col=0, rate_col=H,
                            a_log=f32(a_log), dt_bias=f32(dt), unit_eps=1e-12)
        g = np.exp(-np.exp(a_log) * np.log(2.0))
        o = (D ** -0.5 * g ** far)[:, None] * v[0]
    want = plain.rms_norm(o, normw, eps) * 30.0
    assert np.abs(want).max() > 0.05
    got = out[-1].float().cpu().double().numpy().reshape(H, V)
    tol = 2e-4 if dtype == "float32" else 2e-2
    assert np.abs(got - want).max() <= tol * np.abs(want).max(), (got, want)
    assert bool((state[0] == 0).all()) and bool((state[2] == 0).all())


LATENT = [_lat(3, 10, 8, 14, 22, 26, 0.2, 500.0, 6), _lat(1, 14, 6, 8, 10, 12, 0.3, 50.0, 6),
          _lat(4, 32, 32, 64, 96, 64, 0.125, 1e5, 32), _lat(2, 64, 64, 128, 128, 96, 0.09, 1e4, 64)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", LATENT, ids=[str(i) for i in range(len(LATENT))])
def test_latent_attention_with_neighbours_turned(dtype, layer):
    hidden = 40
    rt = Runtime(TORCH[dtype])
    mixer, m = mixer_of(layer, hidden, rt)
    w, ref = part_weights(mixer, seed=m["dim"], std=0.2)
    mixer.bind(to_dev(w, dtype), rt)
    rng = np.random.default_rng(5)
    hs = [rounded(rng.normal(0, 1, (n, hidden)), dtype) for n in (200, 37)]
    want = [plain.mixer_latent(h, ref, "m.mix.", m, 1e-5) for h in hs]
    moved = [plain.mixer_latent(h, ref, "m.mix.", m, 1e-5, rnd=plain.bfloat16) for h in hs]
    for cuts in ([(0, 200)], PORTIONS):
        line = line_of(4, 256, mixer.cache_need(), TORCH[dtype])
        got = run_mixer(mixer, hs, cuts, hidden, dtype, line=line)
        for g, wnt, mv in zip(got, want, moved):
            check(g, wnt, dtype, f"cuts {cuts}", mv if dtype == "bfloat16" else None)
    rt.check()


# ---------------------------------------------------------------------------- the engine
def engine_of(model, dtype, **kw):
    kw.setdefault("max_tokens", 2048)
    return Engine.from_folder(model.folder, dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_prompts_and_states_after_every_layer_run(small, dtype):
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
        assert len(runs) == len(want_states) == small.runs
        moved = []                 # how far rounding alone moves each state (bfloat16)
        if dtype == "bfloat16":
            small.plain.forward(small.plain_config, small.weights, ids, rnd=small.plain.bfloat16,
                                states=moved)
        for i, (got, ref) in enumerate(zip(runs, want_states)):
            size = max(1.0, np.abs(ref).max())
            err = np.abs(got - ref).max(axis=1) / size
            if dtype == "float32":
                assert err.max() <= F32_TOL, (n, i, err.max())
            else:
                alone = np.abs(moved[i] - ref).max(axis=1) / size
                for what, base, f in (("median", 0.02, np.median),
                                      ("decile", 0.06, lambda a: np.quantile(a, 0.9)),
                                      ("worst", BF16_TOL["worst"], np.max)):
                    assert f(err) <= max(base, 3.0 * f(alone)), (n, i, what, f(err))
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_against_token_by_token_decoding(small, dtype):
    """The last tokens one by one through the cache and the states, across a page border and
    past every window, and a sequence that is decoded from its second token on."""
    eng = engine_of(small, dtype)
    for n, head in ((75, 58), (12, 1), (170, 126)):
        ids = small.tokens(n, seed=100 + n)
        slot = eng.open()
        got = [eng.step([Entry(slot, ids[:head], [head - 1])]).cpu().numpy()]
        for t in range(head, n):
            got.append(eng.step([Entry(slot, [ids[t]])]).cpu().numpy().copy())
        assert eng.length(slot) == n
        eng.close(slot)
        moved = small.rounded(ids, dtype)
        check(np.concatenate(got), small.reference(ids)[head - 1:], dtype,
              f"{n} tokens after a prompt of {head}", None if moved is None else moved[head - 1:])
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [2, 7, 64])
def test_portions_of_prompts(small, dtype, chunk):
    eng = engine_of(small, dtype, prefill_chunk=chunk)
    n = 131
    ids = small.tokens(n, seed=500 + chunk)
    ref, moved = small.reference(ids), small.rounded(ids, dtype)
    slot = eng.open()
    want = [0, 1, 62, 63, 64, 65, n - 1]
    out = eng.step([Entry(slot, ids, want)]).cpu().numpy()
    eng.close(slot)
    check(out, ref[want], dtype, f"{n} tokens in passes of {chunk}",
          None if moved is None else moved[want])
    slot = eng.open()
    got = [eng.step([Entry(slot, ids[a:b], list(range(b - a)))]).cpu().numpy()
           for a, b in ((0, 3), (3, 5), (5, 66), (66, n))]
    eng.close(slot)
    check(np.concatenate(got), ref, dtype, "steps of 3, 2, 61 and 65 tokens", moved)
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_batches_against_each_alone_with_reuse(small, dtype):
    """Batches of unequal requests, one after another in three slots and just enough pages:
    every logit equals that of the request's own whole pass; slots, pages and the slots'
    states are given back and used again (a state that was not set back would show)."""
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
            ref, moved = small.reference(reqs[i]), small.rounded(reqs[i], dtype)
            at_t = sorted(got[i])
            check(np.concatenate([got[i][t] for t in at_t]), ref[at_t], dtype, f"request {i}",
                  None if moved is None else moved[at_t])
    assert all(eng.book.held_pages(g) == 0 for g in range(len(eng.plans)))
    assert eng.book.slots.free == 3
    assert eng.faults() == []
    eng.rt.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_mates_do_not_matter(small_a, dtype):
    small = small_a
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
def test_long_decoding_from_the_first_token(small_a, dtype):
    small = small_a
    eng = engine_of(small, dtype, max_tokens=512)
    n = 200
    ids = small.tokens(n, seed=300)
    slot = eng.open()
    got = [eng.step([Entry(slot, [t])]).cpu().numpy().copy() for t in ids]
    eng.close(slot)
    check(np.concatenate(got), small.reference(ids), dtype, "200 tokens one by one",
          small.rounded(ids, dtype))
    eng.rt.check()


def test_a_step_that_fails_leaves_the_state_as_it_found_it(small_a):
    """A refused step changes nothing, and after it the sequence goes on as if it had not been."""
    small = small_a
    eng = engine_of(small, "float32", max_tokens=256)
    ids = small.tokens(40, seed=9)
    slot = eng.open()
    eng.step([Entry(slot, ids[:30], [])])
    with pytest.raises(Exception):
        eng.step([Entry(slot, [small.doc["vocab"] + 5])])
    out = eng.step([Entry(slot, ids[30:], list(range(10)))]).cpu().numpy()
    check(out, small.reference(ids)[30:], "float32", "after a refused step")


def test_decode_graphs_replay_what_was_computed(small_a):
    small = small_a
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
def test_generation_runs_pick_what_single_steps_pick(small, dtype):
    """The generation loop decodes in runs whose token ids, positions and lengths move on in
    device memory; a sequence alone must get the very tokens that the step function gives it
    one step at a time (the same kernels on the same numbers)."""
    client = LlmClient(small.folder, dtype=dtype, max_batch=2, cache_tokens=1024)
    eng = client.engine
    for n in (1, 70):
        p = small.tokens(n, seed=900 + n)
        got = client.generate([p], max_tokens=8, temperature=0.0, stop=[])[0]
        slot = eng.open()
        logits = eng.step([Entry(slot, p)]).cpu().numpy()
        want = []
        for _ in range(8):
            want.append(int(logits[-1].argmax()))
            logits = eng.step([Entry(slot, [want[-1]])]).cpu().numpy()
        eng.close(slot)
        assert got == want, (n, got, want)


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
                # a 16-bit run may leave the plain choice at a near tie only
                margin = float(logits[order[0]] - logits[order[1]])
                assert dtype == "bfloat16" and margin < 0.06 * logits.std(), (i, a, margin)
                break
            ids.append(a)
    assert all(client.engine.book.held_pages(g) == 0 for g in range(len(client.engine.plans)))


def test_steps_replayed_through_the_trace_runner(small_a, tmp_path):
    """``bin/trace_run`` as a user runs it: requests of unequal lengths start in one step, go on
    by one token together, the shorter ones end earlier, and other requests follow in the
    slots, pages and states that were given back. ``--max-tokens`` counts the tokens that live
    requests hold, no padding."""
    import json
    import subprocess
    import sys
    from tests.conftest import ROOT
    small = small_a
    lens, tails = [1, 70, 130, 9, 66, 3], [2, 5, 3, 4, 1, 6]
    reqs = {f"q{i}": small.tokens(n + t, seed=950 + i) for i, (n, t) in enumerate(zip(lens, tails))}
    steps, expect, n = [], {}, 0
    for batch in (["q0", "q1", "q2"], ["q3", "q4", "q5"]):
        at = {r: lens[int(r[1:])] for r in batch}
        steps.append({"step": n, "end": [],
                      "entries": [{"id": r, "tokens": reqs[r][:at[r]], "want": [at[r] - 1]}
                                  for r in batch]})
        expect[n] = [(r, at[r] - 1) for r in batch]
        n += 1
        live = list(batch)
        while live:
            entries = [{"id": r, "tokens": [reqs[r][at[r]]], "want": [0]} for r in live]
            expect[n] = [(r, at[r]) for r in live]
            for r in live:
                at[r] += 1
            ended = [r for r in live if at[r] >= len(reqs[r])]
            steps.append({"step": n, "entries": entries, "end": ended})
            live = [r for r in live if r not in ended]
            n += 1
    most = max(sum(len(reqs[r]) for r in batch) for batch in (["q0", "q1", "q2"], ["q3", "q4", "q5"]))
    for dtype in DTYPES:
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
                            small.folder, "--dtype", dtype, "--out", str(out), "--max-tokens",
                            str(most)], input="".join(json.dumps(s) + "\n" for s in steps),
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-3000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == \
            [f"done {s['step']}" for s in steps]
        refs = {r: small.reference(ids) for r, ids in reqs.items()}
        moved = {r: small.rounded(ids, dtype) for r, ids in reqs.items()}
        for step, wanted in expect.items():
            got = np.fromfile(str(out / f"{step}.f32"), dtype="<f4").reshape(-1, small.doc["vocab"])
            want = np.stack([refs[r][t] for r, t in wanted])
            check(got, want, dtype, f"step {step}",
                  None if dtype != "bfloat16" else np.stack([moved[r][t] for r, t in wanted]))
