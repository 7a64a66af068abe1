"""A plain, slow implementation of the Laralix decoder in NumPy float64: one function per
mechanism, whole sequences at once, no cache, recurrences token by token. It shares no code
with the library and is the oracle of the library's tests.

The design. x = E[token] * s_e. Layers are pre-norm: x += mixer(N1(x)), x += ff(N2(x)) with
N(x) = x / sqrt(mean(x^2) + eps) * (1 + w). A run of layers [start, stop) may be passed
``times`` times with the same weights; before every pass x += step[t], and before every pass
but the first also x += x0 (the embedding's output). Three mixers:

``parallel``: half the sum of two branches, each normed over the width with a plain weight.
Left: grouped-query attention, q and k normed per head (one weight for all heads), no rotation,
score = cap tanh(scale q.k / cap) - m_h (i - j), m_h = 2^(-8 (h+1) / H), a window of the last
``size`` positions, and a softmax whose denominator has one more term exp(0). Right: the gated
delta rule: q, k, v through a short causal convolution per channel and SiLU, q and k to unit
length (q also times dim^-1/2), beta = sigmoid(.), g = exp(-exp(A) softplus(. + dt)),
S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; o normed per head, times
silu(W_g h).

``parallel_2``: c_l left + c_r right. Left: grouped-query attention whose values are the keys
as projected, q and k normed over their whole rows, a window that also keeps the first
``keep_first`` positions, ordinary softmax. Right: gated linear attention with a decay per key
channel a = sigmoid(W_a2 W_a1 h + b)^(1/tau): S <- diag(a) S + k v^T; o = S^T q.

``latent_attention``: queries through a normed latent; keys and values from a normed latent c
and one rotated key part shared by all heads; rotation of neighbouring pairs (2i, 2i+1).

``weights``: a dict name -> float64 array. ``config``: the dict of config.json. ``rnd`` is
applied to what a 16-bit implementation keeps in 16 bits (the default keeps float64).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np


# ---------------------------------------------------------------------------- small functions
def exact(a):
    return a


def bfloat16(a):
    """a rounded to the nearest bfloat16 (ties to even), as float64."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    """The plain weight."""
    return unit_rms(x, eps) * w


def layer_norm(x, w, eps):
    """The layers' and the model's norm: the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


# ---------------------------------------------------------------------------- positions
def rotate_pairs(x, positions, dims: int, base: float):
    """x [T, ..., n]: of the first ``dims`` values, 2i and 2i+1 turn by position * base^(-2i/dims)."""
    if not dims:
        return x
    out = np.array(x, dtype=np.float64, copy=True)
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------------------- masks
def visible(T: int, size: Optional[int], keep_first: int = 0):
    """[T, T] booleans: i sees j <= i within the last ``size`` positions (None: all) or among
    the first ``keep_first``."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    near = (i - j < size) if size else np.ones((T, T), dtype=bool)
    return (j <= i) & (near | (j < keep_first))


def softmax_rows(s, mask, extra_one: bool):
    """Softmax over the visible keys; ``extra_one``: the denominator has one more term exp(0)."""
    s = np.where(mask, s, -np.inf)
    m = np.max(s, axis=-1, keepdims=True)
    if extra_one:
        m = np.maximum(m, 0.0)
    e = np.exp(s - m)
    den = e.sum(-1, keepdims=True) + (np.exp(-m) if extra_one else 0.0)
    return e / den


def distance_slopes(H: int):
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])


# ---------------------------------------------------------------------------- attention branches
def attention_per_head_norm(h, w, p, m, eps, rnd=exact):
    """The left branch of ``parallel``. p: tensor prefix; m: its sizes."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rnd(h @ w[p + "q"].T).reshape(T, H, D)
    k = rnd(h @ w[p + "k"].T).reshape(T, G, D)
    v = rnd(h @ w[p + "v"].T).reshape(T, G, V)
    q = rnd(rms_norm(q, w[p + "q.norm"], eps))
    k = rnd(rms_norm(k, w[p + "k.norm"], eps))
    mask = visible(T, (m.get("mask") or {}).get("size"), 0)
    slopes = distance_slopes(H)
    dist = (np.arange(T)[:, None] - np.arange(T)[None, :]).astype(np.float64)
    out = np.zeros((T, H, V))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        if m.get("softcap"):
            s = float(m["softcap"]) * np.tanh(s / float(m["softcap"]))
        s = s - slopes[hd] * dist
        out[:, hd] = softmax_rows(s, mask, True) @ v[:, g]
    return rnd(out.reshape(T, H * V)) @ w[p + "o"].T


def attention_keys_as_values(h, w, p, m, eps, rnd=exact):
    """The left branch of ``parallel_2``."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = rnd(h @ w[p + "q"].T)
    kraw = rnd(h @ w[p + "k"].T)
    v = kraw.reshape(T, G, D)
    q = rnd(rms_norm(q, w[p + "q.norm"], eps)).reshape(T, H, D)
    k = rnd(rms_norm(kraw, w[p + "k.norm"], eps)).reshape(T, G, D)
    mk = m.get("mask") or {}
    mask = visible(T, mk.get("size"), int(mk.get("keep_first") or 0))
    out = np.zeros((T, H, D))
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        out[:, hd] = softmax_rows(s, mask, False) @ v[:, g]
    return rnd(out.reshape(T, H * D)) @ w[p + "o"].T


# ---------------------------------------------------------------------------- recurrent branches
def short_conv(x, taps_w):
    """x [T, C], taps_w [C, n]: y_t = sum_j w[:, j] x_(t - (n-1) + j), zeros before the start."""
    T, C = x.shape
    n = taps_w.shape[1]
    pad = np.concatenate([np.zeros((n - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(n):
        y += pad[j:j + T] * taps_w[:, j][None, :]
    return y


def gated_delta(h, w, p, m, eps, rnd=exact):
    """The right branch of ``parallel``."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_conv(rnd(h @ w[p + "q"].T), w[p + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(rnd(h @ w[p + "k"].T), w[p + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(rnd(h @ w[p + "v"].T), w[p + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)                                     # [T, H]
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None, :]))
    gate = silu(rnd(h @ w[p + "g"].T)).reshape(T, H, V)
    o = np.zeros((T, H, V))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((D, V))
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    y = rms_norm(o, w[p + "norm"], eps) * gate
    return rnd(y.reshape(T, H * V)) @ w[p + "o"].T


def gated_linear_attention(h, w, p, m, eps, rnd=exact):
    """The right branch of ``parallel_2``."""
    T = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, V)
    z = rnd(h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"][None, :]
    a = (sigmoid(z) ** (1.0 / float(m["tau"]))).reshape(T, H, D)
    gate = silu(rnd(h @ w[p + "g"].T))
    o = np.zeros((T, H, V))
    for hd in range(H):
        S = np.zeros((D, V))
        for t in range(T):
            S = a[t, hd][:, None] * S + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    y = rms_norm(o, w[p + "norm"], eps).reshape(T, H * V) * gate
    return rnd(y) @ w[p + "o"].T


# ---------------------------------------------------------------------------- the three mixers
def mixer_parallel(h, w, p, m, eps, rnd=exact):
    left = attention_per_head_norm(h, w, p + "left.", m["left"], eps, rnd)
    right = gated_delta(h, w, p + "right.", m["right"], eps, rnd)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


def mixer_parallel_2(h, w, p, m, eps, rnd=exact):
    left = attention_keys_as_values(h, w, p + "left.", m["left"], eps, rnd)
    right = gated_linear_attention(h, w, p + "right.", m["right"], eps, rnd)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def mixer_latent(h, w, p, m, eps, rnd=exact):
    T = h.shape[0]
    H, D, R, V, C = (int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]),
                     int(m["kv_rank"]))
    pos = np.arange(T)
    rot = m.get("rot") or {}
    dims, base = int(rot.get("dims") or 0), float(rot.get("base") or 1.0)
    cq = rnd(rms_norm(rnd(h @ w[p + "dq"].T), w[p + "dq.norm"], eps))
    q = rnd(cq @ w[p + "uq"].T).reshape(T, H, D + R)
    kv = rnd(h @ w[p + "dkv"].T)
    c = rnd(rms_norm(kv[:, :C], w[p + "dkv.norm"], eps))
    kr = rnd(rotate_pairs(kv[:, C:], pos, dims, base))                   # [T, R], all heads'
    qr = rotate_pairs(q[:, :, D:], pos, dims, base)
    ku = (c @ w[p + "uk"].T).reshape(T, H, D)
    v = (c @ w[p + "uv"].T).reshape(T, H, V)
    mask = visible(T, None)
    out = np.zeros((T, H, V))
    for hd in range(H):
        s = (q[:, hd, :D] @ ku[:, hd].T + qr[:, hd] @ kr.T) * float(m["scale"])
        out[:, hd] = softmax_rows(s, mask, False) @ v[:, hd]
    return rnd(out.reshape(T, H * V)) @ w[p + "o"].T


MIXERS = {"parallel": mixer_parallel, "parallel_2": mixer_parallel_2,
          "latent_attention": mixer_latent}


def feed_forward(h, w, p, rnd=exact):
    return rnd(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---------------------------------------------------------------------------- the model
def layer_runs(config) -> List[Tuple[int, int]]:
    """The order of layer runs as (layer, pass): ``pass`` >= 0 for the first layer of a pass
    through the looped run (what is added to x before it), else -1."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop or int(loop["times"]) < 1:
        return [(i, -1) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, -1) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else -1) for i in range(a, b)]
    return runs + [(i, -1) for i in range(b, n)]


def forward(config, w: Dict[str, np.ndarray], tokens, rnd=exact, states: Optional[list] = None):
    """The logits [T, vocab] of one sequence; ``states`` receives x after every layer run."""
    eps = float(config["norm"]["eps"])
    x0 = w["embed"][np.asarray(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    x = x0.copy()
    for i, t in layer_runs(config):
        if t >= 0:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t][None, :]
        layer, p = config["layers"][i], f"l{i}."
        h = rnd(layer_norm(x, w[p + "norm1"], eps))
        x = x + MIXERS[layer["type"]](h, w, p + "mix.", layer["mixer"], eps, rnd)
        if layer.get("mlp") is not None:
            h = rnd(layer_norm(x, w[p + "norm2"], eps))
            x = x + feed_forward(h, w, p + "mlp.", rnd)
        if states is not None:
            states.append(x.copy())
    h = rnd(layer_norm(x, w["final.norm"], eps))
    return (h @ w["head"].T) * float(config.get("logit_scale", 1.0))


def greedy(config, w, prompt, n: int) -> List[int]:
    toks = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(np.argmax(forward(config, w, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out
