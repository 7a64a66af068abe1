"""A plain, slow implementation of the Sezopel decoder in NumPy float64: one function per
mechanism, whole sequences at once, no cache, a token-by-token recurrence. It shares no code
with the library and is the oracle of the library's tests.

The design: the residual x starts as the embedding row times a constant. A layer norms what a
sublayer gives back, not what it reads: x += N1(mixer(x)), x += N2(ff(x)) with
N(y) = y / sqrt(mean(y^2) + eps) * w. After the feed-forward every layer adds an input of its
own from the token: with e the layer's slice of a second embedding table,
t = P (gelu(G x) * e) and x += t / sqrt(mean(t^2) + eps) * n. Mixers: grouped-query softmax
attention (partly rotated heads, q and k brought to unit root mean square after the rotation,
scores capped by c tanh(s / c), a sigmoid gate per head on the heads' outputs; a layer may read
the keys and values that another layer keeps) and retention (rotated q and k, a constant decay
per head, S_t = d S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, each head's o brought to unit root mean
square, a SiLU gate). Feed-forward: W_down relu(W_up x)^2. Output: the norm, the head, and a
cap c tanh(z / c) on the logits.

``weights``: a dict name -> float64 array. ``config``: the dict of config.json.

Every function takes ``rnd``, applied to what a 16-bit implementation would keep in 16 bits (the
results of matrix products, activations, gates, what a sublayer reads, kept keys and values);
the default keeps everything in float64. ``forward(..., rnd=bfloat16)`` therefore shows how far
rounding alone moves the logits of a model, which is what a 16-bit run is measured against.
"""
from __future__ import annotations

import math
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


def soft_cap(z, cap):
    """cap * tanh(z / cap); no cap when ``cap`` is None or 0."""
    return cap * np.tanh(z / cap) if cap else z


# ---------------------------------------------------------------------------- positions
def rotate(x, positions, rot: Optional[Dict]):
    """x [T, heads, dim]: value i of the first ``dims`` turns with value i + dims/2 by the
    angle position * base^(-2i/dims)."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---------------------------------------------------------------------------- mixers
def attention_keys_values(h, weights, prefix, m, eps, positions, rnd=exact):
    """What a layer keeps of its tokens: keys (rotated, then unit root mean square) and values."""
    T = h.shape[0]
    G, D, DV = int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m.get("vdim", m["dim"]))
    k = rnd(h @ weights[prefix + "mix.k"].T).reshape(T, G, D)
    v = rnd(h @ weights[prefix + "mix.v"].T).reshape(T, G, DV)
    k = unit_rms(rotate(k, positions, m.get("rot")), eps)
    return rnd(k), v


def attention_mixer(h, weights, prefix, m, eps, positions, kv, rnd=exact):
    """h [T, width] -> [T, width]; ``kv`` = (keys [T, G, D], values [T, G, DV]) of the same
    tokens (this layer's or another's)."""
    T = h.shape[0]
    H, D = int(m["heads"]), int(m["dim"])
    k, v = kv
    G, DV = k.shape[1], v.shape[2]
    q = rnd(h @ weights[prefix + "mix.q"].T).reshape(T, H, D)
    q = rnd(unit_rms(rotate(q, positions, m.get("rot")), eps))
    gate = sigmoid(rnd(h @ weights[prefix + "mix.g"].T))                # [T, H]
    out = np.zeros((T, H, DV))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].T) * float(m["scale"])
        s = soft_cap(s, m.get("softcap"))
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, head, :] = (p @ v[:, g, :]) * gate[:, head:head + 1]
    return rnd(out).reshape(T, H * DV) @ weights[prefix + "mix.o"].T


def retention_mixer(h, weights, prefix, m, eps, positions, state=None, rnd=exact):
    """Token by token. ``state`` [H, D, DV] or None (zeros); returns (out, state after)."""
    T = h.shape[0]
    H, D, DV = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
    q = rotate(rnd(h @ weights[prefix + "mix.q"].T).reshape(T, H, D), positions, m.get("rot"))
    k = rotate(rnd(h @ weights[prefix + "mix.k"].T).reshape(T, H, D), positions, m.get("rot"))
    k = k * D ** -0.5
    v = rnd(h @ weights[prefix + "mix.v"].T).reshape(T, H, DV)
    gate = silu(rnd(h @ weights[prefix + "mix.g"].T))                   # [T, H * DV]
    decay = np.asarray(m["decay"], dtype=np.float64)
    S = np.zeros((H, D, DV)) if state is None else state.copy()
    o = np.zeros((T, H, DV))
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rnd(unit_rms(o, eps).reshape(T, H * DV) * gate)
    return o @ weights[prefix + "mix.o"].T, S


# ---------------------------------------------------------------------------- feed-forward, side
def dense_ff(h, weights, prefix, rnd=exact):
    a = rnd(np.maximum(rnd(h @ weights[prefix + "mlp.up"].T), 0.0) ** 2)
    return a @ weights[prefix + "mlp.down"].T


def token_side(x, tokens, weights, prefix, layer, dim, eps, rnd=exact):
    """What the layer adds from the token itself: [T, width]."""
    e = weights["side.embed"][np.asarray(tokens)][:, layer * dim:(layer + 1) * dim]
    g = rnd(gelu_tanh(rnd(x @ weights[prefix + "side.gate"].T)) * e)
    y = g @ weights[prefix + "side.proj"].T
    return unit_rms(y, eps) * weights[prefix + "side.norm"]


# ---------------------------------------------------------------------------- the model
def forward(config: Dict, weights: Dict[str, np.ndarray], tokens: List[int],
            states: Optional[List[np.ndarray]] = None, rnd=exact) -> np.ndarray:
    """The logits [T, vocab] of a whole sequence; ``states`` (a list) receives the residual
    after every layer."""
    T = len(tokens)
    eps = float(config["norm"]["eps"])
    positions = np.arange(T)
    x = weights["embed"][np.asarray(tokens)] * float((config.get("embedding") or {}).get("scale", 1.0))
    side = config.get("token_side")
    kept: Dict[int, Tuple[np.ndarray, np.ndarray]] = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "attention":
            if m.get("kv_from") is not None:
                kv = kept[int(m["kv_from"])]
            else:
                kv = kept[i] = attention_keys_values(rnd(x), weights, p, m, eps, positions, rnd)
            y = attention_mixer(rnd(x), weights, p, m, eps, positions, kv, rnd)
        elif layer["type"] == "retention":
            y, _ = retention_mixer(rnd(x), weights, p, m, eps, positions, rnd=rnd)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, weights[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + rms_norm(dense_ff(rnd(x), weights, p, rnd), weights[p + "norm2"], eps)
        if side:
            x = x + token_side(rnd(x), tokens, weights, p, i, int(side["dim"]), eps, rnd)
        if states is not None:
            states.append(x.copy())
    h = rnd(rms_norm(x, weights["final.norm"], eps))
    return soft_cap(h @ weights["head"].T, config.get("logit_softcap"))
