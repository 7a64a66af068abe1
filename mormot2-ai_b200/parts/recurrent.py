"""Mixers that keep a state of fixed size per sequence instead of keys and values
(``csrc/recurrent.cu``). The state is float32, starts at zero, is read when a step begins and
written when it ends; everything that enters the recurrence is float32 on both paths (the
projections' operands are of the activation type, their sums float32).

``wkv`` — token-shifted time mixing with a decaying matrix state per head. With h' the row
before (zeros before a sequence's first), each of r, k, v, g, w reads h + (h' − h) · mu_s
(computed as ONE product [W_s | W_s diag(mu_s)] · [h ; h' − h] for all five);
r, k, v = W_r, W_k, W_v of their mixes (heads × dim), gate = silu(W_g ·), decay
w = exp(−exp(W_w2 tanh(W_w1 ·) + w0)) per head and key channel;
o_t = (S + diag(u) k vᵀ)ᵀ r, S ← diag(w) S + k vᵀ; each head's o over its root mean square,
times ``norm``, times the gate, then W_o. The state is the last h and S.

``mlstm`` — a matrix memory with an exponential input gate and a sigmoid forget gate, both as
logarithms behind a soft cap c: i = c tanh((W_i h + b_i)/c), f = logsigmoid(c tanh((W_f h + b_f)/c));
with a running maximum m (from 0): m' = max(f + m, i), S ← e^(f+m−m') S + e^(i−m') k vᵀ, n
likewise with k, o = Sᵀ q / (max(|n·q|, e^(−m')) + 1e-6) with q scaled by dim^(−1/2); each
head's o over its root mean square, times ``norm``, times sigmoid(W_g h), then W_o. q, k, v,
the output gate and both gates are one product.

``retention`` — linear attention with a constant decay d per head and no softmax or
denominator: q and k (heads × dim) turn by the token's position (``position``), k is then
multiplied by dim^(−1/2); S ← d S + k vᵀ (dim × vdim), o = Sᵀ q with the state that already
holds the token; each head's o over its root mean square (no weight), times silu(W_g h), then
W_o. q, k, v and the gate are one product.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError
from .base import MIXERS, Part, StateNeed, TensorNeed
from .linear import Linear, Pending


def _scan_parts(columns: int) -> int:
    """How many groups of threads share a state column's rows (csrc/recurrent.cu)."""
    return max(1, min(8, 512 // ((columns + 31) // 32 * 32)))


def _scan_smem(dim: int, vdim: int, staged_per_token: int) -> int:
    """Bytes of shared memory of a scan kernel's block: sixteen staged tokens, and the state
    unless a thread's share of a column (at most 32 rows) lies in registers."""
    columns = max(dim, vdim)
    if columns > 512:
        return 1 << 30
    rows = -(-dim // _scan_parts(columns))
    state = 0 if rows <= 32 else dim * vdim + 4
    return 4 * (state + 16 * staged_per_token + 256)


def _retention_fits(dim: int, vdim: int) -> bool:
    """Whether the walk token by token has a slice of a head's value columns (all of them, a
    half, a quarter, ... down to 32) whose block fits 200 KB of shared memory: what
    mb_retention_scan of csrc/recurrent.cu looks for."""
    if not (0 < dim <= 512 and 0 < vdim <= 512):
        return False
    ns = 1
    while True:
        cw = -(-vdim // ns)
        parts = _scan_parts(cw)
        rows = -(-dim // parts)
        state = 0 if rows <= 32 else (dim * cw + 3) // 4 * 4
        if 4 * (state + 16 * (2 * dim + (2 + parts) * cw) + 128) <= 200 * 1024:
            return True
        if cw <= 32:
            return False
        ns *= 2


def _project(linear: Linear, y, x, store: bool):
    """The output product: added into x, or (``store``) written into x, or, where the product
    of a step of few tokens splits its sums, left as ``Pending`` for whoever reads it next (x is
    then not touched)."""
    if store:
        out = linear(y, out=x, defer="any")
        return out if isinstance(out, Pending) else None
    linear(y, add_into=x)
    return None


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


class WkvMixer(Part):
    capturable = True
    can_store = True
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh, self.dim = int(p["hidden_size"]), int(p["heads"]), int(p["dim"])
        self.eps = float(p["eps"])
        # the decay's low rank is a size that only the tensors' shapes give (-1: any)
        self.rank = int(p.get("decay_rank") or -1)
        self.names = {k: prefix + v for k, v in p["names"].items()}
        self.width = self.nh * self.dim
        if _scan_smem(self.dim, self.dim, (6 + _scan_parts(self.dim)) * self.dim) > 200 * 1024:
            raise ConfigError(f"a decaying state of {self.dim} x {self.dim} values per head is "
                              "more than the kernel keeps on one multiprocessor")

    def libraries(self, rt) -> List[str]:
        return ["recurrent"]

    def tensors(self) -> List[TensorNeed]:
        n, W, HD = self.names, self.hidden, self.width
        out = [TensorNeed(n["mu_" + s], (W,), "fraction") for s in self.MIXES]
        out += [TensorNeed(n[s], (HD, W)) for s in ("r", "k", "v", "g")]
        out += [TensorNeed(n["w1"], (self.rank, W)), TensorNeed(n["w2"], (HD, self.rank)),
                TensorNeed(n["w0"], (HD,), "bias"), TensorNeed(n["u"], (self.nh, self.dim), "bias"),
                TensorNeed(n["norm"], (HD,), "vector"), TensorNeed(n["o"], (W, HD))]
        return out

    def state_need(self) -> StateNeed:
        return StateNeed((self.hidden + self.nh * self.dim * self.dim,), "float32", 0.0)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        # W_s (h + (h' - h) mu_s) = [W_s | W_s diag(mu_s)] [h ; h' - h]: the five projections
        # (r, k, v, g and the decay's first, low-rank one) are one product over rows of 2 W
        ws = [weights[n[s]] for s in ("r", "k", "v", "g", "w1")]
        kind = ws[0].dtype if len({w.dtype for w in ws}) == 1 else torch.float32
        rows = []
        for s, w in zip(self.MIXES, ws):
            mu = _f32(weights[n["mu_" + s]])
            rows.append(torch.cat([w.to(kind), (w.float() * mu[None, :]).to(kind)], dim=1))
        self.fused = Linear(torch.cat(rows, dim=0), rt)
        self.low_rank = ws[4].shape[0]
        self.w2 = Linear(weights[n["w2"]], rt)
        self.w0, self.u = _f32(weights[n["w0"]]), _f32(weights[n["u"]]).reshape(-1)
        self.norm = _f32(weights[n["norm"]])
        self.o = Linear(weights[n["o"]], rt)

    def forward(self, h, x, step, line, state, writes_cache: bool, store: bool = False):
        T, dev, dt = h.shape[0], h.device, self.rt.dtype
        HD, R = self.width, self.low_rank
        pair = torch.empty((T, 2 * self.hidden), dtype=dt, device=dev)
        K.token_shift(h, state, step, pair)
        # one row per token: r, k, v, g, the low-rank values, then the decay's logarithm
        z = torch.empty((T, 5 * HD + R), dtype=torch.float32, device=dev)
        self.fused(pair, out=z[:, :4 * HD + R])
        low = torch.empty((T, R), dtype=dt, device=dev)
        K.tanh_rows(z[:, 4 * HD:4 * HD + R], low)
        self.w2(low, out=z[:, 4 * HD + R:])
        y = torch.empty((T, HD), dtype=dt, device=dev)
        K.wkv_scan(z[:, :HD], z[:, HD:2 * HD], z[:, 2 * HD:3 * HD], z[:, 4 * HD + R:],
                   z[:, 3 * HD:4 * HD], self.w0, self.u, self.norm, self.eps, state, h, step, y,
                   self.nh, self.dim)
        return _project(self.o, y, x, store)


class MlstmMixer(Part):
    capturable = True
    can_store = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.cap, self.eps = float(p["gate_cap"]), float(p["eps"])
        if self.cap <= 0:
            raise ConfigError(f"a gate cap of {self.cap}")
        self.names = {k: prefix + v for k, v in p["names"].items()}
        staged = 3 * self.dim + (2 + _scan_parts(max(self.dim, self.vdim))) * self.vdim + 4
        if _scan_smem(self.dim, self.vdim, staged) > 200 * 1024:
            raise ConfigError(f"a matrix memory of {self.dim} x {self.vdim} values per head is "
                              "more than the kernel keeps on one multiprocessor")

    def libraries(self, rt) -> List[str]:
        return ["recurrent"]

    def tensors(self) -> List[TensorNeed]:
        n, W, H = self.names, self.hidden, self.nh
        return [TensorNeed(n["q"], (H * self.dim, W)), TensorNeed(n["k"], (H * self.dim, W)),
                TensorNeed(n["v"], (H * self.vdim, W)), TensorNeed(n["g"], (H * self.vdim, W)),
                TensorNeed(n["i"], (H, W)), TensorNeed(n["f"], (H, W)),
                TensorNeed(n["i_bias"], (H,), "bias"), TensorNeed(n["f_bias"], (H,), "bias"),
                TensorNeed(n["norm"], (H * self.vdim,), "vector"),
                TensorNeed(n["o"], (W, H * self.vdim))]

    def state_need(self) -> StateNeed:
        return StateNeed((self.nh * (self.dim * self.vdim + self.dim + 1),), "float32", 0.0)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        ws = [weights[n[s]] for s in ("q", "k", "v", "g", "i", "f")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.cols, at = [], 0
        for w in ws:
            self.cols.append(at)
            at += w.shape[0]
        self.fused = Linear(torch.cat(ws, dim=0), rt)
        self.bi, self.bf = _f32(weights[n["i_bias"]]), _f32(weights[n["f_bias"]])
        self.norm = _f32(weights[n["norm"]])
        self.o = Linear(weights[n["o"]], rt)

    def forward(self, h, x, step, line, state, writes_cache: bool, store: bool = False):
        T = h.shape[0]
        z = self.fused(h, out_dtype=torch.float32)
        y = torch.empty((T, self.nh * self.vdim), dtype=self.rt.dtype, device=h.device)
        K.mlstm_scan(z, self.cols, self.bi, self.bf, self.cap, self.dim ** -0.5, self.norm,
                     self.eps, state, step, y, self.nh, self.dim, self.vdim)
        return _project(self.o, y, x, store)


class RetentionMixer(Part):
    capturable = True
    can_store = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.eps = float(p["eps"])
        self.decay = [float(d) for d in p["decay"]]
        if len(self.decay) != self.nh:
            raise ConfigError(f"{len(self.decay)} decays for {self.nh} heads")
        self.position = (positions or {}).get(p.get("position", ""))
        if p.get("position") and self.position is None:
            raise ConfigError(f"the mixer names the position encoding \"{p['position']}\", "
                              "which the model does not define")
        self.names = {k: prefix + v for k, v in p["names"].items()}
        self.chunked = None     # True / False: one form of the walk whatever the step's shape
        if not _retention_fits(self.dim, self.vdim):
            raise ConfigError(f"a retention state of {self.dim} x {self.vdim} values per head is "
                              "more than the kernel keeps on one multiprocessor")

    def libraries(self, rt) -> List[str]:
        return ["recurrent"]

    def tensors(self) -> List[TensorNeed]:
        n, W, H = self.names, self.hidden, self.nh
        return [TensorNeed(n["q"], (H * self.dim, W)), TensorNeed(n["k"], (H * self.dim, W)),
                TensorNeed(n["v"], (H * self.vdim, W)), TensorNeed(n["g"], (H * self.vdim, W)),
                TensorNeed(n["o"], (W, H * self.vdim))]

    def state_need(self) -> StateNeed:
        return StateNeed((self.nh * self.dim * self.vdim,), "float32", 0.0)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        ws = [weights[n[s]] for s in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        self.cols, at = [], 0
        for w in ws:
            self.cols.append(at)
            at += w.shape[0]
        self.fused = Linear(torch.cat(ws, dim=0), rt)
        if getattr(rt, "consume_weights", False):
            del ws
            for s in ("q", "k", "v", "g"):
                weights.pop(n[s], None)
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=rt.device)
        self.o = Linear(weights[n["o"]], rt)

    def forward(self, h, x, step, line, state, writes_cache: bool, store: bool = False):
        T = h.shape[0]
        # what enters the recurrence leaves its product as float32 and is never rounded
        z = self.fused(h, out_dtype=torch.float32)
        inv_freq, rot_dim = (self.position.frequencies() if self.position is not None
                             else (None, 0))
        y = torch.empty((T, self.nh * self.vdim), dtype=self.rt.dtype, device=h.device)
        K.retention_scan(z, self.cols, self.decay_dev, self.dim ** -0.5, inv_freq, rot_dim,
                         self.eps, state, step, y, self.nh, self.dim, self.vdim,
                         chunked=self.chunked)
        return _project(self.o, y, x, store)


MIXERS.register("wkv", WkvMixer)
MIXERS.register("retention", RetentionMixer)
MIXERS.register("mlstm", MlstmMixer)
