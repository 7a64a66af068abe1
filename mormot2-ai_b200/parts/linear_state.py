"""Mixers with a matrix state per head that is decayed and written token by token
(``csrc/linear_state.cu``). The state is float32, starts at zero and is carried from step to
step in the engine's state arena; everything that enters the recurrence is float32 on both
paths (the projections' operands are of the activation type, their sums float32).

``gated_linear_attention`` — q = W_q h · dim^(−1/2), k = W_k h (heads × dim), v = W_v h
(heads × vdim) and a decay per key channel a = sigmoid(W_a2 (W_a1 h) + b)^(1/tau):
S ← diag(a) S + k vᵀ, o = Sᵀ q with the state that already holds the token; each head's o
over its root mean square, times ``norm`` [vdim] (one weight for all heads), the heads side
by side times silu(W_g h), then W_o. The low rank of W_a1 is a size that only the stored
tensors give.

``gated_delta`` — the gated delta rule. q and k (kv_heads × dim; head h reads group
h div (heads div kv_heads)) and v (heads × vdim) each pass a causal convolution over time per
channel (``taps`` taps, no bias, zeros before a sequence's start) and SiLU; q and k are then
brought to unit length per head (``unit_eps`` under the root), q also times dim^(−1/2);
beta = sigmoid(W_b h) and g = exp(−exp(A_log) · softplus(W_a h + dt_bias)) per head;
S ← g S; u = beta (v − Sᵀ k); S ← S + k uᵀ; o = Sᵀ q; then the head's norm, the SiLU gate and
W_o as above. The convolutions' last ``taps`` − 1 inputs are part of the state.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError
from .base import MIXERS, Part, StateNeed, TensorNeed
from .linear import Linear
from .recurrent import _f32, _project

MAX_DIM, MAX_VDIM, MAX_TAPS = 256, 1024, 9


def _check_sizes(kind: str, dim: int, vdim: int) -> None:
    if not (0 < dim <= MAX_DIM and 0 < vdim <= MAX_VDIM):
        raise ConfigError(f"{kind}: a state of {dim} x {vdim} values per head (at most "
                          f"{MAX_DIM} x {MAX_VDIM})")


def _fuse(weights: List[torch.Tensor]):
    """The rows of several projections of the same input one after another, and where each
    begins."""
    if len({w.dtype for w in weights}) > 1:
        weights = [w.float() for w in weights]
    cols, at = [], 0
    for w in weights:
        cols.append(at)
        at += w.shape[0]
    return torch.cat(weights, dim=0), cols


class GatedLinearAttention(Part):
    capturable = True
    can_store = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.tau, self.eps = float(p["tau"]), float(p["eps"])
        self.rank = int(p.get("decay_rank") or -1)      # -1: what the stored tensors have
        if self.tau <= 0:
            raise ConfigError(f"tau = {self.tau}")
        _check_sizes("gated linear attention", self.dim, self.vdim)
        self.names = {k: prefix + v for k, v in p["names"].items()}

    def libraries(self, rt) -> List[str]:
        return ["linear_state"]

    def tensors(self) -> List[TensorNeed]:
        n, W, H = self.names, self.hidden, self.nh
        return [TensorNeed(n["q"], (H * self.dim, W)), TensorNeed(n["k"], (H * self.dim, W)),
                TensorNeed(n["v"], (H * self.vdim, W)), TensorNeed(n["g"], (H * self.vdim, W)),
                TensorNeed(n["a1"], (self.rank, W)), TensorNeed(n["a2"], (H * self.dim, self.rank)),
                TensorNeed(n["a2_bias"], (H * self.dim,), "bias"),
                TensorNeed(n["norm"], (self.vdim,), "vector"),
                TensorNeed(n["o"], (W, H * self.vdim))]

    def state_need(self) -> StateNeed:
        return StateNeed((self.nh * self.dim * self.vdim,), "float32", 0.0)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        fused, self.cols = _fuse([weights[n[s]] for s in ("q", "k", "v", "g")])
        self.fused = Linear(fused, rt)
        self.a1, self.a2 = Linear(weights[n["a1"]], rt), Linear(weights[n["a2"]], rt)
        self.a2_bias, self.norm = _f32(weights[n["a2_bias"]]), _f32(weights[n["norm"]])
        self.o = Linear(weights[n["o"]], rt)
        if getattr(rt, "consume_weights", False):
            for s in ("q", "k", "v", "g"):
                weights.pop(n[s], None)

    def forward(self, h, x, step, line, state, writes_cache: bool, store: bool = False):
        T = h.shape[0]
        # what enters the recurrence leaves its product as float32 and is never rounded
        z = self.fused(h, out_dtype=torch.float32)
        za = self.a2(self.a1(h), out_dtype=torch.float32)
        y = torch.empty((T, self.nh * self.vdim), dtype=self.rt.dtype, device=h.device)
        K.linear_state_scan("gla", z, self.cols[:3], 1, z, self.cols[3], self.norm, self.eps,
                            state, step, y, self.nh, self.dim, self.vdim, decay_logits=za,
                            decay_bias=self.a2_bias, inv_tau=1.0 / self.tau)
        return _project(self.o, y, x, store)


class GatedDelta(Part):
    capturable = True
    can_store = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["heads"])
        self.nkv = int(p.get("kv_heads") or self.nh)
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.taps = int(p["taps"])
        self.eps, self.unit_eps = float(p["eps"]), float(p["unit_eps"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"{self.nh} heads on {self.nkv} q/k heads")
        if not 1 <= self.taps <= MAX_TAPS:
            raise ConfigError(f"a convolution of {self.taps} taps (1 to {MAX_TAPS})")
        _check_sizes("gated delta rule", self.dim, self.vdim)
        self.names = {k: prefix + v for k, v in p["names"].items()}
        self.qkw, self.vw = self.nkv * self.dim, self.nh * self.vdim
        self.channels = 2 * self.qkw + self.vw

    def libraries(self, rt) -> List[str]:
        return ["linear_state"]

    def tensors(self) -> List[TensorNeed]:
        n, W, H = self.names, self.hidden, self.nh
        return [TensorNeed(n["q"], (self.qkw, W)), TensorNeed(n["k"], (self.qkw, W)),
                TensorNeed(n["v"], (self.vw, W)), TensorNeed(n["g"], (self.vw, W)),
                TensorNeed(n["q_conv"], (self.qkw, self.taps), "taps"),
                TensorNeed(n["k_conv"], (self.qkw, self.taps), "taps"),
                TensorNeed(n["v_conv"], (self.vw, self.taps), "taps"),
                TensorNeed(n["b"], (H, W)), TensorNeed(n["a"], (H, W)),
                TensorNeed(n["A_log"], (H,), "bias"), TensorNeed(n["dt_bias"], (H,), "bias"),
                TensorNeed(n["norm"], (self.vdim,), "vector"), TensorNeed(n["o"], (W, self.vw))]

    def state_need(self) -> StateNeed:
        return StateNeed((self.nh * self.dim * self.vdim + (self.taps - 1) * self.channels,),
                         "float32", 0.0)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        # q, k, v first (the convolution walks these columns), then the gate and the two
        # scalars per head
        fused, self.cols = _fuse([weights[n[s]] for s in ("q", "k", "v", "g", "b", "a")])
        self.fused = Linear(fused, rt)
        self.conv = torch.cat([_f32(weights[n[s]]) for s in ("q_conv", "k_conv", "v_conv")],
                              dim=0).contiguous()
        self.a_log, self.dt_bias = _f32(weights[n["A_log"]]), _f32(weights[n["dt_bias"]])
        self.norm = _f32(weights[n["norm"]])
        self.o = Linear(weights[n["o"]], rt)
        if getattr(rt, "consume_weights", False):
            for s in ("q", "k", "v", "g", "b", "a"):
                weights.pop(n[s], None)

    def forward(self, h, x, step, line, state, writes_cache: bool, store: bool = False):
        T = h.shape[0]
        z = self.fused(h, out_dtype=torch.float32)
        matrix = self.nh * self.dim * self.vdim
        qkv = torch.empty((T, self.channels), dtype=torch.float32, device=h.device)
        K.short_conv(z, 0, self.conv, state[:, matrix:], step, qkv)
        y = torch.empty((T, self.vw), dtype=self.rt.dtype, device=h.device)
        K.linear_state_scan("delta", qkv, (0, self.qkw, 2 * self.qkw), self.nh // self.nkv, z,
                            self.cols[3], self.norm, self.eps, state, step, y, self.nh, self.dim,
                            self.vdim, scalars=z, beta_col=self.cols[4], rate_col=self.cols[5],
                            a_log=self.a_log, dt_bias=self.dt_bias, unit_eps=self.unit_eps)
        return _project(self.o, y, x, store)


MIXERS.register("gated_linear_attention", GatedLinearAttention)
MIXERS.register("gated_delta", GatedDelta)
