"""Feed-forwards without routing.

``gated_mlp``: x += W_d (act(W_g h + b_g) * (W_u h + b_u)) + b_d with ``activation`` "silu" or
"gelu_tanh" and optional biases. Gate and up are one product. In bfloat16 their rows
alternate and the product's epilogue adds the biases and applies the activation (as the
SwiGLU feed-forward does for SiLU without biases); b_d is placed in the residual rows, which
the last product then accumulates onto, by the norm before the feed-forward where that norm
can (``residual_bias``), else by a kernel of its own. On the 32-bit path the product stores
gate and up and one kernel adds the biases, applies the activation and places b_d.
``none``: a layer without a feed-forward.
``mlp``: W_d act(W_u h) without a gate and without biases, ``activation`` "relu_squared"
(max(z, 0)²), "silu" or "gelu_tanh".

SwiGLU feed-forward: x += (silu(h·Wgᵀ) · (h·Wuᵀ)) · Wdᵀ, no bias
(``decoder.pas:2865-2899``, ``backend.cpu.pas:1827-1833`` of the reference). Gate and up are
one product whose epilogue applies the activation: their rows are laid out alternately (gate
of output 0, up of output 0, gate of output 1, ...), a pure re-layout done once at load."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError
from .base import FEED_FORWARDS, Part, TensorNeed
from .linear import Linear


class SwiGluFfn(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.names = {k: prefix + v for k, v in p["names"].items()}

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        return [TensorNeed(n["gate"], (self.inter, self.hidden)),
                TensorNeed(n["up"], (self.inter, self.hidden)),
                TensorNeed(n["down"], (self.hidden, self.inter))]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        n = self.names
        g, u = weights[n["gate"]], weights[n["up"]]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        pairs = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden)
        self.gate_up = Linear(pairs, rt, swiglu=True)
        if getattr(rt, "consume_weights", False):   # the originals go once they are interleaved
            del g, u
            weights.pop(n["gate"], None)
            weights.pop(n["up"], None)
        self.down = Linear(weights[n["down"]], rt)

    def forward(self, h, x, step):
        """Adds the feed-forward's output into x, or returns it as ``Pending`` split sums for
        the next norm to add."""
        from .linear import Pending
        act = self.gate_up(h)
        out = self.down(act, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


class GatedMlp(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        if p["activation"] not in K.ACTIVATIONS:
            raise ConfigError(f"activation \"{p['activation']}\" is not known "
                              f"(known: {', '.join(sorted(K.ACTIVATIONS))})")
        self.act = K.ACTIVATIONS[p["activation"]]
        self.bias = bool(p.get("bias", False))
        self.names = {k: prefix + v for k, v in p["names"].items()}

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        out = [TensorNeed(n["gate"], (self.inter, self.hidden)),
               TensorNeed(n["up"], (self.inter, self.hidden)),
               TensorNeed(n["down"], (self.hidden, self.inter))]
        if self.bias:
            out += [TensorNeed(n["gate_bias"], (self.inter,), "bias"),
                    TensorNeed(n["up_bias"], (self.inter,), "bias"),
                    TensorNeed(n["down_bias"], (self.hidden,), "bias")]
        return out

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        g, u = weights[n["gate"]], weights[n["up"]]
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.biases = None
        if self.bias:
            b = [weights[n["gate_bias"]], weights[n["up_bias"]], weights[n["down_bias"]]]
            if len({t.dtype for t in b}) > 1:
                b = [t.float() for t in b]
            self.biases = b
        # the fused form: bfloat16 weights (and biases) on the tensor-core kernel
        self.fused = (rt.fast_kernels and g.dtype == torch.bfloat16 and self.hidden % 8 == 0
                      and (self.biases is None or self.biases[0].dtype == torch.bfloat16))
        if self.fused:
            pairs = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden)
            pair_bias = (torch.stack(self.biases[:2], dim=1).reshape(-1).contiguous()
                         if self.biases is not None else None)
            self.gate_up = Linear(pairs, rt, swiglu=True, activation=self.act, pair_bias=pair_bias)
            self.fused = self.gate_up.fast is not None
        if not self.fused:
            self.gate_up = Linear(torch.cat([g, u], dim=0), rt)  # gate rows, then up rows
        if getattr(rt, "consume_weights", False):
            del g, u
            weights.pop(n["gate"], None)
            weights.pop(n["up"], None)
        self.down = Linear(weights[n["down"]], rt)
        # what the norm before this feed-forward may add into the residual for it
        self.residual_bias = self.biases[2] if (self.fused and self.biases is not None) else None

    def forward(self, h, x, step, bias_placed: bool = False):
        """``bias_placed``: the norm before already added ``residual_bias`` into x."""
        from .linear import Pending
        if self.fused:
            act = self.gate_up(h)
            if self.residual_bias is not None and not bias_placed:
                K.add_bias(x, self.residual_bias)
        else:
            gu = self.gate_up(h)
            act = torch.empty((h.shape[0], self.inter), dtype=self.rt.dtype, device=h.device)
            if self.biases is not None:
                K.gated_act(gu, act, self.act, self.biases[0], self.biases[1], x, self.biases[2])
            else:
                K.gated_act(gu, act, self.act)
        out = self.down(act, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


class PlainMlp(Part):
    capturable = True
    can_store = True      # forward(..., store=True) writes its output into x instead of adding

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        if p["activation"] not in K.UNARY_ACTIVATIONS:
            raise ConfigError(f"activation \"{p['activation']}\" is not known "
                              f"(known: {', '.join(sorted(K.UNARY_ACTIVATIONS))})")
        self.act = K.UNARY_ACTIVATIONS[p["activation"]]
        self.names = {k: prefix + v for k, v in p["names"].items()}

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        return [TensorNeed(n["up"], (self.inter, self.hidden)),
                TensorNeed(n["down"], (self.hidden, self.inter))]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        self.up = Linear(weights[self.names["up"]], rt, unary=self.act)
        self.down = Linear(weights[self.names["down"]], rt)

    def forward(self, h, x, step, store: bool = False):
        """Adds the feed-forward's output into x (``store``: writes it there), or returns it as
        ``Pending`` split sums for whoever reads it next (x is then not touched)."""
        from .linear import Pending
        act = self.up(h)          # the activation in the product's epilogue
        if store:
            out = self.down(act, out=x, defer="any")
        else:
            out = self.down(act, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


class NoFeedForward(Part):
    capturable = True

    def forward(self, h, x, step):
        return None


FEED_FORWARDS.register("swiglu", SwiGluFfn)
FEED_FORWARDS.register("gated_mlp", GatedMlp)
FEED_FORWARDS.register("none", NoFeedForward)
FEED_FORWARDS.register("mlp", PlainMlp)
