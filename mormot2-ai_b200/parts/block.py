"""How a layer's parts are arranged around the residual stream.

``prenorm_residual``: x += mixer(norm_mixer(x)); x += feed_forward(norm_ff(x)), the residual
x in float32 throughout (``decoder.pas:2625-2702``, ``:2880-2899`` of the reference).

A mixer or feed-forward may hand its output back as ``Pending`` split sums instead of adding
it into x; the norm that reads x next adds them (one kernel does the sum, the residual add
and the norm). A block that takes part in this says ``accepts_pending = True``, takes the
sums that the block before left in ``pending`` and returns its own.

``hyper_connections``: the residual is ``streams`` copies x_1 .. x_S (all the embedding's output
at first). For each sublayer q with its vectors ``in``, ``out`` [S] and its matrix ``mix``
[S, S] (indexed from, to): u = Σ_s in[s] x_s; y = sublayer(norm(u));
x_t ← Σ_s mix[s, t] x_s + out[t] · y for all t at once. The write-back of one sublayer and the
read (with its layer norm) of the next are one kernel (``csrc/streams.cu``), so a block hands
its last write-back on as pending, as ``prenorm_residual`` hands on split sums.

``output_norm_residual``: the norm stands on what a sublayer gives back, not on what it reads:
x += norm_mixer(mixer(x)); x += norm_ff(feed_forward(x)). The sublayers read the residual
itself, rounded to the activation type; the kernel that norms a sublayer's output and adds it
into x also writes that rounding of the new x, which the next sublayer (or the next block, to
which it is handed on as pending) reads. With ``side`` the block then adds an input of its own
from the token: e = columns [col0, col0 + dim) of the row of a second embedding table,
t = P (act(G x) * e), x += norm_side(t).
"""
from __future__ import annotations

import torch

from ..errors import ConfigError
from .base import BLOCKS, Part, TensorNeed


class PreNormResidualBlock(Part):
    capturable = True

    def __init__(self, spec, prefix: str = "", mixer=None, feed_forward=None, norms=None):
        super().__init__(spec, prefix)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    accepts_pending = True

    def forward(self, x, step, line, state, writes_cache: bool, pending=None):
        h = self._norm("mixer", x, pending)
        pending = self.mixer.forward(h, x, step, line, state, writes_cache)
        if "feed_forward" not in self.norms:      # a layer without a feed-forward
            return pending
        # a feed-forward may name a bias that belongs into the residual before its last product
        # accumulates onto it (``residual_bias``); a norm that can adds it while it has the row
        bias = getattr(self.feed_forward, "residual_bias", None)
        norm = self.norms["feed_forward"]
        if bias is not None and getattr(norm, "accepts_residual_bias", False) \
                and bias.dtype == norm.weight.dtype:
            h = self._norm("feed_forward", x, pending, residual_bias=bias)
            return self.feed_forward.forward(h, x, step, bias_placed=True)
        h = self._norm("feed_forward", x, pending)
        return self.feed_forward.forward(h, x, step)

    def _norm(self, which, x, pending, **more):
        norm = self.norms[which]
        if pending is None:
            return norm.forward(x, **more)
        if getattr(norm, "accepts_pending", False):
            return norm.forward(x, pending=pending, **more)
        settle(x, pending)             # a norm that knows nothing of pending sums
        return norm.forward(x, **more)


def settle(x, pending) -> None:
    """Adds pending split sums into the residual x (or does what else is pending on it)."""
    from .. import kernels as K
    if hasattr(pending, "settle"):
        pending.settle(x)
        return
    K.add_partials(x, pending.partial)


class StreamUpdate:
    """A write-back into the residual streams that has not happened yet: x_t <- sum_s
    mix[s, t] x_s + out[t] * sum_b factor_b y_b."""

    def __init__(self, mix, out, terms):
        self.mix, self.out, self.terms = mix, out, terms

    def as_update(self):
        return (self.mix, self.out, self.terms)

    def settle(self, x) -> None:
        from .. import kernels as K
        K.stream_step(x, update=self.as_update())


class HyperConnectionsBlock(Part):
    capturable = True
    accepts_pending = True

    def __init__(self, spec, prefix: str = "", mixer=None, feed_forward=None, norms=None):
        super().__init__(spec, prefix)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        self.streams = int(spec.params["streams"])
        if not 1 <= self.streams <= 8:
            raise ConfigError(f"{self.streams} residual streams (1 to 8)")
        self.subs = ["mixer"] + (["feed_forward"] if "feed_forward" in norms else [])
        self.names = {q: {k: prefix + v for k, v in spec.params["names"][q].items()}
                      for q in self.subs}
        for q in self.subs:
            if not hasattr(norms[q], "eps") or not hasattr(norms[q], "weight"):
                raise ConfigError("hyper-connections read the streams through a norm with a "
                                  "weight and an eps (layernorm)")

    def libraries(self, rt):
        return ["streams"]

    def tensors(self):
        S = self.streams
        out = []
        for q in self.subs:
            n = self.names[q]
            out += [TensorNeed(n["in"], (S,), "vector"), TensorNeed(n["out"], (S,), "vector"),
                    TensorNeed(n["mix"], (S, S), "identity")]
        return out

    def bind(self, weights, rt) -> None:
        self.rt = rt
        self.w = {q: {k: weights[name].to(torch.float32).contiguous()
                      for k, name in self.names[q].items()} for q in self.subs}

    def _read(self, q, x, pending):
        from .. import kernels as K
        norm = self.norms[q]
        h = torch.empty((x.shape[1], x.shape[2]), dtype=self.rt.dtype, device=x.device)
        if pending is not None and not isinstance(pending, StreamUpdate):
            settle(x, pending)
            pending = None
        K.stream_step(x, update=pending.as_update() if pending is not None else None,
                      read=(self.w[q]["in"], norm.weight, norm.eps, h, None, x.shape[1]))
        return h

    def _sublayer(self, part, h, args, kwargs=None):
        """The sublayer's output as terms [(y, factor)]."""
        y = torch.empty((h.shape[0], h.shape[1]), dtype=torch.float32, device=h.device)
        if getattr(part, "can_store", False):
            pending = part.forward(h, y, *args, store=True)
            if pending is not None and len(pending.partial) <= 16:
                # the sublayer left its output as split sums: each is a term of the write-back
                return [(part_sum, 1.0) for part_sum in pending.partial]
            if pending is not None:      # more terms than the kernel takes: summed here
                y.zero_()
                settle(y, pending)
            return [(y, 1.0)]
        y.zero_()
        pending = part.forward(h, y, *args)
        if pending is not None:
            settle(y, pending)
        return [(y, 1.0)]

    def forward(self, x, step, line, state, writes_cache: bool, pending=None):
        if x.dim() != 3 or x.shape[0] != self.streams:
            raise ConfigError(f"a residual of shape {tuple(x.shape)} for {self.streams} streams")
        h = self._read("mixer", x, pending)
        if hasattr(self.mixer, "forward_branches"):
            terms = self.mixer.forward_branches(h, step, line, state, writes_cache)
        else:
            terms = self._sublayer(self.mixer, h, (step, line, state, writes_cache))
        pending = StreamUpdate(self.w["mixer"]["mix"], self.w["mixer"]["out"], terms)
        if "feed_forward" not in self.subs:
            return pending
        h = self._read("feed_forward", x, pending)
        terms = self._sublayer(self.feed_forward, h, (step,))
        return StreamUpdate(self.w["feed_forward"]["mix"], self.w["feed_forward"]["out"], terms)


class ReadyInput:
    """The residual rounded to the activation type, already made by the block before (nothing
    is owed to x)."""

    def __init__(self, h):
        self.h = h

    def settle(self, x) -> None:
        pass


class OutputNormResidualBlock(Part):
    capturable = True
    accepts_pending = True

    def __init__(self, spec, prefix: str = "", mixer=None, feed_forward=None, norms=None):
        super().__init__(spec, prefix)
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms
        for q, norm in norms.items():
            if not hasattr(norm, "add_normed"):
                raise ConfigError(f"the norm of \"{q}\" cannot norm a sublayer's output into the "
                                  "residual (rmsnorm can)")
        side = spec.params.get("side")
        self.side = None
        if side:
            from .linear import Linear  # noqa: F401  (bound below)
            from .. import kernels as K
            self.side = dict(side)
            if side["activation"] not in K.UNARY_ACTIVATIONS:
                raise ConfigError(f"activation \"{side['activation']}\" is not known")
            self.side_act = K.UNARY_ACTIVATIONS[side["activation"]]
            self.side_names = {k: (v if k == "table" else prefix + v)
                               for k, v in side["names"].items()}

    def tensors(self):
        if not self.side:
            return []
        sd, n = self.side, self.side_names
        hidden, dim = int(sd["hidden_size"]), int(sd["dim"])
        return [TensorNeed(n["table"], (int(sd["vocab_size"]), int(sd["table_width"])), "table"),
                TensorNeed(n["gate"], (dim, hidden)), TensorNeed(n["proj"], (hidden, dim)),
                TensorNeed(n["norm"], (hidden,), "vector")]

    def bind(self, weights, rt) -> None:
        self.rt = rt
        if self.side:
            from .linear import Linear
            n = self.side_names
            self.side_table = weights[n["table"]]
            self.side_gate = Linear(weights[n["gate"]], rt)
            self.side_proj = Linear(weights[n["proj"]], rt)
            self.side_norm = weights[n["norm"]]

    def _operand(self, x):
        """The residual as the sublayers read it (on the 32-bit path: itself)."""
        if self.rt.dtype == torch.float32:
            return x
        from .. import kernels as K
        h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        K.cast_rows(x, h)
        return h

    def _sublayer(self, part, h, args):
        """The sublayer's output: float32 [T, hidden], or its split sums [parts, T, hidden]."""
        y = torch.empty((h.shape[0], h.shape[1]), dtype=torch.float32, device=h.device)
        if getattr(part, "can_store", False):
            pending = part.forward(h, y, *args, store=True)
            return pending.partial if pending is not None else y
        y.zero_()
        pending = part.forward(h, y, *args)
        if pending is not None:
            settle(y, pending)
        return y

    def _next_operand(self, x):
        return None if self.rt.dtype == torch.float32 else \
            torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)

    def forward(self, x, step, line, state, writes_cache: bool, pending=None):
        from .. import kernels as K
        if isinstance(pending, ReadyInput):
            h = pending.h
        else:
            if pending is not None:
                settle(x, pending)
            h = self._operand(x)
        y = self._sublayer(self.mixer, h, (step, line, state, writes_cache))
        h_next = self._next_operand(x)
        self.norms["mixer"].add_normed(y, x, h_next)
        h = h_next if h_next is not None else x
        if "feed_forward" in self.norms:
            y = self._sublayer(self.feed_forward, h, (step,))
            h_next = self._next_operand(x)
            self.norms["feed_forward"].add_normed(y, x, h_next)
            h = h_next if h_next is not None else x
        if self.side:
            sd = self.side
            z = self.side_gate(h)
            g = torch.empty_like(z)
            K.unary_act(z, g, self.side_act, self.side_table, int(sd["col0"]), step.tok_ids)
            from .linear import Pending
            t = self.side_proj(g, out_dtype=torch.float32, defer="any")
            h_next = self._next_operand(x)
            K.norm_add(t.partial if isinstance(t, Pending) else t, self.side_norm,
                       float(sd["eps"]), x, h_next)
            h = h_next if h_next is not None else x
        return ReadyInput(h) if h is not x else None


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
BLOCKS.register("output_norm_residual", OutputNormResidualBlock)
BLOCKS.register("hyper_connections", HyperConnectionsBlock)
