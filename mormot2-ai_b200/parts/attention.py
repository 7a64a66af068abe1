"""Grouped-query attention over the cache, as a mixer: fused q/k/v projection, per-head
RMSNorm of q and k (when the spec names their weights), position encoding, keys and values
into the cache line, causal attention with an optional window, output projection added into
the residual. The steps are the reference's ``AttentionBlock`` (``decoder.pas:2625-2702``);
head h reads KV head h div (heads div kv_heads) (``backend.cpu.pas:1253``).

Options that a design may name: ``v_dim``, a value size that differs from the key size (the
cache then keeps keys and values in pools of their own); ``names["sink"]``, a learned number
per head whose exponential is one more term of the softmax denominator (a key with that
score, not scaled, and a value of zero); ``softcap`` c > 0, which turns every scaled score s into
c tanh(s / c) before the softmax; ``head_norm`` = "unit_after_rotation", which divides q and k
by their root mean square (``head_norm_eps``) after the rotation, without a weight;
``names["g"]``, a projection to one logit per head whose sigmoid multiplies the head's output
before the output projection (its rows ride along in the q/k/v product); ``shared_kv``: the
mixer has no key and value projections and only ever reads the cache line of another layer;
``sink_value``: the sink as a constant, the same for every head (0: one more term exp(0) in
the denominator); ``distance_exponent`` e: head h's scores lose 2^(e (h + 1) / heads) times the
distance between query and key, after the cap; ``keep_first`` n with a ``window``: the first
n positions of a sequence stay visible to all later ones (the cache line then keeps every
page instead of a ring); ``head_norm`` = "whole_rows": q and k are each normed over their
whole projection at once, with weights of that width; ``values`` = "keys_as_projected": there
is no value projection, a token's values are its keys as they leave the projection (before any
norm or rotation).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError, KernelError
from .base import MIXERS, CacheNeed, Part, TensorNeed
from .linear import Linear


class GqaAttention(Part):
    capturable = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["heads"]), int(p["kv_heads"]), int(p["head_dim"])
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"{self.nh} heads on {self.nkv} KV heads")
        self.window = int(p.get("window", 0))
        self.scale = float(p["scale"])
        self.head_norm_eps = p.get("head_norm_eps")
        self.names = {k: prefix + v for k, v in p["names"].items()}
        self.position = (positions or {}).get(p.get("position", ""))
        if p.get("position") and self.position is None:
            raise ConfigError(f"the mixer names the position encoding \"{p['position']}\", "
                              "which the model does not define")
        self.vd = int(p.get("v_dim") or self.hd)
        self.qw, self.kvw, self.vw = self.nh * self.hd, self.nkv * self.hd, self.nkv * self.vd
        self.ow = self.nh * self.vd
        self.sink = None
        self.softcap = float(p.get("softcap") or 0.0)
        if self.softcap < 0:
            raise ConfigError(f"a score cap of {self.softcap}")
        self.head_norm = p.get("head_norm", "weighted_before_rotation")
        if self.head_norm not in ("weighted_before_rotation", "unit_after_rotation",
                                  "whole_rows"):
            raise ConfigError(f"head norm \"{self.head_norm}\" is not known (known: "
                              "unit_after_rotation, weighted_before_rotation, whole_rows)")
        self.whole_rows = self.head_norm == "whole_rows"
        if self.whole_rows and ("q_norm" not in self.names or self.head_norm_eps is None):
            raise ConfigError("a norm over the whole rows of q and k has weights and an eps")
        self.values = p.get("values", "projected")
        if self.values not in ("projected", "keys_as_projected"):
            raise ConfigError(f"values \"{self.values}\" (projected, keys_as_projected)")
        self.v_from_k = self.values == "keys_as_projected"
        if self.v_from_k and (self.vd != self.hd or "v" in self.names):
            raise ConfigError("values that are the keys have the keys' size and no projection")
        self.keep_first = int(p.get("keep_first") or 0)
        if self.keep_first < 0 or (self.keep_first and not self.window):
            raise ConfigError(f"keep_first = {self.keep_first} with a window of {self.window}")
        self.sink_value = p.get("sink_value")
        if self.sink_value is not None and "sink" in self.names:
            raise ConfigError("a sink is either a constant or a tensor")
        self.distance_exponent = p.get("distance_exponent")
        self.slopes = None
        self.unit_after = self.head_norm == "unit_after_rotation"
        if self.unit_after and ("q_norm" in self.names or self.head_norm_eps is None):
            raise ConfigError("a unit norm after the rotation has an eps and no weights")
        self.gate_n = self.nh if "g" in self.names else 0
        # the gates' columns stand behind q (k, v) in the projection's rows: rows of zeros after
        # them keep those rows a multiple of 16 bytes wide, which the tensor-core kernels ask for
        self.gate_w = self.gate_n
        if self.gate_n and self.qw % 8 == 0 and (self.kvw + self.vw) % 8 == 0:
            self.gate_w = (self.gate_n + 7) // 8 * 8
        self.shared_kv = bool(p.get("shared_kv", False))

    can_store = True      # forward(..., store=True) writes its output into x instead of adding

    def libraries(self, rt) -> List[str]:
        return rt.attention_libraries()

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        out = [TensorNeed(n["q"], (self.qw, self.hidden))]
        if not self.shared_kv:
            out.append(TensorNeed(n["k"], (self.kvw, self.hidden)))
            if not self.v_from_k:
                out.append(TensorNeed(n["v"], (self.vw, self.hidden)))
        out.append(TensorNeed(n["o"], (self.hidden, self.ow)))
        if self.gate_n:
            out.append(TensorNeed(n["g"], (self.nh, self.hidden)))
        if "sink" in n:
            out.append(TensorNeed(n["sink"], (self.nh,), "bias"))
        if "q_norm" in n:
            out += [TensorNeed(n["q_norm"], (self.qw if self.whole_rows else self.hd,), "vector"),
                    TensorNeed(n["k_norm"], (self.kvw if self.whole_rows else self.hd,), "vector")]
        return out

    def cache_need(self) -> CacheNeed:
        # kept first positions lie outside a ring of the window's pages: such a line keeps all
        return CacheNeed(self.nkv, self.hd, 0 if self.keep_first else self.window, 2,
                         0 if self.vd == self.hd else self.vd)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        plain = (self.vd == self.hd and "sink" not in self.names and not self.softcap
                 and not self.gate_n and not self.unit_after and self.sink_value is None
                 and self.distance_exponent is None and not self.whole_rows
                 and not self.v_from_k and not self.keep_first)
        if self.sink_value is not None:
            self.sink = torch.full((self.nh,), float(self.sink_value), dtype=torch.float32,
                                   device=rt.device)
        if self.distance_exponent is not None:
            e = float(self.distance_exponent)
            self.slopes = torch.tensor([2.0 ** (e * (h + 1) / self.nh) for h in range(self.nh)],
                                       dtype=torch.float32, device=rt.device)
        if (plain and (self.hd % 16 or self.hd > 256)) or self.hd > 1024 or self.vd > 256:
            raise KernelError(
                f"heads of {self.hd} values (value rows of {self.vd}) are not supported by the "
                "attention kernels (a multiple of 16, at most 256; with a sink, a score cap, a "
                "gate per head or value rows of their own size any size up to 1024 and 256)")
        n = self.names
        wg = weights[n["g"]] if self.gate_n else None
        if wg is not None and self.gate_w > self.gate_n:
            wg = torch.cat([wg, wg.new_zeros((self.gate_w - self.gate_n, wg.shape[1]))], dim=0)
        if self.shared_kv:
            # queries (and the heads' gates) only: keys and values are another layer's
            wq = weights[n["q"]]
            if wg is not None and wg.dtype != wq.dtype:
                wq, wg = wq.float(), wg.float()
            self.qkv, self.split = None, None
            self._q_only = Linear(torch.cat([wq, wg], dim=0) if wg is not None else wq, rt)
            self.o = Linear(weights[n["o"]], rt)
            self.q_norm = self.k_norm = None
            return
        wq, wk = weights[n["q"]], weights[n["k"]]
        # values that are the keys: the product has no rows for them; the kernel that norms q
        # and k copies the keys as they came into the value columns of the row
        wv = wk[:0] if self.v_from_k else weights[n["v"]]
        if wg is not None and not (wq.dtype == wk.dtype == wv.dtype == wg.dtype):
            wq, wk, wv, wg = wq.float(), wk.float(), wv.float(), wg.float()
        if wq.dtype == wk.dtype == wv.dtype:
            # one product for q, k and v: the rows of the three weights one after another (and
            # behind them the rows of the heads' gates, where the design has them)
            self.qkv = Linear(torch.cat([wq, wk, wv] + ([wg] if wg is not None else []), dim=0),
                              rt)
            self._q_only = None      # made when a run first reads another run's cache line
            self.split = None
            if getattr(rt, "consume_weights", False):
                # the engine owns the tensors: the three originals go as soon as they are fused,
                # so that loading never holds much more than the model
                del wq, wk, wv
                for key in ("q", "k", "v"):
                    weights.pop(n.get(key, ""), None)
        else:
            self.qkv = None
            self.split = [Linear(wq, rt), Linear(wk, rt), Linear(wv, rt)]
            self._q_only = self.split[0]
        self.o = Linear(weights[n["o"]], rt)
        self.q_norm = weights.get(n.get("q_norm", ""))
        self.k_norm = weights.get(n.get("k_norm", ""))
        if "sink" in n:
            self.sink = weights[n["sink"]].to(torch.float32).contiguous()

    @property
    def q_only(self) -> Linear:
        """The product for a run that reads keys and values another run wrote: q's rows (and
        the gates') of the fused weight."""
        if self._q_only is None:
            w = self.qkv.weight
            self._q_only = Linear(torch.cat([w[:self.qw], w[w.shape[0] - self.gate_w:]], dim=0)
                                  if self.gate_n else w[:self.qw], self.rt)
        return self._q_only

    def forward(self, h, x, step, line, state, writes_cache: bool, store: bool = False):
        """Adds the mixer's output into x, or returns it as ``Pending`` split sums for the next
        norm to add (a decode step whose output product splits K). ``store``: x receives the
        output instead of a sum onto it, or the split sums are returned and x is left as it is."""
        from .linear import Pending
        T = h.shape[0]
        if writes_cache and self.shared_kv:
            raise ConfigError("a mixer without key and value projections was asked to write "
                              "a cache line")
        nkv = self.nkv if writes_cache else 0
        heads_width = self.qw + nkv * (self.hd + self.vd)
        width = heads_width + self.gate_w
        eps = float(self.head_norm_eps) if self.head_norm_eps is not None else 0.0
        inv_freq, rot_dim = (self.position.frequencies() if self.position is not None
                             else (None, 0))
        split_ok = (writes_cache and self.qkv is not None and rot_dim == self.hd
                    and self.hd in (64, 128, 256) and self.rt.dtype == torch.bfloat16
                    and self.vd == self.hd and not self.gate_n and not self.whole_rows
                    and not self.v_from_k)
        more = {"slopes": self.slopes, "keep_first": self.keep_first}
        qkv = self.qkv(h, defer=True) if split_ok else None
        if isinstance(qkv, Pending):
            # the kernel that norms and rotates q and k adds the split sums up as it reads them
            q = torch.empty((T, self.qw), dtype=self.rt.dtype, device=h.device)
            K.qk_norm_rope_store(None, self.q_norm, self.k_norm, eps, inv_freq, rot_dim, step,
                                 line, self.nh, nkv, self.hd, True, partial=qkv.partial, q_out=q,
                                 unit_after=self.unit_after)
            attn = torch.empty((T, self.qw), dtype=self.rt.dtype, device=h.device)
            self.rt.attention(q, self.qw, attn, step, line, self.nh, self.nkv, self.hd,
                              self.window, self.scale, sink=self.sink, softcap=self.softcap,
                              **more)
            return self._project(attn, x, store)
        if qkv is not None:
            pass
        elif not writes_cache:
            qkv = self.q_only(h)
        elif self.qkv is not None and self.v_from_k:
            # room for the values behind the keys, which the product does not fill
            qkv = torch.empty((T, width), dtype=self.rt.dtype, device=h.device)
            self.qkv(h, out=qkv[:, :self.qw + self.kvw])
        elif self.qkv is not None:
            qkv = self.qkv(h)
        else:
            qkv = torch.empty((T, width), dtype=self.rt.dtype, device=h.device)
            self.split[0](h, out=qkv[:, :self.qw])
            self.split[1](h, out=qkv[:, self.qw:self.qw + self.kvw])
            if not self.v_from_k:
                self.split[2](h, out=qkv[:, self.qw + self.kvw:])
        q_norm, k_norm = self.q_norm, self.k_norm
        if self.whole_rows or self.v_from_k:
            if not writes_cache:
                raise ConfigError("whole-row norms and values from keys with a borrowed cache line")
            if self.whole_rows:
                K.wide_qk_norm(qkv, self.qw, self.kvw, q_norm, k_norm, eps, self.v_from_k)
                q_norm = k_norm = None
            else:       # the copy alone; the per-head norm and the rotation follow as ever
                K.wide_qk_norm(qkv, self.qw, self.kvw, None, None, eps, True)
        K.qk_norm_rope_store(qkv, q_norm, k_norm, eps, inv_freq, rot_dim,
                             step, line, self.nh, nkv, self.hd, writes_cache, vd=self.vd,
                             unit_after=self.unit_after)
        attn = torch.empty((T, self.ow), dtype=self.rt.dtype, device=h.device)
        self.rt.attention(qkv, width, attn, step, line, self.nh, self.nkv, self.hd,
                          self.window, self.scale, vd=self.vd, sink=self.sink,
                          softcap=self.softcap,
                          gate=qkv[:, heads_width:] if self.gate_n else None, gate_stride=width,
                          **more)
        return self._project(attn, x, store)

    def _project(self, attn, x, store: bool):
        from .linear import Pending
        if store:       # stored into x, or left pending (x is then not touched)
            out = self.o(attn, out=x, defer="any")
            return out if isinstance(out, Pending) else None
        out = self.o(attn, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


MIXERS.register("gqa_attention", GqaAttention)
