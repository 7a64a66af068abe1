"""Several mixers side by side: all read the same input, and the result is the sum of their
outputs with a constant factor each. A branch is any registered mixer; at most one of them
may keep keys and values (it gets the cache line), and the branches' fixed-size states lie one
after another in the state of this mixer.

A branch may name ``out_norm`` = {"name", "eps"}: its output is then brought to unit root mean
square over the model width and multiplied by that weight [hidden] before its factor applies
(the factor is folded into the weight once at load)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from ..config.spec import PartSpec
from ..errors import ConfigError
from .base import MIXERS, CacheNeed, Part, StateNeed, TensorNeed


class SideBySide(Part):
    can_store = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        self.branches, self.scales, self.out_norms = [], [], []
        for b in spec.params["branches"]:
            sub = b["mixer"] if isinstance(b["mixer"], PartSpec) else PartSpec(**b["mixer"])
            self.branches.append(MIXERS.build(sub, prefix, positions=positions))
            self.scales.append(float(b.get("scale", 1.0)))
            norm = b.get("out_norm")
            self.out_norms.append((prefix + norm["name"], float(norm["eps"])) if norm else None)
        if any(self.out_norms) and not all(self.out_norms):
            raise ConfigError("either every mixer side by side has an output norm or none")
        self.hidden = int(spec.params.get("hidden_size", 0))
        if any(self.out_norms) and self.hidden <= 0:
            raise ConfigError("output norms of mixers side by side need hidden_size")
        if not 1 <= len(self.branches) <= 4:
            raise ConfigError(f"{len(self.branches)} mixers side by side (1 to 4)")
        if sum(b.cache_need() is not None for b in self.branches) > 1:
            raise ConfigError("more than one of the mixers side by side keeps keys and values")
        self.offsets, at = [], 0
        for b in self.branches:
            need = b.state_need()
            n = 0
            if need is not None:
                if need.dtype != "float32" or need.init != 0.0 or len(need.shape) != 1:
                    raise ConfigError("mixers side by side keep flat float32 state that starts at 0")
                n = int(need.shape[0])
            self.offsets.append((at, n))
            at += n
        self.state_size = at

    @property
    def capturable(self) -> bool:
        return all(getattr(b, "capturable", False) for b in self.branches)

    def libraries(self, rt) -> List[str]:
        out = [] if any(self.out_norms) else ["streams"]
        for b in self.branches:
            out += [n for n in b.libraries(rt) if n not in out]
        return out

    def tensors(self) -> List[TensorNeed]:
        out = [t for b in self.branches for t in b.tensors()]
        out += [TensorNeed(n[0], (self.hidden,), "vector") for n in self.out_norms if n]
        return out

    def cache_need(self) -> Optional[CacheNeed]:
        for b in self.branches:
            if b.cache_need() is not None:
                return b.cache_need()
        return None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.state_size,), "float32", 0.0) if self.state_size else None

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        for b in self.branches:
            b.bind(weights, rt)
        # a branch's factor rides in its norm's weight (float32)
        self.norm_weights = [(weights[n[0]].to(torch.float32) * s).contiguous() if n else None
                             for n, s in zip(self.out_norms, self.scales)]

    def forward_branches(self, h, step, line, state, writes_cache: bool):
        """Runs every branch and returns ``[(y_b float32 [T, hidden], factor_b)]``: whoever
        adds the outputs into the residual does the weighted sum on the way."""
        terms, terms_of = [], []
        for b, scale, (at, n) in zip(self.branches, self.scales, self.offsets):
            terms_of.append(b)
            y = torch.empty((h.shape[0], h.shape[1]), dtype=torch.float32, device=h.device)
            sub_state = state[:, at:at + n] if n else None
            sub_line = line if b.cache_need() is not None else None
            if getattr(b, "can_store", False):
                pending = b.forward(h, y, step, sub_line, sub_state, writes_cache, store=True)
                # a later branch may need a term for a buffer of its own
                left = len(self.branches) - len(terms_of)
                if pending is not None and len(terms) + len(pending.partial) + left <= 16:
                    # the branch left its output as split sums: each is a term of its own
                    terms += [(part, scale) for part in pending.partial]
                    continue
                if pending is not None:      # more terms than a kernel takes: summed here
                    y.zero_()
                    K.add_partials(y, pending.partial)
            else:
                y.zero_()
                pending = b.forward(h, y, step, sub_line, sub_state, writes_cache)
                if pending is not None:
                    K.add_partials(y, pending.partial)
            terms.append((y, scale))
        return terms

    def forward(self, h, x, step, line, state, writes_cache: bool, store: bool = False):
        if any(self.out_norms):
            return self._forward_normed(h, x, step, line, state, writes_cache, store)
        K.add_scaled(x, self.forward_branches(h, step, line, state, writes_cache), store)
        return None

    def _forward_normed(self, h, x, step, line, state, writes_cache: bool, store: bool):
        """x += factor_b * w_b * y_b / rms(y_b) for every branch: one kernel a branch sums the
        branch's split sums (if its output product left any), norms the row and adds it."""
        if store:
            raise ConfigError("mixers side by side with output norms add into the residual")
        for b, (at, n), norm, w in zip(self.branches, self.offsets, self.out_norms,
                                       self.norm_weights):
            sub_state = state[:, at:at + n] if n else None
            sub_line = line if b.cache_need() is not None else None
            y = torch.empty((h.shape[0], h.shape[1]), dtype=torch.float32, device=h.device)
            if getattr(b, "can_store", False):
                pending = b.forward(h, y, step, sub_line, sub_state, writes_cache, store=True)
                if pending is not None and pending.partial.shape[0] <= 8:
                    K.norm_add(pending.partial, w, norm[1], x)
                    continue
                if pending is not None:
                    y.zero_()
                    K.add_partials(y, pending.partial)
            else:
                y.zero_()
                pending = b.forward(h, y, step, sub_line, sub_state, writes_cache)
                if pending is not None:
                    K.add_partials(y, pending.partial)
            K.norm_add(y, w, norm[1], x)
        return None


MIXERS.register("side_by_side", SideBySide)
