"""RMSNorm: y = w · x / sqrt(mean(x²) + eps), the weight multiplying as it is (not 1 + w);
sums in float32 (``backend.cpu.pas:1769-1795``, ``ops.cu:116-130`` of the reference). With
``one_plus`` the stored weight lies around zero and 1 + w multiplies (formed once at load, in
float32).

Dynamic Tanh: y = tanh(alpha · x) · w + b with a learned scalar alpha: a norm that forms no
mean and no variance, value by value in float32.

Layer norm: y = (x − mean) / sqrt(var + eps) · w with the variance as the mean of the squared
deviations and no bias, in float32. Over a residual of several streams it norms their sum."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels as K
from .base import NORMS, Part, TensorNeed


class RmsNorm(Part):
    capturable = True
    accepts_pending = True      # forward(..., pending=) adds split sums into x before it norms

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = prefix + spec.params["name"]
        self.one_plus = bool(spec.params.get("one_plus", False))
        self.optional = bool(spec.params.get("optional", False))   # may be absent (and unused)
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> List[TensorNeed]:
        return [TensorNeed(self.name, (self.size,), "around_zero" if self.one_plus else "vector",
                           optional=self.optional)]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        if self.optional and self.name not in weights:
            return
        self.weight = weights[self.name]
        if self.one_plus:
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()
        self.rt = rt

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, pending=None) -> torch.Tensor:
        """x: the float32 residual [T, size]. ``rows``: only these rows are normed (gathered).
        ``pending``: the split sums of the product before (``parts/linear.py: Pending``), which
        are first added into x."""
        R = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((R, self.size), dtype=self.rt.dtype, device=x.device)
        K.rmsnorm(x, self.weight, self.eps, out, rows, R,
                  pending.partial if pending is not None else None)
        return out

    def add_normed(self, y: torch.Tensor, x: torch.Tensor, h: Optional[torch.Tensor] = None) -> None:
        """x += w · y / rms(y) for a sublayer's output y [T, size] float32 (or its split sums
        [parts, T, size]); ``h`` receives the new x in the activation type."""
        K.norm_add(y, self.weight, self.eps, x, h)


class DynamicTanh(Part):
    """``name`` is the weight; the scalar and the shift are stored beside it as
    ``<name>.alpha`` and ``<name>.b``."""
    capturable = True
    accepts_pending = True
    accepts_residual_bias = True   # forward(..., residual_bias=) adds it into x after norming

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec.params["size"])
        self.name = prefix + spec.params["name"]
        self.optional = bool(spec.params.get("optional", False))   # may be absent (and unused)

    def tensors(self) -> List[TensorNeed]:
        return [TensorNeed(self.name, (self.size,), "vector", optional=self.optional),
                TensorNeed(self.name + ".b", (self.size,), "bias", optional=self.optional),
                TensorNeed(self.name + ".alpha", (), "vector", optional=self.optional)]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        if self.optional and self.name not in weights:
            self.weight = self.bias = self.alpha = None
            return
        self.weight, self.bias = weights[self.name], weights[self.name + ".b"]
        # the scalar stays on the device, as float32 whatever it was stored as
        self.alpha = weights[self.name + ".alpha"].to(torch.float32).reshape(1)
        self.rt = rt

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None, pending=None, residual_bias=None) -> torch.Tensor:
        R = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[0])
        out = torch.empty((R, self.size), dtype=self.rt.dtype, device=x.device)
        K.dynamic_tanh(x, self.weight, self.bias, self.alpha, out, rows, R,
                       pending.partial if pending is not None else None, residual_bias)
        return out


class LayerNorm(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.name = prefix + spec.params["name"]
        self.weight: Optional[torch.Tensor] = None

    def libraries(self, rt) -> List[str]:
        return ["streams"]

    def tensors(self) -> List[TensorNeed]:
        return [TensorNeed(self.name, (self.size,), "vector")]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.weight = weights[self.name]
        self.rt = rt

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None) -> torch.Tensor:
        """x: the float32 residual [T, size], or [streams, T, size], whose sum is normed."""
        R = n_rows if n_rows is not None else (rows.numel() if rows is not None else x.shape[-2])
        out = torch.empty((R, self.size), dtype=self.rt.dtype, device=x.device)
        K.stream_step(x, read=(None, self.weight, self.eps, out, rows, R))
        return out


NORMS.register("rmsnorm", RmsNorm)
NORMS.register("layernorm", LayerNorm)
NORMS.register("dynamic_tanh", DynamicTanh)
