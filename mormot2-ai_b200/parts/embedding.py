"""Token embedding (rows of the table into the float32 residual, times ``scale`` where a
design names one; the reference scales nothing: ``decoder.pas:3292-3309``) and the head (logits = h · Headᵀ in float32, the
head being the embedding when tied: ``model.qwen3.pas:555-579``; a head with ``scale``
multiplies its float32 logits by that constant; one with ``softcap`` c turns them into
c tanh(logits / c))."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from .base import EMBEDDINGS, ENTRIES, HEADS, Part, TensorNeed
from .linear import Linear


class TokenEmbedding(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.name = spec.params["name"]
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.scale = float(spec.params.get("scale", 1.0))

    def tensors(self) -> List[TensorNeed]:
        return [TensorNeed(self.name, (self.vocab, self.hidden), "table")]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.table = weights[self.name]

    def forward(self, ids: torch.Tensor, x: torch.Tensor) -> None:
        """x [T, hidden], or [streams, T, hidden]: every stream starts as the same rows."""
        K.embed(self.table, ids, x, self.scale)


class LmHead(Part):
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.tied = bool(p["tied"])
        self.name = p["tied_to"] if self.tied else p["name"]
        self.stored_name = p["name"]
        self.vocab, self.hidden = int(p["vocab_size"]), int(p["hidden_size"])
        self.scale = float(p.get("scale", 1.0))
        self.softcap = float(p.get("softcap") or 0.0)    # logits <- c tanh(logits / c)

    def tensors(self) -> List[TensorNeed]:
        if self.tied:
            # a stored copy of a tied head is tolerated when it equals the embedding
            return [TensorNeed(self.stored_name, (self.vocab, self.hidden), "table", optional=True,
                               must_equal=self.name)]
        return [TensorNeed(self.name, (self.vocab, self.hidden), "matrix")]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.linear = Linear(weights[self.name], rt)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = self.linear(h, out_dtype=torch.float32)
        if self.scale != 1.0:
            K.scale_rows(logits, self.scale)
        if self.softcap > 0:
            K.softcap_rows(logits, self.softcap)
        return logits


class PassInput(Part):
    """What a pass through looped layers adds to the residual before its first layer: row
    ``row`` of the table ``name`` [rows, size] and, with ``add_embedding``, the embedding's
    output once more (the model keeps a copy of it for the runs that ask)."""
    capturable = True

    def __init__(self, spec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.params
        self.name = prefix + p["name"]
        self.rows, self.row, self.size = int(p["rows"]), int(p["row"]), int(p["size"])
        self.add_embedding = bool(p.get("add_embedding", False))

    def tensors(self) -> List[TensorNeed]:
        return [TensorNeed(self.name, (self.rows, self.size), "bias")]

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.vector = weights[self.name][self.row].contiguous()

    def forward(self, x: torch.Tensor, x0) -> None:
        K.pass_input(x, self.vector, x0 if self.add_embedding else None)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
ENTRIES.register("pass_input", PassInput)
HEADS.register("lm_head", LmHead)
