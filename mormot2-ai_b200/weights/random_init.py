"""Random weights from a configuration and a seed: a model folder (config.json,
model.safetensors) for tests and traces, or tensors made on the device for benchmarks of
large shapes.

Matrices, tables and biases are N(0, std), norm weights 1 + N(0, norm_std), fractions (the
weights of a blend of two rows) uniform in [0, 1), matrices near the identity I + N(0,
norm_std); drawn in float32 from one
seeded generator in the order of the tensor names and then rounded to the stored type (the
reference's fixture tool draws 0.08·randn and 1 + 0.25·randn and rounds to BF16:
``tools/infer-ref/make_reference_qwen3.py:837-844`` of the reference project).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterable

import torch

from ..parts.base import TensorNeed
from .safetensors_file import write_safetensors


def random_tensors(needs: Iterable[TensorNeed], seed: int, std: float = 0.02,
                   norm_std: float = 0.1, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    for n in sorted((n for n in needs if not n.optional), key=lambda n: n.name):
        if any(d < 0 for d in n.shape):
            raise ValueError(f"{n.name}: a size that only a stored tensor gives; the "
                             "configuration of a random model must name it")
        if device == "cpu":
            t = torch.randn(n.shape, generator=gen, dtype=torch.float32)
        else:
            # drawn in the stored type on the device: a large model never exists in float32
            t = torch.empty(n.shape, dtype=dtype, device=device).normal_(0.0, 1.0, generator=gen)
        if n.role == "vector":
            t = t.mul_(norm_std).add_(1.0)
        elif n.role == "taps":
            t = t.mul_(0.5)
        elif n.role == "around_zero":
            t = t.mul_(norm_std)
        elif n.role == "fraction":
            t = t.mul_(0.7071).erf_().add_(1.0).mul_(0.5)      # a normal draw made uniform
        elif n.role == "identity":
            t = t.mul_(norm_std).add_(torch.eye(n.shape[0], n.shape[1], dtype=t.dtype,
                                                device=t.device))
        else:
            t = t.mul_(std)
        out[n.name] = t.to(dtype)
    return out


def write_random_model(folder: str, config, seed: int, std: float = 0.02,
                       norm_std: float = 0.1, dtype: torch.dtype = torch.bfloat16) -> str:
    """Writes ``config.json`` and ``model.safetensors`` of a randomly initialised model of the
    configuration's architecture into ``folder`` and returns it."""
    from ..engine.model import DecoderModel
    os.makedirs(folder, exist_ok=True)
    needs = DecoderModel(config.to_model_spec()).tensors()
    tensors = random_tensors(needs, seed, std, norm_std, dtype)
    doc = config.to_dict()
    doc["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(doc, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder
