"""Latent attention as a mixer: queries and keys/values go through low-rank latents, and the
cache keeps one row per token, the normed key/value latent c (``kv_rank`` values) followed by
one rotated key part r that all heads share (``rot_dim`` values), instead of keys and values
per head.

    c_q = rmsnorm(W_dq h),  q_h = W_uq,h c_q = [q_h,plain (dim) ; q_h,rot (rot_dim)]
    [c' ; r'] = W_dkv h,    c = rmsnorm(c'),  r = rotate(r'),  q_h,rot <- rotate(q_h,rot)
    k_h = [W_uk,h c ; r],   v_h = W_uv,h c,   score = (q_h · k_h) · scale, causal softmax
    out = W_o (concat_h(sum_j p_j v_h,j) * sigmoid(W_g h))          (the gate is optional)

The kernels never form k_h or v_h: q_h,plain is carried into the latent space
(W_uk,hᵀ q_h,plain, a small product per head), every head attends over the same cache rows
[c ; r], and the weighted latent is carried out through W_uv,h (``csrc/latent.cu``). The
projections that read h (W_dq, W_dkv, W_g) are one product.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels as K
from ..errors import ConfigError
from .base import MIXERS, CacheNeed, Part, TensorNeed
from .linear import Linear, Pending


class LatentAttention(Part):
    capturable = True

    def __init__(self, spec, prefix: str = "", positions=None):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.dim, self.rd = int(p["heads"]), int(p["dim"]), int(p["rot_dim"])
        self.vd, self.kvr, self.qr = int(p["vdim"]), int(p["kv_rank"]), int(p["q_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["latent_norm_eps"])
        self.window = int(p.get("window", 0))
        self.gated = bool(p.get("gate", False))
        self.names = {k: prefix + v for k, v in p["names"].items()}
        self.position = (positions or {}).get(p.get("position", ""))
        if p.get("position") and self.position is None:
            raise ConfigError(f"the mixer names the position encoding \"{p['position']}\", "
                              "which the model does not define")
        if min(self.nh, self.dim, self.vd, self.kvr, self.qr) <= 0 or self.rd < 0:
            raise ConfigError(f"latent attention with sizes {p}")

    def libraries(self, rt) -> List[str]:
        return ["latent", "latent_mma"] if rt.fast_kernels else ["latent"]

    def tensors(self) -> List[TensorNeed]:
        n = self.names
        out = [TensorNeed(n["dq"], (self.qr, self.hidden)),
               TensorNeed(n["dq_norm"], (self.qr,), "vector"),
               TensorNeed(n["uq"], (self.nh * (self.dim + self.rd), self.qr)),
               TensorNeed(n["dkv"], (self.kvr + self.rd, self.hidden)),
               TensorNeed(n["dkv_norm"], (self.kvr,), "vector"),
               TensorNeed(n["uk"], (self.nh * self.dim, self.kvr)),
               TensorNeed(n["uv"], (self.nh * self.vd, self.kvr)),
               TensorNeed(n["o"], (self.hidden, self.nh * self.vd))]
        if self.gated:
            out.append(TensorNeed(n["g"], (self.nh * self.vd, self.hidden)))
        return out

    def cache_need(self) -> CacheNeed:
        return CacheNeed(1, self.kvr + self.rd, self.window, planes=1)

    def bind(self, weights: Dict[str, torch.Tensor], rt) -> None:
        self.rt = rt
        n = self.names
        w_dkv, w_uq = weights[n["dkv"]], weights[n["uq"]]
        if getattr(self.position, "pairing", "half") == "neighbours" and self.rd:
            # an encoding that turns neighbours: the rows that produce the shared key part and
            # every head's rotated query part are reordered once, so that the kernels' pairing
            # (i, i + half) turns the same pairs; the scores see no difference
            order = torch.tensor(self.position.half_order(self.rd), device=w_dkv.device)
            w_dkv = torch.cat([w_dkv[:self.kvr], w_dkv[self.kvr:][order]], dim=0)
            per = w_uq.view(self.nh, self.dim + self.rd, self.qr)
            w_uq = torch.cat([per[:, :self.dim], per[:, self.dim:][:, order]],
                             dim=1).reshape(w_uq.shape)
        first = [weights[n["dq"]], w_dkv] + ([weights[n["g"]]] if self.gated else [])
        if len({w.dtype for w in first}) > 1:
            first = [w.float() for w in first]
        # one product for everything that reads h; the query latent first, then the key/value
        # latent with the shared key part behind it, then the gate
        self.down = Linear(torch.cat(first, dim=0), rt)
        self.kv_col, self.gate_col = self.qr, self.qr + self.kvr + self.rd
        self.uq = Linear(w_uq, rt)
        # per head: W_uk,hᵀ as [kv_rank, dim] (the product's output rows), W_uv,h as [vdim, kv_rank]
        self.uk_t = (weights[n["uk"]].view(self.nh, self.dim, self.kvr).transpose(1, 2)
                     .contiguous())
        self.uv = weights[n["uv"]].view(self.nh, self.vd, self.kvr).contiguous()
        self.o = Linear(weights[n["o"]], rt)
        self.q_norm, self.kv_norm = weights[n["dq_norm"]], weights[n["dkv_norm"]]
        if self.q_norm.dtype != self.kv_norm.dtype:
            self.q_norm, self.kv_norm = self.q_norm.float(), self.kv_norm.float()
        if getattr(rt, "consume_weights", False):
            for key in ["dq", "dkv", "uk"] + (["g"] if self.gated else []):
                weights.pop(n[key], None)

    def forward(self, h, x, step, line, state, writes_cache: bool):
        T, dev, dt = h.shape[0], h.device, self.rt.dtype
        nh, dim, rd, vd, kvr, qr = self.nh, self.dim, self.rd, self.vd, self.kvr, self.qr
        inv_freq, rot_dims = (self.position.frequencies() if self.position is not None
                              else (None, 0))
        amplitude = float(getattr(self.position, "amplitude", 1.0))
        if rot_dims > rd:
            raise ConfigError(f"{rot_dims} rotating values of a part of {rd}")
        # [T, qr + kvr + rd (+ nh vd)], or (few tokens) the product's split sums, which the kernel
        # that norms the latents adds up as it reads them
        f = self.down(h, defer=True)
        cq = torch.empty((T, qr), dtype=dt, device=dev)
        if isinstance(f, Pending):
            gate = torch.empty((T, nh * vd), dtype=dt, device=dev) if self.gated else None
            K.latent_prep(None, 0, self.kv_col, qr, kvr, rd, self.q_norm, self.kv_norm, self.eps,
                          inv_freq, rot_dims, amplitude, step, line, cq, writes_cache,
                          partial=f.partial, gate_out=gate, gate_col=self.gate_col)
        else:
            gate = f[:, self.gate_col:] if self.gated else None
            K.latent_prep(f, 0, self.kv_col, qr, kvr, rd, self.q_norm, self.kv_norm, self.eps,
                          inv_freq, rot_dims, amplitude, step, line, cq, writes_cache)
        q = self.uq(cq)                                                # [T, nh (dim + rd)]
        ql = torch.empty((T, nh * (kvr + rd)), dtype=dt, device=dev)
        K.heads_gemm(q, dim + rd, self.uk_t, ql, kvr + rd, tail=rd, rot_dims=rot_dims,
                     inv_freq=inv_freq, amplitude=amplitude, tok_pos=step.tok_pos)
        ol = torch.empty((T, nh * kvr), dtype=dt, device=dev)
        self.rt.latent_attention(ql, ol, step, line, nh, kvr, rd, self.window, self.scale)
        heads = torch.empty((T, nh * vd), dtype=dt, device=dev)
        K.heads_gemm(ol, kvr, self.uv, heads, vd, gate=gate)
        out = self.o(heads, add_into=x, defer=True)
        return out if isinstance(out, Pending) else None


MIXERS.register("latent_attention", LatentAttention)
