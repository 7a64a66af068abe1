"""The typed configuration of the Laralix decoder, read from its own config.json keys.

config.json: ``architecture`` = "Laralix", ``vocab``, ``width``, ``norm.eps``,
``embedding.scale`` (absent: 1), ``logit_scale`` (absent: 1), ``loop`` with ``start``, ``stop``
and ``times`` (absent: every layer runs once) and ``layers``, a list whose entries have
``type`` ("parallel", "parallel_2" or "latent_attention"), the mixer's sizes in ``mixer`` and
the feed-forward in ``mlp`` (``kind`` "dense" with ``ff``, or null). Tensor names: ``embed``,
``loop.step``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``.

Layers are pre-norm with RMS norms whose weight is stored around zero (``one_plus``); the
feed-forward is W_down (silu(W_gate h) * W_up h). The layers ``start`` .. ``stop`` - 1 run
``times`` times in a row with the same weights, every pass with cache lines of its own; before
a pass the row of ``loop.step`` with the pass's number is added to the residual and, from the
second pass on, the embedding's output as well.

``parallel``: two mixers side by side whose outputs are each normed over the width
(``mix.left.out``, ``mix.right.out``) and averaged. Left (``mix.left.*``): grouped-query
attention with a weighted norm per head of q and k, no rotation, ``scale``, ``softcap``, a bias
-2^(-8 (h + 1) / heads) * distance, a window ``mask.size`` and one more term exp(0) in the
softmax's denominator. Right (``mix.right.*``): the gated delta rule with short convolutions
of ``conv`` taps.

``parallel_2``: ``left_scale`` * left + ``right_scale`` * right. Left: grouped-query attention
whose values are the keys as projected, q and k normed over their whole rows, a window
``mask.size`` that also keeps the first ``mask.keep_first`` positions. Right: gated linear
attention with a decay per key channel, sigmoid(.)^(1 / ``tau``); the low rank of the decay's
two projections is read from the stored tensors (``rank``, if present, names it for a model
of random weights).

``latent_attention``: queries through a latent of ``q_rank``, keys and values from a latent of
``kv_rank`` and a shared rotated key part of ``rot_dim`` values; ``rot.dims`` of them turn, in
pairs of neighbours, with ``rot.base``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .busavik import MAX_POSITIONS, _dict, _int, _num
from .spec import LayerSpec, ModelSpec, PartSpec, Run

# the distance bias of the design: head h's slope is 2^(DISTANCE_EXPONENT * (h + 1) / heads)
DISTANCE_EXPONENT = -8.0
# the eps under the root when the delta rule's q and k are brought to unit length
UNIT_EPS = 1e-6


@dataclass(frozen=True)
class LaralixConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    loop: Optional[Tuple[int, int, int]]          # (start, stop, times) or None
    layers: Tuple[Dict[str, Any], ...]            # as in config.json, checked
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Laralix"
    MODEL_TYPE = "laralix"

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return MAX_POSITIONS

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, doc: Dict[str, Any], source: str = "config") -> "LaralixConfig":
        if not isinstance(doc, dict):
            raise ConfigError(f"{source} is no JSON object")
        if doc.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"{source}: architecture \"{doc.get('architecture')}\" is not "
                              f"{cls.ARCHITECTURE}")
        layers = doc.get("layers")
        if not isinstance(layers, list) or not 0 < len(layers) <= 1024:
            raise ConfigError(f"{source}: \"layers\" is missing, empty or too long")
        for i, layer in enumerate(layers):
            cls._check_layer(layer, f"{source}: layer {i}")
        norm = _dict(doc, "norm", source)
        scale = 1.0
        if doc.get("embedding") is not None:
            emb = _dict(doc, "embedding", source)
            if emb.get("scale") is not None:
                scale = _num(emb, "scale", source + " embedding")
        loop = None
        if doc.get("loop") is not None:
            lp = _dict(doc, "loop", source)
            start = _int(lp, "start", source + " loop", lo=0, hi=len(layers) - 1)
            stop = _int(lp, "stop", source + " loop", lo=start + 1, hi=len(layers))
            loop = (start, stop, _int(lp, "times", source + " loop", hi=1024))
        return cls(vocab=_int(doc, "vocab", source, hi=1 << 22),
                   width=_int(doc, "width", source, hi=1 << 16),
                   norm_eps=_num(norm, "eps", source + " norm"), embedding_scale=scale,
                   logit_scale=(_num(doc, "logit_scale", source)
                                if doc.get("logit_scale") is not None else 1.0),
                   loop=loop, layers=tuple(layers))

    @staticmethod
    def _heads(m: Dict[str, Any], source: str) -> Tuple[int, int]:
        heads = _int(m, "heads", source, hi=1 << 12)
        kv = _int(m, "kv_heads", source, hi=1 << 12) if m.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"{source}: {heads} heads on {kv} key/value heads")
        _int(m, "dim", source, hi=1 << 12)
        if m.get("vdim") is not None:
            _int(m, "vdim", source, hi=1 << 12)
        return heads, kv

    @staticmethod
    def _mask(m: Dict[str, Any], source: str) -> Tuple[int, int]:
        if m.get("mask") is None:
            return 0, 0
        mk = _dict(m, "mask", source)
        size = _int(mk, "size", source + " mask", hi=1 << 24) if mk.get("size") is not None else 0
        keep = (_int(mk, "keep_first", source + " mask", lo=0, hi=1 << 24)
                if mk.get("keep_first") is not None else 0)
        return size, (keep if size else 0)    # without a window every position is visible anyway

    @classmethod
    def _check_layer(cls, layer: Any, source: str) -> None:
        if not isinstance(layer, dict):
            raise ConfigError(f"{source} is no object")
        kind = layer.get("type")
        m = _dict(layer, "mixer", source)
        ms = source + " mixer"
        if kind in ("parallel", "parallel_2"):
            left, right = _dict(m, "left", ms), _dict(m, "right", ms)
            cls._heads(left, ms + " left")
            cls._heads(right, ms + " right")
            _num(left, "scale", ms + " left")
            cls._mask(left, ms + " left")
            if kind == "parallel":
                if left.get("softcap") is not None and _num(left, "softcap", ms + " left") < 0:
                    raise ConfigError(f"{source}: a score cap of {left['softcap']}")
                _int(right, "conv", ms + " right", hi=8)
            else:
                if left.get("vdim") is not None and int(left["vdim"]) != int(left["dim"]):
                    raise ConfigError(f"{source}: the values are the keys, so value rows of "
                                      f"{left['vdim']} cannot differ from keys of {left['dim']}")
                if _num(right, "tau", ms + " right") <= 0:
                    raise ConfigError(f"{source}: tau = {right['tau']}")
                _num(m, "left_scale", ms)
                _num(m, "right_scale", ms)
        elif kind == "latent_attention":
            _int(m, "heads", ms, hi=1 << 12)
            _int(m, "dim", ms, hi=1 << 12)
            rd = _int(m, "rot_dim", ms, lo=0, hi=1 << 12)
            _int(m, "vdim", ms, hi=1 << 12)
            _int(m, "kv_rank", ms, hi=1 << 16)
            _int(m, "q_rank", ms, hi=1 << 16)
            _num(m, "scale", ms)
            if m.get("rot") is not None:
                rot = _dict(m, "rot", ms)
                dims = _int(rot, "dims", ms + " rot", lo=0, hi=1 << 12)
                if dims % 2 or dims > rd:
                    raise ConfigError(f"{source}: {dims} rotating values of a part of {rd}")
                if dims and _num(rot, "base", ms + " rot") <= 0:
                    raise ConfigError(f"{source}: a rotary base of {rot['base']}")
        else:
            raise ConfigError(f"{source}: mixer type \"{kind}\" is not known "
                              "(known: latent_attention, parallel, parallel_2)")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
            raise ConfigError(f"{source}: feed-forward kind "
                              f"\"{mlp.get('kind') if isinstance(mlp, dict) else mlp}\" "
                              "is not known (known: dense)")
        _int(mlp, "ff", source + " mlp", hi=1 << 22)

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> Dict[str, Any]:
        doc: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale},
                               "logit_scale": self.logit_scale, "layers": list(self.layers)}
        if self.loop is not None:
            doc["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return doc

    # ------------------------------------------------------------------ the model as data
    def order(self) -> List[Tuple[int, int]]:
        """The order of layer runs as (layer, pass): ``pass`` is the number of the pass
        through the looped layers that this run opens, -1 for every other run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, -1) for i in range(n)]
        a, b, times = self.loop
        runs = [(i, -1) for i in range(a)]
        for t in range(times):
            runs += [(i, t if i == a else -1) for i in range(a, b)]
        return runs + [(i, -1) for i in range(b, n)]

    def _attention(self, m: Dict[str, Any], prefix: str, kind: str) -> PartSpec:
        heads = int(m["heads"])
        size, keep = self._mask(m, "mask")
        names = {"q": prefix + "q", "k": prefix + "k", "o": prefix + "o",
                 "q_norm": prefix + "q.norm", "k_norm": prefix + "k.norm"}
        params: Dict[str, Any] = {
            "hidden_size": self.width, "heads": heads,
            "kv_heads": int(m.get("kv_heads") or heads), "head_dim": int(m["dim"]),
            "scale": float(m["scale"]), "window": size, "keep_first": keep,
            "head_norm_eps": self.norm_eps, "names": names}
        if kind == "parallel":
            names["v"] = prefix + "v"
            params.update({"v_dim": int(m.get("vdim") or m["dim"]),
                           "softcap": float(m.get("softcap") or 0.0),
                           "distance_exponent": DISTANCE_EXPONENT, "sink_value": 0.0})
        else:
            params.update({"head_norm": "whole_rows", "values": "keys_as_projected"})
        return PartSpec("gqa_attention", params)

    def _mixer(self, layer: Dict[str, Any], positions: Dict[str, PartSpec]) -> PartSpec:
        m, kind = layer["mixer"], layer["type"]
        c = self
        if kind == "latent_attention":
            rot = m.get("rot") or {}
            position = ""
            if int(rot.get("dims") or 0):
                spec = PartSpec("rope_pairs", {"theta": float(rot["base"]),
                                               "rot_dim": int(rot["dims"]), "rounding": "once"})
                position = next((n for n, have in positions.items() if have == spec), "")
                if not position:
                    position = f"rot{len(positions)}"
                    positions[position] = spec
            return PartSpec("latent_attention", {
                "hidden_size": c.width, "heads": int(m["heads"]), "dim": int(m["dim"]),
                "rot_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]),
                "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]),
                "scale": float(m["scale"]), "latent_norm_eps": c.norm_eps, "gate": False,
                "position": position,
                "names": {"dq": "mix.dq", "dq_norm": "mix.dq.norm", "uq": "mix.uq",
                          "dkv": "mix.dkv", "dkv_norm": "mix.dkv.norm", "uk": "mix.uk",
                          "uv": "mix.uv", "o": "mix.o"}})
        left, right = m["left"], m["right"]
        r = "mix.right."
        heads, dim = int(right["heads"]), int(right["dim"])
        vdim = int(right.get("vdim") or dim)
        if kind == "parallel":
            rec = PartSpec("gated_delta", {
                "hidden_size": c.width, "heads": heads,
                "kv_heads": int(right.get("kv_heads") or heads), "dim": dim, "vdim": vdim,
                "taps": int(right["conv"]), "eps": c.norm_eps, "unit_eps": UNIT_EPS,
                "names": {k: r + v for k, v in {
                    "q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv",
                    "v_conv": "v.conv", "b": "b", "a": "a", "A_log": "A_log",
                    "dt_bias": "dt_bias", "g": "g", "norm": "norm", "o": "o"}.items()}})
            norm = lambda name: {"name": name, "eps": c.norm_eps}
            branches = [
                {"mixer": self._attention(left, "mix.left.", kind), "scale": 0.5,
                 "out_norm": norm("mix.left.out")},
                {"mixer": rec, "scale": 0.5, "out_norm": norm("mix.right.out")}]
        else:
            rec = PartSpec("gated_linear_attention", {
                "hidden_size": c.width, "heads": heads, "dim": dim, "vdim": vdim,
                "tau": float(right["tau"]), "eps": c.norm_eps,
                # the decay's low rank is what the stored tensors have; a configuration that a
                # random model is drawn from names it as "rank"
                "decay_rank": int(right["rank"]) if right.get("rank") is not None else None,
                "names": {k: r + v for k, v in {
                    "q": "q", "k": "k", "v": "v", "g": "g", "a1": "a1", "a2": "a2",
                    "a2_bias": "a2.b", "norm": "norm", "o": "o"}.items()}})
            branches = [
                {"mixer": self._attention(left, "mix.left.", kind), "scale": float(m["left_scale"])},
                {"mixer": rec, "scale": float(m["right_scale"])}]
        return PartSpec("side_by_side", {"hidden_size": c.width, "branches": branches})

    def to_model_spec(self) -> ModelSpec:
        c = self
        positions: Dict[str, PartSpec] = {}
        layers: List[LayerSpec] = []
        norm = lambda name: PartSpec("rmsnorm", {"name": name, "size": c.width,
                                                 "eps": c.norm_eps, "one_plus": True})
        for i, layer in enumerate(c.layers):
            mlp = layer.get("mlp")
            norms = {"mixer": norm("norm1")}
            if mlp is None:
                ff = PartSpec("none")
                # a layer without a feed-forward may still store its second norm: tolerated, unused
                norms["spare"] = PartSpec("rmsnorm", {"name": "norm2", "size": c.width,
                                                      "eps": c.norm_eps, "optional": True})
            else:
                ff = PartSpec("swiglu", {"hidden_size": c.width,
                                         "intermediate_size": int(mlp["ff"]),
                                         "names": {"gate": "mlp.gate", "up": "mlp.up",
                                                   "down": "mlp.down"}})
                norms["feed_forward"] = norm("norm2")
            layers.append(LayerSpec(block=PartSpec("prenorm_residual"),
                                    mixer=c._mixer(layer, positions), feed_forward=ff,
                                    norms=norms, prefix=f"l{i}."))
        schedule = []
        for n, (l, t) in enumerate(c.order()):
            before = None
            if t >= 0:
                before = PartSpec("pass_input", {"name": "loop.step", "rows": c.loop[2], "row": t,
                                                 "size": c.width, "add_embedding": t > 0})
            schedule.append(Run(layer=l, cache_line=n, writes_cache=True, before=before))
        return ModelSpec(
            architecture=c.ARCHITECTURE, vocab_size=c.vocab, hidden_size=c.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": c.vocab,
                                                   "hidden_size": c.width,
                                                   "scale": c.embedding_scale}),
            positions=positions, layers=tuple(layers), schedule=tuple(schedule),
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": c.vocab,
                                      "hidden_size": c.width, "scale": c.logit_scale}),
            # a model without a loop may still store the passes' vectors: tolerated, unused
            tolerated=() if c.loop is not None else (("loop.step", (-1, c.width)),))
