"""The typed configuration of the Sezopel decoder, read from its own config.json keys.

config.json: ``architecture`` = "Sezopel", ``vocab``, ``width``, ``norm.eps``,
``embedding.scale`` (absent: 1), ``logit_softcap`` (absent: none), ``token_side.dim`` (absent:
no input from the token after a layer's feed-forward) and ``layers``, a list whose entries have
``type`` ("attention" or "retention"), the mixer's sizes in ``mixer`` and the feed-forward in
``mlp`` (``kind`` "dense" with ``ff``, or null). Tensor names: ``embed``, ``side.embed``,
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``,
``final.norm``, ``head``.

Mixer ``attention``: ``heads``, ``kv_heads`` (absent: ``heads``), ``dim``, ``vdim`` (absent:
``dim``), ``scale``, ``softcap`` (absent: none), ``rot`` with ``base`` and ``dims`` (absent: no
rotation) and optionally ``kv_from``: j, which gives the layer no key and value projections:
it reads what layer j keeps. Mixer ``retention``: ``heads``, ``dim``, ``vdim`` (absent:
``dim``), ``decay`` (one per head), ``rot``.

Every layer norms what its sublayers give back (``output_norm_residual``); q and k are brought
to unit root mean square after the rotation; the heads' outputs pass a sigmoid gate (one
logit per head); the feed-forward is W_down relu(W_up x)².
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import ConfigError
from .busavik import MAX_POSITIONS, _dict, _int, _num
from .spec import LayerSpec, ModelSpec, PartSpec, Run


@dataclass(frozen=True)
class SezopelConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float                          # 0: none
    side_dim: int                                 # 0: no input from the token after a layer
    layers: Tuple[Dict[str, Any], ...]            # as in config.json, checked
    extra: Dict[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Sezopel"
    MODEL_TYPE = "sezopel"

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
    def from_dict(cls, doc: Dict[str, Any], source: str = "config") -> "SezopelConfig":
        if not isinstance(doc, dict):
            raise ConfigError(f"{source} is no JSON object")
        if doc.get("architecture") != cls.ARCHITECTURE:
            raise ConfigError(f"{source}: architecture \"{doc.get('architecture')}\" is not "
                              f"{cls.ARCHITECTURE}")
        layers = doc.get("layers")
        if not isinstance(layers, list) or not 0 < len(layers) <= 1024:
            raise ConfigError(f"{source}: \"layers\" is missing, empty or too long")
        for i, layer in enumerate(layers):
            cls._check_layer(layer, i, layers, f"{source}: layer {i}")
        norm = _dict(doc, "norm", source)
        if norm.get("kind", "rms") not in ("rms", "rmsnorm"):
            raise ConfigError(f"{source}: norm kind \"{norm.get('kind')}\" is not known (known: rms)")
        scale = 1.0
        if doc.get("embedding") is not None:
            emb = _dict(doc, "embedding", source)
            if emb.get("scale") is not None:
                scale = _num(emb, "scale", source + " embedding")
        cap = 0.0
        if doc.get("logit_softcap") is not None:
            cap = _num(doc, "logit_softcap", source)
            if cap < 0:
                raise ConfigError(f"{source}: a logit cap of {cap}")
        side = 0
        if doc.get("token_side") is not None:
            side = _int(_dict(doc, "token_side", source), "dim", source + " token_side",
                        hi=1 << 16)
        return cls(vocab=_int(doc, "vocab", source, hi=1 << 22),
                   width=_int(doc, "width", source, hi=1 << 16),
                   norm_eps=_num(norm, "eps", source + " norm"),
                   embedding_scale=scale, logit_softcap=cap, side_dim=side,
                   layers=tuple(layers))

    @staticmethod
    def _check_rot(m: Dict[str, Any], dim: int, source: str) -> None:
        if m.get("rot") is None:
            return
        rot = _dict(m, "rot", source)
        dims = _int(rot, "dims", source + " rot", lo=0, hi=1 << 12)
        if dims % 2 or dims > dim:
            raise ConfigError(f"{source}: {dims} rotating values of a head of {dim}")
        if dims and _num(rot, "base", source + " rot") <= 0:
            raise ConfigError(f"{source}: a rotary base of {rot['base']}")

    @classmethod
    def _check_layer(cls, layer: Any, i: int, layers: List[Any], source: str) -> None:
        if not isinstance(layer, dict):
            raise ConfigError(f"{source} is no object")
        kind = layer.get("type")
        m = _dict(layer, "mixer", source)
        ms = source + " mixer"
        if kind == "attention":
            heads, dim = _int(m, "heads", ms, hi=1 << 12), _int(m, "dim", ms, hi=1 << 12)
            kv = _int(m, "kv_heads", ms, hi=1 << 12) if m.get("kv_heads") is not None else heads
            if heads % kv:
                raise ConfigError(f"{source}: {heads} heads on {kv} key/value heads")
            if m.get("vdim") is not None:
                _int(m, "vdim", ms, hi=1 << 12)
            _num(m, "scale", ms)
            if m.get("softcap") is not None and _num(m, "softcap", ms) < 0:
                raise ConfigError(f"{source}: a score cap of {m['softcap']}")
            cls._check_rot(m, dim, ms)
            if m.get("kv_from") is not None:
                j = _int(m, "kv_from", ms, lo=0, hi=len(layers) - 1)
                other = layers[j] if isinstance(layers[j], dict) else {}
                om = other.get("mixer") if isinstance(other.get("mixer"), dict) else {}
                if j >= i or other.get("type") != "attention" or om.get("kv_from") is not None:
                    raise ConfigError(f"{source}: kv_from names layer {j}, which is no earlier "
                                      "attention layer with keys and values of its own")
                same = lambda key, default=None: (om.get(key, default) == m.get(key, default))
                if not (same("heads") and same("dim") and same("rot")
                        and om.get("kv_heads", om.get("heads")) == kv
                        and om.get("vdim", om.get("dim")) == m.get("vdim", dim)):
                    raise ConfigError(f"{source}: kv_from names layer {j}, whose heads, sizes or "
                                      "rotation differ")
        elif kind == "retention":
            heads, dim = _int(m, "heads", ms, hi=1 << 12), _int(m, "dim", ms, hi=1 << 12)
            if m.get("vdim") is not None:
                _int(m, "vdim", ms, hi=1 << 12)
            decay = m.get("decay")
            if (not isinstance(decay, list) or len(decay) != heads
                    or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay)):
                raise ConfigError(f"{source}: \"decay\" is no list of {heads} numbers")
            cls._check_rot(m, dim, ms)
        else:
            raise ConfigError(f"{source}: mixer type \"{kind}\" is not known "
                              "(known: attention, retention)")
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
                               "layers": list(self.layers)}
        if self.logit_softcap:
            doc["logit_softcap"] = self.logit_softcap
        if self.side_dim:
            doc["token_side"] = {"dim": self.side_dim}
        return doc

    # ------------------------------------------------------------------ the model as data
    @staticmethod
    def _positions(rot: Optional[Dict[str, Any]], positions: Dict[str, PartSpec]) -> str:
        """The name of the encoding with these constants (layers with equal ones share it)."""
        if not rot or not int(rot["dims"]):
            spec = PartSpec("none", {})
        else:
            spec = PartSpec("rope_half", {"theta": float(rot["base"]),
                                          "rot_dim": int(rot["dims"]), "rounding": "once"})
        for name, have in positions.items():
            if have == spec:
                return name
        name = f"rot{len(positions)}"
        positions[name] = spec
        return name

    def to_model_spec(self) -> ModelSpec:
        c = self
        positions: Dict[str, PartSpec] = {}
        layers: List[LayerSpec] = []
        schedule: List[Run] = []
        for i, layer in enumerate(c.layers):
            m, mlp = layer["mixer"], layer.get("mlp")
            dim = int(m["dim"])
            vdim = int(m.get("vdim") or dim)
            if layer["type"] == "attention":
                shared = m.get("kv_from") is not None
                names = {"q": "mix.q", "o": "mix.o", "g": "mix.g"}
                if not shared:
                    names.update({"k": "mix.k", "v": "mix.v"})
                mixer = PartSpec("gqa_attention", {
                    "hidden_size": c.width, "heads": int(m["heads"]),
                    "kv_heads": int(m.get("kv_heads") or m["heads"]), "head_dim": dim,
                    "v_dim": vdim, "scale": float(m["scale"]),
                    "softcap": float(m.get("softcap") or 0.0),
                    "head_norm": "unit_after_rotation", "head_norm_eps": c.norm_eps,
                    "shared_kv": shared, "position": c._positions(m.get("rot"), positions),
                    "names": names})
                schedule.append(Run(layer=i, cache_line=int(m["kv_from"]) if shared else i,
                                    writes_cache=not shared))
            else:
                mixer = PartSpec("retention", {
                    "hidden_size": c.width, "heads": int(m["heads"]), "dim": dim, "vdim": vdim,
                    "decay": [float(d) for d in m["decay"]], "eps": c.norm_eps,
                    "position": c._positions(m.get("rot"), positions),
                    "names": {"q": "mix.q", "k": "mix.k", "v": "mix.v", "g": "mix.g",
                              "o": "mix.o"}})
                schedule.append(Run(layer=i, cache_line=i, writes_cache=True))
            norm = lambda name: PartSpec("rmsnorm", {"name": name, "size": c.width,
                                                     "eps": c.norm_eps})
            norms = {"mixer": norm("norm1")}
            if mlp is None:
                ff = PartSpec("none")
            else:
                ff = PartSpec("mlp", {"hidden_size": c.width, "intermediate_size": int(mlp["ff"]),
                                      "activation": "relu_squared",
                                      "names": {"up": "mlp.up", "down": "mlp.down"}})
                norms["feed_forward"] = norm("norm2")
            params: Dict[str, Any] = {}
            if c.side_dim:
                params["side"] = {
                    "hidden_size": c.width, "dim": c.side_dim, "col0": i * c.side_dim,
                    "table_width": len(c.layers) * c.side_dim, "vocab_size": c.vocab,
                    "eps": c.norm_eps, "activation": "gelu_tanh",
                    "names": {"table": "side.embed", "gate": "side.gate", "proj": "side.proj",
                              "norm": "side.norm"}}
            layers.append(LayerSpec(block=PartSpec("output_norm_residual", params), mixer=mixer,
                                    feed_forward=ff, norms=norms, prefix=f"l{i}."))
        return ModelSpec(
            architecture=c.ARCHITECTURE, vocab_size=c.vocab, hidden_size=c.width,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"name": "embed", "vocab_size": c.vocab,
                                                   "hidden_size": c.width,
                                                   "scale": c.embedding_scale}),
            positions=positions, layers=tuple(layers), schedule=tuple(schedule),
            final_norm=PartSpec("rmsnorm", {"name": "final.norm", "size": c.width,
                                            "eps": c.norm_eps}),
            head=PartSpec("lm_head", {"name": "head", "tied": False, "vocab_size": c.vocab,
                                      "hidden_size": c.width, "softcap": c.logit_softcap}))
