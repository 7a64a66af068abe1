"""Small Sezopel configurations for the tests, their random model folders and the plain
implementation's view of them.

P: an input from the token after every layer, an embedding scale, capped logits; attention with
   value rows of another size than its keys, heads only partly rotated, capped scores, two
   later layers that read the first layer's keys and values; retention with slow decays, a full
   rotation and more key than value channels; a layer without a feed-forward.
Q: none of the options (no token input, no scale, no caps, no rotation in the attention, as
   many key/value heads as heads, value rows as large as keys); a single head; sizes that are
   not multiples of four; retention first, partly rotated, with a decay of exactly one.
R: sizes that the tensor-core kernels take (heads of 64 values that rotate as a whole,
   multiples of 32); retention between two attention layers; a shared cache line read by the
   last layer; decays close to one.
S: heads of 128 values on one key/value head, a head count that is no power of two, retention
   heads of 128 x 64.
"""
import json
import os

import numpy as np


def _att(heads, dim, scale, kv=None, vdim=None, rot=None, softcap=None, kv_from=None, ff=None):
    m = {"heads": heads, "dim": dim, "scale": scale}
    if kv is not None:
        m["kv_heads"] = kv
    if vdim is not None:
        m["vdim"] = vdim
    if rot is not None:
        m["rot"] = rot
    if softcap is not None:
        m["softcap"] = softcap
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _ret(heads, dim, decay, vdim=None, rot=None, ff=None):
    m = {"heads": heads, "dim": dim, "decay": decay}
    if vdim is not None:
        m["vdim"] = vdim
    if rot is not None:
        m["rot"] = rot
    return {"type": "retention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _p():
    rot = {"base": 1e4, "dims": 16}
    return {"architecture": "Sezopel", "vocab": 211, "width": 80, "norm": {"eps": 1e-5},
            "embedding": {"scale": 5.0}, "logit_softcap": 9.0, "token_side": {"dim": 12},
            "layers": [
                _att(4, 24, 2.5, kv=2, vdim=40, rot=rot, softcap=7.0, ff=96),
                _att(4, 24, 1.5, kv=2, vdim=40, rot=rot, softcap=3.0, kv_from=0, ff=72),
                _ret(3, 20, [0.9, 0.99, 0.999], vdim=12, rot={"base": 500.0, "dims": 20}, ff=56),
                _att(4, 24, 4.0, kv=2, vdim=40, rot=rot, softcap=20.0, kv_from=0),
                _ret(2, 8, [0.5, 0.97], vdim=36, rot={"base": 1e5, "dims": 4})]}


def _q():
    return {"architecture": "Sezopel", "vocab": 130, "width": 50, "norm": {"eps": 1e-6},
            "layers": [
                _ret(1, 10, [1.0], rot={"base": 300.0, "dims": 6}, ff=34),
                _att(3, 10, 3.0, ff=18),
                _att(1, 14, 6.0, vdim=6, rot={"base": 77.0, "dims": 14}),
                _ret(5, 6, [0.8, 0.9, 0.95, 0.99, 0.999], vdim=9, ff=22)]}


def _r():
    rot = {"base": 5e5, "dims": 64}
    return {"architecture": "Sezopel", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
            "embedding": {"scale": 8.0}, "logit_softcap": 30.0, "token_side": {"dim": 32},
            "layers": [
                _att(4, 64, 3.0, kv=1, rot=rot, softcap=10.0, ff=256),
                _ret(2, 64, [0.99, 0.9995], rot={"base": 1e6, "dims": 64}, ff=128),
                _att(4, 64, 5.0, kv=1, rot=rot, softcap=4.0, kv_from=0, ff=192)]}


def _s():
    rot = {"base": 1e4, "dims": 128}
    return {"architecture": "Sezopel", "vocab": 190, "width": 192, "norm": {"eps": 1e-6},
            "embedding": {"scale": 3.0}, "token_side": {"dim": 8},
            "layers": [
                _att(3, 128, 6.0, kv=1, rot=rot, softcap=15.0, ff=160),
                _ret(2, 128, [0.98, 0.998], vdim=64, rot={"base": 1e4, "dims": 32}, ff=96),
                _att(3, 128, 2.0, kv=1, rot=rot, kv_from=0)]}


SMALL = {"P": _p, "Q": _q, "R": _r, "S": _s}

# name -> (seed, std of matrices, prompt lengths of the whole-prompt tests, decode steps)
HOW = {"P": (31, 0.12, [1, 9, 64, 150], 9), "Q": (32, 0.15, [2, 63, 65, 131], 7),
       "R": (33, 0.09, [5, 128, 200], 6), "S": (34, 0.08, [3, 130], 5)}


def small_doc(name):
    return SMALL[name]()


class SmallModel:
    def __init__(self, name, folder):
        from mormot2_ai_b200 import SezopelConfig, write_random_model
        from tests.plain import sezopel_plain as plain
        from tests.plain.qwen3_plain import read_safetensors
        self.name, self.doc = name, small_doc(name)
        self.seed, std, self.prompt_lens, self.decode_steps = HOW[name]
        self.config = SezopelConfig.from_dict(self.doc)
        self.folder = write_random_model(folder, self.config, self.seed, std=std, norm_std=0.2)
        with open(os.path.join(folder, "config.json")) as f:
            self.plain_config = json.load(f)
        self.weights = {k: np.asarray(v, dtype=np.float64)
                        for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
        self.plain = plain

    def tokens(self, n, seed=0):
        rng = np.random.default_rng(1000 * self.seed + seed)
        return rng.integers(0, self.doc["vocab"], n).tolist()

    def reference(self, ids, states=None):
        return self.plain.forward(self.plain_config, self.weights, ids, states)

    def rounded(self, ids, dtype="bfloat16"):
        """The plain logits with everything that a 16-bit run keeps in 16 bits rounded so (None
        for float32): how far rounding alone moves them."""
        if dtype != "bfloat16":
            return None
        return self.plain.forward(self.plain_config, self.weights, ids, rnd=self.plain.bfloat16)
