"""Small Laralix configurations for the tests, their random model folders and the plain
implementation's view of them.

A: a loop of two passes over the first two layers; sizes that are no multiples of four; fewer
   rotating values than the rotated part; key/value groups; a window that decoding passes;
   kept first positions; a convolution of four taps.
B: no loop, no embedding scale, no logit factor, no cap, no window in the first layer; one head;
   as many key/value heads as heads; a convolution of two taps; a layer without feed-forward;
   a kept prefix longer than the window.
C: sizes that the tensor-core kernels take (heads of 64, multiples of 32); a loop of three
   passes over the last two layers; windows longer than a page.
D: heads of 128 values; states of 128 x 128; a latent of 128 values; a single pass "loop".
"""
import json
import os

import numpy as np


def _ff(ff):
    return {"kind": "dense", "ff": ff} if ff else None


def _par(heads, kv, dim, vdim, scale, size, rheads, rkv, rdim, rvdim, conv, softcap=None, ff=None):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        left["mask"] = {"size": size}
    if softcap:
        left["softcap"] = softcap
    right = {"heads": rheads, "kv_heads": rkv, "dim": rdim, "vdim": rvdim, "conv": conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": _ff(ff)}


def _par2(heads, kv, dim, scale, size, keep, rheads, rdim, rvdim, tau, ls, rs, ff=None, rank=5):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
            "mask": {"size": size, "keep_first": keep}}
    right = {"heads": rheads, "dim": rdim, "vdim": rvdim, "tau": tau, "rank": rank}
    return {"type": "parallel_2", "mixer": {"left": left, "right": right, "left_scale": ls,
                                            "right_scale": rs}, "mlp": _ff(ff)}


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base, dims, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                      "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                      "rot": {"base": base, "dims": dims}}, "mlp": _ff(ff)}


def _a():
    return {"architecture": "Laralix", "vocab": 150, "width": 72, "norm": {"eps": 1e-5},
            "embedding": {"scale": 6.0}, "logit_scale": 0.25,
            "loop": {"start": 0, "stop": 2, "times": 2},
            "layers": [
                _par(4, 2, 18, 10, 0.3, 21, 4, 2, 10, 14, 4, softcap=6.0, ff=90),
                _lat(3, 10, 8, 14, 22, 26, 0.2, 500.0, 6, ff=50),
                _par2(6, 3, 12, 0.25, 19, 5, 2, 14, 6, 8.0, 0.7, 1.2, ff=66)]}


def _b():
    return {"architecture": "Laralix", "vocab": 97, "width": 40, "norm": {"eps": 1e-6},
            "layers": [
                _par2(1, 1, 20, 0.2, 9, 13, 3, 6, 10, 3.0, 1.0, 0.5, ff=44),
                _par(2, 2, 12, 12, 0.35, 0, 1, 1, 16, 8, 2),
                _lat(1, 14, 6, 8, 10, 12, 0.3, 50.0, 6, ff=30)]}


def _c():
    return {"architecture": "Laralix", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
            "embedding": {"scale": 8.0}, "logit_scale": 2.0,
            "loop": {"start": 1, "stop": 3, "times": 3},
            "layers": [
                _lat(4, 32, 32, 64, 96, 64, 0.125, 1e5, 32, ff=192),
                _par(4, 2, 64, 64, 0.125, 70, 2, 1, 64, 64, 3, softcap=20.0, ff=256),
                _par2(4, 1, 64, 0.1, 72, 9, 2, 32, 64, 12.0, 0.9, 0.6, ff=160)]}


def _d():
    return {"architecture": "Laralix", "vocab": 200, "width": 192, "norm": {"eps": 1e-6},
            "embedding": {"scale": 4.0}, "loop": {"start": 0, "stop": 3, "times": 1},
            "layers": [
                _par(3, 1, 128, 128, 0.09, 100, 2, 2, 128, 128, 3, softcap=40.0, ff=224),
                _par2(2, 2, 128, 0.08, 66, 70, 2, 128, 64, 20.0, 1.1, 0.4, ff=128),
                _lat(2, 64, 64, 128, 128, 96, 0.09, 1e4, 64)]}


SMALL = {"A": _a, "B": _b, "C": _c, "D": _d}

# name -> (seed, std of matrices, prompt lengths of the whole-prompt tests, decode steps)
HOW = {"A": (41, 0.12, [1, 9, 64, 150], 9), "B": (42, 0.16, [2, 63, 65, 131], 7),
       "C": (43, 0.09, [5, 128, 200], 6), "D": (44, 0.07, [3, 130], 5)}


def small_doc(name):
    return SMALL[name]()


class SmallModel:
    def __init__(self, name, folder):
        from mormot2_ai_b200 import LaralixConfig, write_random_model
        from tests.plain import laralix_plain as plain
        from tests.plain.qwen3_plain import read_safetensors
        self.name, self.doc = name, small_doc(name)
        self.seed, std, self.prompt_lens, self.decode_steps = HOW[name]
        self.config = LaralixConfig.from_dict(self.doc)
        self.folder = write_random_model(folder, self.config, self.seed, std=std, norm_std=0.2)
        with open(os.path.join(folder, "config.json")) as f:
            self.plain_config = json.load(f)
        self.weights = {k: np.asarray(v, dtype=np.float64)
                        for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}
        self.plain = plain
        self.runs = len(plain.layer_runs(self.plain_config))

    def tokens(self, n, seed=0):
        rng = np.random.default_rng(1000 * self.seed + seed)
        return rng.integers(0, self.doc["vocab"], n).tolist()

    def reference(self, ids, states=None):
        return self.plain.forward(self.plain_config, self.weights, ids, states=states)

    def rounded(self, ids, dtype="bfloat16"):
        """The plain logits with everything that a 16-bit run keeps in 16 bits rounded so (None
        for float32): how far rounding alone moves them."""
        if dtype != "bfloat16":
            return None
        return self.plain.forward(self.plain_config, self.weights, ids, rnd=self.plain.bfloat16)
