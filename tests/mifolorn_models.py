"""Tiny Mifolorn configurations for the tests: every mixer, layers with and without a feed-forward, models with and
without a loop, a per-layer token input, a soft cap and frequency scaling, and sizes chosen so that nothing that could
be confused is equal (heads and query/key heads, key and value size, rotated and whole head size, taps) or happens to
be 1 by accident."""
from __future__ import annotations

import os

import numpy as np
import torch

import helpers


def attention(heads, kv_heads, dim, vdim, scale, rot=None, softcap=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if rot is not None:
        m["rot"] = rot
    if softcap:
        m["softcap"] = softcap
    return m


def delta(heads, kv_heads, dim, vdim, conv):
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}


def mlstm(heads, dim, vdim, cap):
    return {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def parallel(left, right, left_scale, right_scale):
    return {"left": left, "left_scale": left_scale, "right": right, "right_scale": right_scale}


def config(width, vocab, eps, layers, std, scale=1.0, side=0, loop=None):
    c = {"architecture": "Mifolorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": scale},
         "layers": layers, "initializer_range": std}
    if side:
        c["token_side"] = {"dim": side}
    if loop:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}

CONFIGS = {
    # a loop over the two middle layers, three passes; a token input; partly rotated heads with frequency scaling and a cap
    "U": config(48, 131, 1e-6, [
        layer("delta", delta(3, 3, 16, 8, 2), 40),
        layer("parallel", parallel(attention(4, 2, 16, 16, 0.3, {"base": 900.0, "dims": 8, "scaling": YARN}, 20.0),
                                   delta(2, 1, 8, 12, 3), 0.7, 1.3), 56),
        layer("mlstm", mlstm(2, 8, 12, 8.0), None),
        layer("delta", delta(4, 2, 8, 20, 5), 24),
    ], 0.12, scale=3.0, side=6, loop=(1, 3, 3)),
    # no loop, no token input, no cap, rotation of the whole head without scaling, values narrower than keys
    "V": config(64, 200, 1e-5, [
        layer("mlstm", mlstm(3, 16, 8, 15.0), 72),
        layer("parallel", parallel(attention(2, 2, 32, 24, 0.2, {"base": 10000.0, "dims": 32}),
                                   delta(1, 1, 64, 16, 4), 1.0, 0.5), None),
        layer("delta", delta(2, 2, 24, 24, 3), 48),
    ], 0.1),
    # heads of 64 with three query heads per key head (the tensor-core attention's shapes), the whole model twice
    "W": config(128, 300, 1e-5, [
        layer("parallel", parallel(attention(3, 1, 64, 64, 0.125, {"base": 20000.0, "dims": 32, "scaling": YARN}, 30.0),
                                   delta(4, 2, 32, 16, 4), 0.9, 1.2), 160),
        layer("mlstm", mlstm(2, 32, 64, 10.0), 96),
    ], 0.08, scale=2.0, side=16, loop=(0, 2, 2)),
    # sizes that no vector load divides: a width of 8 * 5, feed-forwards of 4 * 13 and 2 * 15, a token input of 5, an odd
    # vocabulary, six rotated dims, key and value sizes of 12 / 10 / 20 / 28 / 36, a head wider than 128, a convolution of
    # one tap; the loop covers the first two layers and the last layer has no feed-forward
    "X": config(40, 103, 1e-6, [
        layer("parallel", parallel(attention(3, 1, 24, 40, 0.25, {"base": 10000.0, "dims": 6, "scaling": YARN}, 10.0),
                                   delta(3, 1, 20, 28, 3), 1.0, 1.0), 52),
        layer("mlstm", mlstm(3, 20, 36, 6.0), 30),
        layer("delta", delta(6, 2, 12, 10, 2), 44),
        layer("parallel", parallel(attention(2, 2, 136, 72, 0.09, {"base": 3000.0, "dims": 136, "scaling": YARN}, 60.0),
                                   delta(1, 1, 72, 40, 1), 2.0, 0.25), None),
    ], 0.15, scale=3.0, side=5, loop=(0, 2, 2)),
}
SEEDS = {"U": 31, "V": 32, "W": 33, "X": 34}


def make_model_dir(tmpdir, which: str, dtype=torch.float32) -> str:
    from hk_b200.config import config_from_dict
    from hk_b200.weights import write_random_model
    raw = CONFIGS[which]
    d = os.path.join(str(tmpdir), f"mifolorn_{which}_{str(dtype).split('.')[-1]}")
    write_random_model(d, config_from_dict(raw), SEEDS[which], std=raw["initializer_range"], norm_std=0.1, dtype=dtype)
    return d


def prompts(which: str, rng: np.random.Generator, lengths):
    return [rng.integers(0, CONFIGS[which]["vocab"], n).tolist() for n in lengths]


load_plain = helpers.load_plain
