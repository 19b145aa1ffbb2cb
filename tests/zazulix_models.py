"""Tiny Zazulix configurations for the tests: every mixer and feed-forward, layers in several orders, with and without
the keys a layer may go without (window, rotation, convolution, groups, shared expert, feed-forward), and sizes chosen
so that nothing that could be confused is equal (heads and key/value heads, key and value size, rotated and whole map
size, experts and groups) or happens to be 1 by accident.  The convolutions' taps are made larger than the other
weights, so that the attention behind them is not flat."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import helpers


def latent(heads, dim, vdim, kv_rank, scale, window=None):
    m = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "scale": scale, "vdim": vdim}
    if window:
        m["mask"] = {"size": window}
    return m


def attention(heads, kv_heads, dim, vdim, scale, diff, conv=None, rot=None):
    m = {"diff": diff, "dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if conv:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = rot
    return m


def retention(heads, dim, vdim, decay, rot=None):
    m = {"decay": decay, "dim": dim, "heads": heads, "vdim": vdim}
    if rot is not None:
        m["rot"] = rot
    return m


def dense(ff, limit):
    return {"ff": ff, "kind": "dense", "limit": limit}


def moe(ff, experts, top, scale, groups=None, shared=None):
    r = {"experts": experts, "scale": scale, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"expert": {"ff": ff}, "kind": "moe", "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(width, vocab, eps, layers, std):
    return {"architecture": "Zazulix", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers,
            "initializer_range": std}


CONFIGS = {
    # cache rows of 16 numbers (the tensor-core decode kernels' smallest head); a window shorter than a page run; an
    # attention without convolution and with as many key/value heads as heads; a layer without feed-forward
    "A": config(48, 131, 1e-6, [
        layer("attention", attention(4, 2, 8, 16, 0.3, 0.3, conv=3, rot={"base": 900.0, "dims": 4}), moe(24, 6, 2, 1.5, (3, 2), 40)),
        layer("retention", retention(3, 8, 12, [0.9, 0.97, 0.995], rot={"base": 10000.0, "dims": 8}), dense(40, 1.0)),
        layer("latent_attention", latent(3, 8, 12, 16, 0.35, window=7), moe(16, 5, 3, 0.8)),
        layer("attention", attention(2, 2, 12, 10, 0.25, 0.6), None),
    ], 0.12),
    # a cache row of 24 numbers and values wider than two maps (no tensor-core kernel takes either); groups of three
    # experts of which two are kept; a shared expert; a convolution of four taps without rotation
    "B": config(64, 200, 1e-5, [
        layer("latent_attention", latent(2, 16, 8, 24, 0.2, window=33), dense(72, 0.8)),
        layer("retention", retention(2, 24, 8, [0.96, 0.999], rot={"base": 50000.0, "dims": 12}), moe(24, 9, 3, 2.0, (3, 2))),
        layer("attention", attention(6, 2, 16, 40, 0.2, 0.45, conv=4), moe(32, 8, 2, 1.0, (4, 1), 48)),
        layer("retention", retention(4, 8, 16, [0.5, 0.9, 0.99, 1.0]), dense(48, 2.5)),
    ], 0.1),
    # the tensor-core kernels' sizes: cache rows of 64 numbers with groups of four and eight query heads, a cache row of
    # 144 numbers (the wide latent kernel), retention heads of 64; all experts chosen; every group kept
    "C": config(128, 300, 1e-5, [
        layer("attention", attention(2, 1, 32, 64, 0.18, 0.4, conv=2, rot={"base": 20000.0, "dims": 16}), moe(40, 4, 4, 1.3, (2, 2), 64)),
        layer("latent_attention", latent(8, 32, 48, 64, 0.2, window=37), dense(160, 1.2)),
        layer("retention", retention(2, 64, 64, [0.97, 0.998], rot={"base": 500000.0, "dims": 32}), moe(40, 6, 2, 1.0, (2, 1), 24)),
        layer("latent_attention", latent(4, 16, 48, 144, 0.25), moe(40, 6, 2, 1.0, (3, 1))),
    ], 0.08),
    # sizes that no vector load divides: a width of 8 * 5, an odd vocabulary, maps of 6 with 2 rotated dims, one tap, a
    # latent of 10, groups of one expert, one expert per token, no window
    "D": config(40, 103, 1e-6, [
        layer("retention", retention(3, 10, 6, [0.8, 0.9, 0.95]), moe(12, 6, 1, 2.5, (6, 2), 20)),
        layer("attention", attention(3, 1, 6, 10, 0.4, 0.2, conv=1, rot={"base": 100.0, "dims": 2}), dense(30, 0.7)),
        layer("latent_attention", latent(5, 6, 10, 10, 0.4), None),
        layer("attention", attention(1, 1, 20, 14, 0.2, 0.5, conv=2, rot={"base": 3000.0, "dims": 20}), moe(20, 3, 2, 1.0)),
    ], 0.15),
}
SEEDS = {"A": 41, "B": 42, "C": 43, "D": 44}
SHARPEN = {".conv": 6.0, ".correction": 2.0}       # factors on the tensors whose names end so


def make_model_dir(tmpdir, which: str, dtype=torch.float32) -> str:
    """Seeded random weights of configuration `which` with the convolutions' taps and the routers' corrections made
    larger; matrices stored as `dtype`."""
    from hk_b200.config import config_from_dict, resolve_architecture
    from hk_b200.weights import random_tensors
    from hk_b200.weights.safetensors_io import save_file
    raw = CONFIGS[which]
    cfg = config_from_dict(raw)
    _, build = resolve_architecture(cfg.architecture)
    specs = build(cfg, 8).param_specs()
    tensors = random_tensors(specs, SEEDS[which], raw["initializer_range"], 0.1, "cuda" if torch.cuda.is_available() else "cpu",
                             dtype_of=lambda s: torch.float32 if s.kind == "vector" else dtype)
    tensors = {k: v.cpu() for k, v in tensors.items()}
    for name in tensors:
        for ending, factor in SHARPEN.items():
            if name.endswith(ending):
                tensors[name] = tensors[name] * factor
    d = os.path.join(str(tmpdir), f"zazulix_{which}_{str(dtype).split('.')[-1]}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg.to_dict(), f, indent=1)
    save_file(tensors, os.path.join(d, "model.safetensors"))
    return d


def prompts(which: str, rng: np.random.Generator, lengths):
    return [rng.integers(0, CONFIGS[which]["vocab"], n).tolist() for n in lengths]


def routed_prefixes(cfg: dict):
    """The tensor prefixes of the routed feed-forwards, in running order."""
    return [f"l{i}.mlp." for i, e in enumerate(cfg["layers"]) if e.get("mlp") and e["mlp"]["kind"] == "moe"]


load_plain = helpers.load_plain
