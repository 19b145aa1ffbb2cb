"""Typed configuration of the Zazulix decoder, read from its own config.json keys.

config.json of this design is nested: `width`, `vocab`, `norm.eps` and a list `layers`, one entry per layer in running
order.  An entry has `type` (which mixer: latent_attention, attention or retention), `mixer` (that mixer's sizes and
constants) and `mlp` (null for none; `kind` dense with `ff` and `limit`, or `kind` moe with `expert.ff`, `router`
(`experts`, `top`, `scale`, `groups.count`, `groups.keep`) and `shared.ff`).  Every size and constant of a model stands
here and nowhere else in the package; what the design fixes for all of its models stands in the parts' parameters that
the model's builder sets.  A key that a layer may go without (`mask`, `rot`, `conv`, `kv_heads`, `vdim`, `groups`,
`shared`, the router's `scale`, `mlp`) is read as absent.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .base import ConfigError, ModelConfig, need_int, opt_float, opt_int
from .padodra import PadodraRotation, _need_dict, _need_float

MIXERS = ("latent_attention", "attention", "retention")


def _rotation(raw: dict, where: str, limit: int) -> Optional[PadodraRotation]:
    if raw.get("rot") is None:
        return None
    return PadodraRotation.from_dict(_need_dict(raw, "rot", where), where + "rot.", limit, ())


@dataclass
class ZazulixLatentAttention:
    """Attention over one cached vector of `kv_rank` numbers per token, without positions, over the last `window` tokens
    (0: all)."""
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int = 0

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "ZazulixLatentAttention":
        dim = need_int(raw, "dim")
        window = 0
        if raw.get("mask") is not None:
            window = need_int(_need_dict(raw, "mask", where), "size")
        return cls(need_int(raw, "heads"), dim, opt_int(raw, "vdim", dim), need_int(raw, "kv_rank"),
                   _need_float(raw, "scale", where), window)

    def to_dict(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass
class ZazulixAttention:
    """Differential attention: `heads` query heads of two maps of `dim` over `kv_heads` key/value heads; `conv` taps of
    the short convolutions (0: none); `diff` the constant in lambda and in the output's factor."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    conv: int = 0
    rot: Optional[PadodraRotation] = None

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "ZazulixAttention":
        heads, dim = need_int(raw, "heads"), need_int(raw, "dim")
        kv_heads = opt_int(raw, "kv_heads", heads)
        if heads % kv_heads:
            raise ConfigError(f"config.json {where}'heads' = {heads} is not a multiple of 'kv_heads' = {kv_heads}")
        return cls(heads, kv_heads, dim, opt_int(raw, "vdim", dim), _need_float(raw, "scale", where),
                   _need_float(raw, "diff", where), opt_int(raw, "conv", 0, minimum=1), _rotation(raw, where, dim))

    def to_dict(self) -> dict:
        d = {"diff": self.diff, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale,
             "vdim": self.vdim}
        if self.conv:
            d["conv"] = self.conv
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass
class ZazulixRetention:
    heads: int
    dim: int
    vdim: int
    decay: List[float]
    rot: Optional[PadodraRotation] = None

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "ZazulixRetention":
        heads, dim = need_int(raw, "heads"), need_int(raw, "dim")
        decay = raw.get("decay")
        if not isinstance(decay, list) or len(decay) != heads or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay):
            raise ConfigError(f"config.json {where}'decay' must be a list of {heads} numbers (one per head)")
        return cls(heads, dim, opt_int(raw, "vdim", dim), [float(x) for x in decay], _rotation(raw, where, dim))

    def to_dict(self) -> dict:
        d = {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


_MIXER_CLASSES = {"latent_attention": ZazulixLatentAttention, "attention": ZazulixAttention, "retention": ZazulixRetention}


@dataclass
class ZazulixMlp:
    """`kind` dense: `ff`, `limit`.  `kind` moe: `ff` is an expert's size, `experts`, `top`, `route_scale`, the groups
    (`group_count` 0: none) and `shared_ff` (0: no shared expert)."""
    kind: str
    ff: int
    limit: float = 0.0
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    group_count: int = 0
    group_keep: int = 0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "ZazulixMlp":
        kind = raw.get("kind")
        if kind == "dense":
            limit = _need_float(raw, "limit", where)
            if not limit > 0:
                raise ConfigError(f"config.json {where}'limit' = {limit} must be positive")
            return cls("dense", need_int(raw, "ff"), limit)
        if kind != "moe":
            raise ConfigError(f"config.json {where}'kind' = {kind!r} is not supported (supported: dense, moe)")
        r = _need_dict(raw, "router", where)
        experts, top = need_int(r, "experts"), need_int(r, "top")
        if top > experts:
            raise ConfigError(f"config.json {where}router.'top' = {top} exceeds 'experts' = {experts}")
        count = keep = 0
        if r.get("groups") is not None:
            g = _need_dict(r, "groups", where + "router.")
            count, keep = need_int(g, "count"), need_int(g, "keep")
            if experts % count or keep > count:
                raise ConfigError(f"config.json {where}router.'groups' = {count} (keep {keep}) does not divide the {experts} experts")
        shared = 0
        if raw.get("shared") is not None:
            shared = need_int(_need_dict(raw, "shared", where), "ff")
        return cls("moe", need_int(_need_dict(raw, "expert", where), "ff"), 0.0, experts, top, opt_float(r, "scale", 1.0),
                   count, keep, shared)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense", "limit": self.limit}
        r = {"experts": self.experts, "scale": self.route_scale, "top": self.top}
        if self.group_count:
            r["groups"] = {"count": self.group_count, "keep": self.group_keep}
        d = {"expert": {"ff": self.ff}, "kind": "moe", "router": r}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass
class ZazulixLayer:
    kind: str
    mixer: object
    mlp: Optional[ZazulixMlp]


@dataclass
class ZazulixConfig(ModelConfig):
    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-6
    layers: List[ZazulixLayer] = field(default_factory=list)
    initializer_range: float = 0.05

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: dict) -> "ZazulixConfig":
        width, vocab = need_int(raw, "width"), need_int(raw, "vocab")
        eps = _need_float(_need_dict(raw, "norm", ""), "eps", "norm.")
        if not eps > 0:
            raise ConfigError(f"config.json 'norm.eps' = {eps} must be positive")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json 'layers' must be a list with at least one layer")
        layers: List[ZazulixLayer] = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json layers[{i}] must be an object")
            kind = e.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"config.json {where}'type' = {kind!r} is not supported (supported: {', '.join(MIXERS)})")
            mixer = _MIXER_CLASSES[kind].from_dict(_need_dict(e, "mixer", where), where + "mixer.")
            mlp = None if e.get("mlp") is None else ZazulixMlp.from_dict(_need_dict(e, "mlp", where), where + "mlp.")
            layers.append(ZazulixLayer(kind, mixer, mlp))
        return cls(architecture="Zazulix", width=width, vocab=vocab, norm_eps=eps, layers=layers,
                   initializer_range=opt_float(raw, "initializer_range", 0.05))

    def to_dict(self) -> dict:
        out = [{"mixer": layer.mixer.to_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict(), "type": layer.kind}
               for layer in self.layers]
        return {"architecture": self.architecture, "layers": out, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                "width": self.width, "initializer_range": self.initializer_range}
