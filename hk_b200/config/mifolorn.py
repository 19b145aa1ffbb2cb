"""Typed configuration of the Mifolorn decoder, read from its own config.json keys.

config.json of this design is nested: `width`, `vocab`, `norm.eps`, `embedding.scale`, `token_side.dim` (the size of
the per-layer token input; absent: the layers have none), `loop` (`start`, `stop`, `times`: layers start .. stop - 1
run `times` times in a row with the same tensors; absent: every layer runs once) and a list `layers`, one entry per
layer.  An entry has `type` (mlstm, delta or parallel), `mixer` (that mixer's sizes and constants; for `parallel` the
two sides under `left` and `right` with `left_scale` and `right_scale`) and `mlp` (null for none; `kind` dense with
`ff`).  Every size and constant of a model stands here and nowhere else in the package; what the design fixes for all
of its models stands in the parts and in the model's builder.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .base import ConfigError, ModelConfig, need_int, opt_float, opt_int
from .padodra import PadodraMlp, PadodraRotation, _need_dict, _need_float, _opt_positive

MIXERS = ("mlstm", "delta", "parallel")


@dataclass
class MifolornAttention:
    """The softmax side of a parallel mixer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0                        # 0: none
    rot: Optional[PadodraRotation] = None

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "MifolornAttention":
        heads, dim = need_int(raw, "heads"), need_int(raw, "dim")
        kv_heads = opt_int(raw, "kv_heads", heads)
        if heads % kv_heads:
            raise ConfigError(f"config.json {where}'heads' = {heads} is not a multiple of 'kv_heads' = {kv_heads}")
        rot = None
        if raw.get("rot") is not None:
            rot = PadodraRotation.from_dict(_need_dict(raw, "rot", where), where + "rot.", dim,
                                            ("factor", "original", "fast", "slow"))
        return cls(heads, kv_heads, dim, opt_int(raw, "vdim", dim), _need_float(raw, "scale", where),
                   _opt_positive(raw, "softcap", where), rot)

    def to_dict(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass
class MifolornDelta:
    """A gated delta rule: `kv_heads` query/key heads of `dim` serve `heads` value heads of `vdim`; `conv` taps."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "MifolornDelta":
        heads, dim = need_int(raw, "heads"), need_int(raw, "dim")
        kv_heads = opt_int(raw, "kv_heads", heads)
        if heads % kv_heads:
            raise ConfigError(f"config.json {where}'heads' = {heads} is not a multiple of 'kv_heads' = {kv_heads}")
        return cls(heads, kv_heads, dim, opt_int(raw, "vdim", dim), need_int(raw, "conv", minimum=1))

    def to_dict(self) -> dict:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}


@dataclass
class MifolornMLSTM:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "MifolornMLSTM":
        cap = _need_float(raw, "gate_cap", where)
        if not cap > 0:
            raise ConfigError(f"config.json {where}'gate_cap' = {cap} must be positive")
        dim = need_int(raw, "dim")
        return cls(need_int(raw, "heads"), dim, opt_int(raw, "vdim", dim), cap)

    def to_dict(self) -> dict:
        return {"dim": self.dim, "gate_cap": self.gate_cap, "heads": self.heads, "vdim": self.vdim}


@dataclass
class MifolornParallel:
    left: MifolornAttention
    right: MifolornDelta
    left_scale: float = 1.0
    right_scale: float = 1.0

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "MifolornParallel":
        return cls(MifolornAttention.from_dict(_need_dict(raw, "left", where), where + "left."),
                   MifolornDelta.from_dict(_need_dict(raw, "right", where), where + "right."),
                   opt_float(raw, "left_scale", 1.0), opt_float(raw, "right_scale", 1.0))

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "left_scale": self.left_scale, "right": self.right.to_dict(),
                "right_scale": self.right_scale}


_MIXER_CLASSES = {"mlstm": MifolornMLSTM, "delta": MifolornDelta, "parallel": MifolornParallel}


@dataclass
class MifolornLayer:
    kind: str
    mixer: object
    mlp: Optional[PadodraMlp]


@dataclass
class MifolornLoop:
    start: int
    stop: int
    times: int


@dataclass
class MifolornConfig(ModelConfig):
    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    side_dim: int = 0                           # 0: no per-layer token input
    loop: Optional[MifolornLoop] = None
    layers: List[MifolornLayer] = field(default_factory=list)
    initializer_range: float = 0.05

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: dict) -> "MifolornConfig":
        width, vocab = need_int(raw, "width"), need_int(raw, "vocab")
        eps = _need_float(_need_dict(raw, "norm", ""), "eps", "norm.")
        if not eps > 0:
            raise ConfigError(f"config.json 'norm.eps' = {eps} must be positive")
        emb_scale = 1.0
        if raw.get("embedding") is not None:
            emb_scale = opt_float(_need_dict(raw, "embedding", ""), "scale", 1.0)
        side_dim = 0
        if raw.get("token_side") is not None:
            side_dim = need_int(_need_dict(raw, "token_side", ""), "dim")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json 'layers' must be a list with at least one layer")
        layers: List[MifolornLayer] = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json layers[{i}] must be an object")
            kind = e.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"config.json {where}'type' = {kind!r} is not supported (supported: {', '.join(MIXERS)})")
            mixer = _MIXER_CLASSES[kind].from_dict(_need_dict(e, "mixer", where), where + "mixer.")
            mlp = None if e.get("mlp") is None else PadodraMlp.from_dict(_need_dict(e, "mlp", where), where + "mlp.")
            layers.append(MifolornLayer(kind, mixer, mlp))
        loop = None
        if raw.get("loop") is not None:
            lp = _need_dict(raw, "loop", "")
            loop = MifolornLoop(need_int(lp, "start", minimum=0), need_int(lp, "stop", minimum=0), need_int(lp, "times"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"config.json 'loop' = {loop.start}..{loop.stop} does not lie within the {len(layers)} layers")
        return cls(architecture="Mifolorn", width=width, vocab=vocab, norm_eps=eps, embedding_scale=emb_scale,
                   side_dim=side_dim, loop=loop, layers=layers, initializer_range=opt_float(raw, "initializer_range", 0.05))

    def to_dict(self) -> dict:
        out = [{"mixer": layer.mixer.to_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict(), "type": layer.kind}
               for layer in self.layers]
        d = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": out,
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width,
             "initializer_range": self.initializer_range}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return d
