"""The Zazulix decoder put together from parts, by its configuration.

A layer is pre-norm (`PreNormBlock`): x <- x + mixer(N1(x)), x <- x + ff(N2(x)); every norm of the model multiplies by
1 + its stored weight (`RMSNorm(weight_offset=1)`).  The mixer is, layer by layer,

  * `latent_attention`: attention over one cached vector per token (`LatentAttention` without a rotated part), over a
    sliding window, with an element-wise sigmoid gate on the heads' outputs;
  * `attention`: a differential attention (`DifferentialAttention`: two score maps per head over the same values, short
    convolutions behind the projections, rotation of the first `rot.dims` dims of every map in halves, a weightless norm
    per head and one gate number per head);
  * `retention`: linear attention with a fixed decay per head (`Retention`).

The feed-forward is dense with the clamped activation (`SwiGLUFeedForward(act="swish_clamped")`, slope 1.702), a mixture
of experts (`RoutedFeedForward` with sigmoid scores, a correction for the choice alone, groups of experts, weights over
their sum + 1e-20 times the router's factor, and a shared expert behind a gate of one number per token), or absent.
The logits come from the embedding table behind the final norm.  Tensor names: `embed`, `l<i>.norm1|norm2`,
`l<i>.mix.*`, `l<i>.mlp.*` (`e<j>.`, `shared.`, `router`, `correction`), `final.norm`.
"""
from __future__ import annotations

from ..config import ZazulixConfig, register_architecture
from ..parts import (DifferentialAttention, LatentAttention, OutputHead, PreNormBlock, RMSNorm, Retention, RotaryEmbedding,
                     RoutedFeedForward, SwiGLUFeedForward, TokenEmbedding)
from .spec import ModelSpec

SWISH_SLOPE = 1.702         # the sigmoid's slope in the dense feed-forward's activation
ROUTE_NORM_EPS = 1e-20      # added to the sum of the chosen experts' scores
GLU_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def _rotation(rot, positions: int, made: dict):
    if rot is None:
        return None
    key = (rot.base, rot.dims)
    if key not in made:
        made[key] = RotaryEmbedding(rot.base, rot.dims, positions, pairing="half")
    return made[key]


def _norm(d: int, eps: float, name: str) -> RMSNorm:
    return RMSNorm(d, eps, name, weight_offset=1.0)


def _feed_forward(d: int, mlp, prefix: str):
    if mlp.kind == "dense":
        return SwiGLUFeedForward(d, mlp.ff, prefix, act="swish_clamped", names=GLU_NAMES, limit=mlp.limit, slope=SWISH_SLOPE)
    shared = SwiGLUFeedForward(d, mlp.shared_ff, prefix + "shared.", names=GLU_NAMES) if mlp.shared_ff else None
    return RoutedFeedForward(d, mlp.ff, mlp.experts, mlp.top, prefix, scores="sigmoid", correction=True,
                             groups=mlp.group_count, keep=mlp.group_keep, weight_scale=mlp.route_scale,
                             norm_eps=ROUTE_NORM_EPS, shared=shared, shared_gated=shared is not None)


def build_zazulix(cfg: ZazulixConfig, max_positions: int = 0) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    positions = max(int(max_positions), 1)
    ropes: dict = {}
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.kind == "latent_attention":
            mixer = LatentAttention(d, m.heads, m.dim, 0, m.vdim, m.kv_rank, p + "mix.", eps, m.scale, gate=True,
                                    window=m.window or None)
        elif layer.kind == "attention":
            mixer = DifferentialAttention(d, m.heads, m.kv_heads, m.dim, m.vdim, p + "mix.", m.diff, eps, scale=m.scale,
                                          position=_rotation(m.rot, positions, ropes), taps=m.conv)
        else:
            mixer = Retention(d, m.heads, m.dim, m.vdim, m.decay, p + "mix.", eps, position=_rotation(m.rot, positions, ropes))
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn, ffn_norm = _feed_forward(d, layer.mlp, p + "mlp."), _norm(d, eps, p + "norm2")
        blocks.append(PreNormBlock(_norm(d, eps, p + "norm1"), mixer, ffn_norm, ffn))
    embedding = TokenEmbedding(cfg.vocab, d, "embed")
    head = OutputHead(d, cfg.vocab, _norm(d, eps, "final.norm"), "head", tied_to="embed")
    return ModelSpec(cfg, embedding, blocks, head)


register_architecture("Zazulix", ZazulixConfig, build_zazulix, "zazulix")
