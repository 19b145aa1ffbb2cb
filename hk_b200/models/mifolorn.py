"""The Mifolorn decoder put together from parts, by its configuration.

A layer is pre-norm (`PreNormBlock`): x <- x + mixer(N1(x)), x <- x + ff(N2(x)), and then, where the model has a
per-layer token input, x <- x + side(x) (`TokenSideInput`, the layer's own slice of the table `side.embed`).  The
mixer is, layer by layer,

  * `mlstm`: a matrix memory with exponential gates (`MLSTM`);
  * `delta`: a gated delta rule behind short convolutions (`GatedDeltaRule`);
  * `parallel`: a grouped-query attention (`GQAAttention`: biases on q, k and v, a weighted per-head norm of q and k
    before the rotation, rotation of the first `rot.dims` dims in halves with YaRN frequency scaling and magnitude, a
    soft cap on the scores, plain causal softmax, an output gate) beside a gated delta rule, both reading the same
    input, summed with a factor each (`ParallelMixer`).

The feed-forward is a SwiGLU or absent.  The embedding is multiplied by `embedding.scale`; the logits come from the
embedding table itself (without that factor) behind the final norm.  `loop`: the layers start .. stop - 1 run `times`
times in a row with the same tensors, every run with caches and states of its own, and before every pass but the first
the embedding's output is added to the stream (`LayerCall.add_embedding`).  Tensor names: `embed`, `side.embed`,
`l<i>.norm1|norm2`, `l<i>.mix.*` (`l<i>.mix.left.*`, `l<i>.mix.right.*`), `l<i>.mlp.*`, `l<i>.side.*`, `final.norm`.
"""
from __future__ import annotations

from ..config import MifolornConfig, register_architecture
from ..parts import (GQAAttention, GatedDeltaRule, MLSTM, OutputHead, ParallelMixer, PreNormBlock, RMSNorm, RopeScaling,
                     RotaryEmbedding, SwiGLUFeedForward, TokenEmbedding, TokenSideInput)
from .spec import LayerCall, ModelSpec


def _rotation(rot, positions: int, made: dict):
    if rot is None:
        return None
    s = rot.scaling
    key = (rot.base, rot.dims, tuple(sorted(s.items())))
    if key not in made:
        scaling = None
        if s:
            scaling = RopeScaling("yarn", factor=s["factor"], orig_ctx=s["original"], beta_fast=s["fast"], beta_slow=s["slow"])
        made[key] = RotaryEmbedding(rot.base, rot.dims, positions, pairing="half", scaling=scaling)
    return made[key]


def _attention(d, m, prefix, eps, positions, ropes):
    return GQAAttention(d, m.heads, m.kv_heads, m.dim, prefix, qk_norm_eps=eps, position=_rotation(m.rot, positions, ropes),
                        scale=m.scale, qkv_bias=True, v_head_dim=m.vdim, softcap=m.softcap or None, gate=True,
                        names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g",
                               "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"})


def _delta(d, m, prefix, eps, out_scale=1.0):
    return GatedDeltaRule(d, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, prefix, norm_eps=eps, out_scale=out_scale)


def layer_calls(n_layers: int, loop) -> list:
    """The schedule of a model whose layers start .. stop - 1 run `times` times."""
    if loop is None or loop.stop <= loop.start:
        return [LayerCall(i) for i in range(n_layers)]
    calls = [LayerCall(i) for i in range(loop.start)]
    for r in range(loop.times):
        calls += [LayerCall(i, add_embedding=(r > 0 and i == loop.start)) for i in range(loop.start, loop.stop)]
    return calls + [LayerCall(i) for i in range(loop.stop, n_layers)]


def build_mifolorn(cfg: MifolornConfig, max_positions: int = 0) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    positions = max(int(max_positions), 1)
    ropes: dict = {}
    blocks = []
    n = len(cfg.layers)
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.kind == "mlstm":
            mixer = MLSTM(d, m.heads, m.dim, m.vdim, m.gate_cap, p + "mix.", norm_eps=eps)
        elif layer.kind == "delta":
            mixer = _delta(d, m, p + "mix.", eps)
        else:
            mixer = ParallelMixer(_attention(d, m.left, p + "mix.left.", eps, positions, ropes),
                                  _delta(d, m.right, p + "mix.right.", eps), m.left_scale, m.right_scale)
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = SwiGLUFeedForward(d, layer.mlp.ff, p + "mlp.", names={"gate": "gate", "up": "up", "down": "down"})
            ffn_norm = RMSNorm(d, eps, p + "norm2")
        side = None
        if cfg.side_dim:
            side = TokenSideInput(d, cfg.vocab, "side.embed", n * cfg.side_dim, i * cfg.side_dim, cfg.side_dim, p + "side.", eps)
        blocks.append(PreNormBlock(RMSNorm(d, eps, p + "norm1"), mixer, ffn_norm, ffn, after=side))
    embedding = TokenEmbedding(cfg.vocab, d, "embed", scale=cfg.embedding_scale)
    head = OutputHead(d, cfg.vocab, RMSNorm(d, eps, "final.norm"), "head", tied_to="embed")
    return ModelSpec(cfg, embedding, blocks, head, layer_calls(n, cfg.loop))


register_architecture("Mifolorn", MifolornConfig, build_mifolorn, "mifolorn")
