"""Two mixers side by side: both read the same input, and the layer receives
    left_scale * left(h) + right_scale * right(h).
Either side is any mixer part (an attention over pages beside a recurrent mixer with a state, for instance); the
pair keeps the caches of both, the left one's first.  A side that can carry a factor on its result (it has a
settable `out_scale`: an attention's output gate, a recurrent mixer's output norm) is given its factor when the pair
is made, and then both sides add their output projection straight onto the float32 residual stream.  Otherwise
each side stores its float32 result in a buffer of its own and one kernel adds both, with their factors, onto the
residual stream.  Either way the sum is taken in 32-bit."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Part, register_part


def mixer_cache_specs(mixer) -> list:
    """A mixer's caches as a list: `cache_specs()` where it keeps several, else its one `cache_spec()`."""
    if hasattr(mixer, "cache_specs"):
        return list(mixer.cache_specs())
    return [mixer.cache_spec()]


def mixer_caches(mixer, caches):
    """What a mixer's forward is handed out of `caches` (one per spec): the list, or the single cache."""
    return list(caches) if hasattr(mixer, "cache_specs") else caches[0]


def _takes_scale(mixer) -> bool:
    """Whether the mixer carries a factor on its result by itself (set before its tensors are bound)."""
    return hasattr(mixer, "out_scale") and bool(getattr(mixer, "gate", True))      # an attention carries it on its gate


class ParallelMixer(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, left, right, left_scale: float = 1.0, right_scale: float = 1.0):
        self.left, self.right = left, right
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        self._n_left = len(mixer_cache_specs(left))
        self._carried = all(_takes_scale(m) for m in (left, right))
        if self._carried:
            left.out_scale, right.out_scale = self.left_scale, self.right_scale

    @property
    def hidden(self) -> int:
        return self.left.hidden

    def children(self):
        return (self.left, self.right)

    def cache_specs(self):
        return mixer_cache_specs(self.left) + mixer_cache_specs(self.right)

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        if self._carried:
            self.left.forward(xb, residual, ctx, mixer_caches(self.left, cache[:self._n_left]), write_cache, accumulate=accumulate)
            self.right.forward(xb, residual, ctx, mixer_caches(self.right, cache[self._n_left:]), write_cache, accumulate=True)
            return
        y_left = torch.empty(residual.shape, dtype=torch.float32, device=residual.device)
        y_right = torch.empty_like(y_left)
        self.left.forward(xb, y_left, ctx, mixer_caches(self.left, cache[:self._n_left]), write_cache, accumulate=False)
        self.right.forward(xb, y_right, ctx, mixer_caches(self.right, cache[self._n_left:]), write_cache, accumulate=False)
        ops.scaled_sum(residual, y_left, self.left_scale, y_right, self.right_scale, accumulate=accumulate)


register_part("mixer", "parallel", ParallelMixer)
