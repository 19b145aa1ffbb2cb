"""SwiGLU feed-forward: residual += (silu(xb Wg^T) * (xb Wu^T)) Wd^T, no biases
(src/engine/cpu_backend.zig:308-323, src/engine/ops.zig:65-80).  Gate and up are one
product over the concatenated weight [2F, d] (the reference fuses them into one parallel
region: src/engine/matmul.zig:93-96).  The gate's activation is a parameter (`act`: silu, or gelu_tanh =
0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), which makes it a GeGLU), and so are the tensors' names.
`act="swish_clamped"` is the clamped form: with g = min(gate, limit) and u = clamp(up, -limit, limit) the hidden
vector is g * sigmoid(slope * g) * (u + 1); `limit` and `slope` are parameters."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .base import MATRIX, VECTOR, ParamSpec, Part, Precision, register_part


class SwiGLUFeedForward(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, hidden: int, intermediate: int, prefix: str, act: str = "silu", names=None, limit: float = 0.0,
                 slope: float = 1.0):
        if act not in ops.GLU_ACTS:
            raise ValueError(f"activation '{act}' is not one of {', '.join(ops.GLU_ACTS)}")
        if act == "swish_clamped" and not limit > 0:
            raise ValueError("the clamped activation needs a positive limit")
        self.hidden, self.F, self.prefix, self.act = hidden, intermediate, prefix, act
        self.limit, self.slope = float(limit), float(slope)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        self.w_gate_up = self.w_down = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm = self.prefix, self.names
        return {
            p + nm["gate"]: ParamSpec((self.F, self.hidden), MATRIX),
            p + nm["up"]: ParamSpec((self.F, self.hidden), MATRIX),
            p + nm["down"]: ParamSpec((self.hidden, self.F), MATRIX),
        }

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        gate, up = tensors[p + nm["gate"]], tensors[p + nm["up"]]
        # One matrix [all gate rows | all up rows]: one product gives both halves, and the tensor-core kernels take a
        # tile's rows half from each so that SwiGLU runs in their epilogue (cf. the reference's fused gate/up product,
        # shaders/swiglu_pair.comp:2).
        if gate.dtype != up.dtype:                  # one of them kept in 32-bit: both are
            gate, up = gate.float(), up.float()
        self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[p + nm["down"]]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, accumulate: bool = True) -> None:
        h = torch.empty((xb.shape[0], self.F), dtype=xb.dtype, device=xb.device)
        ops.gemm_swiglu(xb, self.w_gate_up, h, self.act, self.limit, self.slope)
        ops.gemm(h, self.w_down, residual, accumulate=accumulate)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)


class PolyNormFeedForward(Part):
    """residual += W_down act(W_up xb) with the polynomial activation
        act(z) = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3,   N(v) = v / sqrt(mean(v^2) + eps) over a token's F values,
    powers element by element; the four numbers are a tensor of the model (`act`).  The up product's result is
    float32, the three means and the activation are computed in float32 and narrowed for the down product."""
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, hidden: int, intermediate: int, prefix: str, eps: float, names=None):
        self.hidden, self.F, self.prefix, self.eps = hidden, intermediate, prefix, float(eps)
        self.names = {"up": "up", "down": "down", "act": "act"}
        self.names.update(names or {})
        self.w_up = self.w_down = self.coef = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm = self.prefix, self.names
        return {
            p + nm["up"]: ParamSpec((self.F, self.hidden), MATRIX),
            p + nm["down"]: ParamSpec((self.hidden, self.F), MATRIX),
            p + nm["act"]: ParamSpec((4,), VECTOR, "one_plus_normal"),
        }

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        self.w_up, self.w_down, self.coef = tensors[p + nm["up"]], tensors[p + nm["down"]], tensors[p + nm["act"]]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, accumulate: bool = True) -> None:
        n = xb.shape[0]
        z = torch.empty((n, self.F), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_up, z)
        h = torch.empty((n, self.F), dtype=xb.dtype, device=xb.device)
        ops.polynorm(z, self.coef, self.eps, h)
        ops.gemm(h, self.w_down, residual, accumulate=accumulate)


class RoutedFeedForward(Part):
    """A mixture of `experts` SwiGLU feed-forwards of which every token uses `top`:
        router logits z = W_router xb in float32; the `top` largest are chosen (the lower index wins a tie) and
        weighted by the softmax over the chosen logits; residual += sum_k weight_k * W_down_e (silu(W_gate_e xb) * W_up_e xb).
    The choice never leaves the device (`csrc/routed.cu`): tokens are sorted by expert there and the experts'
    products run as one grouped product over tiles of the sorted rows, so the launches depend on the number of
    rows alone.  The experts' weights are stacked at binding: [E, 2F, d] (gate rows, then up rows) and [E, d, F].

    `scores="sigmoid"` is another router: every expert's score is s = sigmoid(z) by itself; the choice is made on
    s + correction (`correction=True`: a tensor [E] of the model, used for the choice alone), among the experts of the best
    `keep` of `groups` equal groups of neighbours when `groups` is given (a group's score is the sum of its two largest
    choice scores; the experts of the other groups count as minus infinity), and the weights are the chosen experts' s over
    their sum + `norm_eps`, times `weight_scale`.  `shared`: one more feed-forward part that every token uses; its result is
    added to the experts' sum, times sigmoid(W_sg xb) (one number per token, tensor `shared_gate` [1, d], whose product
    rides along with the router's in 32-bit) when `shared_gated` is set."""
    graph_safe = True   # reads the batch from device tensors only; launches depend on the row count alone
    kernel_libraries = ("routed",)
    route_log = None    # a list, when someone wants to see the choices: every eager forward appends a copy of its
                        # chosen experts int32 [rows, top] (a replayed graph runs no Python and appends nothing)

    def __init__(self, hidden: int, intermediate: int, n_experts: int, top: int, prefix: str, names=None,
                 scores: str = "softmax", correction: bool = False, groups: int = 0, keep: int = 0, weight_scale: float = 1.0,
                 norm_eps: float = 0.0, shared=None, shared_gated: bool = False):
        if not 1 <= top <= n_experts or top > 32:
            raise ValueError(f"top = {top} must be in 1..min(experts, 32) (experts = {n_experts})")
        if scores not in ("softmax", "sigmoid"):
            raise ValueError(f"scores '{scores}' is neither 'softmax' nor 'sigmoid'")
        if scores == "softmax" and (correction or groups or weight_scale != 1.0 or shared_gated):
            raise ValueError("a correction, groups, a factor on the weights and a gated shared part belong to scores='sigmoid'")
        if groups and (n_experts % groups or not 1 <= keep <= groups):
            raise ValueError(f"{n_experts} experts do not form {groups} equal groups of which {keep} are kept")
        if shared_gated and shared is None:
            raise ValueError("shared_gated needs a shared part")
        self.hidden, self.F, self.E, self.top, self.prefix = hidden, intermediate, n_experts, top, prefix
        self.scores, self.correction, self.groups, self.keep = scores, bool(correction), int(groups), int(keep)
        self.weight_scale, self.norm_eps = float(weight_scale), float(norm_eps)
        self.shared, self.shared_gated = shared, bool(shared_gated)
        self.names = {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down",
                      "correction": "correction", "shared_gate": "shared.sg"}
        self.names.update(names or {})
        self.w_router = self.w_gate_up = self.w_down = self.w_correction = None

    def children(self):
        return (self.shared,) if self.shared is not None else ()

    def _expert(self, e: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(e) + self.names[which]

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        specs = {self.prefix + self.names["router"]: ParamSpec((self.E, self.hidden), MATRIX)}
        if self.correction:
            specs[self.prefix + self.names["correction"]] = ParamSpec((self.E,), VECTOR)
        if self.shared_gated:
            specs[self.prefix + self.names["shared_gate"]] = ParamSpec((1, self.hidden), MATRIX)
        for e in range(self.E):
            specs[self._expert(e, "gate")] = ParamSpec((self.F, self.hidden), MATRIX)
            specs[self._expert(e, "up")] = ParamSpec((self.F, self.hidden), MATRIX)
            specs[self._expert(e, "down")] = ParamSpec((self.hidden, self.F), MATRIX)
        return specs

    def own_bind(self, tensors, precision: Precision) -> None:
        self.w_router = tensors[self.prefix + self.names["router"]].float().contiguous()    # the router runs in 32-bit
        if self.shared_gated:       # the shared part's gate is one more row of the router's product
            self.w_router = torch.cat([self.w_router, tensors[self.prefix + self.names["shared_gate"]].float()]).contiguous()
        if self.correction:
            self.w_correction = tensors[self.prefix + self.names["correction"]]
        dt = precision.compute
        self.w_gate_up = torch.stack([torch.cat([tensors[self._expert(e, "gate")].to(dt), tensors[self._expert(e, "up")].to(dt)])
                                      for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down")].to(dt) for e in range(self.E)]).contiguous()
        self._tile_rows = ops.route_tile_rows()

    TC_MIN_PAIRS = 1024     # from this many (row, choice) pairs on, a bfloat16 step takes the tcgen05 grouped product

    def _forward_tc(self, xb, residual, ids, weights, accumulate: bool, shared_y=None, shared_gate=None) -> bool:
        """Prompt-sized steps in bfloat16: the rows are gathered into expert order with every expert's rows padded to whole
        128-row tiles, and both products run on the tcgen05 kernel with a tile's expert choosing its weights."""
        from ..csrc import gemm_fast
        n, dev = xb.shape[0], xb.device
        pairs, pad = n * self.top, gemm_fast.GROUPED_ROWS
        m_max = -(-(pairs + self.E * (pad - 1)) // pad) * pad
        perm = torch.empty(m_max, dtype=torch.int32, device=dev)
        inv = torch.empty(pairs, dtype=torch.int32, device=dev)
        groups = torch.empty(m_max // pad, dtype=torch.int32, device=dev)
        ops.route_sort_padded(ids, self.E, pad, perm, inv, groups)
        xs = torch.empty((m_max, self.hidden), dtype=xb.dtype, device=dev)
        ops.route_gather(xb, perm, self.top, xs)
        h = torch.empty((m_max, self.F), dtype=xb.dtype, device=dev)
        if not ops.grouped_gemm_tc(xs, self.w_gate_up, h, groups, gated=True):
            return False
        ys = torch.empty((m_max, self.hidden), dtype=torch.float32, device=dev)
        if not ops.grouped_gemm_tc(h, self.w_down, ys, groups, gated=False):
            return False
        ops.route_combine(ys, inv, weights, residual, accumulate=accumulate, shared=shared_y, shared_gate=shared_gate)
        return True

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, accumulate: bool = True) -> None:
        n, dev = xb.shape[0], xb.device
        pairs = n * self.top
        ids = torch.empty((n, self.top), dtype=torch.int32, device=dev)
        weights = torch.empty((n, self.top), dtype=torch.float32, device=dev)
        shared_gate = torch.empty((n, 1), dtype=torch.float32, device=dev) if self.shared_gated else None
        ops.route_topk(xb, self.w_router, ids, weights, self.scores, self.w_correction, self.groups, self.keep, self.weight_scale,
                       self.norm_eps, shared_gate)
        if RoutedFeedForward.route_log is not None:
            RoutedFeedForward.route_log.append(ids.clone())
        shared_y = None
        if self.shared is not None:
            shared_y = torch.empty((n, self.hidden), dtype=torch.float32, device=dev)
            self.shared.forward(xb, shared_y, ctx, accumulate=False)
        if xb.dtype == torch.bfloat16 and pairs >= self.TC_MIN_PAIRS and self.hidden % 8 == 0 and self.F % 8 == 0 \
                and self._forward_tc(xb, residual, ids, weights, accumulate, shared_y, shared_gate):
            return
        max_tiles = pairs // self._tile_rows + min(self.E, pairs)
        offsets = torch.empty(self.E + 1, dtype=torch.int32, device=dev)
        perm = torch.empty(pairs, dtype=torch.int32, device=dev)
        inv = torch.empty(pairs, dtype=torch.int32, device=dev)
        tiles = torch.empty((max_tiles, 2), dtype=torch.int32, device=dev)
        ops.route_sort(ids, self.E, offsets, perm, inv, tiles)
        h = torch.empty((pairs, self.F), dtype=xb.dtype, device=dev)
        ops.grouped_gemm(xb, self.w_gate_up, h, tiles, offsets, perm, self.top, gather=True, gated=True)
        ys = torch.empty((pairs, self.hidden), dtype=torch.float32, device=dev)
        ops.grouped_gemm(h, self.w_down, ys, tiles, offsets, perm, self.top, gather=False, gated=False)
        ops.route_combine(ys, inv, weights, residual, accumulate=accumulate, shared=shared_y, shared_gate=shared_gate)


register_part("feed_forward", "polynorm", PolyNormFeedForward)
register_part("feed_forward", "routed_swiglu", RoutedFeedForward)
