"""Recurrent mixers: a state of fixed size per request, advanced token by token.

Both keep their state in float32 in the request's state slot (`StateSpec`) and find the rows of every request
of a step through one host-built table, `segments` int32 [requests of the step, 3] = (slot, first row, rows),
shared by all recurrent mixers of a model.  The scans (`csrc/recurrent.cu`) walk a request's rows in order, so
what a position computes does not depend on how the prompt was cut, on the batch or on the slot.  Projections
are products in the compute type with float32 results; everything from there to the state and the scan's
output is float32.

`GeneralDeltaRule` (per head a matrix state S [key_dim, value_dim], zero at the start):
      r, k, v, g = W_r h, W_k h, W_v h, W_g h;   decay logits wl = W_w2 tanh(W_w1 h) + w0;   al = W_a h + a0
      d = exp(-decay_scale * sigmoid(wl)),  a = sigmoid(al),  u = k / sqrt(sum(k^2) + key_eps)        per head
      S <- diag(d) S - (a * u) (u^T S) + k v^T        (both terms read the old S);    o = S^T r
      y = W_o ((o / rms(o) per head) * norm_weight * sigmoid(g))
  `decay_scale` and `key_eps` are parameters (exp(-1/2) and 1e-6 by default); the width of W_w1 is read from the
  configuration or, at binding, from the tensor.

`MinGRU` (one scalar state per channel, zero at the start; the gates read only the current token):
      z = sigmoid(W_z h + b_z);  x = W_x h + b_x;  c = x + 1/2 for x >= 0, sigmoid(x) below
      S <- (1 - z) S + z c;   y = W_o (S * silu(W_g h))

`GatedDeltaRule` (per head a matrix state S [key_dim, value_dim], zero at the start; `kv_heads` query/key heads serve
`n_heads` value heads, head h reading query/key head h // (n_heads / kv_heads)):
      q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     a short causal convolution per channel
      q <- q / sqrt(sum(q^2) + unit_eps) * key_dim^(-1/2),   k <- k / sqrt(sum(k^2) + unit_eps)        per head
      beta = sigmoid(W_b h),   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))                      one per head
      S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
      y = W_o ((o / rms(o) per head) * norm_weight[value_dim] * silu(W_g h))
  The request's state is S and the last taps - 1 inputs of the convolution (two `StateSpec`s).

`MLSTM` (per head a matrix S [key_dim, value_dim], a vector n [key_dim] and a running maximum m that starts at 0):
      q = W_q h * key_dim^(-1/2), k = W_k h, v = W_v h
      i = cap tanh((W_i h + b_i) / cap),   f = logsigmoid(cap tanh((W_f h + b_f) / cap))              one per head
      m' = max(f + m, i);   S <- e^(f + m - m') S + e^(i - m') k v^T;   n <- e^(f + m - m') n + e^(i - m') k
      o = S^T q / (max(|n . q|, e^(-m')) + den_eps)
      y = W_o ((o / rms(o) per head) * norm_weight[n_heads * value_dim] * sigmoid(W_g h))
  n is kept as one more column of S (its value is always 1), m in a `StateSpec` of its own.

`Retention` (per head a matrix state S [key_dim, value_dim], zero at the start; a fixed decay per head, no softmax and no
denominator):
      q, k = rot(W_q h), rot(W_k h) * k_scale;   v = W_v h          rot: the position encoding handed in (or none)
      S <- decay_h S + k v^T;   o = S^T q
      y = W_o ((o / rms(o) per head) * silu(W_g h))
  `decay` (one number per head) and `k_scale` (key_dim^(-1/2) by default) are parameters.

`ShortConvolution` is the causal convolution over a request's last `taps` rows per channel as a part of its own (tensors
[channels, taps] by group of channels, an optional silu, the request's last taps - 1 inputs as its state), for mixers
other than the gated delta rule that put one behind their projections.

A mixer with several caches says so with `cache_specs()` and is handed the list.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from ..csrc import ops
from .base import MATRIX, VECTOR, ParamSpec, Part, Precision, StateSpec, StepTables, register_part

SEGMENTS_KEY = ("request_segments",)


def segment_tables(ctx) -> StepTables:
    """(slot, first row, rows) of every request of the step.  Its shape depends on the number of requests alone."""
    seg = np.stack([np.asarray(ctx.slots, dtype=np.int32), np.asarray(ctx.q_starts, dtype=np.int32),
                    np.asarray(ctx.q_lens, dtype=np.int32)], axis=1)
    return StepTables({"segments": seg})


class _SegmentScan(Part):
    graph_safe = True           # the batch is read from device tensors and the segment table only
    kernel_libraries = ("recurrent",)

    def step_tables_key(self):
        return SEGMENTS_KEY

    def step_tables(self, ctx):
        return segment_tables(ctx)

    @staticmethod
    def _segments(ctx) -> torch.Tensor:
        return ctx.tables[SEGMENTS_KEY][0]["segments"]


class GeneralDeltaRule(_SegmentScan):
    def __init__(self, hidden: int, n_heads: int, key_dim: int, prefix: str, norm_eps: float,
                 value_dim: Optional[int] = None, decay_rank: Optional[int] = None,
                 decay_scale: float = math.exp(-0.5), key_eps: float = 1e-6, names: Optional[Dict[str, str]] = None):
        self.hidden, self.H, self.dk = hidden, n_heads, key_dim
        self.dv = key_dim if value_dim is None else int(value_dim)
        self.prefix, self.norm_eps = prefix, float(norm_eps)
        self.decay_rank = decay_rank         # None: whatever the file's tensor has (known at binding)
        self.decay_scale, self.key_eps = float(decay_scale), float(key_eps)
        self.names = {"r": "r", "k": "k", "v": "v", "g": "g", "a": "a", "a_bias": "a.b", "w1": "w1", "w2": "w2",
                      "w_bias": "w0", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_w2 = self.w_o = self.a_bias = self.w_bias = self.norm_weight = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, d = self.prefix, self.names, self.hidden
        K, V = self.H * self.dk, self.H * self.dv
        R = self.decay_rank if self.decay_rank is not None else -1      # -1: any size along that axis
        return {
            p + nm["r"]: ParamSpec((K, d), MATRIX), p + nm["k"]: ParamSpec((K, d), MATRIX),
            p + nm["v"]: ParamSpec((V, d), MATRIX), p + nm["g"]: ParamSpec((V, d), MATRIX),
            p + nm["a"]: ParamSpec((K, d), MATRIX), p + nm["a_bias"]: ParamSpec((K,), VECTOR),
            p + nm["w1"]: ParamSpec((R, d), MATRIX), p + nm["w2"]: ParamSpec((K, R), MATRIX),
            p + nm["w_bias"]: ParamSpec((K,), VECTOR), p + nm["norm"]: ParamSpec((V,), VECTOR, "one_plus_normal"),
            p + nm["o"]: ParamSpec((d, V), MATRIX),
        }

    def cache_spec(self):
        return StateSpec((self.H, self.dk, self.dv), torch.float32)

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("r", "k", "v", "g", "a", "w1")]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        # one product gives r, k, v, g, the removal logits and the hidden layer of the decay's low-rank projection
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()
        self.rank = int(tensors[p + nm["w1"]].shape[0])
        self.w_w2 = tensors[p + nm["w2"]]
        if int(self.w_w2.shape[1]) != self.rank:
            raise ValueError(f"'{p + nm['w2']}' takes {int(self.w_w2.shape[1])} inputs, '{p + nm['w1']}' gives {self.rank}")
        self.w_o = tensors[p + nm["o"]]
        self.a_bias, self.w_bias = tensors[p + nm["a_bias"]], tensors[p + nm["w_bias"]]
        self.norm_weight = tensors[p + nm["norm"]]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n = xb.shape[0]
        K, V = self.H * self.dk, self.H * self.dv
        proj = torch.empty((n, self.w_in.shape[0]), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_in, proj)
        r, k, v = proj[:, :K], proj[:, K:2 * K], proj[:, 2 * K:2 * K + V]
        g, al = proj[:, 2 * K + V:2 * K + 2 * V], proj[:, 2 * K + 2 * V:3 * K + 2 * V]
        hid = torch.empty((n, self.rank), dtype=xb.dtype, device=xb.device)
        ops.tanh_cols(proj[:, 3 * K + 2 * V:], hid)
        wl = torch.empty((n, K), dtype=torch.float32, device=xb.device)
        ops.gemm(hid, self.w_w2, wl)
        o = torch.empty((n, V), dtype=torch.float32, device=xb.device)
        ops.delta_rule_scan(r, k, v, al, wl, self.a_bias, self.w_bias, self._segments(ctx), cache.state, o,
                            self.H, self.dk, self.dv, self.decay_scale, self.key_eps)
        og = torch.empty((n, V), dtype=xb.dtype, device=xb.device)
        ops.head_norm_gate(o, g, self.norm_weight, self.norm_eps, og, self.H, self.dv)
        ops.gemm(og, self.w_o, residual, accumulate=accumulate)


class MinGRU(_SegmentScan):
    def __init__(self, hidden: int, width: int, prefix: str, names: Optional[Dict[str, str]] = None):
        self.hidden, self.width, self.prefix = hidden, width, prefix
        self.names = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "g": "g", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_o = self.z_bias = self.x_bias = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, d, W = self.prefix, self.names, self.hidden, self.width
        return {
            p + nm["z"]: ParamSpec((W, d), MATRIX), p + nm["z_bias"]: ParamSpec((W,), VECTOR),
            p + nm["x"]: ParamSpec((W, d), MATRIX), p + nm["x_bias"]: ParamSpec((W,), VECTOR),
            p + nm["g"]: ParamSpec((W, d), MATRIX), p + nm["o"]: ParamSpec((d, W), MATRIX),
        }

    def cache_spec(self):
        return StateSpec((self.width,), torch.float32)

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("z", "x", "g")]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()
        self.w_o = tensors[p + nm["o"]]
        self.z_bias, self.x_bias = tensors[p + nm["z_bias"]], tensors[p + nm["x_bias"]]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n = xb.shape[0]
        proj = torch.empty((n, 3 * self.width), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_in, proj)
        out = torch.empty((n, self.width), dtype=xb.dtype, device=xb.device)
        ops.mingru_scan(proj, self.z_bias, self.x_bias, self._segments(ctx), cache.state, out)
        ops.gemm(out, self.w_o, residual, accumulate=accumulate)


class GatedDeltaRule(_SegmentScan):
    def __init__(self, hidden: int, n_heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int, prefix: str,
                 norm_eps: float, unit_eps: float = 1e-6, q_scale: Optional[float] = None, out_scale: float = 1.0,
                 names: Optional[Dict[str, str]] = None):
        if n_heads % kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {kv_heads} query/key heads")
        if taps < 1:
            raise ValueError("the short convolution needs at least one tap")
        self.hidden, self.H, self.G, self.dk, self.dv, self.taps = hidden, n_heads, kv_heads, key_dim, value_dim, int(taps)
        self.prefix, self.norm_eps, self.unit_eps = prefix, float(norm_eps), float(unit_eps)
        self.q_scale = float(q_scale) if q_scale is not None else key_dim ** -0.5
        self.out_scale = float(out_scale)      # a factor on the mixer's result (carried by the output norm's weight)
        self.names = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "b": "b",
                      "a": "a", "a_log": "A_log", "dt_bias": "dt_bias", "g": "g", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_o = self.conv = self.a_log = self.dt_bias = self.norm_weight = None

    @property
    def channels(self) -> int:
        return 2 * self.G * self.dk + self.H * self.dv

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, d = self.prefix, self.names, self.hidden
        K, V = self.G * self.dk, self.H * self.dv
        return {
            p + nm["q"]: ParamSpec((K, d), MATRIX), p + nm["k"]: ParamSpec((K, d), MATRIX),
            p + nm["v"]: ParamSpec((V, d), MATRIX), p + nm["g"]: ParamSpec((V, d), MATRIX),
            p + nm["q_conv"]: ParamSpec((K, self.taps), VECTOR), p + nm["k_conv"]: ParamSpec((K, self.taps), VECTOR),
            p + nm["v_conv"]: ParamSpec((V, self.taps), VECTOR),
            p + nm["b"]: ParamSpec((self.H, d), MATRIX), p + nm["a"]: ParamSpec((self.H, d), MATRIX),
            p + nm["a_log"]: ParamSpec((self.H,), VECTOR), p + nm["dt_bias"]: ParamSpec((self.H,), VECTOR),
            p + nm["norm"]: ParamSpec((self.dv,), VECTOR, "one_plus_normal"), p + nm["o"]: ParamSpec((d, V), MATRIX),
        }

    def cache_specs(self):
        # one tap keeps no inputs; its tail is a row that nobody reads (a state of no size has no slot to live in)
        return [StateSpec((self.H, self.dk, self.dv), torch.float32), StateSpec((max(self.taps - 1, 1), self.channels), torch.float32)]

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("q", "k", "v", "g", "b", "a")]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        # one product gives the convolutions' inputs, the output gate's logits and the two per-head logits
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()
        self.conv = torch.cat([tensors[p + nm[c]] for c in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.w_o = tensors[p + nm["o"]]
        self.a_log, self.dt_bias = tensors[p + nm["a_log"]], tensors[p + nm["dt_bias"]]
        self.norm_weight = tensors[p + nm["norm"]]
        if self.out_scale != 1.0:
            self.norm_weight = (self.norm_weight * self.out_scale).contiguous()

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n = xb.shape[0]
        K, V, C, H = self.G * self.dk, self.H * self.dv, self.channels, self.H
        state, tail = cache[0].state, cache[1].state
        segs = self._segments(ctx)
        proj = torch.empty((n, self.w_in.shape[0]), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_in, proj)
        act = torch.empty((n, C), dtype=torch.float32, device=xb.device)
        ops.short_conv(proj[:, :C], self.conv, segs, tail, act)
        o = torch.empty((n, V), dtype=torch.float32, device=xb.device)
        ops.gated_delta_scan(act[:, :K], act[:, K:2 * K], act[:, 2 * K:], proj[:, C + V:C + V + H], proj[:, C + V + H:],
                             self.a_log, self.dt_bias, segs, state, o, H, self.G, self.dk, self.dv, self.q_scale, self.unit_eps)
        og = torch.empty((n, V), dtype=xb.dtype, device=xb.device)
        ops.head_out_gate(o, proj[:, C:C + V], self.norm_weight, self.norm_eps, og, H, self.dv, act="silu")
        ops.gemm(og, self.w_o, residual, accumulate=accumulate)


class Retention(_SegmentScan):
    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, decay, prefix: str, norm_eps: float,
                 position=None, k_scale: Optional[float] = None, names: Optional[Dict[str, str]] = None):
        decay = [float(x) for x in decay]
        if len(decay) != n_heads:
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        if position is not None and (position.rotary_dim > key_dim or position.pairing != "half"):
            raise ValueError("the rotation must fit the key size and pair dim i with i + dims/2")
        self.hidden, self.H, self.dk, self.dv = hidden, n_heads, key_dim, value_dim
        self.decay_values, self.prefix, self.norm_eps, self.position = decay, prefix, float(norm_eps), position
        self.k_scale = float(k_scale) if k_scale is not None else key_dim ** -0.5
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_o = self.decay = None

    def children(self):
        return (self.position,) if self.position is not None else ()

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, d = self.prefix, self.names, self.hidden
        K, V = self.H * self.dk, self.H * self.dv
        return {p + nm["q"]: ParamSpec((K, d), MATRIX), p + nm["k"]: ParamSpec((K, d), MATRIX),
                p + nm["v"]: ParamSpec((V, d), MATRIX), p + nm["g"]: ParamSpec((V, d), MATRIX),
                p + nm["o"]: ParamSpec((d, V), MATRIX)}

    def cache_spec(self):
        return StateSpec((self.H, self.dk, self.dv), torch.float32)

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("q", "k", "v", "g")]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()
        self.w_o = tensors[p + nm["o"]]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(precision.device)

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n = xb.shape[0]
        K, V = self.H * self.dk, self.H * self.dv
        proj = torch.empty((n, self.w_in.shape[0]), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_in, proj)
        cos = sin = None
        rot = 0
        if self.position is not None:
            cos, sin, rot = self.position.tables()
        o = torch.empty((n, V), dtype=torch.float32, device=xb.device)
        ops.retention_scan(proj[:, :K], proj[:, K:2 * K], proj[:, 2 * K:2 * K + V], cos, sin, rot, ctx.positions, self.decay,
                           self._segments(ctx), cache.state, o, self.H, self.dk, self.dv, self.k_scale)
        og = torch.empty((n, V), dtype=xb.dtype, device=xb.device)
        ops.head_out_gate(o, proj[:, 2 * K + V:], None, self.norm_eps, og, self.H, self.dv, act="silu")
        ops.gemm(og, self.w_o, residual, accumulate=accumulate)


class ShortConvolution(_SegmentScan):
    """y[t, c] = act(sum_j w[c, j] x[t - (taps - 1) + j, c]) over a request's rows, zeros before its start.  `groups`:
    (tensor name, channels) in the order of the channels; the tensors [channels, taps] are laid side by side at binding."""

    def __init__(self, groups, taps: int, act: str = "none"):
        if taps < 1 or act not in ("none", "silu"):
            raise ValueError("the short convolution needs at least one tap, and act 'none' or 'silu'")
        self.groups, self.taps, self.act = [(str(nm), int(c)) for nm, c in groups], int(taps), act
        self.channels = sum(c for _, c in self.groups)
        self.weight = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        return {nm: ParamSpec((c, self.taps), VECTOR) for nm, c in self.groups}

    def cache_spec(self):
        # one tap keeps no inputs; its tail is a row that nobody reads (a state of no size has no slot to live in)
        return StateSpec((max(self.taps - 1, 1), self.channels), torch.float32)

    def own_bind(self, tensors, precision: Precision) -> None:
        self.weight = torch.cat([tensors[nm] for nm, _ in self.groups], dim=0).contiguous()

    def forward(self, x: torch.Tensor, ctx, cache, out: torch.Tensor) -> None:
        """x and out: float32 column slices [n, channels]; `cache`: the state of `cache_spec()`."""
        ops.short_conv(x, self.weight, self._segments(ctx), cache.state, out, act=self.act)


class MLSTM(_SegmentScan):
    def __init__(self, hidden: int, n_heads: int, key_dim: int, value_dim: int, gate_cap: float, prefix: str, norm_eps: float,
                 den_eps: float = 1e-6, q_scale: Optional[float] = None, names: Optional[Dict[str, str]] = None):
        if not gate_cap > 0:
            raise ValueError("the gates' cap must be positive")
        self.hidden, self.H, self.dk, self.dv = hidden, n_heads, key_dim, value_dim
        self.dvp = ops.mlstm_padded(value_dim)
        self.cap, self.prefix, self.norm_eps, self.den_eps = float(gate_cap), prefix, float(norm_eps), float(den_eps)
        self.q_scale = float(q_scale) if q_scale is not None else key_dim ** -0.5
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b",
                      "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_o = self.i_bias = self.f_bias = self.norm_weight = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, d = self.prefix, self.names, self.hidden
        K, V, H = self.H * self.dk, self.H * self.dv, self.H
        return {
            p + nm["q"]: ParamSpec((K, d), MATRIX), p + nm["k"]: ParamSpec((K, d), MATRIX),
            p + nm["v"]: ParamSpec((V, d), MATRIX), p + nm["g"]: ParamSpec((V, d), MATRIX),
            p + nm["i"]: ParamSpec((H, d), MATRIX), p + nm["i_bias"]: ParamSpec((H,), VECTOR),
            p + nm["f"]: ParamSpec((H, d), MATRIX), p + nm["f_bias"]: ParamSpec((H,), VECTOR),
            p + nm["norm"]: ParamSpec((V,), VECTOR, "one_plus_normal"), p + nm["o"]: ParamSpec((d, V), MATRIX),
        }

    def cache_specs(self):
        return [StateSpec((self.H, self.dk, self.dvp), torch.float32), StateSpec((self.H,), torch.float32)]

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("q", "k", "v", "g", "i", "f")]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()
        self.w_o = tensors[p + nm["o"]]
        self.i_bias, self.f_bias = tensors[p + nm["i_bias"]], tensors[p + nm["f_bias"]]
        self.norm_weight = tensors[p + nm["norm"]]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n = xb.shape[0]
        K, V, H = self.H * self.dk, self.H * self.dv, self.H
        proj = torch.empty((n, self.w_in.shape[0]), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_in, proj)
        o = torch.empty((n, H * self.dvp), dtype=torch.float32, device=xb.device)
        gates = torch.empty((n, H, 3), dtype=torch.float32, device=xb.device)
        ops.mlstm_scan(proj[:, :K], proj[:, K:2 * K], proj[:, 2 * K:2 * K + V], proj[:, 2 * K + 2 * V:2 * K + 2 * V + H],
                       proj[:, 2 * K + 2 * V + H:], self.i_bias, self.f_bias, self._segments(ctx), cache[0].state,
                       cache[1].state, o, gates, H, self.dk, self.dv, self.cap, self.q_scale)
        og = torch.empty((n, V), dtype=xb.dtype, device=xb.device)
        ops.head_out_gate(o, proj[:, 2 * K + V:2 * K + 2 * V], self.norm_weight, self.norm_eps, og, H, self.dv, act="sigmoid",
                          gates=gates, den_eps=self.den_eps)
        ops.gemm(og, self.w_o, residual, accumulate=accumulate)


register_part("mixer", "general_delta_rule", GeneralDeltaRule)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
register_part("mixer", "mlstm", MLSTM)
register_part("mixer", "mingru", MinGRU)
register_part("mixer", "retention", Retention)
