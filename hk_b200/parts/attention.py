"""Grouped-query attention over a paged cache, as a mixer part.

Steps, in the reference's order (src/engine/cpu_backend.zig:266-304):
  q, k, v = xb Wq^T, xb Wk^T, xb Wv^T   (one fused product; no bias: src/engine/config.zig:313)
  per-head RMS norm of q and of k with a weight [head_dim] shared by the heads, before the
  rotation (src/engine/ops.zig:32-38, src/kernels_impl.zig:55-66) - optional here
  rotate-half rotation of q and k by position (src/engine/ops.zig:176-181) - optional here
  the step's k and v go to the cache before any score is taken (cpu_backend.zig:290-295)
  scores scale * q . k_j over the visible keys, softmax in float32, weighted values
  (src/engine/attention.zig:45-103), q head h reading kv head h // (H/G) (attention.zig:56)
  residual += att Wo^T (cpu_backend.zig:303-304)

Sizes, the norm's eps, the position encoding (with its pairing of dims), the window, the scale and
biases on the projections are parameters.  The
reference's attention has no window (src/engine/config.zig:271-279 refuses one); `window=w`
limits the keys of position p to (p - w, p] and lets the cache give pages back.

Further parameters, for designs other than the reference's:
  `qk_norm_after` puts the per-head norm of q and k behind the rotation; `qk_norm_weight=False` makes it a norm
  without a weight (x over its root mean square);
  `value_from_key` drops the v projection: a token's value is its key as projected, before rotation and norm,
  of which the first `v_head_dim` dims are kept (the cache then holds both forms of the key);
  `sink` adds a term to the softmax's denominator, a key of score 0 that has no value:
  p_j = exp(s_j) / (1 + sum exp(s_j)); with `sink_weights` that score is a number per query head learned with the
  model (tensor `sink` [H]): p_j = exp(s_j) / (exp(sink_h) + sum exp(s_j));
  `v_head_dim` without `value_from_key` gives the values a width of their own (W_v is [G * v_head_dim, hidden]);
  `softcap` c bounds the scores: s <- c tanh(s / c), after the scale and before the softmax;
  `chunk` s cuts the sequence into blocks of s positions counted from position 0: a token sees the keys of its own
  block up to itself and none of an earlier block;
  `gate` multiplies the concatenated heads' outputs, before W_o, element by element with sigmoid(W_g x) of the
  mixer's own input (tensor `g` [H * v_head_dim, hidden], fused into the q/k/v product); `out_scale` is a factor on
  the mixer's result that the gate carries;
  `names` renames the tensors (keys q, k, v, o, q_norm, k_norm, sink, gate, and q_bias, k_bias, v_bias, o_bias).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import KVCacheSpec, MATRIX, VECTOR, ParamSpec, Part, Precision, StepTables, register_part
from .position import RotaryEmbedding


def flash_step_tables(ctx, H: int, G: int, hd: int, window: int, chunk: int, sm_count: int, tensor_prompt: bool = True):
    """The flash kernels' work items for one step, as a part's host-built tables.  `tensor_prompt` = False keeps prompt
    portions off the tcgen05 kernels' tiles of 128 and 256 rows (for a kernel of its own that takes 64-row items)."""
    from ..csrc import attention_fast
    tc = attention_fast.tc_prefill_supported(hd, H // G) and ops.forced("attention") != "flash_cp" and tensor_prompt
    rows = 128 if tc else 64
    # the kernel with two query tiles per CTA is the faster one per row, but halves the number of work items: it
    # is taken when its items still fill the SMs (measured on the 8B layer: equal at 1,024 prompt tokens = 128
    # items, 1.6 times faster at 2,048, 1.3 times slower at 512), where the pages allow it
    if tc and attention_fast.tc2_prefill_supported(hd, H // G, ctx.page_tokens):
        group = H // G
        items = G * sum(-(-(int(q) * group) // 256) for q in ctx.q_lens if int(q) * group > 128)
        if items * 20 >= sm_count * 17:
            rows = 256
    fixed = attention_fast.decode_splits(ctx.n_tokens, G, sm_count) if ctx.fixed_shape else 0
    got = attention_fast.plan_arrays(ctx.slots, ctx.q_starts, ctx.q_lens, ctx.start_positions, ctx.n_tokens,
                                     window, H, G, sm_count, fixed_splits=fixed,
                                     max_context=ctx.max_context if ctx.fixed_shape else 0,
                                     prefill_rows=rows, chunk=chunk)
    if got is None:
        return None
    items, merge, info = got
    arrays = {"items": items}
    if merge is not None:
        arrays["merge"] = merge
    return StepTables(arrays, info)


def flash_plan(ctx, key):
    """The step's plan on the device from the tables named `key`, or None (the generic kernel takes the step)."""
    got = ctx.tables.get(key) if key is not None else None
    if got is None or got[1] is None:
        return None
    from ..csrc import attention_fast
    arrays, info = got
    return attention_fast.plan_on_device(info, arrays["items"], arrays.get("merge"))


class GQAAttention(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, prefix: str,
                 qk_norm_eps: Optional[float] = None, position: Optional[RotaryEmbedding] = None,
                 window: Optional[int] = None, scale: Optional[float] = None, qkv_bias: bool = False,
                 o_bias: bool = False, qk_norm_after: bool = False, qk_norm_weight: bool = True,
                 value_from_key: bool = False, v_head_dim: Optional[int] = None, sink: bool = False,
                 names: Optional[Dict[str, str]] = None, sink_weights: bool = False, softcap: Optional[float] = None,
                 chunk: Optional[int] = None, gate: bool = False, out_scale: float = 1.0):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        if head_dim > 256 or head_dim < 2:
            raise ValueError(f"head_dim {head_dim} is outside 2..256")
        if position is not None and position.rotary_dim > head_dim:
            raise ValueError("the rotary width exceeds head_dim")
        self.hidden, self.H, self.G, self.hd = hidden, n_heads, n_kv_heads, head_dim
        self.vd = head_dim if v_head_dim is None else int(v_head_dim)
        if not 1 <= self.vd <= 256 or (self.vd > head_dim and value_from_key):
            raise ValueError(f"value size {self.vd} must be in 1..256, and at most head_dim when the values are the keys")
        if sink_weights and not sink:
            raise ValueError("sink_weights needs sink")
        self.sink_weights, self.gate = bool(sink_weights), bool(gate)
        if out_scale != 1.0 and not gate:
            raise ValueError("out_scale rides on the output gate: it needs gate=True")
        self.out_scale = float(out_scale)      # a factor on the mixer's result (carried by the output gate)
        self.softcap = float(softcap) if softcap else 0.0
        self.chunk = int(chunk) if chunk else 0
        if self.softcap < 0 or self.chunk < 0:
            raise ValueError("softcap and chunk must be positive (or absent)")
        self.qk_norm_after, self.qk_norm_weight = bool(qk_norm_after), bool(qk_norm_weight)
        self.value_from_key, self.sink = bool(value_from_key), bool(sink)
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                      "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sink", "gate": "g_proj.weight",
                      "q_bias": "q_proj.bias",
                      "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias"}
        self.names.update(names or {})
        self.prefix = prefix
        self.qk_norm_eps = qk_norm_eps
        self.position = position
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        # biases on the projections: the reference turns `qkv_bias` on by architecture (src/engine/config.zig:313)
        self.qkv_bias, self.o_bias = bool(qkv_bias), bool(o_bias)
        self.b_qkv = self.b_o = None
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.sinks = None
        self._tables_key = None        # set at bind: the flash kernels' work items, when they take these sizes
        self._sm_count = 0

    # -- declaration ---------------------------------------------------------------------
    def kernel_libraries(self, bfloat16: bool):
        """The flash kernels are compiled only for a model one of whose attention parts can use them."""
        from ..csrc import attention_fast
        if not bfloat16 or not self._flash_takes():
            return ()
        return ("attention_flash", "attention_prefill_tc") if attention_fast.tc_prefill_supported(self.hd, self.H // self.G) \
            else ("attention_flash",)

    def _flash_takes(self) -> bool:
        """Whether the flash kernels take this mixer's sizes (they know every option of the scores: sink, cap, blocks)."""
        from ..csrc import attention_fast
        return self.vd == self.hd and attention_fast.supported(self.hd, self.H // self.G)

    def children(self):
        return (self.position,) if self.position is not None else ()

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, H, G, hd, d, nm = self.prefix, self.H, self.G, self.hd, self.hidden, self.names
        specs = {
            p + nm["q"]: ParamSpec((H * hd, d), MATRIX),
            p + nm["k"]: ParamSpec((G * hd, d), MATRIX),
            p + nm["o"]: ParamSpec((d, H * self.vd), MATRIX),
        }
        if not self.value_from_key:
            specs[p + nm["v"]] = ParamSpec((G * self.vd, d), MATRIX)
        if self.sink_weights:
            specs[p + nm["sink"]] = ParamSpec((H,), VECTOR)
        if self.gate:
            specs[p + nm["gate"]] = ParamSpec((H * self.vd, d), MATRIX)
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            specs[p + nm["q_norm"]] = ParamSpec((hd,), VECTOR, "one_plus_normal")
            specs[p + nm["k_norm"]] = ParamSpec((hd,), VECTOR, "one_plus_normal")
        if self.qkv_bias:
            specs[p + nm["q_bias"]] = ParamSpec((H * hd,), VECTOR)
            specs[p + nm["k_bias"]] = ParamSpec((G * hd,), VECTOR)
            if not self.value_from_key:
                specs[p + nm["v_bias"]] = ParamSpec((G * self.vd,), VECTOR)
        if self.o_bias:
            specs[p + nm["o_bias"]] = ParamSpec((d,), VECTOR)
        return specs

    def cache_spec(self):
        return KVCacheSpec(self.G, self.hd, self.window, None if self.vd == self.hd else self.vd)

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        parts = "qk" if self.value_from_key else "qkv"
        qkv = [tensors[p + nm[c]] for c in parts]
        self._qkv_width = sum(int(t.shape[0]) for t in qkv)
        if self.gate:                        # the gate's logits are further columns of the same product
            qkv.append(tensors[p + nm["gate"]])
        if self.sink_weights:
            self.sinks = tensors[p + nm["sink"]]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in qkv) else qkv[0].dtype    # one kept in 32-bit: all are
        self.w_qkv = torch.cat([t.to(wide) for t in qkv], dim=0).contiguous()
        self.w_o = tensors[p + nm["o"]]
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[p + nm[c + "_bias"]] for c in parts]).contiguous()
        if self.o_bias:
            self.b_o = tensors[p + nm["o_bias"]]
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm = tensors[p + nm["q_norm"]]
            self.k_norm = tensors[p + nm["k_norm"]]
        from ..csrc import attention_fast
        if precision.compute == torch.bfloat16 and self._flash_takes():
            self._tables_key = ("paged_attention_items", self.window or 0, self.H, self.G, self.hd, self.sink, self.chunk, bool(self.softcap))
            self._sm_count = torch.cuda.get_device_properties(precision.device).multi_processor_count

    # -- the step's work items (host-built; see parts.base) --------------------------------
    def step_tables_key(self):
        return self._tables_key

    def step_tables(self, ctx):
        """Cuts the batch into the flash kernels' work items (csrc/attention_fast.py).  In a step whose shape must
        not change (a captured decode graph) every request's keys go to the same number of splits."""
        return flash_step_tables(ctx, self.H, self.G, self.hd, self.window or 0, self.chunk, self._sm_count)

    def _plan(self, ctx):
        return flash_plan(ctx, self._tables_key)

    # -- one step ------------------------------------------------------------------------
    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        """`accumulate=False` stores the mixer's result in `residual` instead of adding it (a block that norms the
        result before the residual sum)."""
        n = xb.shape[0]
        H, G, hd = self.H, self.G, self.hd
        plan = self._plan(ctx) if xb.dtype == torch.bfloat16 else None
        proj = torch.empty((n, self.w_qkv.shape[0]), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_qkv, proj)
        qkv = proj[:, :self._qkv_width] if self.gate else proj
        gate = proj[:, self._qkv_width:] if self.gate else None
        q = torch.empty((n, H * hd), dtype=xb.dtype, device=xb.device)
        cos = sin = None
        rot = 0
        pairing = "half"
        if self.position is not None:
            cos, sin, rot = self.position.tables()
            pairing = getattr(self.position, "pairing", "half")
        # the projections' bias rides on the fused kernel's load
        ops.qk_norm_rope_kv_write(
            qkv, q, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, cos, sin, rot, ctx.positions,
            ctx.slot_of_token, cache.block_table, cache.k_pages, cache.v_pages, H, G, hd, cache.page_tokens,
            write_kv=write_cache, bias=self.b_qkv, pairing=pairing, norm_after=self.qk_norm_after,
            tied_v=self.value_from_key)
        att = torch.empty((n, H * self.vd), dtype=xb.dtype, device=xb.device)
        ops.paged_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions, ctx.slot_of_token,
                            att, H, G, hd, cache.page_tokens, self.window or 0, self.scale,
                            plan=plan, sink=self.sink, sinks=self.sinks, softcap=self.softcap, chunk=self.chunk, gate=gate,
                            gate_scale=self.out_scale)
        ops.gemm(att, self.w_o, residual, accumulate=accumulate, bias=self.b_o)


register_part("mixer", "gqa_attention", GQAAttention)


class DifferentialAttention(Part):
    """Grouped-query attention with two score maps per head over the same values ("differential attention").

        q = W_q h [H, 2, dim],  k = W_k h [G, 2, dim],  v = W_v h [G, vdim]      a head's two maps side by side
        optionally a short causal convolution per channel of q, k and v (`taps`), straight behind the projections
        rotation of the first `position.rotary_dim` dims of every map of q and k
        a_j = softmax(scale * q_j k_j^T) v  for j = 1, 2     (causal; `window` limits the keys)
        lambda = exp(sum(lq1 * lk1)) - exp(sum(lq2 * lk2)) + diff                one number for the mixer
        o = a_1 - lambda * a_2;   o <- o / sqrt(mean(o^2) + norm_eps) * (1 - diff)   per head, no weight
        y = W_o (o * sigmoid(W_g h)_head)                                        `gate`: one number per head

    It runs on the ordinary paged attention kernels as 2 H query heads over G key/value heads: the cache row of a key
    head holds both maps' keys side by side, and a map's query is zero outside its own half, so both maps of all heads
    of a group read the same keys and values once.  Where the cache rows have a head size the tensor-core kernels know
    (2 dim = vdim), those run; else the generic kernel.  The cache is `KVCacheSpec(G, 2 dim, window, vdim)` and, with a
    convolution, its last taps - 1 inputs per request.  `names` renames the tensors (keys q, k, v, o, gate, q_conv, k_conv,
    v_conv, lq1, lk1, lq2, lk2)."""
    graph_safe = True   # reads the batch from device tensors only
    MAPS = 2

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, prefix: str, diff: float,
                 norm_eps: float, scale: Optional[float] = None, position: Optional[RotaryEmbedding] = None,
                 window: Optional[int] = None, taps: int = 0, gate: bool = True, names: Optional[Dict[str, str]] = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        if position is not None and (position.rotary_dim > head_dim or position.pairing != "half"):
            raise ValueError("the rotation must fit a map's size and pair dim i with i + dims/2")
        if self.MAPS * head_dim > 640 or v_head_dim > 640 or min(head_dim, v_head_dim) < 1:
            raise ValueError("a cache row of a differential attention holds at most 640 numbers")
        self.hidden, self.H, self.G, self.dk, self.vd = hidden, n_heads, n_kv_heads, head_dim, v_head_dim
        self.prefix, self.diff, self.norm_eps = prefix, float(diff), float(norm_eps)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position, self.window, self.gate = position, window, bool(gate)
        self.names = {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_conv": "q.conv", "k_conv": "k.conv",
                      "v_conv": "v.conv", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
        self.names.update(names or {})
        M = self.MAPS
        self.channels = (n_heads + n_kv_heads) * M * head_dim + n_kv_heads * v_head_dim
        self.conv = None
        if taps:
            from .recurrent import ShortConvolution
            nm = self.names
            self.conv = ShortConvolution([(prefix + nm["q_conv"], n_heads * M * head_dim), (prefix + nm["k_conv"], n_kv_heads * M * head_dim),
                                          (prefix + nm["v_conv"], n_kv_heads * v_head_dim)], taps, act="none")
        self.w_in = self.w_o = None
        self.lam = 0.0
        self._tables_key = None
        self._sm_count = 0

    def _flash_takes(self) -> bool:
        from ..csrc import attention_fast
        return self.vd == self.MAPS * self.dk and attention_fast.supported(self.vd, self.MAPS * self.H // self.G)

    def kernel_libraries(self, bfloat16: bool):
        from ..csrc import attention_fast
        if not bfloat16 or not self._flash_takes():
            return ()
        return ("attention_flash", "attention_prefill_tc") if attention_fast.tc_prefill_supported(self.vd, self.MAPS * self.H // self.G) \
            else ("attention_flash",)

    def children(self):
        return tuple(p for p in (self.position, self.conv) if p is not None)

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, H, G, dk, vd, d, M = self.prefix, self.names, self.H, self.G, self.dk, self.vd, self.hidden, self.MAPS
        specs = {p + nm["q"]: ParamSpec((H * M * dk, d), MATRIX), p + nm["k"]: ParamSpec((G * M * dk, d), MATRIX),
                 p + nm["v"]: ParamSpec((G * vd, d), MATRIX), p + nm["o"]: ParamSpec((d, H * vd), MATRIX)}
        for key in ("lq1", "lk1", "lq2", "lk2"):
            specs[p + nm[key]] = ParamSpec((dk,), VECTOR)
        if self.gate:
            specs[p + nm["gate"]] = ParamSpec((H, d), MATRIX)
        return specs

    def cache_specs(self):
        pages = KVCacheSpec(self.G, self.MAPS * self.dk, self.window, self.vd)
        return [pages, self.conv.cache_spec()] if self.conv is not None else [pages]

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("q", "k", "v")] + ([tensors[p + nm["gate"]]] if self.gate else [])
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()     # one product: q, k, v and the heads' gates
        self.w_o = tensors[p + nm["o"]]
        l = [tensors[p + nm[key]].float() for key in ("lq1", "lk1", "lq2", "lk2")]
        # lambda in 32-bit, once: it is the same for every token
        self.lam = float((torch.exp((l[0] * l[1]).sum()) - torch.exp((l[2] * l[3]).sum()) + self.diff).item())
        if precision.compute == torch.bfloat16 and self._flash_takes():
            self._tables_key = ("paged_attention_items", self.window or 0, self.MAPS * self.H, self.G, self.vd, False, 0, False)
            self._sm_count = torch.cuda.get_device_properties(precision.device).multi_processor_count

    def step_tables_key(self):
        return self._tables_key

    def step_tables(self, ctx):
        return flash_step_tables(ctx, self.MAPS * self.H, self.G, self.vd, self.window or 0, 0, self._sm_count)

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n, dev, dt = xb.shape[0], xb.device, xb.dtype
        H, G, dk, vd, M, C = self.H, self.G, self.dk, self.vd, self.MAPS, self.channels
        pages = cache[0]
        proj = torch.empty((n, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        ops.gemm(xb, self.w_in, proj)
        x = proj[:, :C]
        if self.conv is not None:
            x = torch.empty((n, C), dtype=torch.float32, device=dev)
            self.conv.forward(proj[:, :C], ctx, cache[1], x)
        cos = sin = None
        rot = 0
        if self.position is not None:
            cos, sin, rot = self.position.tables()
        q = torch.empty((n, H * M * M * dk), dtype=dt, device=dev)
        ops.maps_rope_kv_write(x, q, cos, sin, rot, ctx.positions, ctx.slot_of_token, pages.block_table, pages.k_pages,
                               pages.v_pages, H, G, M, dk, pages.page_tokens, write_kv=write_cache)
        plan = flash_plan(ctx, self._tables_key) if dt == torch.bfloat16 else None
        att = torch.empty((n, M * H * vd), dtype=dt, device=dev)
        ops.paged_attention(q, pages.k_pages, pages.v_pages, pages.block_table, ctx.positions, ctx.slot_of_token, att,
                            M * H, G, M * dk, pages.page_tokens, self.window or 0, self.scale, plan=plan)
        og = torch.empty((n, H * vd), dtype=dt, device=dev)
        ops.diff_heads_out(att, proj[:, C:C + H] if self.gate else None, og, H, vd, self.lam, self.norm_eps, 1.0 - self.diff)
        ops.gemm(og, self.w_o, residual, accumulate=accumulate)


register_part("mixer", "differential_attention", DifferentialAttention)
