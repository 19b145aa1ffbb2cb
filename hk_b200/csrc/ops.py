"""Python face of the CUDA kernels: argument checks, kernel choice, launch on torch's
current stream.

Every function takes torch CUDA tensors, checks what the kernel assumes (device, dtype,
contiguity, sizes) and raises `KernelError` with a clear message when a kernel refuses a
shape; nothing falls back to the CPU or to a library.  Kernel choice (tensor-core GEMM or
generic GEMM, flash or generic attention) is by shape alone, never by batch content, and
can be pinned with `force()` by tests.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Optional

import torch

from . import build

F32, BF16 = 0, 1
_ERR_UNSUPPORTED = 100001


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, not {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, not {t.dim()}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


_launches = 0


def launch_count() -> int:
    """How many kernel launches this module has issued so far (for benchmarks' bookkeeping)."""
    return _launches


def count_launches(n: int) -> None:
    """Adds kernel launches made outside this module's wrappers (a replayed CUDA graph's nodes)."""
    global _launches
    _launches += n


def _check(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += launches
        return
    if code == _ERR_UNSUPPORTED:
        raise KernelError(f"{what}: the kernel refuses these sizes or types")
    raise KernelError(f"{what}: CUDA error {code}")


# ---- kernel choice --------------------------------------------------------------------

_forced = {"gemm": None, "attention": None}


def forced(kind: str) -> Optional[str]:
    """The kernel family pinned for `kind` ('gemm' or 'attention'), or None."""
    return _forced[kind]


@contextlib.contextmanager
def force(gemm: Optional[str] = None, attention: Optional[str] = None):
    """Pins the kernel family inside the block: gemm in {'generic','tc','smallm','stream'},
    attention in {'generic','flash','flash_cp'} ('flash_cp': the flash kernels without the TMA-fed decode
    variant).  A pinned kernel that refuses the shape raises."""
    old = dict(_forced)
    if gemm is not None:
        _forced["gemm"] = gemm
    if attention is not None:
        _forced["attention"] = attention
    try:
        yield
    finally:
        _forced.update(old)


# ---- embedding ------------------------------------------------------------------------


def _narrow_target(narrow: Optional[torch.Tensor], like: torch.Tensor, what: str):
    """The optional bfloat16 copy that a row-wise kernel writes beside its float32 result."""
    if narrow is None:
        return None
    _need(narrow, "narrow", torch.bfloat16, 2)
    if narrow.shape != like.shape:
        raise KernelError(f"{what}: the narrowed copy must have the result's shape")
    return narrow


def embedding(table: torch.Tensor, token_ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
              narrow: Optional[torch.Tensor] = None) -> None:
    """out[t, :] = table[token_ids[t], :] widened to float32, times `scale`; `narrow` (bfloat16, out's shape) receives
    the same rows rounded."""
    narrow = _narrow_target(narrow, out, "embedding")
    _need(table, "table", dims=2)
    _need(token_ids, "token_ids", torch.int32, 1)
    _need(out, "out", torch.float32, 2)
    n, d = out.shape
    if token_ids.shape[0] != n or table.shape[1] != d:
        raise KernelError(f"embedding: out {tuple(out.shape)} does not fit ids {tuple(token_ids.shape)} and table {tuple(table.shape)}")
    lib = build.load("elementwise")
    _check(lib.hk_embedding(_ptr(table), _dt(table), _ptr(token_ids), _ptr(out), n, d, table.shape[0],
                            ctypes.c_float(scale), _ptr(narrow), _stream()),
           "embedding")


# ---- rms norm -------------------------------------------------------------------------


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = x[rows[r] or r, :] * rsqrt(mean(x^2) + eps) * weight  (x, weight float32)."""
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    _need(out, "out", dims=2)
    d = x.shape[1]
    n_out = out.shape[0]
    if weight.shape[0] != d or out.shape[1] != d:
        raise KernelError("rms_norm: widths of x, weight and out differ")
    if rows is None:
        if n_out != x.shape[0]:
            raise KernelError("rms_norm: out has other rows than x")
    else:
        _need(rows, "rows", torch.int32, 1)
        if rows.shape[0] < n_out:
            raise KernelError("rms_norm: fewer row indices than output rows")
    lib = build.load("elementwise")
    _check(lib.hk_rms_norm(_ptr(x), _ptr(weight), _ptr(rows), _ptr(out), _dt(out), n_out, d,
                           ctypes.c_float(eps), _stream()), "rms_norm")


# ---- swiglu ---------------------------------------------------------------------------


GLU_ACTS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0, act: str = "silu", limit: float = 0.0,
           slope: float = 1.0) -> None:
    """out[t, j] = act(gate) * up for gate_up float32 [n, 2F]; act is silu or the tanh form of gelu; or, with act
    'swish_clamped', g sigmoid(slope g) (u + 1) with g = min(gate, limit) and u = clamp(up, -limit, limit).  With block = 0
    the row is laid out [F gates | F ups]; with block = b (dividing F) it is [b gates | b ups | b gates | ...]."""
    if act not in GLU_ACTS:
        raise KernelError(f"swiglu: activation {act!r} is not one of {', '.join(GLU_ACTS)}")
    _need(gate_up, "gate_up", torch.float32, 2)
    _need(out, "out", dims=2)
    n, f = out.shape
    block = block or f
    if gate_up.shape[0] != n or gate_up.shape[1] != 2 * f or f % block:
        raise KernelError("swiglu: gate_up must be [n, 2F] for out [n, F], and the block must divide F")
    lib = build.load("elementwise")
    _check(lib.hk_swiglu(_ptr(gate_up), _ptr(out), _dt(out), n, f, int(block), GLU_ACTS[act], ctypes.c_float(limit),
                         ctypes.c_float(slope), _stream()), "swiglu")


def _as_weights(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """A product runs in its weights' type: where a matrix is kept in 32-bit although the engine computes in
    bfloat16 (its file stored it so), the activations are widened for that product (and narrowed for the next)."""
    if a.dtype == w.dtype:
        return a
    if w.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"weights must be float32 or bfloat16, not {w.dtype}")
    return a.to(w.dtype)


def gemm_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, act: str = "silu", limit: float = 0.0,
                slope: float = 1.0) -> None:
    """out[M, F] = act(gate) * up (act: silu, the tanh form of gelu, or the clamped form of `swiglu` with its limit and
    slope) of a @ w_gate_up^T, w_gate_up [2F, K] = [F gate rows | F up rows].  Fused into
    the tensor-core product's epilogue when that takes the shape (a tile of the product then holds gate rows and
    the up rows that match them), else a product to float32 followed by the swiglu kernel."""
    _need(a, "a", dims=2)
    _need(w_gate_up, "w", dims=2)
    _need(out, "out", a.dtype, 2)
    if w_gate_up.dtype != a.dtype:              # weights kept in 32-bit on the bfloat16 path: this product runs in 32-bit
        wide = torch.empty(out.shape, dtype=w_gate_up.dtype, device=out.device)
        gemm_swiglu(_as_weights(a, w_gate_up), w_gate_up, wide, act, limit, slope)
        out.copy_(wide)
        return
    M, F = out.shape
    if a.shape[0] != M or w_gate_up.shape != (2 * F, a.shape[1]):
        raise KernelError("gemm_swiglu: shapes do not fit")
    if a.dtype == torch.bfloat16 and _forced["gemm"] in (None, "tc", "stream"):
        from . import gemm_fast
        if gemm_fast.run_swiglu(a, w_gate_up, out, _forced["gemm"], act=GLU_ACTS[act], limit=limit, slope=slope):
            return
    gu = torch.empty((M, 2 * F), dtype=torch.float32, device=a.device)
    gemm(a, w_gate_up, gu)
    swiglu(gu, out, 0, act, limit, slope)


# ---- per-head norm + rotation + cache write ---------------------------------------------


PAIRINGS = {"half": 0, "adjacent": 1}


def qk_norm_rope_kv_write(qkv, q_out, q_weight, k_weight, eps, cos, sin, rotary_dim, positions,
                          slot_of_token, block_table, k_pages, v_pages, n_heads, n_kv_heads, head_dim,
                          page_tokens, write_kv=True, bias=None, pairing="half", norm_after=False, tied_v=False) -> None:
    """Splits the fused projection qkv[n, (H+G)*hd + G*vd] (float32; vd = v_pages' width, hd unless the values have a
    width of their own): q heads are normalised (if
    q_weight), rotated (if rotary_dim > 0) and stored to q_out[n, H*hd]; k heads likewise and
    stored, with the v heads, into the token's cache page [page, G, page_tokens, hd].
    `bias` (float32 [(H+2G)*hd]) is added to the projection first.  `pairing`: "half" rotates dims
    (i, i + rotary_dim/2), "adjacent" dims (2i, 2i+1).  `norm_after`: the per-head norm comes behind the
    rotation, and a missing weight then means a weight of ones.  `tied_v`: qkv is [n, (H+G)*hd] and a token's
    value is its key as projected (before norm and rotation), of which the first v_pages.shape[-1] dims are kept."""
    if pairing not in PAIRINGS:
        raise KernelError(f"qk_norm_rope_kv_write: pairing {pairing!r} is neither 'half' nor 'adjacent'")
    if not isinstance(qkv, torch.Tensor) or not qkv.is_cuda or qkv.dtype != torch.float32 or qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("qkv must be a float32 CUDA matrix with unit column stride (it may be a column slice)")
    _need(q_out, "q_out", dims=2)
    n = qkv.shape[0]
    H, G, hd = n_heads, n_kv_heads, head_dim
    vd = int(v_pages.shape[3]) if write_kv else (hd if tied_v else (qkv.shape[1] - (H + G) * hd) // max(G, 1))
    width = (H + G) * hd + (0 if tied_v else G * vd)
    if bias is not None:
        _need(bias, "bias", torch.float32, 1)
        if bias.shape[0] != width:
            raise KernelError("qk_norm_rope_kv_write: bias must have one entry per projected column")
    if qkv.shape[1] != width or tuple(q_out.shape) != (n, H * hd):
        raise KernelError("qk_norm_rope_kv_write: qkv or q_out has the wrong shape")
    if head_dim > 256:
        raise KernelError(f"qk_norm_rope_kv_write: head_dim {head_dim} is above 256")
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _need(w, name, torch.float32, 1)
            if w.shape[0] != hd:
                raise KernelError(f"{name} must have head_dim entries")
    if rotary_dim > 0:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape or rotary_dim % 2 or rotary_dim > hd:
            raise KernelError("rotation tables must be [positions, rotary_dim/2]")
    _need(positions, "positions", torch.int32, 1)
    _need(slot_of_token, "slot_of_token", torch.int32, 1)
    if write_kv:
        _need(block_table, "block_table", torch.int32, 2)
        _need(k_pages, "k_pages", q_out.dtype, 4)
        _need(v_pages, "v_pages", q_out.dtype, 4)
        if tuple(k_pages.shape[1:]) != (G, page_tokens, hd) or tuple(v_pages.shape[:3]) != tuple(k_pages.shape[:3]) \
                or not 1 <= v_pages.shape[3] <= 256 or (v_pages.shape[3] > hd and tied_v):
            raise KernelError("cache pages must be [pages, G, page_tokens, head_dim] (values: their own width)")
    lib = build.load("elementwise")
    _check(lib.hk_qk_norm_rope_kv_write(
        _ptr(qkv), _ptr(q_out), _dt(q_out), _ptr(q_weight), _ptr(k_weight), ctypes.c_float(eps),
        _ptr(cos if rotary_dim > 0 else None), _ptr(sin if rotary_dim > 0 else None), int(rotary_dim),
        _ptr(positions), _ptr(slot_of_token), _ptr(block_table if write_kv else None),
        int(block_table.shape[1]) if write_kv else 0, _ptr(k_pages if write_kv else None),
        _ptr(v_pages if write_kv else None), n, H, G, hd, int(page_tokens), 1 if write_kv else 0, _ptr(bias),
        PAIRINGS[pairing], 1 if norm_after else 0, 1 if tied_v else 0, vd, ctypes.c_longlong(qkv.stride(0)), _stream()),
        "qk_norm_rope_kv_write")


def maps_rope_kv_write(x, q_out, cos, sin, rotary_dim: int, positions, slot_of_token, block_table, k_pages, v_pages,
                       n_heads: int, n_kv_heads: int, maps: int, key_dim: int, page_tokens: int, write_kv: bool = True) -> None:
    """For an attention whose heads carry `maps` score maps over the same values: splits the float32 row
    x[n, H*maps*dk | G*maps*dk | G*vd] (a column slice), turns q and k by position on the first `rotary_dim` dims of
    every map (dim i paired with i + rotary_dim/2), writes the queries as H*maps heads of maps*dk numbers (a map's query at
    its own place, zeros elsewhere) to q_out[n, H*maps*maps*dk] and the keys (a head's maps side by side) and values into
    the token's place in k_pages [pages, G, page_tokens, maps*dk] and v_pages [pages, G, page_tokens, vd]."""
    H, G, M, dk = n_heads, n_kv_heads, maps, key_dim
    _need(q_out, "q_out", dims=2)
    _need(v_pages, "v_pages", q_out.dtype, 4)
    _need(k_pages, "k_pages", q_out.dtype, 4)
    vd = int(v_pages.shape[3])
    ld = _cols(x, "x", (H + G) * M * dk + G * vd)
    n = x.shape[0]
    if tuple(q_out.shape) != (n, H * M * M * dk) or tuple(k_pages.shape[1:]) != (G, page_tokens, M * dk) \
            or tuple(v_pages.shape[:3]) != tuple(k_pages.shape[:3]):
        raise KernelError("maps_rope_kv_write: shapes do not fit")
    if rotary_dim > 0:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape or rotary_dim % 2 or rotary_dim > dk:
            raise KernelError("maps_rope_kv_write: rotation tables must be [positions, rotary_dim/2]")
    _need(positions, "positions", torch.int32, 1)
    _need(slot_of_token, "slot_of_token", torch.int32, 1)
    _need(block_table, "block_table", torch.int32, 2)
    lib = build.load("elementwise")
    _check(lib.hk_maps_rope_kv_write(
        _ptr(x), ctypes.c_longlong(ld), _ptr(q_out), _dt(q_out), _ptr(cos if rotary_dim > 0 else None),
        _ptr(sin if rotary_dim > 0 else None), int(rotary_dim), _ptr(positions), _ptr(slot_of_token), _ptr(block_table),
        int(block_table.shape[1]), _ptr(k_pages), _ptr(v_pages), n, H, G, M, dk, vd, int(page_tokens), 1 if write_kv else 0,
        _stream()), "maps_rope_kv_write")


def diff_heads_out(a, gate, out, n_heads: int, value_dim: int, lam: float, eps: float, out_scale: float = 1.0) -> None:
    """The heads of a differential attention: a[n, H*2*vd] holds, per head, the two maps' weighted values a1 | a2;
    o = a1 - lam * a2, out[t, h] = o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate[t, h]) (gate: a float32 column slice
    [n, H], or None).  a float32 or out's type; float32 arithmetic."""
    H, vd = n_heads, value_dim
    _need(a, "a", dims=2)
    _need(out, "out", dims=2)
    n = out.shape[0]
    ldg = 0
    if gate is not None:
        ldg = _cols(gate, "gate", H)
    if tuple(a.shape) != (n, 2 * H * vd) or tuple(out.shape) != (n, H * vd) or (gate is not None and gate.shape[0] != n) \
            or (a.dtype != torch.float32 and a.dtype != out.dtype):
        raise KernelError("diff_heads_out: shapes or types do not fit")
    lib = build.load("elementwise")
    _check(lib.hk_diff_heads_out(_ptr(a), _dt(a), _ptr(gate), ctypes.c_longlong(ldg), _ptr(out), _dt(out), n, H, vd,
                                 ctypes.c_float(lam), ctypes.c_float(eps), ctypes.c_float(out_scale), _stream()), "diff_heads_out")


# ---- matrix product -------------------------------------------------------------------


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out[t, :] += bias (both float32)."""
    _need(out, "out", torch.float32, 2)
    _need(bias, "bias", torch.float32, 1)
    if bias.shape[0] != out.shape[1]:
        raise KernelError("add_bias: one bias entry per output column")
    lib = build.load("elementwise")
    _check(lib.hk_add_bias(_ptr(out), _ptr(bias), out.shape[0], out.shape[1], _stream()), "add_bias")


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False,
         bias: Optional[torch.Tensor] = None) -> None:
    """out[M, N] (float32) = a[M, K] @ w[N, K]^T (+ out when `accumulate`) (+ bias[N], float32).
    a and w share a type: float32 (plain FMA) or bfloat16 (fp32 accumulation)."""
    if bias is not None:
        gemm(a, w, out, accumulate)
        add_bias(out, bias)
        return
    _need(a, "a", dims=2)
    _need(w, "w", dims=2)
    _need(out, "out", torch.float32, 2)
    a = _as_weights(a, w)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    choice = _forced["gemm"]
    if a.dtype == torch.bfloat16 and choice != "generic":
        from . import gemm_fast
        if gemm_fast.run(a, w, out, accumulate, choice):
            return
        if choice is not None:
            raise KernelError(f"gemm: the '{choice}' kernel refuses M={M} N={N} K={K}")
    lib = build.load("gemm_generic")
    _check(lib.hk_gemm_generic(_ptr(a), _ptr(w), _dt(a), _ptr(out), M, N, K, ctypes.c_longlong(K),
                               ctypes.c_longlong(K), ctypes.c_longlong(N), 1 if accumulate else 0, _stream()),
           "gemm")


# ---- attention ------------------------------------------------------------------------


def paged_attention(q, k_pages, v_pages, block_table, positions, slot_of_token, out, n_heads, n_kv_heads,
                    head_dim, page_tokens, window: int, scale: float, plan=None, sink: bool = False, sinks=None,
                    softcap: float = 0.0, chunk: int = 0, gate=None, gate_scale: float = 1.0) -> None:
    """out[t, h, :] = softmax_j(scale * q[t, h] . k[j]) v[j] over the keys j in
    [max(0, p - window + 1), p] (all of [0, p] when window <= 0) of the token's request, read
    through its block-table row; p = positions[t].  `plan` carries the per-request tiling the
    flash kernel wants; without it (or for sizes it refuses) the generic kernel runs.  Values may have a width of
    their own (v_pages [pages, G, page_tokens, vd], out [n, H*vd]; generic kernel).  `v_pages` None: the cache keeps
    one tensor per token and a token's value is the first vd = out.shape[1] / H dims of its key row.
    `sink`: one more term in the softmax's denominator, a key without a value whose score is 0, or `sinks[h]` when
    that float32 [H] tensor is given: p_j = exp(s_j) / (exp(sink) + sum exp(s_j)).
    `softcap` c > 0: scores become c * tanh(score / c).  `chunk` s > 0: a token sees no key before the start of its own
    block of s positions.  `gate` (a float32 column slice [n, H*vd] of a projection's output): the result is
    multiplied by gate_scale * sigmoid(gate)."""
    _need(q, "q", dims=2)
    _need(out, "out", q.dtype, 2)
    _need(k_pages, "k_pages", q.dtype, 4)
    if v_pages is not None:
        _need(v_pages, "v_pages", q.dtype, 4)
    _need(block_table, "block_table", torch.int32, 2)
    _need(positions, "positions", torch.int32, 1)
    _need(slot_of_token, "slot_of_token", torch.int32, 1)
    n = q.shape[0]
    H, G, hd = n_heads, n_kv_heads, head_dim
    if H < 1 or G < 1 or H % G != 0:
        raise KernelError(f"paged_attention: {H} heads are not a multiple of {G} groups")
    vd = int(v_pages.shape[3]) if v_pages is not None else int(out.shape[1]) // H
    if tuple(q.shape) != (n, H * hd) or tuple(out.shape) != (n, H * vd):
        raise KernelError("paged_attention: q must be [n, H*head_dim] and out [n, H*value_dim]")
    if tuple(k_pages.shape[1:]) != (G, page_tokens, hd) or (v_pages is not None and tuple(k_pages.shape[:3]) != tuple(v_pages.shape[:3])) \
            or vd < 1 or (v_pages is None and vd > hd):
        raise KernelError("paged_attention: cache pages must be [pages, G, page_tokens, head_dim]")
    if max(hd, vd) > 640:
        raise KernelError(f"paged_attention: a head of {max(hd, vd)} dims is above 640")
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, 1)
        if sinks.shape[0] != H or not sink:
            raise KernelError("paged_attention: sinks must hold one score per query head (and sink be set)")
    gate_ld = 0
    if gate is not None:
        gate_ld = _cols(gate, "gate", H * vd)
        if gate.shape[0] != n:
            raise KernelError("paged_attention: one row of gate logits per token")
    choice = _forced["attention"]
    if q.dtype == torch.bfloat16 and choice != "generic" and plan is not None and v_pages is not None and vd == hd:
        from . import attention_fast
        done = attention_fast.run(q, k_pages, v_pages, block_table, out, H, G, hd, page_tokens, window, scale, plan,
                                  allow_tma=choice != "flash_cp", sink=sink, sinks=sinks, softcap=softcap, chunk=chunk,
                                  gate=gate, gate_scale=gate_scale)
        if done:
            if gate is not None and done != attention_fast.GATED:
                sigmoid_gate(out, gate, out, gate_scale)
            return
        if choice is not None:
            raise KernelError(f"paged_attention: the '{choice}' kernel refuses head_dim={hd} page_tokens={page_tokens}")
    lib = build.load("attention_generic")
    _check(lib.hk_attention_generic(
        _ptr(q), _ptr(k_pages), _ptr(v_pages if v_pages is not None else k_pages), _dt(q), _ptr(block_table),
        int(block_table.shape[1]), _ptr(positions), _ptr(slot_of_token), _ptr(out), n, H, G, hd, int(page_tokens), int(window),
        ctypes.c_float(scale), vd, 1 if sink else 0, _ptr(sinks), ctypes.c_float(softcap), int(chunk),
        vd if v_pages is not None else hd, _ptr(gate), ctypes.c_longlong(gate_ld), ctypes.c_float(gate_scale), _stream()),
        "paged_attention")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out = x * scale * sigmoid(gate) element by element; x [n, W] float32 or out's type, gate a float32 column slice [n, W] of
    a projection's output (any row stride)."""
    _need(x, "x", dims=2)
    _need(out, "out", dims=2)
    n, W = out.shape
    ld = _cols(gate, "gate", W)
    if x.shape != out.shape or gate.shape[0] != n or (x.dtype != torch.float32 and x.dtype != out.dtype):
        raise KernelError("sigmoid_gate: shapes or types do not fit")
    lib = build.load("elementwise")
    _check(lib.hk_sigmoid_gate(_ptr(x), _dt(x), _ptr(gate), ctypes.c_longlong(ld), _ptr(out), _dt(out), n, W, ctypes.c_float(scale),
                               _stream()), "sigmoid_gate")


def latent_prep(proj, q_plain, q_full, c_weight, eps, cos, sin, rotary_dim, pairing, positions, slot_of_token, block_table,
                pages, n_heads, plain_dim, rot_dim, rank, page_tokens, write_kv=True) -> None:
    """What a token brings to a latent attention, from the fused projection proj float32 [n, >= H*(dn+dr) + r + dr]
    = [H query heads of (dn plain | dr to rotate) | r compressed dims | dr dims of the shared rotated key | ...]:
    q_plain[n, H*dn] takes the queries' plain parts, q_full[n, H*(r+dr)] their rotated parts in its last dr dims per
    head (the first r are left for the absorbed product), and the token's cache row [page, 0, place, r+dr] takes the
    compressed dims RMS-normed with `c_weight` and the rotated key part."""
    if pairing not in PAIRINGS:
        raise KernelError(f"latent_prep: pairing {pairing!r} is neither 'half' nor 'adjacent'")
    H, dn, dr, r = n_heads, plain_dim, rot_dim, rank
    _need(q_plain, "q_plain", dims=2)
    _need(q_full, "q_full", q_plain.dtype, 2)
    _need(c_weight, "c_weight", torch.float32, 1)
    n = q_plain.shape[0]
    if not isinstance(proj, torch.Tensor) or not proj.is_cuda or proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1 \
            or proj.shape[0] != n or proj.shape[1] < H * (dn + dr) + r + dr:
        raise KernelError("latent_prep: the projection must be float32 [n, >= H*(dn+dr) + r + dr] with unit column stride")
    if tuple(q_plain.shape) != (n, H * dn) or tuple(q_full.shape) != (n, H * (r + dr)) or c_weight.shape[0] != r:
        raise KernelError("latent_prep: q_plain, q_full or the norm weight has the wrong shape")
    if rotary_dim > 0:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape or rotary_dim % 2 or rotary_dim > dr:
            raise KernelError("rotation tables must be [positions, rotary_dim/2]")
    _need(positions, "positions", torch.int32, 1)
    _need(slot_of_token, "slot_of_token", torch.int32, 1)
    if write_kv:
        _need(block_table, "block_table", torch.int32, 2)
        _need(pages, "pages", q_plain.dtype, 4)
        if tuple(pages.shape[1:]) != (1, page_tokens, r + dr):
            raise KernelError("latent_prep: cache pages must be [pages, 1, page_tokens, rank + rot_dim]")
    lib = build.load("elementwise")
    _check(lib.hk_latent_prep(
        _ptr(proj), ctypes.c_longlong(proj.stride(0)), _ptr(q_plain), _ptr(q_full), _dt(q_plain), _ptr(c_weight),
        ctypes.c_float(eps), _ptr(cos if rotary_dim > 0 else None), _ptr(sin if rotary_dim > 0 else None), int(rotary_dim),
        PAIRINGS[pairing], _ptr(positions), _ptr(slot_of_token), _ptr(block_table if write_kv else None),
        int(block_table.shape[1]) if write_kv else 0, _ptr(pages if write_kv else None), n, H, dn, dr, r, int(page_tokens),
        1 if write_kv else 0, _stream()), "latent_prep")


def gemm_heads(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_heads: int, gate: Optional[torch.Tensor] = None) -> None:
    """One small product per head: out[t, h, :N] = a[t, h, :K] @ w[h]^T for w [H, N, K].  `a` and `out` are 3-D views
    [n, H, K] and [n, H, N] with any row and head strides and unit stride along the last dimension (so either may be
    a slice of wider heads).  out takes a's type or float32.  `gate` (a float32 column slice [n, H * N] of a projection's
    output): the result is multiplied by sigmoid(gate), head h reading columns h * N .. of it."""
    H = n_heads
    for name, t in (("a", a), ("out", out)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dim() != 3 or t.stride(2) != 1 or t.shape[1] != H:
            raise KernelError(f"gemm_heads: {name} must be a CUDA view [n, heads, width] with unit stride along the width")
    _need(w, "w", a.dtype, 3)
    n, _, K = a.shape
    N = out.shape[2]
    if tuple(w.shape) != (H, N, K) or out.shape[0] != n:
        raise KernelError("gemm_heads: shapes do not fit")
    gate_ld = 0
    if gate is not None:
        gate_ld = _cols(gate, "gate", H * N)
        if gate.shape[0] != n:
            raise KernelError("gemm_heads: one row of gate logits per row")
    if a.dtype == torch.bfloat16 and _forced["gemm"] != "generic":
        lib = build.load("gemm_heads")
        code = lib.hk_gemm_heads_mma(_ptr(a), _ptr(w), _ptr(out), _dt(out), n, N, K, H, ctypes.c_longlong(a.stride(0)),
                                     ctypes.c_longlong(a.stride(1)), ctypes.c_longlong(out.stride(0)),
                                     ctypes.c_longlong(out.stride(1)), _ptr(gate), ctypes.c_longlong(gate_ld), _stream())
        if code != _ERR_UNSUPPORTED:
            _check(code, "gemm_heads (mma)")
            return
    lib = build.load("gemm_generic")
    _check(lib.hk_gemm_heads(_ptr(a), _ptr(w), _dt(a), _ptr(out), _dt(out), n, N, K, H, ctypes.c_longlong(a.stride(0)),
                             ctypes.c_longlong(a.stride(1)), ctypes.c_longlong(out.stride(0)), ctypes.c_longlong(out.stride(1)),
                             _ptr(gate), ctypes.c_longlong(gate_ld), _stream()), "gemm_heads")


# ---- sampling -------------------------------------------------------------------------


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first maximum of logits[r, :] (float32)."""
    _need(logits, "logits", torch.float32, 2)
    _need(out, "out", torch.int32, 1)
    if out.shape[0] != logits.shape[0]:
        raise KernelError("argmax: one output per row")
    lib = build.load("sampling")
    _check(lib.hk_argmax(_ptr(logits), logits.shape[0], logits.shape[1], _ptr(out), _stream()), "argmax")


def adjust_logits(logits, offsets, ids, counts, bias, repeat_penalty, freq_penalty, presence_penalty) -> None:
    """Applies repetition, frequency and presence penalties and logit biases in place: entries
    offsets[r]..offsets[r+1] of (ids, counts, bias) belong to row r."""
    _need(logits, "logits", torch.float32, 2)
    rows = logits.shape[0]
    for name, t, dt, n in (("offsets", offsets, torch.int32, rows + 1), ("ids", ids, torch.int32, None),
                           ("counts", counts, torch.int32, ids.shape[0]), ("bias", bias, torch.float32, ids.shape[0]),
                           ("repeat_penalty", repeat_penalty, torch.float32, rows),
                           ("freq_penalty", freq_penalty, torch.float32, rows),
                           ("presence_penalty", presence_penalty, torch.float32, rows)):
        _need(t, name, dt, 1)
        if n is not None and t.shape[0] != n:
            raise KernelError(f"adjust_logits: {name} has {t.shape[0]} entries, expected {n}")
    lib = build.load("sampling")
    _check(lib.hk_adjust_logits(_ptr(logits), rows, logits.shape[1], _ptr(offsets), _ptr(ids), _ptr(counts), _ptr(bias),
                                _ptr(repeat_penalty), _ptr(freq_penalty), _ptr(presence_penalty), _stream()),
           "adjust_logits")


def sample(logits, temperature, top_k, top_p, min_p, seeds, counters, out) -> None:
    """One token per row by the chain top-k -> top-p -> min-p -> temperature -> draw; rows with
    temperature <= 0 take the first maximum.  seeds and counters are int64 per row."""
    _need(logits, "logits", torch.float32, 2)
    rows = logits.shape[0]
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
                        ("seeds", seeds, torch.int64), ("counters", counters, torch.int64), ("out", out, torch.int32)):
        _need(t, name, dt, 1)
        if t.shape[0] != rows:
            raise KernelError(f"sample: {name} must have one entry per row")
    lib = build.load("sampling")
    _check(lib.hk_sample(_ptr(logits), rows, logits.shape[1], _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p),
                         _ptr(seeds), _ptr(counters), _ptr(out), _stream()), "sample")


# ---- a layer that norms both sides of its sublayers --------------------------------------


def rms_norm_add(y: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor,
                 narrow: Optional[torch.Tensor] = None) -> None:
    """residual[r, :] += y[r, :] * rsqrt(mean(y^2) + eps) * weight (all float32): the norm behind a sublayer, fused
    with the residual sum.  `narrow` (bfloat16, residual's shape) receives the new residual rounded: the next
    sublayer's input where sublayers read the residual stream itself."""
    narrow = _narrow_target(narrow, residual, "rms_norm_add")
    _need(y, "y", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    _need(residual, "residual", torch.float32, 2)
    if y.shape != residual.shape or weight.shape[0] != y.shape[1]:
        raise KernelError("rms_norm_add: y, residual and weight do not fit")
    lib = build.load("elementwise")
    _check(lib.hk_rms_norm_add(_ptr(y), _ptr(weight), _ptr(residual), y.shape[0], y.shape[1], ctypes.c_float(eps), _ptr(narrow),
                               _stream()), "rms_norm_add")


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3 per row, N(v) = v / sqrt(mean(v^2) + eps), powers element by
    element; z float32 [n, F], coef float32 [4] on the device."""
    _need(z, "z", torch.float32, 2)
    _need(coef, "coef", torch.float32, 1)
    _need(out, "out", dims=2)
    if out.shape != z.shape or coef.shape[0] != 4:
        raise KernelError("polynorm: out must have z's shape and coef four entries")
    lib = build.load("elementwise")
    _check(lib.hk_polynorm(_ptr(z), _ptr(coef), _ptr(out), _dt(out), z.shape[0], z.shape[1], ctypes.c_float(eps), _stream()),
           "polynorm")


def _cols(x: torch.Tensor, name: str, width: int) -> int:
    """Checks a float32 column slice [n, width] of a row-major matrix; returns its row stride."""
    if not isinstance(x, torch.Tensor) or not x.is_cuda or x.dtype != torch.float32 or x.dim() != 2:
        raise KernelError(f"{name} must be a float32 CUDA matrix")
    if x.shape[1] != width or x.stride(1) != 1:
        raise KernelError(f"{name} must be [n, {width}] with unit column stride")
    return int(x.stride(0))


def tanh_cols(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = tanh(x) for a column slice x (float32, any row stride) of a fused projection's output."""
    _need(out, "out", dims=2)
    ld = _cols(x, "x", out.shape[1])
    if x.shape[0] != out.shape[0]:
        raise KernelError("tanh_cols: rows differ")
    lib = build.load("elementwise")
    _check(lib.hk_tanh_cols(_ptr(x), ctypes.c_longlong(ld), _ptr(out), _dt(out), out.shape[0], out.shape[1], _stream()), "tanh_cols")


# ---- recurrent mixers ---------------------------------------------------------------------


def delta_rule_scan(r, k, v, a_logit, w_logit, a_bias, w_bias, segments, state, out, n_heads: int, key_dim: int,
                    value_dim: int, decay_scale: float, key_eps: float) -> None:
    """Generalised delta rule over the rows of every segment (slot, first row, rows) of `segments` int32 [n_seg, 3]:
        S <- diag(d) S - (a * u) (u^T S) + k v^T,  out = S^T r      per head, S = state[slot, head] float32 [dk, dv]
    d = exp(-decay_scale * sigmoid(w_logit + w_bias)), a = sigmoid(a_logit + a_bias), u = k / sqrt(sum k^2 + key_eps).
    r, k, a_logit [n, H*dk] and v [n, H*dv] are float32 column slices of ONE matrix (one row stride); w_logit is
    float32 [n, H*dk] with its own.  out: float32 [n, H*dv]."""
    H, dk, dv = n_heads, key_dim, value_dim
    ld = _cols(r, "r", H * dk)
    if _cols(k, "k", H * dk) != ld or _cols(a_logit, "a_logit", H * dk) != ld or _cols(v, "v", H * dv) != ld:
        raise KernelError("delta_rule_scan: r, k, v and a_logit must be slices of one matrix")
    ldw = _cols(w_logit, "w_logit", H * dk)
    _need(a_bias, "a_bias", torch.float32, 1)
    _need(w_bias, "w_bias", torch.float32, 1)
    _need(segments, "segments", torch.int32, 2)
    _need(state, "state", torch.float32, 4)
    _need(out, "out", torch.float32, 2)
    n = r.shape[0]
    if tuple(state.shape[1:]) != (H, dk, dv) or tuple(out.shape) != (n, H * dv) or segments.shape[1] != 3 \
            or a_bias.shape[0] != H * dk or w_bias.shape[0] != H * dk:
        raise KernelError("delta_rule_scan: shapes do not fit")
    lib = build.load("recurrent")
    # what every token brings to the scan (decay, removal times unit key, unit key, key, receptance, value), made by a
    # kernel of its own for all tokens at once
    rec = torch.empty(n * H * int(lib.hk_delta_rule_record(dk, dv)), dtype=torch.float32, device=out.device)
    _check(lib.hk_delta_rule_scan(_ptr(r), _ptr(k), _ptr(v), _ptr(a_logit), ctypes.c_longlong(ld), _ptr(w_logit),
                                  ctypes.c_longlong(ldw), _ptr(a_bias), _ptr(w_bias), _ptr(segments), int(segments.shape[0]), n,
                                  _ptr(rec), _ptr(state), _ptr(out), H, dk, dv, ctypes.c_float(decay_scale),
                                  ctypes.c_float(key_eps), _stream()), "delta_rule_scan", launches=2)


def head_norm_gate(o, gate_logit, weight, eps: float, out, n_heads: int, value_dim: int) -> None:
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h]^2) + eps) * weight[h, :] * sigmoid(gate_logit[t, h, :])."""
    H, dv = n_heads, value_dim
    _need(o, "o", torch.float32, 2)
    ldg = _cols(gate_logit, "gate_logit", H * dv)
    _need(weight, "weight", torch.float32, 1)
    _need(out, "out", dims=2)
    if tuple(o.shape) != (out.shape[0], H * dv) or out.shape != o.shape or weight.shape[0] != H * dv:
        raise KernelError("head_norm_gate: shapes do not fit")
    lib = build.load("recurrent")
    _check(lib.hk_head_norm_gate(_ptr(o), _ptr(gate_logit), ctypes.c_longlong(ldg), _ptr(weight), _ptr(out), _dt(out),
                                 o.shape[0], H, dv, ctypes.c_float(eps), _stream()), "head_norm_gate")


def mingru_scan(proj, z_bias, x_bias, segments, state, out) -> None:
    """minGRU over the rows of every segment: proj float32 [n, 3W] = [z logits | candidate inputs | gate inputs];
    S <- (1 - z) S + z c, z = sigmoid(zl + z_bias), c = x + 1/2 (x >= 0) or sigmoid(x), x = xl + x_bias;
    out = S * silu(gate input).  state float32 [slots, W]."""
    _need(proj, "proj", torch.float32, 2)
    _need(segments, "segments", torch.int32, 2)
    _need(state, "state", torch.float32, 2)
    _need(out, "out", dims=2)
    W = state.shape[1]
    for name, b in (("z_bias", z_bias), ("x_bias", x_bias)):
        if b is not None:
            _need(b, name, torch.float32, 1)
            if b.shape[0] != W:
                raise KernelError(f"mingru_scan: {name} must have one entry per channel")
    if proj.shape[1] != 3 * W or tuple(out.shape) != (proj.shape[0], W) or segments.shape[1] != 3:
        raise KernelError("mingru_scan: shapes do not fit")
    lib = build.load("recurrent")
    _check(lib.hk_mingru_scan(_ptr(proj), ctypes.c_longlong(3 * W), _ptr(z_bias), _ptr(x_bias), _ptr(segments),
                              int(segments.shape[0]), _ptr(state), _ptr(out), _dt(out), W, _stream()), "mingru_scan")


def short_conv(x, weight, segments, tail, out, act: str = "silu") -> None:
    """out[t, c] = act(sum_j weight[c, j] * x[t - (taps - 1) + j, c]) over the rows of every segment (the last column
    of `weight` is the current token's); act 'silu' or 'none'.  Rows before a segment's first come from `tail` float32 [slots, taps - 1, C],
    the request's last taps - 1 inputs (zero at its start), which is moved on (with one tap: one row that is left alone).
    x and out: float32 column slices [n, C]."""
    C = int(weight.shape[0])
    ldx, ldy = _cols(x, "x", C), _cols(out, "out", C)
    _need(weight, "weight", torch.float32, 2)
    _need(segments, "segments", torch.int32, 2)
    _need(tail, "tail", torch.float32, 3)
    taps = int(weight.shape[1])
    if x.shape[0] != out.shape[0] or tuple(tail.shape[1:]) != (max(taps - 1, 1), C) or segments.shape[1] != 3 or taps < 1 \
            or act not in ("silu", "none"):
        raise KernelError("short_conv: shapes do not fit")
    lib = build.load("recurrent")
    _check(lib.hk_short_conv(_ptr(x), ctypes.c_longlong(ldx), _ptr(weight), _ptr(segments), int(segments.shape[0]), int(x.shape[0]),
                             _ptr(tail), _ptr(out), ctypes.c_longlong(ldy), C, taps, 1 if act == "silu" else 0, _stream()),
           "short_conv")


def gated_delta_scan(q, k, v, b_logit, a_logit, a_log, dt_bias, segments, state, out, n_heads: int, n_qk_heads: int,
                     key_dim: int, value_dim: int, q_scale: float, unit_eps: float) -> None:
    """Gated delta rule over the rows of every segment, per head, S = state[slot, head] float32 [dk, dv]:
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  out = S^T q
    with q, k made unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times q_scale, beta = sigmoid(b_logit),
    g = exp(-exp(a_log) * softplus(a_logit + dt_bias)).  q, k [n, G*dk] and v [n, H*dv]: float32 column slices of ONE
    matrix; b_logit, a_logit [n, H] slices of one; value head h reads query/key head h // (H/G).  out float32 [n, H*dv]."""
    H, G, dk, dv = n_heads, n_qk_heads, key_dim, value_dim
    ld = _cols(q, "q", G * dk)
    if _cols(k, "k", G * dk) != ld or _cols(v, "v", H * dv) != ld:
        raise KernelError("gated_delta_scan: q, k and v must be slices of one matrix")
    ldg = _cols(b_logit, "b_logit", H)
    if _cols(a_logit, "a_logit", H) != ldg:
        raise KernelError("gated_delta_scan: b_logit and a_logit must be slices of one matrix")
    _need(a_log, "a_log", torch.float32, 1)
    _need(dt_bias, "dt_bias", torch.float32, 1)
    _need(segments, "segments", torch.int32, 2)
    _need(state, "state", torch.float32, 4)
    _need(out, "out", torch.float32, 2)
    n = q.shape[0]
    if tuple(state.shape[1:]) != (H, dk, dv) or tuple(out.shape) != (n, H * dv) or segments.shape[1] != 3 \
            or a_log.shape[0] != H or dt_bias.shape[0] != H or H % G:
        raise KernelError("gated_delta_scan: shapes do not fit")
    lib = build.load("recurrent")
    rec = torch.empty(n * H * int(lib.hk_delta_rule_record(dk, dv)), dtype=torch.float32, device=out.device)
    _check(lib.hk_gated_delta_scan(_ptr(q), _ptr(k), _ptr(v), ctypes.c_longlong(ld), _ptr(b_logit), _ptr(a_logit),
                                   ctypes.c_longlong(ldg), _ptr(a_log), _ptr(dt_bias), _ptr(segments), int(segments.shape[0]), n,
                                   _ptr(rec), _ptr(state), _ptr(out), H, G, dk, dv, ctypes.c_float(q_scale),
                                   ctypes.c_float(unit_eps), _stream()), "gated_delta_scan", launches=2)


def retention_scan(q, k, v, cos, sin, rotary_dim: int, positions, decay, segments, state, out, n_heads: int, key_dim: int,
                   value_dim: int, k_scale: float) -> None:
    """Retention over the rows of every segment, per head, S = state[slot, head] float32 [dk, dv]:
        S <- decay[h] S + k v^T;  out = S^T q
    with q and k turned by position on their first `rotary_dim` dims (dim i paired with i + rotary_dim / 2; tables
    cos, sin float32 [positions, rotary_dim / 2]; 0: no rotation) and k then times k_scale.  q, k [n, H*dk] and v
    [n, H*dv]: float32 column slices of ONE matrix; decay float32 [H]; out float32 [n, H*dv]."""
    H, dk, dv = n_heads, key_dim, value_dim
    ld = _cols(q, "q", H * dk)
    if _cols(k, "k", H * dk) != ld or _cols(v, "v", H * dv) != ld:
        raise KernelError("retention_scan: q, k and v must be slices of one matrix")
    _need(decay, "decay", torch.float32, 1)
    _need(positions, "positions", torch.int32, 1)
    _need(segments, "segments", torch.int32, 2)
    _need(state, "state", torch.float32, 4)
    _need(out, "out", torch.float32, 2)
    n = q.shape[0]
    if rotary_dim > 0:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape or rotary_dim % 2 or rotary_dim > dk:
            raise KernelError("retention_scan: rotation tables must be [positions, rotary_dim/2]")
    if tuple(state.shape[1:]) != (H, dk, dv) or tuple(out.shape) != (n, H * dv) or segments.shape[1] != 3 \
            or decay.shape[0] != H or positions.shape[0] != n:
        raise KernelError("retention_scan: shapes do not fit")
    lib = build.load("recurrent")
    rec = torch.empty(n * H * int(lib.hk_delta_rule_record(dk, dv)), dtype=torch.float32, device=out.device)
    _check(lib.hk_retention_scan(_ptr(q), _ptr(k), _ptr(v), ctypes.c_longlong(ld), _ptr(cos if rotary_dim > 0 else None),
                                 _ptr(sin if rotary_dim > 0 else None), int(rotary_dim), _ptr(positions), _ptr(decay), _ptr(segments),
                                 int(segments.shape[0]), n, _ptr(rec), _ptr(state), _ptr(out), H, dk, dv, ctypes.c_float(k_scale),
                                 _stream()), "retention_scan", launches=2)


def mlstm_padded(value_dim: int) -> int:
    """The value size of the mLSTM's state and scan output: value_dim + 1 (the normaliser's column) rounded up to 4."""
    return (int(value_dim) + 1 + 3) & ~3


def mlstm_scan(q, k, v, i_logit, f_logit, i_bias, f_bias, segments, state, m_state, out, gates, n_heads: int, key_dim: int,
               value_dim: int, cap: float, q_scale: float) -> None:
    """Matrix memory with exponential gates over the rows of every segment, per head (S, n zero and m = 0 at a
    request's start): i = cap tanh((i_logit + i_bias) / cap), f = logsigmoid(cap tanh((f_logit + f_bias) / cap)),
        m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k alone.
    state float32 [slots, H, dk, dvp] holds S and, as column dv, n (dvp = mlstm_padded(dv)); m_state [slots, H].
    out float32 [n, H*dvp]: per head S^T (q q_scale) and, at column dv, n . (q q_scale); gates float32 [n, H, 3]
    receives (e^(f + m - m'), e^(i - m'), e^(-m')) per token.  q, k, v, i_logit, f_logit: slices of ONE float32 matrix."""
    H, dk, dv = n_heads, key_dim, value_dim
    dvp = mlstm_padded(dv)
    ld = _cols(q, "q", H * dk)
    if _cols(k, "k", H * dk) != ld or _cols(v, "v", H * dv) != ld or _cols(i_logit, "i_logit", H) != ld \
            or _cols(f_logit, "f_logit", H) != ld:
        raise KernelError("mlstm_scan: q, k, v and the gates' logits must be slices of one matrix")
    _need(i_bias, "i_bias", torch.float32, 1)
    _need(f_bias, "f_bias", torch.float32, 1)
    _need(segments, "segments", torch.int32, 2)
    _need(state, "state", torch.float32, 4)
    _need(m_state, "m_state", torch.float32, 2)
    _need(out, "out", torch.float32, 2)
    _need(gates, "gates", torch.float32, 3)
    n = q.shape[0]
    if tuple(state.shape[1:]) != (H, dk, dvp) or tuple(m_state.shape[1:]) != (H,) or tuple(out.shape) != (n, H * dvp) \
            or tuple(gates.shape) != (n, H, 3) or segments.shape[1] != 3 or i_bias.shape[0] != H or f_bias.shape[0] != H:
        raise KernelError("mlstm_scan: shapes do not fit")
    lib = build.load("recurrent")
    rec = torch.empty(n * H * int(lib.hk_delta_rule_record(dk, dvp)), dtype=torch.float32, device=out.device)
    _check(lib.hk_mlstm_scan(_ptr(q), _ptr(k), _ptr(v), _ptr(i_logit), _ptr(f_logit), ctypes.c_longlong(ld), _ptr(i_bias),
                             _ptr(f_bias), _ptr(segments), int(segments.shape[0]), n, _ptr(rec), _ptr(gates), _ptr(state),
                             _ptr(m_state), _ptr(out), H, dk, dv, ctypes.c_float(cap), ctypes.c_float(q_scale), _stream()),
           "mlstm_scan", launches=3)


def head_out_gate(o, gate_logit, weight, eps: float, out, n_heads: int, value_dim: int, act: str = "sigmoid",
                  gates=None, den_eps: float = 0.0) -> None:
    """out[t, h, :] = N(o[t, h, :dv] / den) * weight * act(gate_logit[t, h, :]), N = x / sqrt(mean(x^2) + eps) over the
    head's dv values.  o float32 [n, H*ldo] with ldo >= dv floats per head; weight [H*dv], or [dv] shared by the heads, or
    None (a norm without a weight); act 'sigmoid' or 'silu'.  With `gates` (float32 [n, H, 3], as `mlstm_scan` leaves it) den = max(|o[t, h, dv]|,
    gates[t, h, 2]) + den_eps; without, den = 1."""
    H, dv = n_heads, value_dim
    _need(o, "o", torch.float32, 2)
    ldg = _cols(gate_logit, "gate_logit", H * dv)
    if weight is not None:
        _need(weight, "weight", torch.float32, 1)
    _need(out, "out", dims=2)
    n = out.shape[0]
    if o.shape[0] != n or o.shape[1] % H or tuple(out.shape) != (n, H * dv) or (weight is not None and weight.shape[0] not in (dv, H * dv)) \
            or gate_logit.shape[0] != n or act not in ("sigmoid", "silu"):
        raise KernelError("head_out_gate: shapes do not fit")
    ldo = o.shape[1] // H
    if gates is not None:
        _need(gates, "gates", torch.float32, 3)
        if tuple(gates.shape) != (n, H, 3):
            raise KernelError("head_out_gate: gates must be [n, H, 3]")
    shared = 1 if (weight is not None and weight.shape[0] == dv and H > 1) else 0
    lib = build.load("recurrent")
    _check(lib.hk_head_out_gate(_ptr(o), int(ldo), _ptr(gate_logit), ctypes.c_longlong(ldg), _ptr(weight), shared,
                                0 if act == "sigmoid" else 1, _ptr(gates), ctypes.c_float(den_eps), _ptr(out), _dt(out), n, H, dv,
                                ctypes.c_float(eps), _stream()), "head_out_gate")


# ---- small element-wise kernels of layers with several streams -------------------------------


def scaled_sum(out, a, alpha: float, b=None, beta: float = 0.0, accumulate: bool = True) -> None:
    """out (+)= alpha * a + beta * b, all float32 of one shape (b may be absent); stored instead of added without
    `accumulate`."""
    _need(out, "out", torch.float32)
    _need(a, "a", torch.float32)
    if b is not None:
        _need(b, "b", torch.float32)
    if a.shape != out.shape or (b is not None and b.shape != out.shape):
        raise KernelError("scaled_sum: shapes differ")
    lib = build.load("elementwise")
    _check(lib.hk_scaled_sum(_ptr(out), _ptr(a), ctypes.c_float(alpha), _ptr(b), ctypes.c_float(beta),
                             ctypes.c_longlong(out.numel()), 1 if accumulate else 0, _stream()), "scaled_sum")


def narrow(x, out) -> None:
    """out = x (float32) rounded to out's type, element by element."""
    _need(x, "x", torch.float32)
    _need(out, "out")
    if x.shape != out.shape:
        raise KernelError("narrow: shapes differ")
    lib = build.load("elementwise")
    _check(lib.hk_narrow(_ptr(x), _ptr(out), _dt(out), ctypes.c_longlong(x.numel()), _stream()), "narrow")


def token_gate(z, table, col0: int, token_ids, out, act: str = "gelu_tanh") -> None:
    """out[t, j] = act(z[t, j]) * table[token_ids[t], col0 + j] for the W = out.shape[1] columns from col0 on; z a
    float32 column slice [n, W]; act 'gelu_tanh' or 'silu'."""
    _need(out, "out", dims=2)
    n, W = out.shape
    ld = _cols(z, "z", W)
    _need(table, "table", dims=2)
    _need(token_ids, "token_ids", torch.int32, 1)
    if z.shape[0] != n or token_ids.shape[0] != n or act not in ("gelu_tanh", "silu"):
        raise KernelError("token_gate: shapes do not fit")
    lib = build.load("elementwise")
    _check(lib.hk_token_gate(_ptr(z), ctypes.c_longlong(ld), _ptr(table), _dt(table), ctypes.c_longlong(table.shape[1]), int(col0),
                             _ptr(token_ids), _ptr(out), _dt(out), n, W, 0 if act == "gelu_tanh" else 1, _stream()), "token_gate")


# ---- routed feed-forward -------------------------------------------------------------------


def route_tile_rows() -> int:
    """Rows per tile of the grouped products."""
    return int(build.load("routed").hk_route_tile_rows())


def route_topk(x, w_router, ids, weights, scores: str = "softmax", correction=None, groups: int = 0, keep: int = 0,
               scale: float = 1.0, norm_eps: float = 0.0, extra_out=None) -> None:
    """Per row of x [n, d]: the `top` = ids.shape[1] largest of the E float32 router logits x . w_router[e]
    (w_router float32 [E, d]; the lower index wins a tie), and the softmax over the chosen logits.
    scores 'sigmoid': every expert's score is s = sigmoid(logit); the choice is made on s + correction (float32 [E], or
    None), among the experts of the best `keep` of `groups` equal groups of neighbours when groups > 0 (a group's score: the
    sum of its two largest choice scores; the others count as minus infinity); weights = s / (sum of the chosen s +
    norm_eps) * scale.  `extra_out` float32 [n, X]: w_router has X more rows behind the experts', and the sigmoids of their
    logits are written there."""
    _need(x, "x", dims=2)
    _need(w_router, "w_router", torch.float32, 2)
    _need(ids, "ids", torch.int32, 2)
    _need(weights, "weights", torch.float32, 2)
    n, d = x.shape
    extra = 0
    if extra_out is not None:
        _need(extra_out, "extra_out", torch.float32, 2)
        extra = int(extra_out.shape[1])
        if extra_out.shape[0] != n:
            raise KernelError("route_topk: one row of extra_out per row of x")
    E = int(w_router.shape[0]) - extra
    if w_router.shape[1] != d or ids.shape[0] != n or ids.shape != weights.shape or scores not in ("softmax", "sigmoid") or E < 1:
        raise KernelError("route_topk: shapes do not fit")
    if correction is not None:
        _need(correction, "correction", torch.float32, 1)
        if correction.shape[0] != E:
            raise KernelError("route_topk: one correction per expert")
    lib = build.load("routed")
    _check(lib.hk_route_topk(_ptr(x), _dt(x), _ptr(w_router), _ptr(ids), _ptr(weights), n, d, E, ids.shape[1],
                             1 if scores == "sigmoid" else 0, _ptr(correction), int(groups), int(keep), ctypes.c_float(scale),
                             ctypes.c_float(norm_eps), extra, _ptr(extra_out), _stream()), "route_topk")


def route_sort(ids, n_experts: int, offsets, perm, inv, tiles) -> None:
    """Lays the (row, choice) pairs out by expert: offsets int32 [E+1], perm [pairs] (sorted place -> pair), inv [pairs]
    (pair -> sorted place), tiles int32 [max_tiles, 2] = (expert, first sorted place) of every tile of
    `route_tile_rows()` rows, -1 for unused tiles."""
    for name, t in (("ids", ids), ("offsets", offsets), ("perm", perm), ("inv", inv), ("tiles", tiles)):
        _need(t, name, torch.int32)
    pairs = ids.numel()
    if offsets.numel() != n_experts + 1 or perm.numel() != pairs or inv.numel() != pairs or tiles.dim() != 2 or tiles.shape[1] != 2:
        raise KernelError("route_sort: shapes do not fit")
    lib = build.load("routed")
    _check(lib.hk_route_sort(_ptr(ids), pairs, n_experts, _ptr(offsets), _ptr(perm), _ptr(inv), _ptr(tiles), tiles.shape[0],
                             _stream()), "route_sort")


def grouped_gemm(a, w, out, tiles, offsets, perm, top: int, gather: bool, gated: bool) -> None:
    """A product per expert over the sorted rows.  w [E, N, K] (gated: [E, 2N, K] = N gate rows then N up rows);
    row p of the product reads a[perm[p] // top] (gather) or a[p]; out[p, :N] = a . w[e]^T in float32, or
    silu(gate) * up in a's type when gated."""
    _need(a, "a", dims=2)
    _need(w, "w", a.dtype, 3)
    _need(out, "out", dims=2)
    K = a.shape[1]
    N = out.shape[1]
    if w.shape[2] != K or w.shape[1] != (2 * N if gated else N) or out.dtype != (a.dtype if gated else torch.float32):
        raise KernelError("grouped_gemm: shapes or types do not fit")
    lib = build.load("routed")
    _check(lib.hk_grouped_gemm(_ptr(a), _ptr(w), _dt(a), _ptr(out), _ptr(tiles), tiles.shape[0], _ptr(offsets), _ptr(perm),
                               int(top), 1 if gather else 0, N, K, 1 if gated else 0, _stream()), "grouped_gemm")


def route_combine(ys, inv, weights, y, accumulate: bool = False, shared=None, shared_gate=None) -> None:
    """y[t, :] (+)= sum_k weights[t, k] * ys[inv[t, k], :], the choices in their order (all float32); with `shared`
    (float32 [n, d]) also + shared_gate[t] * shared[t, :] (shared_gate float32 [n] or [n, 1]; None: 1)."""
    _need(ys, "ys", torch.float32, 2)
    _need(inv, "inv", torch.int32)
    _need(weights, "weights", torch.float32, 2)
    _need(y, "y", torch.float32, 2)
    n, top = weights.shape
    if y.shape[0] != n or ys.shape[1] != y.shape[1] or inv.numel() != n * top or ys.shape[0] < n * top:
        raise KernelError("route_combine: shapes do not fit")
    if shared is not None:
        _need(shared, "shared", torch.float32, 2)
        if shared.shape != y.shape or (shared_gate is not None and (shared_gate.dtype != torch.float32 or shared_gate.numel() != n
                                                                    or not shared_gate.is_contiguous())):
            raise KernelError("route_combine: the shared result must be [n, d] and its gate [n]")
    lib = build.load("routed")
    _check(lib.hk_route_combine(_ptr(ys), _ptr(inv), _ptr(weights), _ptr(y), n, y.shape[1], top, 1 if accumulate else 0,
                                _ptr(shared), _ptr(shared_gate if shared is not None else None), _stream()), "route_combine")


def route_sort_padded(ids, n_experts: int, pad: int, perm, inv, groups) -> None:
    """The layout for the tcgen05 grouped product: every expert's rows start on a multiple of `pad`.  perm int32 [M_max]
    (sorted place -> pair, -1 for padding), inv [pairs], groups [M_max / pad] (tile -> expert or -1);
    M_max >= pairs + E * (pad - 1) and a multiple of pad."""
    for name, t in (("ids", ids), ("perm", perm), ("inv", inv), ("groups", groups)):
        _need(t, name, torch.int32)
    pairs, m_max = ids.numel(), perm.numel()
    if inv.numel() != pairs or groups.numel() * pad != m_max:
        raise KernelError("route_sort_padded: shapes do not fit")
    lib = build.load("routed")
    _check(lib.hk_route_sort_padded(_ptr(ids), pairs, n_experts, int(pad), _ptr(perm), _ptr(inv), _ptr(groups), m_max, _stream()),
           "route_sort_padded")


def route_gather(x, perm, top: int, xs) -> None:
    """xs[p, :] = x[perm[p] // top, :] (zeros where perm[p] < 0), bfloat16 rows of a multiple of 8 elements."""
    _need(x, "x", torch.bfloat16, 2)
    _need(xs, "xs", torch.bfloat16, 2)
    _need(perm, "perm", torch.int32, 1)
    if xs.shape[0] != perm.shape[0] or xs.shape[1] != x.shape[1]:
        raise KernelError("route_gather: shapes do not fit")
    lib = build.load("routed")
    _check(lib.hk_route_gather(_ptr(x), _ptr(perm), int(top), _ptr(xs), xs.shape[0], xs.shape[1], _stream()), "route_gather")


def grouped_gemm_tc(a, w, out, groups, gated: bool) -> bool:
    """The grouped product on the tcgen05 kernel: a bf16 [M, K] in tiles of 128 rows, tile t belonging to expert groups[t]
    (-1: skipped); w bf16 [E, N, K] (gated: [E, 2N, K]); out float32 [M, N], or bf16 silu(gate) * up when gated.  False when
    the kernel refuses the shape."""
    from . import gemm_fast
    return gemm_fast.run_grouped(a, w, out, groups, gated)
