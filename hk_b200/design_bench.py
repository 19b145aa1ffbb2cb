"""Throughput of a model design beside the closest existing one at equal size (`bench.py --design NAME`).

For each size: a prompt of 2,048 tokens in one step (tokens/s) and decode steps at batch 8 and 64 over 2,048-token
contexts (tokens/s), through `Engine.step` with random weights in bfloat16, timed on the device with CUDA events
(warm-up first; a prefill reads or writes far more than L2 holds, a decode step streams every weight).  Then the
design's own kernels one by one at that size, each with the bytes it must move and the floating-point operations
it must do, so that its distance from the roofline (the larger of bytes / measured copy bandwidth and operations /
peak) can be read beside the like kernel of the other model.  L2 is flushed between the timed launches of a kernel.
"""
from __future__ import annotations

import json
import math
import sys
import time

FP32_TFLOPS = 2 * 148 * 128 * 1.9e-3        # fp32 FMA peak of 148 SMs x 128 lanes at 1.9 GHz (nominal): the scans' ceiling


def kedanex_shape(width: int, groups: int = 2, vocab: int = 32000, window: int = 1024) -> dict:
    """Layer sizes that resemble a real model's: delta rule with heads of 64, attention with heads of 128 and four
    query heads per key head, a minGRU as wide as the model, a dense feed-forward of three times the width and eight
    experts of half the width of which two are used; one layer of every group runs with the first layer's tensors."""
    heads64, heads128 = width // 64, width // 128
    delta = {"type": "general_delta", "mixer": {"dim": 64, "heads": heads64, "decay_rank": 64}}
    att = {"type": "attention", "mixer": {"dim": 128, "heads": heads128, "kv_heads": max(1, heads128 // 4), "vdim": 128,
                                          "mask": {"size": window}, "rot": {"base": 1000000.0, "dims": 128},
                                          "scale": 1.0 / math.sqrt(128.0)}}
    gru = {"type": "mingru", "mixer": {"width": width}}
    dense = {"kind": "dense", "ff": 3 * width}
    moe = {"kind": "moe", "expert": {"ff": width // 2}, "router": {"experts": 8, "top": 2}}
    layers = []
    for g in range(groups):
        first = len(layers)
        layers += [dict(delta, mlp=dense), dict(att, mlp=moe), dict(gru, mlp=moe), dict(delta, mlp=dense, weights_of=first)]
    return {"architecture": "Kedanex", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "layers": layers,
            "initializer_range": 0.02}


def qwen3_shape(width: int, layers: int, vocab: int = 32000) -> dict:
    return dict(architectures=["Qwen3ForCausalLM"], hidden_size=width, num_hidden_layers=layers, intermediate_size=3 * width,
                num_attention_heads=width // 128, num_key_value_heads=max(1, width // 512), head_dim=128, vocab_size=vocab,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=8192,
                initializer_range=0.02)


def _events():
    import torch
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def model_points(raw: dict, prompt: int, batches, steps: int, warmup: int, reps: int) -> dict:
    import numpy as np
    import torch

    from .config import config_from_dict
    from .csrc import ops
    from .engine import Engine, StepEntry
    cfg = config_from_dict(raw)
    rng = np.random.default_rng(3)
    vocab = cfg.vocab_size
    out = {}
    per_req = -(-(prompt + warmup + steps + 8) // 64) * 64
    for batch in batches:
        eng = Engine(config=cfg, random_seed=5, dtype="bfloat16", max_tokens=batch * per_req, page_tokens=64, max_requests=batch,
                     max_context=per_req, max_batch_tokens=max(prompt, batch))
        if "params" not in out:
            out["params"] = int(sum(int(np.prod(s.shape)) for s in eng.model.param_specs().values()))
        if "prefill" not in out:
            ids = rng.integers(0, vocab, prompt).tolist()
            times = []
            for i in range(reps + 2):
                eng.open_request("p")
                a, b = _events()
                torch.cuda.synchronize()
                a.record()
                eng.step([StepEntry("p", ids, [prompt - 1])])
                b.record()
                torch.cuda.synchronize()
                eng.close_request("p")
                if i > 1:
                    times.append(a.elapsed_time(b))
            ms = float(np.median(times))
            out["prefill"] = {"tokens": prompt, "ms": ms, "tok_s": prompt / ms * 1e3}
        names = [f"d{i}" for i in range(batch)]
        for r in names:
            eng.open_request(r)
        group = max(1, eng.max_batch_tokens // prompt)
        for i in range(0, batch, group):
            eng.step([StepEntry(r, rng.integers(0, vocab, prompt).tolist(), []) for r in names[i:i + group]])
        toks = rng.integers(0, vocab, (warmup + steps, batch))
        pick = torch.empty(batch, dtype=torch.int32, device=eng.device)

        def one(s):
            ops.argmax(eng.step([StepEntry(r, [int(toks[s, i])], [0]) for i, r in enumerate(names)]), pick)

        for s in range(warmup):
            one(s)
        a, b = _events()
        torch.cuda.synchronize()
        l0 = ops.launch_count()
        a.record()
        for s in range(warmup, warmup + steps):
            one(s)
        b.record()
        torch.cuda.synchronize()
        eng.check_kernel_status()
        ms = a.elapsed_time(b) / steps
        out[f"decode_b{batch}"] = {"ms": ms, "tok_s": batch / ms * 1e3, "launches_per_step": (ops.launch_count() - l0) / steps}
        for r in names:
            eng.close_request(r)
        del eng
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    return out


def _time_kernel(fn, reps: int = 7, replay: bool = False):
    """Median device time in microseconds of `fn()`, L2 flushed before every timed call.  `replay`: the call is captured
    in a CUDA graph once and the graph's replay is timed, as decode steps run: the host's part of the call is left out."""
    import torch
    flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device="cuda")
    if replay:
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        fn = graph.replay
    times = []
    for i in range(reps + 3):
        flush.fill_(float(i))
        a, b = _events()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(a.elapsed_time(b) * 1e3)
    times.sort()
    return times[len(times) // 2]


def kernel_points(width: int, n: int, peaks: dict) -> dict:
    """The design's kernels alone at `n` rows of a layer of this width, and the like kernels of the Qwen3 decoder."""
    import numpy as np
    import torch

    from .csrc import ops
    dev = "cuda"
    bw, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    out = {}

    def note(name, us, nbytes, flops, peak_flops, like=None):
        floor = max(nbytes / bw, flops / peak_flops if peak_flops else 0.0) * 1e6
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "flops": int(flops), "roofline_us": round(floor, 2),
                     "of_roofline": round(floor / us, 3), **({"like": like} if like else {})}

    def segs(count, rows):
        return torch.tensor([[i, i * rows, rows] for i in range(count)], dtype=torch.int32, device=dev)

    # ---- delta rule scan: one request of n rows; and n requests of one row (a decode step)
    H, dk = width // 64, 64
    K = H * dk
    proj = torch.randn(n, 4 * K, device=dev) * 0.5
    wl = torch.randn(n, K, device=dev)
    ab, wb = torch.zeros(K, device=dev), torch.zeros(K, device=dev)
    o = torch.empty(n, K, device=dev)
    for label, count, rows in (("delta_rule_scan (1 request)", 1, n), ("delta_rule_scan (8 requests)", 8, n // 8),
                               ("delta_rule_scan (decode, 64 requests)", 64, 1)):
        state = torch.zeros(count, H, dk, dk, device=dev)
        m = count * rows
        sg = segs(count, rows)
        us = _time_kernel(lambda: ops.delta_rule_scan(proj[:m, :K], proj[:m, K:2 * K], proj[:m, 2 * K:3 * K], proj[:m, 3 * K:], wl[:m], ab,
                                                      wb, sg, state, o[:m], H, dk, dk, math.exp(-0.5), 1e-6))
        note(label, us, 4 * (6 * m * K + 2 * count * H * dk * dk), 8.0 * m * H * dk * dk, FP32_TFLOPS * 1e12,
             like="paged attention (same rows)")
    g = torch.randn(n, K, device=dev)
    og = torch.empty(n, K, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.head_norm_gate(o, g, torch.ones(K, device=dev), 1e-5, og, H, dk))
    note("head_norm_gate", us, n * K * (4 + 4 + 2), 0, 0, like="rms_norm")
    # ---- minGRU scan
    proj3 = torch.randn(n, 3 * width, device=dev)
    outb = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
    zb = torch.zeros(width, device=dev)
    for label, count, rows in (("mingru_scan (1 request)", 1, n), ("mingru_scan (8 requests)", 8, n // 8), ("mingru_scan (decode, 64 requests)", 64, 1)):
        state = torch.zeros(count, width, device=dev)
        m = count * rows
        sg = segs(count, rows)
        us = _time_kernel(lambda: ops.mingru_scan(proj3[:m], zb, zb, sg, state, outb[:m]))
        note(label, us, m * width * (12 + 2), 0, 0, like="swiglu / rms_norm (row-wise)")
    # ---- norms and the polynomial activation
    x = torch.randn(n, width, device=dev)
    res = torch.randn(n, width, device=dev)
    wn = torch.ones(width, device=dev)
    us = _time_kernel(lambda: ops.rms_norm_add(x, wn, 1e-5, res))
    note("rms_norm_add", us, n * width * 12, 0, 0, like="rms_norm")
    xb = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.rms_norm(x, wn, 1e-5, xb))
    note("rms_norm (Qwen3 and this design)", us, n * width * 6, 0, 0)
    F = 3 * width
    z = torch.randn(n, F, device=dev)
    hb = torch.empty(n, F, dtype=torch.bfloat16, device=dev)
    coef = torch.ones(4, device=dev)
    us = _time_kernel(lambda: ops.polynorm(z, coef, 1e-5, hb))
    note("polynorm", us, n * F * 6, 0, 0, like="swiglu")
    gu = torch.randn(n, 2 * F, device=dev)
    us = _time_kernel(lambda: ops.swiglu(gu, hb))
    note("swiglu (Qwen3, unfused form)", us, n * F * 10, 0, 0)
    # ---- routed feed-forward: route, sort, the two grouped products, combine
    E, top, Fe = 8, 2, width // 2
    xb.copy_(torch.randn(n, width, device=dev))
    wr = torch.randn(E, width, device=dev) * 0.1
    ids = torch.empty(n, top, dtype=torch.int32, device=dev)
    wts = torch.empty(n, top, device=dev)
    us = _time_kernel(lambda: ops.route_topk(xb, wr, ids, wts))
    note("route_topk", us, n * width * 2 + E * width * 4, 2.0 * n * E * width, FP32_TFLOPS * 1e12)
    pairs = n * top
    tile_rows = ops.route_tile_rows()
    max_tiles = pairs // tile_rows + min(E, pairs)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    perm = torch.empty(pairs, dtype=torch.int32, device=dev)
    inv = torch.empty(pairs, dtype=torch.int32, device=dev)
    tiles = torch.empty(max_tiles, 2, dtype=torch.int32, device=dev)
    us = _time_kernel(lambda: ops.route_sort(ids, E, offsets, perm, inv, tiles))
    note("route_sort", us, pairs * 16, 0, 0)
    wgu = (torch.randn(E, 2 * Fe, width, device=dev) * 0.02).bfloat16()
    wd = (torch.randn(E, width, Fe, device=dev) * 0.02).bfloat16()
    h = torch.empty(pairs, Fe, dtype=torch.bfloat16, device=dev)
    ys = torch.empty(pairs, width, device=dev)
    used = min(E, pairs)
    us = _time_kernel(lambda: ops.grouped_gemm(xb, wgu, h, tiles, offsets, perm, top, gather=True, gated=True))
    note("grouped gate/up product + SwiGLU (mma.sync)", us, used * 2 * Fe * width * 2 + n * width * 2 + pairs * Fe * 2, 2.0 * pairs * 2 * Fe * width, tc,
         like="gate/up product with SwiGLU epilogue (same FLOPs)")
    us = _time_kernel(lambda: ops.grouped_gemm(h, wd, ys, tiles, offsets, perm, top, gather=False, gated=False))
    note("grouped down product (mma.sync)", us, used * Fe * width * 2 + pairs * (Fe * 2 + width * 4), 2.0 * pairs * Fe * width, tc,
         like="down product (same FLOPs)")
    if pairs >= 1024:
        # the form that prompt-sized steps take: rows gathered into padded expert order, both products on the tcgen05 kernel
        from .csrc import gemm_fast
        pad = gemm_fast.GROUPED_ROWS
        m_max = -(-(pairs + E * (pad - 1)) // pad) * pad
        perm_p = torch.empty(m_max, dtype=torch.int32, device=dev)
        inv_p = torch.empty(pairs, dtype=torch.int32, device=dev)
        groups = torch.empty(m_max // pad, dtype=torch.int32, device=dev)
        us = _time_kernel(lambda: ops.route_sort_padded(ids, E, pad, perm_p, inv_p, groups))
        note("route_sort_padded", us, pairs * 16, 0, 0)
        xs = torch.empty(m_max, width, dtype=torch.bfloat16, device=dev)
        us = _time_kernel(lambda: ops.route_gather(xb, perm_p, top, xs))
        note("route_gather", us, (n + m_max) * width * 2, 0, 0)
        hp = torch.empty(m_max, Fe, dtype=torch.bfloat16, device=dev)
        ysp = torch.empty(m_max, width, device=dev)
        us = _time_kernel(lambda: ops.grouped_gemm_tc(xs, wgu, hp, groups, gated=True))
        note("grouped gate/up product + SwiGLU (tcgen05)", us, used * 2 * Fe * width * 2 + pairs * (width + Fe) * 2, 2.0 * pairs * 2 * Fe * width, tc,
             like="gate/up product with SwiGLU epilogue (same FLOPs)")
        us = _time_kernel(lambda: ops.grouped_gemm_tc(hp, wd, ysp, groups, gated=False))
        note("grouped down product (tcgen05)", us, used * Fe * width * 2 + pairs * (Fe * 2 + width * 4), 2.0 * pairs * Fe * width, tc,
             like="down product (same FLOPs)")
    y = torch.empty(n, width, device=dev)
    us = _time_kernel(lambda: ops.route_combine(ys, inv, wts, y))
    note("route_combine", us, pairs * width * 4 + n * width * 4, 0, 0)
    # the like products of the dense decoder: the same FLOPs as the routed pair (pairs rows, Fe wide)
    wq = (torch.randn(2 * Fe, width, device=dev) * 0.02).bfloat16()
    a2 = torch.randn(pairs, width, device=dev).bfloat16()
    us = _time_kernel(lambda: ops.gemm_swiglu(a2, wq, h))
    note("dense gate/up product + SwiGLU (Qwen3; rows = pairs)", us, 2 * Fe * width * 2 + pairs * (width + Fe) * 2, 2.0 * pairs * 2 * Fe * width, tc)
    wd2 = wd[0].contiguous()
    us = _time_kernel(lambda: ops.gemm(h, wd2, ys))
    note("dense down product (Qwen3; rows = pairs)", us, Fe * width * 2 + pairs * (Fe * 2 + width * 4), 2.0 * pairs * Fe * width, tc)
    return out


def padodra_shape(width: int, groups: int = 2, vocab: int = 32000, block: int = 1024) -> dict:
    """Layer sizes that resemble a real model's: attention with heads of 128 and four query heads per key head, a soft cap,
    a mask of blocks of 1,024 positions and a sink; latent attention with per head 128 plain and 64 rotated query dims,
    values of 128 and a cached latent of 512 (a cache row of 576 numbers); GeGLU feed-forwards of three times the width."""
    heads = width // 128
    att = {"type": "attention", "mixer": {"dim": 128, "heads": heads, "kv_heads": max(1, heads // 4), "vdim": 128,
                                          "mask": {"size": block}, "softcap": 30.0, "scale": 1.0 / math.sqrt(128.0),
                                          "rot": {"base": 500000.0, "dims": 128,
                                                  "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}}
    lat = {"type": "latent_attention", "mixer": {"dim": 128, "heads": heads, "kv_rank": 512, "rot_dim": 64, "vdim": 128,
                                                 "scale": 1.0 / math.sqrt(192.0),
                                                 "rot": {"base": 10000.0, "dims": 64,
                                                         "scaling": {"factor": 40.0, "fast": 32.0, "slow": 1.0, "original": 4096}}}}
    dense = {"kind": "dense", "ff": 3 * width}
    layers = []
    for g in range(groups):
        layers += [dict(att, mlp=dense), dict(lat, mlp=dense), dict(lat, mlp=dense), dict(att, mlp=dense)]
    return {"architecture": "Padodra", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "embedding": {"scale": math.sqrt(width)},
            "logit_scale": 0.5, "layers": layers, "initializer_range": 0.02}


def padodra_kernel_points(width: int, n: int, context: int, peaks: dict) -> dict:
    """The design's kernels alone at a layer of this width, each beside the like kernel of the Qwen3 decoder: with
    context = 0 one request of n prompt tokens, else n requests that each bring one token over `context` cached ones."""
    import numpy as np
    import torch

    from .csrc import attention_fast, ops
    dev = "cuda"
    bw, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    out = {}

    def note(name, us, nbytes, flops, peak_flops, like=None):
        floor = max(nbytes / bw, flops / peak_flops if peak_flops else 0.0) * 1e6
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "flops": int(flops), "roofline_us": round(floor, 2),
                     "of_roofline": round(floor / us, 3), **({"like": like} if like else {})}

    H, G, hd, pt, block = width // 128, max(1, width // 512), 128, 64, 1024
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    decode = context > 0
    reqs = n if decode else 1
    per = (context + 1) if decode else n
    ppr = -(-per // pt)                                   # pages per request
    table = torch.arange(reqs * ppr, dtype=torch.int32, device=dev).view(reqs, ppr).contiguous()
    slots = list(range(reqs))
    q_starts = list(range(n)) if decode else [0]
    q_lens = [1] * n if decode else [n]
    starts = [context] * n if decode else [0]
    positions = torch.tensor([context] * n if decode else list(range(n)), dtype=torch.int32, device=dev)
    slot_of = torch.tensor(list(range(n)) if decode else [0] * n, dtype=torch.int32, device=dev)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    pairs_plain = n * (context + 1) if decode else n * (n + 1) // 2
    pairs_block = sum(min(p % block, p) + 1 for p in ([context] * n if decode else range(n)))

    # ---- grouped-query attention: with the soft cap, the mask of blocks and the sink; and plain (Qwen3's)
    kp = (torch.randn(reqs * ppr, G, pt, hd, device=dev) * 0.5).bfloat16()
    vp = (torch.randn(reqs * ppr, G, pt, hd, device=dev) * 0.5).bfloat16()
    q = (torch.randn(n, H * hd, device=dev) * 0.5).bfloat16()
    att = torch.empty(n, H * hd, dtype=torch.bfloat16, device=dev)
    sinks = torch.zeros(H, device=dev)
    fixed = attention_fast.decode_splits(n, G, sm) if decode else 0
    rows = 256 if (not decode and attention_fast.tc2_prefill_supported(hd, H // G, pt)) else (128 if not decode else 64)
    plan = attention_fast.build_plan(slots, q_starts, q_lens, starts, n, 0, H, G, sm, up, fixed_splits=fixed,
                                     max_context=context + 64 if decode else 0, prefill_rows=rows, chunk=block)
    us = _time_kernel(lambda: ops.paged_attention(q, kp, vp, table, positions, slot_of, att, H, G, hd, pt, 0, hd ** -0.5, plan=plan,
                                                  sink=True, sinks=sinks, softcap=30.0, chunk=block))
    keys_read = (min(context % block, context) + 1) * n if decode else n
    note("attention with cap, blocks and sink", us, keys_read * G * hd * 4 + n * H * hd * 4, 4.0 * pairs_block * H * hd, tc,
         like="attention (Qwen3)")
    plan0 = attention_fast.build_plan(slots, q_starts, q_lens, starts, n, 0, H, G, sm, up, fixed_splits=fixed,
                                      max_context=context + 64 if decode else 0, prefill_rows=rows)
    us = _time_kernel(lambda: ops.paged_attention(q, kp, vp, table, positions, slot_of, att, H, G, hd, pt, 0, hd ** -0.5, plan=plan0))
    note("attention (Qwen3)", us, (n * (context + 1) if decode else n) * G * hd * 4 + n * H * hd * 4, 4.0 * pairs_plain * H * hd, tc)
    gate = torch.randn(n, H * hd, device=dev)
    us = _time_kernel(lambda: ops.sigmoid_gate(att, gate, att))
    note("sigmoid_gate", us, n * H * hd * 8, 0, 0, like="swiglu (Qwen3, unfused form)")

    # ---- latent attention: H heads over one cache row of 576 numbers whose first 512 are the value
    r, dr, dn, dv = 512, 64, 128, 128
    dk = r + dr
    rows_l = (torch.randn(reqs * ppr, 1, pt, dk, device=dev) * 0.3).bfloat16()
    ql = (torch.randn(n, H * dk, device=dev) * 0.3).bfloat16()
    lat = torch.empty(n, H * r, dtype=torch.bfloat16, device=dev)
    fixed_l = attention_fast.decode_splits(n, 1, sm) if decode else 0
    plan_l = attention_fast.build_plan(slots, q_starts, q_lens, starts, n, 0, H, 1, sm, up, fixed_splits=fixed_l,
                                       max_context=context + 64 if decode else 0, prefill_rows=64)
    us = _time_kernel(lambda: attention_fast.run_latent(ql, rows_l, table, lat, H, dk, r, pt, 0, 192 ** -0.5, plan_l, single_tokens=decode))
    note("latent attention (rows of 576, values of 512)", us, (n * (context + 1) if decode else n) * dk * 2 + n * H * (dk + r) * 2,
         2.0 * pairs_plain * H * (dk + r), tc, like="attention (Qwen3)")
    proj = torch.randn(n, H * (dn + dr) + dk + H * dv, device=dev)
    q_plain = torch.empty(n, H * dn, dtype=torch.bfloat16, device=dev)
    cn = torch.ones(r, device=dev)
    cos = torch.ones(per + 1, dr // 2, device=dev)
    sin = torch.zeros(per + 1, dr // 2, device=dev)
    us = _time_kernel(lambda: ops.latent_prep(proj, q_plain, ql, cn, 1e-6, cos, sin, dr, "half", positions, slot_of, table, rows_l,
                                              H, dn, dr, r, pt))
    note("latent_prep", us, n * (H * (dn + dr) + dk) * 6, 0, 0, like="qk_norm_rope_kv_write (Qwen3)")
    qkv = torch.randn(n, (H + 2 * G) * hd, device=dev)
    qn = torch.ones(hd, device=dev)
    cos2 = torch.ones(per + 1, hd // 2, device=dev)
    sin2 = torch.zeros(per + 1, hd // 2, device=dev)
    us = _time_kernel(lambda: ops.qk_norm_rope_kv_write(qkv, q, qn, qn, 1e-6, cos2, sin2, hd, positions, slot_of, table, kp, vp, H, G, hd, pt))
    note("qk_norm_rope_kv_write (Qwen3)", us, n * (H + 2 * G) * hd * 6, 0, 0)
    w_uk = (torch.randn(H, r, dn, device=dev) * 0.05).bfloat16()
    w_uv = (torch.randn(H, dv, r, device=dev) * 0.05).bfloat16()
    o = torch.empty(n, H * dv, device=dev)
    us = _time_kernel(lambda: ops.gemm_heads(q_plain.view(n, H, dn), w_uk, ql.view(n, H, dk)[:, :, :r], H))
    note("query into the latent space (a product per head)", us, H * r * dn * 2 + n * H * (dn + r) * 2, 2.0 * n * H * r * dn, tc,
         like="dense product of equal FLOPs (Qwen3)")
    glat = torch.randn(n, H * dv, device=dev)
    ob = torch.empty(n, H * dv, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.gemm_heads(lat.view(n, H, r), w_uv, ob.view(n, H, dv), H, gate=glat))
    note("values out of the latent space, gated (a product per head)", us, H * r * dv * 2 + n * H * (r * 2 + dv * 6), 2.0 * n * H * r * dv, tc,
         like="dense product of equal FLOPs (Qwen3)")
    wd = (torch.randn(H * dn, r, device=dev) * 0.05).bfloat16()       # [N = H * 128, K = 512]: the same FLOPs as one of the two
    a2 = (torch.randn(n, r, device=dev) * 0.3).bfloat16()
    od = torch.empty(n, H * dn, device=dev)
    us = _time_kernel(lambda: ops.gemm(a2, wd, od))
    note("dense product of equal FLOPs (Qwen3)", us, H * dn * r * 2 + n * (r * 2 + H * dn * 4), 2.0 * n * H * dn * r, tc)

    # ---- the layer's row-wise kernels and the feed-forward's first product
    x = torch.randn(n, width, device=dev)
    res = torch.randn(n, width, device=dev)
    wn = torch.ones(width, device=dev)
    xb = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.rms_norm_add(x, wn, 1e-6, res, xb))
    note("rms_norm_add with the narrowed copy", us, n * width * 14, 0, 0, like="rms_norm (Qwen3)")
    us = _time_kernel(lambda: ops.rms_norm(x, wn, 1e-6, xb))
    note("rms_norm (Qwen3)", us, n * width * 6, 0, 0)
    F = 3 * width
    wgu = (torch.randn(2 * F, width, device=dev) * 0.02).bfloat16()
    xb.copy_(torch.randn(n, width, device=dev))
    hb = torch.empty(n, F, dtype=torch.bfloat16, device=dev)
    for act, name in (("gelu_tanh", "gate/up product with the gelu gate in its epilogue"), ("silu", "gate/up product with SwiGLU epilogue (Qwen3)")):
        us = _time_kernel(lambda: ops.gemm_swiglu(xb, wgu, hb, act))
        note(name, us, 2 * F * width * 2 + n * (width + F) * 2, 4.0 * n * F * width, tc,
             like=None if act == "silu" else "gate/up product with SwiGLU epilogue (Qwen3)")
    gu = torch.randn(n, 2 * F, device=dev)
    us = _time_kernel(lambda: ops.swiglu(gu, hb))
    note("swiglu (Qwen3, unfused form)", us, n * F * 10, 0, 0)
    return out


def mifolorn_shape(width: int, passes: int = 2, vocab: int = 32000) -> dict:
    """Layer sizes that resemble a real model's: an attention with heads of 128, four query heads per key head, half of
    every head rotated with scaled frequencies, a soft cap and an output gate, beside a gated delta rule with heads of 64
    (two value heads per query/key head, four taps); a matrix memory and a gated delta rule with as many heads of 64 as
    the width holds; feed-forwards of three times the width; a token input of 64 per layer; the four layers run
    `passes` times."""
    heads128, heads64 = width // 128, width // 64
    rot = {"base": 1000000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    left = {"dim": 128, "heads": heads128, "kv_heads": max(1, heads128 // 4), "vdim": 128, "scale": 1.0 / math.sqrt(128.0),
            "softcap": 50.0, "rot": rot}
    right = {"dim": 64, "heads": heads128, "kv_heads": max(1, heads128 // 2), "vdim": 64, "conv": 4}
    par = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.8, "right_scale": 1.1}}
    mem = {"type": "mlstm", "mixer": {"dim": 64, "heads": heads64, "vdim": 64, "gate_cap": 15.0}}
    dlt = {"type": "delta", "mixer": {"dim": 64, "heads": heads64, "kv_heads": max(1, heads64 // 2), "vdim": 64, "conv": 4}}
    dense = {"kind": "dense", "ff": 3 * width}
    layers = [dict(par, mlp=dense), dict(par, mlp=dense), dict(mem, mlp=dense), dict(dlt, mlp=dense)]
    return {"architecture": "Mifolorn", "width": width, "vocab": vocab, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "token_side": {"dim": 64}, "loop": {"start": 0, "stop": len(layers), "times": passes}, "layers": layers,
            "initializer_range": 0.02}


def mifolorn_kernel_points(width: int, n: int, decode: bool, peaks: dict) -> dict:
    """The design's kernels alone at a layer of this width, each beside the like kernel of the Kedanex decoder: one
    request of n prompt tokens, or (decode) n requests that each bring one token (the attention over 2,047 cached ones;
    these are timed as replays of a captured graph)."""
    import numpy as np
    import torch

    from .csrc import attention_fast, ops
    dev = "cuda"
    bw, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    out = {}

    def note(name, us, nbytes, flops, peak_flops, like=None):
        floor = max(nbytes / bw, flops / peak_flops if peak_flops else 0.0) * 1e6
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "flops": int(flops), "roofline_us": round(floor, 2),
                     "of_roofline": round(floor / us, 3), **({"like": like} if like else {})}

    count, rows = (n, 1) if decode else (1, n)
    _time_kernel = lambda fn: globals()["_time_kernel"](fn, replay=decode)      # decode steps replay a captured graph
    sg = torch.tensor([[i, i * rows, rows] for i in range(count)], dtype=torch.int32, device=dev)
    H, G, dk, dv, taps = width // 64, width // 128, 64, 64, 4
    K, V = G * dk, H * dv
    C = 2 * K + V
    fp32 = FP32_TFLOPS * 1e12

    # ---- gated delta rule: the short convolution, the scan (its preparation and the walk), the output's norm and gate
    proj = torch.randn(n, C + V + 2 * H, device=dev) * 0.5
    act = torch.empty(n, C, device=dev)
    conv = torch.randn(C, taps, device=dev) * 0.3
    tail = torch.zeros(count, taps - 1, C, device=dev)
    us = _time_kernel(lambda: ops.short_conv(proj[:, :C], conv, sg, tail, act))
    note("short_conv (q, k and v of a gated delta rule)", us, n * C * 8 + count * (taps - 1) * C * 8, 2.0 * n * C * taps, fp32,
         like="rms_norm_add (row-wise)")
    state = torch.zeros(count, H, dk, dv, device=dev)
    o = torch.empty(n, V, device=dev)
    a_log, dt_bias = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
    us = _time_kernel(lambda: ops.gated_delta_scan(act[:, :K], act[:, K:2 * K], act[:, 2 * K:], proj[:, C + V:C + V + H], proj[:, C + V + H:],
                                                   a_log, dt_bias, sg, state, o, H, G, dk, dv, dk ** -0.5, 1e-6))
    note("gated_delta_scan", us, 4 * (n * (2 * K + 2 * V + 2 * H) + 2 * count * H * dk * dv), 8.0 * n * H * dk * dv, fp32,
         like="delta_rule_scan (Kedanex)")
    # the like kernel: the generalised delta rule at the same heads (its decays and removal strengths are vectors per head)
    KK = H * dk
    projk = torch.randn(n, 4 * KK, device=dev) * 0.5
    wl = torch.randn(n, KK, device=dev)
    zb = torch.zeros(KK, device=dev)
    ok = torch.empty(n, KK, device=dev)
    us = _time_kernel(lambda: ops.delta_rule_scan(projk[:, :KK], projk[:, KK:2 * KK], projk[:, 2 * KK:3 * KK], projk[:, 3 * KK:], wl, zb, zb, sg,
                                                  state, ok, H, dk, dk, math.exp(-0.5), 1e-6))
    note("delta_rule_scan (Kedanex)", us, 4 * (6 * n * KK + 2 * count * H * dk * dk), 8.0 * n * H * dk * dk, fp32)
    og = torch.empty(n, V, dtype=torch.bfloat16, device=dev)
    wn = torch.ones(dv, device=dev)
    us = _time_kernel(lambda: ops.head_out_gate(o, proj[:, C:C + V], wn, 1e-5, og, H, dv, act="silu"))
    note("head_out_gate (delta rule: shared weight, silu)", us, n * V * (4 + 4 + 2), 0, 0, like="head_norm_gate (Kedanex)")
    wk = torch.ones(V, device=dev)
    us = _time_kernel(lambda: ops.head_norm_gate(o, proj[:, C:C + V], wk, 1e-5, og, H, dv))
    note("head_norm_gate (Kedanex)", us, n * V * (4 + 4 + 2), 0, 0)

    # ---- matrix memory: the gates' walk, the preparation and the scan; its output's normaliser, norm and gate
    dvp = ops.mlstm_padded(dv)
    projm = torch.randn(n, 2 * KK + 2 * V + 2 * H, device=dev) * 0.5
    st_m = torch.zeros(count, H, dk, dvp, device=dev)
    m_st = torch.zeros(count, H, device=dev)
    om = torch.empty(n, H * dvp, device=dev)
    gates = torch.empty(n, H, 3, device=dev)
    ib = torch.zeros(H, device=dev)

    def memory():
        st_m.zero_()
        m_st.zero_()
        ops.mlstm_scan(projm[:, :KK], projm[:, KK:2 * KK], projm[:, 2 * KK:2 * KK + V], projm[:, 2 * KK + 2 * V:2 * KK + 2 * V + H],
                       projm[:, 2 * KK + 2 * V + H:], ib, ib, sg, st_m, m_st, om, gates, H, dk, dv, 15.0, dk ** -0.5)

    us = _time_kernel(memory)
    note("mlstm_scan", us, 4 * (n * (2 * KK + 2 * V + 2 * H) + 2 * count * H * dk * dvp), 5.0 * n * H * dk * (dv + 1), fp32,
         like="delta_rule_scan (Kedanex)")
    us = _time_kernel(lambda: ops.head_out_gate(om, projm[:, 2 * KK + V:2 * KK + 2 * V], wk, 1e-5, og, H, dv, act="sigmoid", gates=gates,
                                                den_eps=1e-6))
    note("head_out_gate (matrix memory: normaliser, sigmoid)", us, n * V * (4 + 4 + 2), 0, 0, like="head_norm_gate (Kedanex)")

    # ---- attention: heads of 128 with a soft cap and the output gate; and Kedanex's, with its window and sink
    Ha, Ga, hd, pt, context = width // 128, max(1, width // 512), 128, 64, 2047
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    per = (context + 1) if decode else n
    ppr = -(-per // pt)
    table = torch.arange(count * ppr, dtype=torch.int32, device=dev).view(count, ppr).contiguous()
    slots = list(range(count))
    q_starts = list(range(n)) if decode else [0]
    q_lens = [1] * n if decode else [n]
    starts = [context] * n if decode else [0]
    positions = torch.tensor([context] * n if decode else list(range(n)), dtype=torch.int32, device=dev)
    slot_of = torch.tensor(list(range(n)) if decode else [0] * n, dtype=torch.int32, device=dev)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    pairs = n * (context + 1) if decode else n * (n + 1) // 2
    kp = (torch.randn(count * ppr, Ga, pt, hd, device=dev) * 0.5).bfloat16()
    vp = (torch.randn(count * ppr, Ga, pt, hd, device=dev) * 0.5).bfloat16()
    q = (torch.randn(n, Ha * hd, device=dev) * 0.5).bfloat16()
    att = torch.empty(n, Ha * hd, dtype=torch.bfloat16, device=dev)
    gate = torch.randn(n, Ha * hd, device=dev)
    fixed = attention_fast.decode_splits(n, Ga, sm) if decode else 0
    rws = 256 if (not decode and attention_fast.tc2_prefill_supported(hd, Ha // Ga, pt)) else (128 if not decode else 64)
    plan = attention_fast.build_plan(slots, q_starts, q_lens, starts, n, 0, Ha, Ga, sm, up, fixed_splits=fixed,
                                     max_context=context + 64 if decode else 0, prefill_rows=rws)
    keys = (n * (context + 1) if decode else n) * Ga * hd * 4
    us = _time_kernel(lambda: ops.paged_attention(q, kp, vp, table, positions, slot_of, att, Ha, Ga, hd, pt, 0, hd ** -0.5, plan=plan,
                                                  softcap=50.0, gate=gate, gate_scale=0.8))
    note("attention with soft cap and output gate", us, keys + n * Ha * hd * (4 + 4 + 4), 4.0 * pairs * Ha * hd, tc,
         like="attention with a sink (Kedanex; no window here)")
    us = _time_kernel(lambda: ops.paged_attention(q, kp, vp, table, positions, slot_of, att, Ha, Ga, hd, pt, 0, hd ** -0.5, plan=plan,
                                                  sink=True))
    note("attention with a sink (Kedanex; no window here)", us, keys + n * Ha * hd * 4, 4.0 * pairs * Ha * hd, tc)
    qkv = torch.randn(n, (Ha + 2 * Ga) * hd, device=dev)
    bias = torch.zeros((Ha + 2 * Ga) * hd, device=dev)
    qn = torch.ones(hd, device=dev)
    cos = torch.ones(per + 1, 32, device=dev)
    sin = torch.zeros(per + 1, 32, device=dev)
    us = _time_kernel(lambda: ops.qk_norm_rope_kv_write(qkv, q, qn, qn, 1e-5, cos, sin, 64, positions, slot_of, table, kp, vp, Ha, Ga, hd, pt,
                                                        bias=bias))
    note("qk_norm_rope_kv_write with biases and half-rotated heads", us, n * (Ha + 2 * Ga) * hd * 6, 0, 0,
         like="qk_norm_rope_kv_write (whole heads rotated, no bias)")
    cos2 = torch.ones(per + 1, hd // 2, device=dev)
    sin2 = torch.zeros(per + 1, hd // 2, device=dev)
    us = _time_kernel(lambda: ops.qk_norm_rope_kv_write(qkv, q, qn, qn, 1e-5, cos2, sin2, hd, positions, slot_of, table, kp, vp, Ha, Ga, hd, pt))
    note("qk_norm_rope_kv_write (whole heads rotated, no bias)", us, n * (Ha + 2 * Ga) * hd * 6, 0, 0)

    # ---- the per-layer token input and the layer's row-wise kernels
    side = 64
    x = torch.randn(n, width, device=dev)
    xb = torch.empty(n, width, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.narrow(x, xb))
    note("narrow (the token input reads the stream itself)", us, n * width * 6, 0, 0, like="rms_norm")
    z = torch.randn(n, side, device=dev)
    tab = (torch.randn(32000, 4 * side, device=dev) * 0.1).bfloat16()
    ids = torch.randint(0, 32000, (n,), dtype=torch.int32, device=dev)
    g = torch.empty(n, side, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.token_gate(z, tab, side, ids, g))
    note("token_gate", us, n * side * (4 + 2 + 2), 0, 0, like="swiglu (row-wise)")
    res = torch.randn(n, width, device=dev)
    wnn = torch.ones(width, device=dev)
    us = _time_kernel(lambda: ops.rms_norm_add(x, wnn, 1e-5, res))
    note("rms_norm_add (row-wise)", us, n * width * 12, 0, 0)
    us = _time_kernel(lambda: ops.rms_norm(x, wnn, 1e-5, xb))
    note("rms_norm", us, n * width * 6, 0, 0)
    gu = torch.randn(n, 2 * side, device=dev)
    us = _time_kernel(lambda: ops.swiglu(gu, g))
    note("swiglu (row-wise)", us, n * side * 10, 0, 0)
    return out


def zazulix_shape(width: int, groups: int = 2, vocab: int = 32000, window: int = 1024) -> dict:
    """Layer sizes that resemble a real model's: a latent attention with heads of 128 over a cached vector of 512 and a
    window; a differential attention with maps of 64, values of 128, four query heads per key/value head, four taps and
    whole maps rotated; two retention layers with heads of 64; a dense feed-forward of three times the width and eight
    experts of half the width in two groups, of which two are used, beside a shared expert."""
    heads128, heads64 = width // 128, width // 64
    lat = {"type": "latent_attention", "mixer": {"dim": 128, "heads": heads128, "kv_rank": 512, "vdim": 128, "mask": {"size": window},
                                                 "scale": 1.0 / math.sqrt(128.0)}}
    att = {"type": "attention", "mixer": {"dim": 64, "heads": heads128, "kv_heads": max(1, heads128 // 4), "vdim": 128, "conv": 4,
                                          "diff": 0.4, "rot": {"base": 100000.0, "dims": 64}, "scale": 0.125}}
    ret = {"type": "retention", "mixer": {"dim": 64, "heads": heads64, "vdim": 64, "rot": {"base": 500000.0, "dims": 32},
                                          "decay": [1.0 - 2.0 ** (-5.0 - 5.0 * h / max(heads64 - 1, 1)) for h in range(heads64)]}}
    dense = {"kind": "dense", "ff": 3 * width, "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": width // 2}, "router": {"experts": 8, "top": 2, "scale": 2.5, "groups": {"count": 2, "keep": 1}},
           "shared": {"ff": width // 2}}
    layers = []
    for g in range(groups):
        layers += [dict(lat, mlp=dense), dict(att, mlp=moe), dict(ret, mlp=moe), dict(ret, mlp=moe)]
    return {"architecture": "Zazulix", "width": width, "vocab": vocab, "norm": {"eps": 1e-6}, "layers": layers,
            "initializer_range": 0.02}


def zazulix_kernel_points(width: int, n: int, decode: bool, peaks: dict) -> dict:
    """The design's kernels alone at a layer of this width, each beside the like kernel of the Kedanex (or Mifolorn)
    decoder: one request of n prompt tokens, or (decode) n requests that each bring one token (the attention over 2,047
    cached ones; these are timed as replays of a captured graph)."""
    import numpy as np
    import torch

    from .csrc import attention_fast, ops
    dev = "cuda"
    bw, tc = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    out = {}

    def note(name, us, nbytes, flops, peak_flops, like=None):
        floor = max(nbytes / bw, flops / peak_flops if peak_flops else 0.0) * 1e6
        out[name] = {"us": round(us, 1), "bytes": int(nbytes), "flops": int(flops), "roofline_us": round(floor, 2),
                     "of_roofline": round(floor / us, 3), **({"like": like} if like else {})}

    count, rows = (n, 1) if decode else (1, n)
    _time_kernel = lambda fn: globals()["_time_kernel"](fn, replay=decode)      # decode steps replay a captured graph
    sg = torch.tensor([[i, i * rows, rows] for i in range(count)], dtype=torch.int32, device=dev)
    fp32 = FP32_TFLOPS * 1e12
    pt, context = 64, 2047
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    per = (context + 1) if decode else n
    ppr = -(-per // pt)
    table = torch.arange(count * ppr, dtype=torch.int32, device=dev).view(count, ppr).contiguous()
    slots = list(range(count))
    q_starts = list(range(n)) if decode else [0]
    q_lens = [1] * n if decode else [n]
    starts = [context] * n if decode else [0]
    positions = torch.tensor([context] * n if decode else list(range(n)), dtype=torch.int32, device=dev)
    slot_of = torch.tensor(list(range(n)) if decode else [0] * n, dtype=torch.int32, device=dev)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    pairs = n * (context + 1) if decode else n * (n + 1) // 2

    # ---- differential attention: convolution, rotation and cache write, the attention itself, the heads' combination
    H, G, dk, vd, taps = width // 128, max(1, width // 512), 64, 128, 4
    C = (H + G) * 2 * dk + G * vd
    proj = torch.randn(n, C + H, device=dev) * 0.5
    act = torch.empty(n, C, device=dev)
    conv = torch.randn(C, taps, device=dev) * 0.3
    tail = torch.zeros(count, taps - 1, C, device=dev)
    us = _time_kernel(lambda: ops.short_conv(proj[:, :C], conv, sg, tail, act, act="none"))
    note("short_conv (q, k and v of the differential attention, no activation)", us, n * C * 8 + count * (taps - 1) * C * 8,
         2.0 * n * C * taps, fp32, like="short_conv (Mifolorn: silu)")
    us = _time_kernel(lambda: ops.short_conv(proj[:, :C], conv, sg, tail, act))
    note("short_conv (Mifolorn: silu)", us, n * C * 8 + count * (taps - 1) * C * 8, 2.0 * n * C * taps, fp32)
    kp = (torch.randn(count * ppr, G, pt, 2 * dk, device=dev) * 0.5).bfloat16()
    vp = (torch.randn(count * ppr, G, pt, vd, device=dev) * 0.5).bfloat16()
    q2 = torch.empty(n, 2 * H * 2 * dk, dtype=torch.bfloat16, device=dev)
    cos = torch.ones(per + 1, dk // 2, device=dev)
    sin = torch.zeros(per + 1, dk // 2, device=dev)
    us = _time_kernel(lambda: ops.maps_rope_kv_write(act, q2, cos, sin, dk, positions, slot_of, table, kp, vp, H, G, 2, dk, pt))
    note("maps_rope_kv_write (two maps a head)", us, n * C * 4 + n * (2 * H * 2 * dk + G * 2 * dk + G * vd) * 2, 0, 0,
         like="qk_norm_rope_kv_write (Kedanex's attention)")
    hd = 128
    qkv = torch.randn(n, (H + 2 * G) * hd, device=dev)
    q1 = torch.empty(n, H * hd, dtype=torch.bfloat16, device=dev)
    cos2 = torch.ones(per + 1, hd // 2, device=dev)
    sin2 = torch.zeros(per + 1, hd // 2, device=dev)
    us = _time_kernel(lambda: ops.qk_norm_rope_kv_write(qkv, q1, None, None, 1e-5, cos2, sin2, hd, positions, slot_of, table, kp, vp, H, G,
                                                        hd, pt, norm_after=True))
    note("qk_norm_rope_kv_write (Kedanex's attention)", us, n * (H + 2 * G) * hd * 6, 0, 0)
    fixed = attention_fast.decode_splits(n, G, sm) if decode else 0

    def plan_for(heads):
        rws = 256 if (not decode and attention_fast.tc2_prefill_supported(hd, heads // G, pt)) else (128 if not decode else 64)
        return attention_fast.build_plan(slots, q_starts, q_lens, starts, n, 0, heads, G, sm, up, fixed_splits=fixed,
                                         max_context=context + 64 if decode else 0, prefill_rows=rws)

    keys = (n * (context + 1) if decode else n) * G * hd * 4
    q2.normal_(0.0, 0.5)
    att2 = torch.empty(n, 2 * H * vd, dtype=torch.bfloat16, device=dev)
    plan2 = plan_for(2 * H)
    us = _time_kernel(lambda: ops.paged_attention(q2, kp, vp, table, positions, slot_of, att2, 2 * H, G, hd, pt, 0, 0.125, plan=plan2))
    # the operations that the design asks for: two maps of dk against the keys, two sums over the values; the kernel
    # multiplies rows of 2 dk (half of them zeros)
    note("differential attention (2 H heads over rows of two maps)", us, keys + n * 2 * H * (hd + vd) * 2,
         (4.0 * dk + 4.0 * vd) * pairs * H, tc, like="attention with a sink (Kedanex; no window here)")
    q1.normal_(0.0, 0.5)
    att1 = torch.empty(n, H * hd, dtype=torch.bfloat16, device=dev)
    plan1 = plan_for(H)
    us = _time_kernel(lambda: ops.paged_attention(q1, kp, vp, table, positions, slot_of, att1, H, G, hd, pt, 0, hd ** -0.5, plan=plan1,
                                                  sink=True))
    note("attention with a sink (Kedanex; no window here)", us, keys + n * H * hd * 4, 4.0 * pairs * H * hd, tc)
    og = torch.empty(n, H * vd, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.diff_heads_out(att2, proj[:, C:C + H], og, H, vd, 0.5, 1e-6, 0.5))
    note("diff_heads_out (difference, norm, gate)", us, n * H * vd * 6, 0, 0, like="head_norm_gate (Kedanex)")

    # ---- retention: the scan (its preparation and the walk), the output's norm and gate
    Hr, dr = width // 64, 64
    KK = Hr * dr
    projr = torch.randn(n, 4 * KK, device=dev) * 0.5
    state = torch.zeros(count, Hr, dr, dr, device=dev)
    o = torch.empty(n, KK, device=dev)
    decay = torch.full((Hr,), 0.99, device=dev)
    cosr = torch.ones(per + 1, dr // 2, device=dev)
    sinr = torch.zeros(per + 1, dr // 2, device=dev)
    us = _time_kernel(lambda: ops.retention_scan(projr[:, :KK], projr[:, KK:2 * KK], projr[:, 2 * KK:3 * KK], cosr, sinr, dr, positions, decay,
                                                 sg, state, o, Hr, dr, dr, dr ** -0.5))
    note("retention_scan", us, 4 * (4 * n * KK + 2 * count * Hr * dr * dr), 4.0 * n * Hr * dr * dr, fp32, like="delta_rule_scan (Kedanex)")
    wl = torch.randn(n, KK, device=dev)
    zb = torch.zeros(KK, device=dev)
    us = _time_kernel(lambda: ops.delta_rule_scan(projr[:, :KK], projr[:, KK:2 * KK], projr[:, 2 * KK:3 * KK], projr[:, 3 * KK:], wl, zb, zb, sg,
                                                  state, o, Hr, dr, dr, math.exp(-0.5), 1e-6))
    note("delta_rule_scan (Kedanex)", us, 4 * (6 * n * KK + 2 * count * Hr * dr * dr), 8.0 * n * Hr * dr * dr, fp32)
    ogr = torch.empty(n, KK, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.head_out_gate(o, projr[:, 3 * KK:], None, 1e-6, ogr, Hr, dr, act="silu"))
    note("head_out_gate (retention: no weight, silu)", us, n * KK * (4 + 4 + 2), 0, 0, like="head_norm_gate (Kedanex)")
    wk = torch.ones(KK, device=dev)
    us = _time_kernel(lambda: ops.head_norm_gate(o, projr[:, 3 * KK:], wk, 1e-5, ogr, Hr, dr))
    note("head_norm_gate (Kedanex)", us, n * KK * (4 + 4 + 2), 0, 0)

    # ---- the router with sigmoid scores, groups and the shared expert's gate; the combination with the shared result
    E, top = 8, 2
    xb = (torch.randn(n, width, device=dev) * 0.5).bfloat16()
    wr = torch.randn(E + 1, width, device=dev) * 0.05
    corr = torch.randn(E, device=dev) * 0.1
    ids = torch.empty(n, top, dtype=torch.int32, device=dev)
    wts = torch.empty(n, top, device=dev)
    sgate = torch.empty(n, 1, device=dev)
    us = _time_kernel(lambda: ops.route_topk(xb, wr, ids, wts, "sigmoid", corr, 2, 1, 2.5, 1e-20, sgate))
    note("route_topk (sigmoid scores, correction, groups, shared gate)", us, n * width * 2 + (E + 1) * width * 4, 2.0 * n * (E + 1) * width, fp32,
         like="route_topk (Kedanex: softmax over the chosen)")
    wr8 = wr[:E].contiguous()
    us = _time_kernel(lambda: ops.route_topk(xb, wr8, ids, wts))
    note("route_topk (Kedanex: softmax over the chosen)", us, n * width * 2 + E * width * 4, 2.0 * n * E * width, fp32)
    ys = torch.randn(n * top, width, device=dev)
    inv = torch.randperm(n * top, device=dev).to(torch.int32)
    res = torch.randn(n, width, device=dev)
    shared = torch.randn(n, width, device=dev)
    us = _time_kernel(lambda: ops.route_combine(ys, inv, wts, res, accumulate=True, shared=shared, shared_gate=sgate))
    note("route_combine (with the gated shared expert)", us, n * width * 4 * (top + 3), 0, 0, like="route_combine (Kedanex)")
    us = _time_kernel(lambda: ops.route_combine(ys, inv, wts, res, accumulate=True))
    note("route_combine (Kedanex)", us, n * width * 4 * (top + 2), 0, 0)

    # ---- the dense feed-forward's first product with the clamped activation, beside the one with silu
    F = 3 * width
    wgu = (torch.randn(2 * F, width, device=dev) * 0.02).bfloat16()
    hbuf = torch.empty(n, F, dtype=torch.bfloat16, device=dev)
    us = _time_kernel(lambda: ops.gemm_swiglu(xb, wgu, hbuf, "swish_clamped", 7.0, 1.702))
    note("gate/up product with the clamped activation", us, 2 * F * width * 2 + n * (width + F) * 2, 4.0 * n * F * width, tc,
         like="gate/up product with silu")
    us = _time_kernel(lambda: ops.gemm_swiglu(xb, wgu, hbuf, "silu"))
    note("gate/up product with silu", us, 2 * F * width * 2 + n * (width + F) * 2, 4.0 * n * F * width, tc)
    return out


def run(design: str, args, peaks: dict) -> dict:
    if design not in ("kedanex", "padodra", "mifolorn", "zazulix"):
        raise SystemExit(f"bench.py --design: unknown design '{design}' (known: kedanex, padodra, mifolorn, zazulix)")
    widths = [int(w) for w in str(args.design_widths).split(",")]
    sizes = {}
    for width in widths:
        t0 = time.time()
        ours = {"kedanex": kedanex_shape, "padodra": padodra_shape, "mifolorn": mifolorn_shape, "zazulix": zazulix_shape}[design](width)
        runs = len(ours["layers"]) * (ours["loop"]["times"] if "loop" in ours else 1)
        beside, theirs = ("kedanex", kedanex_shape(width, runs // 4)) if design in ("mifolorn", "zazulix") else ("qwen3", qwen3_shape(width, runs))
        entry = {design: model_points(ours, 2048, (8, 64), args.steps, max(args.warmup, 3), 5),
                 beside: model_points(theirs, 2048, (8, 64), args.steps, max(args.warmup, 3), 5),
                 "layer_runs": runs}
        if design == "mifolorn":
            entry["kernels_prefill_2048_rows"] = mifolorn_kernel_points(width, 2048, False, peaks)
            entry["kernels_decode_64_rows"] = mifolorn_kernel_points(width, 64, True, peaks)
        elif design == "zazulix":
            entry["kernels_prefill_2048_rows"] = zazulix_kernel_points(width, 2048, False, peaks)
            entry["kernels_decode_64_rows"] = zazulix_kernel_points(width, 64, True, peaks)
        elif design == "kedanex":
            entry["kernels_prefill_2048_rows"] = kernel_points(width, 2048, peaks)
            entry["kernels_decode_64_rows"] = {k: v for k, v in kernel_points(width, 64, peaks).items() if "request" not in k or "decode" in k}
        else:
            entry["kernels_prefill_2048_rows"] = padodra_kernel_points(width, 2048, 0, peaks)
            entry["kernels_decode_64_rows"] = padodra_kernel_points(width, 64, 2047, peaks)
            entry["kernels_decode_8_rows"] = padodra_kernel_points(width, 8, 2047, peaks)
        sizes[f"width{width}"] = entry
        print(f"[bench] design {design}, width {width}: {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    k = sizes[f"width{widths[-1]}"]
    return {"metric": f"{design} prefill and decode tok/s beside {'Kedanex' if design in ('mifolorn', 'zazulix') else 'Qwen3'} at equal width and depth", "value": k[design]["decode_b8"]["tok_s"],
            "unit": "tokens/s (decode, batch 8, largest width)", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic: seeded uniform token ids, random-init weights",
            "impl": "ours", "design": design, "sizes": sizes, "peaks": peaks}


if __name__ == "__main__":
    print(json.dumps(kedanex_shape(2048), indent=1))
