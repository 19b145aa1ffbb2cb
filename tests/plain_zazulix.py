"""A plain, slow implementation of the Zazulix decoder in numpy float64: one function per mechanism, a Python
loop per recurrence, no code shared with the package.  `cfg` is the content of a config.json of this design
(a dict), `w` maps tensor names to float64 arrays.

Notation: h is a sublayer's input (one row per token of ONE sequence, positions from 0), W x a product with a
weight stored [out, in], rms(x) = x / sqrt(mean(x^2) + eps).
"""
import math

import numpy as np

round_inputs = None      # a function that rounds an array as the serving engine's storage type does, or None
route_choices = None     # a dict {(tensor prefix of a routed feed-forward): int array [T, top]}: experts to use instead
                         # of the plain choice (the tests replay the engine's own choices where a call was close)
route_margins = None     # a dict that receives, per routed feed-forward, the gap between the last chosen and the first
                         # refused choice score of every token


def product(h, weight):
    """h W^T; with `round_inputs` set, the rows are rounded first: a coarse model of what 16-bit inputs of the
    products do, by which the tests know how far rounding alone moves the logits of a position."""
    return (round_inputs(h) if round_inputs is not None else h) @ weight.T


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def layer_norm(x, weight, eps):
    """The design's norm: the stored weight lies around zero and 1 is added to it."""
    return rms(x, eps) * (1.0 + weight)


def rotate(x, positions, rot):
    """x [T, ..., dim]: the first rot.dims dims of the last axis turned, dim i paired with i + dims/2, by the
    angle position * base^(-2i/dims)."""
    if not rot:
        return x
    dims, base = int(rot["dims"]), float(rot["base"])
    f = base ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(a).reshape(shape), np.sin(a).reshape(shape)
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.copy()
    out[..., :dims // 2] = u * c - v * s
    out[..., dims // 2:dims] = v * c + u * s
    return out


def short_conv(x, taps_weight):
    """x [T, C], taps_weight [C, taps]: causal per channel, the last column weighs the current token, zeros before
    the sequence's start."""
    T, C = x.shape
    taps = taps_weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += padded[j:j + T] * taps_weight[:, j][None, :]
    return y


def softmax_rows(s, visible):
    s = np.where(visible, s, -np.inf)
    s = s - s.max(axis=1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=1, keepdims=True)


# ---- mixers ---------------------------------------------------------------------------------------------------

def latent_attention(h, w, p, m, eps):
    """Attention whose keys and values of every head are products of one small vector per token (the latent), without
    positions, over a sliding window, with an element-wise sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
    q = product(h, w[p + "q"]).reshape(T, H, dk)
    c = rms(product(h, w[p + "dkv"]), eps) * w[p + "dkv.norm"]
    if round_inputs is not None:                 # the cache and the queries are kept in the storage type
        q, c = round_inputs(q), round_inputs(c)
    k = (c @ w[p + "uk"].T).reshape(T, H, dk)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    pos = np.arange(T)
    back = pos[:, None] - pos[None, :]
    visible = back >= 0
    if m.get("mask"):
        visible &= back < int(m["mask"]["size"])
    out = np.zeros((T, H, dv))
    for hh in range(H):
        out[:, hh] = softmax_rows((q[:, hh] @ k[:, hh].T) * float(m["scale"]), visible) @ v[:, hh]
    y = out.reshape(T, H * dv) * sigmoid(product(h, w[p + "g"]))
    return product(y, w[p + "o"])


def differential_attention(h, w, p, m, eps):
    """Grouped-query attention with two score maps per head over the same values: the second map's output, times
    lambda, is taken off the first one's; short convolutions behind the projections, rotation, a weightless norm per head
    and one gate number per head."""
    T = h.shape[0]
    H, G, dk = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
    dv, diff = int(m.get("vdim", dk)), float(m["diff"])
    q, k, v = product(h, w[p + "q"]), product(h, w[p + "k"]), product(h, w[p + "v"])
    if m.get("conv"):
        q, k, v = short_conv(q, w[p + "q.conv"]), short_conv(k, w[p + "k.conv"]), short_conv(v, w[p + "v.conv"])
    pos = np.arange(T)
    q = rotate(q.reshape(T, H, 2, dk), pos, m.get("rot"))
    k = rotate(k.reshape(T, G, 2, dk), pos, m.get("rot"))
    v = v.reshape(T, G, dv)
    if round_inputs is not None:
        q, k, v = round_inputs(q), round_inputs(k), round_inputs(v)
    lam = math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"]))) + diff
    visible = pos[None, :] <= pos[:, None]
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        a = [softmax_rows((q[:, hh, j] @ k[:, g, j].T) * float(m["scale"]), visible) @ v[:, g] for j in range(2)]
        out[:, hh] = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
    out = out * sigmoid(product(h, w[p + "g"]))[:, :, None]
    return product(out.reshape(T, H * dv), w[p + "o"])


def retention(h, w, p, m, eps):
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q, no softmax, no denominator."""
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
    pos = np.arange(T)
    q = rotate(product(h, w[p + "q"]).reshape(T, H, dk), pos, m.get("rot"))
    k = rotate(product(h, w[p + "k"]).reshape(T, H, dk), pos, m.get("rot")) * dk ** -0.5
    v = product(h, w[p + "v"]).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for hh in range(H):
        S = np.zeros((dk, dv))
        for t in range(T):
            S = float(m["decay"][hh]) * S + np.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    y = rms(out, eps).reshape(T, H * dv) * silu(product(h, w[p + "g"]))
    return product(y, w[p + "o"])


MIXERS = {"latent_attention": latent_attention, "attention": differential_attention, "retention": retention}


# ---- feed-forwards ----------------------------------------------------------------------------------------------

def clamped_feed_forward(h, w, p, limit):
    g = np.minimum(product(h, w[p + "gate"]), limit)
    u = np.clip(product(h, w[p + "up"]), -limit, limit)
    return product(g * sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def expert(h, w, p):
    return product(silu(product(h, w[p + "gate"])) * product(h, w[p + "up"]), w[p + "down"])


def route(z, correction, top, groups):
    """z [E] router logits of one token.  Returns (chosen experts in order of choice, their weights before the
    router's factor, the smallest gap by which a choice was made: last kept against first refused group score, last
    chosen against best refused choice score)."""
    s = sigmoid(z)
    choice = s + correction
    E = len(z)
    allowed = np.ones(E, dtype=bool)
    margin = np.inf
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        size = E // count
        score = np.array([np.sort(choice[g * size:(g + 1) * size])[::-1][:2].sum() for g in range(count)])
        order = sorted(range(count), key=lambda g: (-score[g], g))
        allowed[:] = False
        for g in order[:keep]:
            allowed[g * size:(g + 1) * size] = True
        if keep < count:
            margin = score[order[keep - 1]] - score[order[keep]]
    masked = np.where(allowed, choice, -np.inf)
    order = sorted(range(E), key=lambda e: (-masked[e], e))
    chosen = order[:top]
    if top < E:
        margin = min(margin, masked[chosen[-1]] - masked[order[top]])
    weights = s[chosen] / (s[chosen].sum() + 1e-20)
    return chosen, weights, margin


def routed_feed_forward(h, w, p, mlp):
    r = mlp["router"]
    E, top, factor = int(r["experts"]), int(r["top"]), float(r.get("scale", 1.0))
    T = h.shape[0]
    hr = round_inputs(h) if round_inputs is not None else h
    z = hr @ w[p + "router"].T
    corr = w[p + "correction"] if (p + "correction") in w else np.zeros(E)
    y = np.zeros((T, w[p + "e0.down"].shape[0]))
    outs = {}
    margins = np.zeros(T)
    for t in range(T):
        chosen, weights, margins[t] = route(z[t], corr, top, r.get("groups"))
        if route_choices is not None and p in route_choices:
            chosen = [int(e) for e in route_choices[p][t]]
            s = sigmoid(z[t])[chosen]
            weights = s / (s.sum() + 1e-20)
        for e, wt in zip(chosen, weights):
            if e not in outs:
                outs[e] = expert(h, w, f"{p}e{e}.")
            y[t] += factor * wt * outs[e][t]
    if route_margins is not None:
        route_margins[p] = margins
    if mlp.get("shared"):
        y = y + expert(h, w, p + "shared.") * sigmoid(product(h, w[p + "shared.sg"]))
    return y


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return clamped_feed_forward(h, w, p, float(mlp["limit"]))
    return routed_feed_forward(h, w, p, mlp)


# ---- the model ----------------------------------------------------------------------------------------------------

def layer(x, w, cfg, i):
    entry, eps = cfg["layers"][i], float(cfg["norm"]["eps"])
    p = f"l{i}."
    x = x + MIXERS[entry["type"]](layer_norm(x, w[p + "norm1"], eps), w, p + "mix.", entry["mixer"], eps)
    if entry.get("mlp") is not None:
        x = x + feed_forward(layer_norm(x, w[p + "norm2"], eps), w, p + "mlp.", entry["mlp"])
    return x


def forward(cfg, w, tokens, trace=None):
    """Logits [T, vocab] of one sequence from its first token.  `trace`: a list that receives the residual stream
    after every layer."""
    x = w["embed"][np.asarray(tokens)]
    for i in range(len(cfg["layers"])):
        x = layer(x, w, cfg, i)
        if trace is not None:
            trace.append(x.copy())
    return product(layer_norm(x, w["final.norm"], float(cfg["norm"]["eps"])), w["embed"])
