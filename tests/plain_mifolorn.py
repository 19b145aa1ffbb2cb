"""A plain, slow implementation of the Mifolorn decoder in numpy float64: one function per mechanism, a Python
loop per recurrence, no code shared with the package.  `cfg` is the content of a config.json of this design
(a dict), `w` maps tensor names to float64 arrays.

Notation: h is a sublayer's input (one row per token of ONE sequence, positions from 0), W x a product with a
weight stored [out, in].
"""
import math

import numpy as np

round_inputs = None      # a function that rounds an array as the serving engine's storage type does, or None


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


def softplus(x):
    return np.logaddexp(0.0, x)


def logsigmoid(x):
    return -np.logaddexp(0.0, -x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ---- rotation ------------------------------------------------------------------------------------------------

def rotation_frequencies(rot):
    """Per pair i < dims/2: the angle's factor and the magnitude that multiplies cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def corr(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(corr(float(sc["fast"]))), 0)
    hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims dims of each head turned, dim i paired with i + dims/2."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, mag = rotation_frequencies(rot)
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(a) * mag)[:, None, :], (np.sin(a) * mag)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    out = x.copy()
    out[..., :dims // 2] = u * c - v * s
    out[..., dims // 2:dims] = v * c + u * s
    return out


# ---- mixers ---------------------------------------------------------------------------------------------------

def softmax_attention(h, w, p, m, eps):
    """Grouped-query attention with biases, weighted per-head norms of q and k, rotation, a soft cap and an output
    gate.  `p`: the tensors' prefix (with the trailing dot), `m`: the mixer's entry of the configuration."""
    T = h.shape[0]
    H, G, dk = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"])
    dv = int(m.get("vdim", dk))
    q = (product(h, w[p + "q"]) + w[p + "q.b"]).reshape(T, H, dk)
    k = (product(h, w[p + "k"]) + w[p + "k.b"]).reshape(T, G, dk)
    v = (product(h, w[p + "v"]) + w[p + "v.b"]).reshape(T, G, dv)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    pos = np.arange(T)
    q, k = rotate(q, pos, m.get("rot")), rotate(k, pos, m.get("rot"))
    if round_inputs is not None:               # the cache and the queries are kept in the storage type
        q, k, v = round_inputs(q), round_inputs(k), round_inputs(v)
    cap = m.get("softcap")
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        if cap:
            s = cap * np.tanh(s / cap)
        s = np.where(pos[None, :] <= pos[:, None], s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        e = np.exp(s)
        out[:, hh] = (e / e.sum(axis=1, keepdims=True)) @ v[:, g]
    y = out.reshape(T, H * dv) * sigmoid(product(h, w[p + "g"]))
    return product(y, w[p + "o"])


def short_conv(x, taps_weight):
    """x [T, C], taps_weight [C, taps]: causal per channel, the last column is the current token's, zeros before
    the start."""
    T, C = x.shape
    taps = taps_weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for j in range(taps):
        y += padded[j:j + T] * taps_weight[:, j][None, :]
    return y


def gated_delta(h, w, p, m, eps):
    T = h.shape[0]
    H, G, dk, dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    q = silu(short_conv(product(h, w[p + "q"]), w[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(product(h, w[p + "k"]), w[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(product(h, w[p + "v"]), w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * dk ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(product(h, w[p + "b"]))                                             # [T, H]
    decay = np.exp(-np.exp(w[p + "A_log"]) * softplus(product(h, w[p + "a"]) + w[p + "dt_bias"]))
    out = np.zeros((T, H, dv))
    for hh in range(H):
        g = hh // (H // G)
        S = np.zeros((dk, dv))
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    y = rms(out, eps) * w[p + "norm"] * silu(product(h, w[p + "g"])).reshape(T, H, dv)
    return product(y.reshape(T, H * dv), w[p + "o"])


def mlstm(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv, cap = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["gate_cap"])
    q = (product(h, w[p + "q"])).reshape(T, H, dk) * dk ** -0.5
    k = (product(h, w[p + "k"])).reshape(T, H, dk)
    v = (product(h, w[p + "v"])).reshape(T, H, dv)
    ig = cap * np.tanh((product(h, w[p + "i"]) + w[p + "i.b"]) / cap)
    fg = logsigmoid(cap * np.tanh((product(h, w[p + "f"]) + w[p + "f.b"]) / cap))
    out = np.zeros((T, H, dv))
    for hh in range(H):
        S, nrm, mx = np.zeros((dk, dv)), np.zeros(dk), 0.0
        for t in range(T):
            new = max(fg[t, hh] + mx, ig[t, hh])
            keep, take = math.exp(fg[t, hh] + mx - new), math.exp(ig[t, hh] - new)
            S = keep * S + take * np.outer(k[t, hh], v[t, hh])
            nrm = keep * nrm + take * k[t, hh]
            mx = new
            out[t, hh] = S.T @ q[t, hh] / (max(abs(nrm @ q[t, hh]), math.exp(-mx)) + 1e-6)
    y = rms(out, eps).reshape(T, H * dv) * w[p + "norm"] * sigmoid(product(h, w[p + "g"]))
    return product(y, w[p + "o"])


def parallel(h, w, p, m, eps):
    return float(m["left_scale"]) * softmax_attention(h, w, p + "left.", m["left"], eps) \
        + float(m["right_scale"]) * gated_delta(h, w, p + "right.", m["right"], eps)


MIXERS = {"mlstm": mlstm, "delta": gated_delta, "parallel": parallel}


# ---- the rest of a layer -----------------------------------------------------------------------------------------

def feed_forward(h, w, p):
    return product(silu(product(h, w[p + "gate"])) * product(h, w[p + "up"]), w[p + "down"])


def token_side_input(x, tokens, w, i, dim, eps):
    """What layer i adds from its own slice of the second embedding table."""
    e = w["side.embed"][np.asarray(tokens)][:, i * dim:(i + 1) * dim]
    y = product(gelu_tanh(product(x, w[f"l{i}.side.gate"])) * e, w[f"l{i}.side.proj"])
    return rms(y, eps) * w[f"l{i}.side.norm"]


def layer(x, tokens, w, cfg, i):
    entry, eps = cfg["layers"][i], float(cfg["norm"]["eps"])
    p = f"l{i}."
    x = x + MIXERS[entry["type"]](rms(x, eps) * w[p + "norm1"], w, p + "mix.", entry["mixer"], eps)
    if entry.get("mlp") is not None:
        x = x + feed_forward(rms(x, eps) * w[p + "norm2"], w, p + "mlp.")
    side = cfg.get("token_side")
    if side:
        x = x + token_side_input(x, tokens, w, i, int(side["dim"]), eps)
    return x


def layer_runs(cfg):
    """The order in which the layers run: (layer, whether the embedding output is added first)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for r in range(times):
        runs += [(i, r > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def forward(cfg, w, tokens, trace=None):
    """Logits [T, vocab] of one sequence from its first token.  `trace`: a list that receives the residual stream
    after every layer run."""
    scale = float((cfg.get("embedding") or {}).get("scale", 1.0))
    x0 = w["embed"][np.asarray(tokens)] * scale
    x = x0
    for i, add in layer_runs(cfg):
        if add:
            x = x + x0
        x = layer(x, tokens, w, cfg, i)
        if trace is not None:
            trace.append(x.copy())
    return product(rms(x, float(cfg["norm"]["eps"])) * w["final.norm"], w["embed"])
