"""The mechanisms of the Zazulix decoder one by one: each part alone against its function of the plain
implementation (`plain_zazulix`), whole, cut into portions down to two tokens, token by token, in batches of
unequal requests, and after slots and pages were freed and taken again.  Where random weights would hide a fault, the
weights or inputs are made so that it shows."""
import numpy as np
import pytest
import torch

import plain_zazulix as P
from test_kedanex_parts_gpu import close
from test_mifolorn_parts_gpu import Harness, under_every_cut
from test_parts_gpu import DTYPES, IDS, bind_random

pytestmark = pytest.mark.gpu


def rope(rot, positions=2048):
    from hk_b200.parts import RotaryEmbedding
    return RotaryEmbedding(rot["base"], rot["dims"], positions, pairing="half") if rot else None


# ------------------------------------------------------------------------------------ differential attention

def diff_part(d, H, G, dk, dv, taps, rot, diff=0.4, scale=None, window=None):
    from hk_b200.parts import DifferentialAttention
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "diff": diff, "scale": scale if scale is not None else 3.0 / dk}
    if taps:
        m["conv"] = taps
    if rot:
        m["rot"] = rot
    part = DifferentialAttention(d, H, G, dk, dv, "m.", diff, 1e-5, scale=m["scale"], position=rope(rot), taps=taps, window=window)
    return part, m


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,G,dk,dv,taps,rot", [
    (40, 4, 2, 8, 16, 3, {"base": 900.0, "dims": 4}),        # cache rows of 16: the tensor-core kernels' smallest head
    (48, 6, 2, 16, 32, 4, None),                             # rows of 32, three heads a group, no rotation
    (64, 2, 1, 32, 64, 2, {"base": 10000.0, "dims": 20}),    # rows of 64: the tcgen05 prompt kernel
    (24, 2, 2, 12, 10, 0, {"base": 50.0, "dims": 12}),       # values narrower than two maps, no convolution, G = H
    (32, 3, 1, 6, 20, 1, {"base": 100.0, "dims": 2}),        # values wider than two maps, one tap
    (32, 1, 1, 24, 24, 5, {"base": 3000.0, "dims": 8}),      # one head
    (64, 4, 2, 48, 96, 3, {"base": 50000.0, "dims": 16}),    # rows of 96: the mma.sync kernels for prompts too
    (64, 8, 2, 64, 128, 4, {"base": 50000.0, "dims": 64}),   # rows of 128, eight rows a group
])
def test_differential_attention_under_every_cut(dtype, d, H, G, dk, dv, taps, rot):
    part, m = diff_part(d, H, G, dk, dv, taps, rot)
    prec, w = bind_random(part, dtype, std=0.35)
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 70}, lambda x: P.differential_attention(x, w, "m.", m, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("dk,dv", [(32, 64), (12, 20)])
def test_differential_attention_finds_one_key_among_hundreds(dtype, dk, dv):
    """The first map's query reads the input as its key does, eight times as large, the convolution passes the current
    token alone and nothing is rotated: a token looks at the tokens whose input resembles its own.  Queries and keys read
    the first half of the input, values the second.  The last three tokens repeat the first half of the inputs at positions
    3, 15 (a page's last row) and 16 (a page's first), 400 tokens back; without those keys the result is another one."""
    d, H, G, taps, T = 48, 2, 1, 3, 420
    part, m = diff_part(d, H, G, dk, dv, taps, None, scale=1.0 / dk)
    prec, w = bind_random(part, dtype, std=0.25)
    with torch.no_grad():
        wk = part.w_in[H * 2 * dk:H * 2 * dk + dk].clone()          # key head 0, map 1
        for h in range(H):
            part.w_in[h * 2 * dk:h * 2 * dk + dk] = wk * 8.0
        part.w_in[:(H + G) * 2 * dk, d // 2:] = 0
        part.w_in[(H + G) * 2 * dk:(H + G) * 2 * dk + G * dv, :d // 2] = 0
        part.conv.weight.zero_()
        part.conv.weight[:, -1] = 1.0
    for h in range(H):
        w["m.q"][h * 2 * dk:h * 2 * dk + dk] = w["m.k"][:dk] * 8.0
    w["m.q"][:, d // 2:] = 0
    w["m.k"][:, d // 2:] = 0
    w["m.v"][:, :d // 2] = 0
    for c in ("q", "k", "v"):
        w[f"m.{c}.conv"] = np.zeros_like(w[f"m.{c}.conv"])
        w[f"m.{c}.conv"][:, -1] = 1.0
    x = torch.randn(T, d, device="cuda")
    quiet = torch.ones(T, 1, device="cuda") * 0.3          # every other token's key is small, so that none competes
    quiet[[3, 15, 16]] = 1.0
    x[:, :d // 2] *= quiet
    for i, src in enumerate((3, 15, 16)):
        x[T - 3 + i, :d // 2] = x[src, :d // 2]
    x = x.to(dtype)
    xs = x.double().cpu().numpy()
    want = P.differential_attention(xs, w, "m.", m, 1e-5)
    lost = P.differential_attention(xs[17:], w, "m.", m, 1e-5)
    assert np.abs(want[-3:] - lost[-3:]).max() > 0.2 * np.abs(want[-3:]).max()
    hs = Harness(part, prec, dtype, {"a": x}, page_tokens=16)
    for steps in ([[("a", T)]], [[("a", T - 11)]] + [[("a", 1)]] * 11, [[("a", 2)], [("a", 250)], [("a", 165)], [("a", 2)], [("a", 1)]]):
        close(hs.run(steps)["a"][-3:], want[-3:], dtype, "far keys")


# ------------------------------------------------------------------------------------ latent attention over a window

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,dk,dv,r,window", [(40, 3, 8, 12, 16, 7), (64, 8, 32, 48, 64, 37), (48, 2, 16, 8, 24, 33),
                                                (40, 5, 6, 10, 10, None), (64, 4, 16, 48, 144, 21), (32, 1, 8, 8, 32, 1)])
def test_latent_attention_without_positions_over_a_window(dtype, d, H, dk, dv, r, window):
    """Sharp scores (a large factor), so that a token's result hangs on few keys: a window that is one token off shows at
    every token whose strongest key lies at the window's edge, which the test first makes sure of."""
    from hk_b200.parts import LatentAttention
    scale = 6.0 / dk
    part = LatentAttention(d, H, dk, 0, dv, r, "m.", 1e-5, scale, gate=True, window=window)
    prec, w = bind_random(part, dtype, std=0.35)
    m = {"heads": H, "dim": dk, "vdim": dv, "kv_rank": r, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if window and window > 1:
        x = np.random.default_rng(0).standard_normal((90, d))
        base = P.latent_attention(x, w, "m.", m, 1e-5)
        for other in (window - 1, window + 1):
            off = P.latent_attention(x, w, "m.", dict(m, mask={"size": other}), 1e-5)
            assert (np.abs(off - base).max(axis=1) > 0.1 * np.abs(base).max()).sum() >= 3
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 90}, lambda x: P.latent_attention(x, w, "m.", m, 1e-5))


# ------------------------------------------------------------------------------------ retention

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,dk,dv,rot,decay", [
    (40, 3, 8, 12, {"base": 10000.0, "dims": 8}, [0.9, 0.97, 0.995]), (48, 2, 24, 8, {"base": 50000.0, "dims": 12}, [0.96, 0.999]),
    (64, 2, 64, 64, {"base": 200000.0, "dims": 64}, [0.98, 0.999]), (40, 3, 10, 6, None, [0.8, 0.9, 0.95]),
    (32, 1, 136, 7, {"base": 100.0, "dims": 2}, [1.0]), (32, 4, 8, 16, {"base": 500.0, "dims": 6}, [0.5, 0.9, 0.99, 1.0])])
def test_retention_under_every_cut(dtype, d, H, dk, dv, rot, decay):
    from hk_b200.parts import Retention
    part = Retention(d, H, dk, dv, decay, "m.", 1e-5, position=rope(rot))
    prec, w = bind_random(part, dtype, std=0.3)
    m = {"heads": H, "dim": dk, "vdim": dv, "decay": decay}
    if rot:
        m["rot"] = rot
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 64}, lambda x: P.retention(x, w, "m.", m, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_retention_keeps_what_a_token_wrote_300_tokens_back(dtype):
    """Query and key read the first 16 input dims one to one, nothing is rotated, the decay is 1: position 3 and the last
    token have their key in dims 8..15, every other token in dims 0..7 (where the last token's query is zero), so the last
    token reads what position 3 wrote and its own value.  A state that is lost, cleared or decayed gives its own alone."""
    from hk_b200.parts import Retention
    d, H, dk, dv, T = 32, 2, 16, 8, 301
    part = Retention(d, H, dk, dv, [1.0, 1.0], "m.", 1e-5)
    prec, w = bind_random(part, dtype, std=0.2)
    eye = torch.zeros(H * dk, d, device="cuda")
    for h in range(H):
        eye[h * dk:(h + 1) * dk, :dk] = torch.eye(dk, device="cuda")
    with torch.no_grad():
        part.w_in[:H * dk] = eye
        part.w_in[H * dk:2 * H * dk] = eye
        part.w_in[2 * H * dk:2 * H * dk + H * dv, :dk] = 0
    w["m.q"] = w["m.k"] = eye.double().cpu().numpy()
    w["m.v"][:, :dk] = 0
    x = torch.randn(T, d, device="cuda")
    x[:, 8:16] = 0
    x[3, :8] = 0
    x[3, 8:16] = torch.randn(8, device="cuda")
    x[300, :16] = x[3, :16]
    x = x.to(dtype)
    m = {"heads": H, "dim": dk, "vdim": dv, "decay": [1.0, 1.0]}
    want = P.retention(x.double().cpu().numpy(), w, "m.", m, 1e-5)
    lost = P.retention(x[4:].double().cpu().numpy(), w, "m.", m, 1e-5)
    assert np.abs(want[-1] - lost[-1]).max() > 0.1 * np.abs(want[-1]).max()
    hs = Harness(part, prec, dtype, {"a": x})
    for steps in ([[("a", T)]], [[("a", 290)]] + [[("a", 1)]] * 11, [[("a", 2)], [("a", 150)], [("a", 147)], [("a", 2)]]):
        close(hs.run(steps)["a"][-3:], want[-3:], dtype, "far write")


# ------------------------------------------------------------------------------------ short convolution without activation

@pytest.mark.parametrize("taps", [1, 2, 5])
def test_short_convolution_without_activation_across_the_edges_of_portions(taps):
    from hk_b200.csrc import ops
    C, n = 37, 29
    wt = torch.randn(C, taps, device="cuda")
    x = torch.randn(n, C + 3, device="cuda")
    tail = torch.zeros(2, max(taps - 1, 1), C, device="cuda")
    got, p = [], 0
    for c in (1, 2, 1, 6, 2, 17):
        y = torch.full((c, C), float("nan"), device="cuda")
        ops.short_conv(x[p:p + c, 1:1 + C], wt, torch.tensor([[1, 0, c]], dtype=torch.int32, device="cuda"), tail, y, act="none")
        got.append(y)
        p += c
    want = P.short_conv(x[:, 1:1 + C].double().cpu().numpy(), wt.double().cpu().numpy())
    np.testing.assert_allclose(torch.cat(got).double().cpu().numpy(), want, rtol=1e-5, atol=1e-5)
    assert torch.all(tail[0] == 0.0)


# ------------------------------------------------------------------------------------ feed-forwards

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,F,limit,rows", [(40, 52, 0.7, 9), (64, 160, 1.0, 70), (128, 320, 2.5, 300), (128, 320, 1.5, 12),
                                            (192, 256, 1.0, 5), (256, 1024, 1.2, 2048)])
def test_clamped_feed_forward(dtype, d, F, limit, rows):
    """Rows and sizes that reach every kernel with the activation in its epilogue (the generic product with the
    activation's own kernel, the streaming product, the tcgen05 product with and without K slices)."""
    from hk_b200.parts import SwiGLUFeedForward
    part = SwiGLUFeedForward(d, F, "f.", act="swish_clamped", names={"gate": "gate", "up": "up", "down": "down"}, limit=limit, slope=1.702)
    prec, w = bind_random(part, dtype, std=0.2)
    x = (torch.randn(rows, d, device="cuda") * 1.5).to(dtype)
    xs = x.double().cpu().numpy()
    assert (np.abs(xs @ w["f.up"].T) > limit).mean() > 0.05 and ((xs @ w["f.gate"].T) > limit).mean() > 0.02     # the limits bite
    y = torch.zeros(rows, d, device="cuda")
    part.forward(x, y, None, accumulate=False)
    close(y.double().cpu().numpy(), P.clamped_feed_forward(xs, w, "f.", limit), dtype, "clamped")


def routed_part(d, F, E, top, scale, groups, shared):
    from hk_b200.parts import RoutedFeedForward, SwiGLUFeedForward
    names = {"gate": "gate", "up": "up", "down": "down"}
    sh = SwiGLUFeedForward(d, shared, "f.shared.", names=names) if shared else None
    part = RoutedFeedForward(d, F, E, top, "f.", scores="sigmoid", correction=True, groups=groups[0] if groups else 0,
                             keep=groups[1] if groups else 0, weight_scale=scale, norm_eps=1e-20, shared=sh, shared_gated=bool(shared))
    mlp = {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": top, "scale": scale}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        mlp["shared"] = {"ff": shared}
    return part, mlp


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,F,E,top,scale,groups,shared,rows,shift", [
    (40, 12, 6, 1, 2.5, (6, 2), 20, 33, 0.0),          # groups of one expert
    (48, 24, 10, 3, 1.3, (2, 1), 40, 57, -3.0),        # every choice score negative: a refused group must not count as 0
    (64, 32, 9, 3, 2.0, (3, 2), 0, 300, 0.0),          # no shared expert; prompt-sized rows
    (32, 16, 4, 4, 1.0, (2, 2), 24, 20, 0.5),          # all experts, all groups
    (128, 64, 8, 2, 1.0, None, 96, 600, 0.0),          # no groups; the tensor-core grouped product's sizes
])
def test_sigmoid_router_with_groups_and_a_gated_shared_expert(dtype, d, F, E, top, scale, groups, shared, rows, shift):
    from hk_b200.parts import RoutedFeedForward
    part, mlp = routed_part(d, F, E, top, scale, groups, shared)
    prec, w = bind_random(part, dtype, std=0.2)
    with torch.no_grad():
        part.w_correction.mul_(3.0).add_(shift)
    w["f.correction"] = part.w_correction.double().cpu().numpy()
    x = torch.randn(rows, d, device="cuda").to(dtype)
    xs = x.double().cpu().numpy()
    corr = w["f.correction"]
    RoutedFeedForward.route_log = log = []
    try:
        y = torch.zeros(rows, d, device="cuda")
        part.forward(x, y, None, accumulate=False)
    finally:
        RoutedFeedForward.route_log = None
    ids = log[0].cpu().numpy()
    # the engine's experts against the plain router's wherever the choice was clear (groups and experts alike)
    free = [P.route(xs[t] @ w["f.router"].T, corr, top, mlp["router"].get("groups")) for t in range(rows)]
    own, margins = np.asarray([f[0] for f in free]), np.asarray([f[2] for f in free])
    clear = margins >= (1e-4 if dtype == torch.float32 else 2e-2)
    assert clear.mean() > 0.5
    assert (np.sort(own[clear], axis=1) == np.sort(ids[clear], axis=1)).all()
    if shift < 0:
        assert (P.sigmoid(xs @ w["f.router"].T) + corr).max() < 0
    # the result along the engine's experts
    P.route_choices = {"f.": ids}
    try:
        want = P.routed_feed_forward(xs, w, "f.", mlp)
    finally:
        P.route_choices = None
    close(y.double().cpu().numpy(), want, dtype, "routed")
