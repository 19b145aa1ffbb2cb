"""The mechanisms of the Mifolorn decoder one by one: each part alone against its function of the plain
implementation (`plain_mifolorn`), whole, cut into portions down to two tokens, token by token, in batches of
unequal requests, and after slots and pages were freed and taken again.  Where random weights would hide a fault, the
weights or inputs are made so that it shows."""
import numpy as np
import pytest
import torch

import plain_mifolorn as P
from test_kedanex_parts_gpu import close, schedules
from test_parts_gpu import DTYPES, IDS, bind_random, make_ctx

pytestmark = pytest.mark.gpu


class Harness:
    """Runs a mixer part (with one cache or several) over several requests under a schedule of steps."""

    def __init__(self, part, prec, dtype, inputs, page_tokens=4, slots=3, pages=256):
        from hk_b200.cache.device import PagedCache
        from hk_b200.parts.parallel import mixer_cache_specs, mixer_caches
        self.part, self.prec, self.dtype, self.inputs = part, prec, dtype, inputs
        self.cache = PagedCache([mixer_cache_specs(part)], prec, page_tokens, pages, slots, 2048)
        self.handed = mixer_caches(part, self.cache.layers[0])

    def run(self, steps):
        names = sorted({r for st in steps for r, _ in st})
        slot = {r: self.cache.open() for r in names}
        fed = {r: 0 for r in names}
        got = {r: [] for r in names}
        for st in steps:
            spans = [(slot[r], fed[r], c) for r, c in st]
            ctx = make_ctx(self.prec, spans, self.cache, page_tokens=self.cache.page_tokens, part=self.part)
            ctx.page_tokens = self.cache.page_tokens
            xb = torch.cat([self.inputs[r][fed[r]:fed[r] + c] for r, c in st])
            y = torch.full((xb.shape[0], self.part.hidden), float("nan"), device="cuda")
            self.part.forward(xb, y, ctx, self.handed, accumulate=False)
            at = 0
            for r, c in st:
                got[r].append(y[at:at + c].double().cpu().numpy())
                at += c
                fed[r] += c
        for r in names:
            self.cache.close(slot[r])
        return {r: np.concatenate(v) for r, v in got.items()}


def under_every_cut(part, prec, dtype, lengths, plain, std_in=1.0):
    d = part.hidden
    inputs = {r: (torch.randn(n, d, device="cuda") * std_in).to(dtype) for r, n in lengths.items()}
    want = {r: plain(x.double().cpu().numpy()) for r, x in inputs.items()}
    hs = Harness(part, prec, dtype, inputs)
    first = None
    for name, steps in schedules(lengths).items():
        got = hs.run(steps)                 # the slots and pages of the run before are taken again
        for r in lengths:
            close(got[r], want[r], dtype, f"{name} {r}")
        if first is None:
            first = got
        elif dtype == torch.float32:
            for r in lengths:
                np.testing.assert_allclose(got[r], first[r], rtol=2e-5, atol=2e-6)


# ------------------------------------------------------------------------------------ gated delta rule


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,G,dk,dv,taps", [(40, 2, 1, 16, 8, 4), (24, 3, 3, 8, 12, 2), (72, 1, 1, 64, 64, 3), (48, 4, 2, 40, 20, 5),
                                              (32, 2, 2, 136, 6, 4), (24, 6, 2, 6, 7, 3), (32, 4, 4, 32, 32, 7), (24, 2, 1, 8, 12, 1)])
def test_gated_delta_rule_under_every_cut(dtype, d, H, G, dk, dv, taps):
    from hk_b200.parts import GatedDeltaRule
    part = GatedDeltaRule(d, H, G, dk, dv, taps, "m.", norm_eps=1e-5)
    prec, w = bind_random(part, dtype, std=0.3)
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "conv": taps}
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 64}, lambda x: P.gated_delta(x, w, "m.", m, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_gated_delta_rule_keeps_a_key_from_far_back(dtype):
    """A delta rule forgets a key when later keys overlap it, so the test keeps them apart: query and key read the
    first 16 input dims one to one (and the convolution passes the current token alone), the values read the other 16;
    position 3 and the last token have their key in dims 8..15, every other token in dims 0..7.  With a decay of 1 the
    last token, which brings a value of its own, reads a mixture of its value and that of position 3.  A state that is
    lost, cleared or decayed on the way gives its own value alone."""
    from hk_b200.parts import GatedDeltaRule
    d, H, G, dk, dv, taps, T = 32, 2, 1, 16, 8, 3, 301
    part = GatedDeltaRule(d, H, G, dk, dv, taps, "m.", norm_eps=1e-5)
    prec, w = bind_random(part, dtype, std=0.2)
    eye = torch.zeros(dk, d, device="cuda")
    eye[:, :dk] = torch.eye(dk, device="cuda")
    with torch.no_grad():
        part.w_in[:dk] = eye
        part.w_in[dk:2 * dk] = eye
        part.w_in[2 * dk:2 * dk + H * dv, :dk] = 0                 # the values do not see the key's dims
        part.w_in[2 * dk + 2 * H * dv:2 * dk + 2 * H * dv + H] = 0     # beta = 1/2
        part.a_log.fill_(-30.0)
        part.conv.zero_()
        part.conv[:, -1] = 1.0
    w["m.q"] = w["m.k"] = eye.double().cpu().numpy()
    w["m.v"][:, :dk] = 0
    w["m.b"][:] = 0
    w["m.A_log"] = np.full(H, -30.0)
    for c in ("q", "k", "v"):
        w[f"m.{c}.conv"] = np.zeros_like(w[f"m.{c}.conv"])
        w[f"m.{c}.conv"][:, -1] = 1.0
    x = torch.randn(T, d, device="cuda")
    x[:, 8:16] = 0
    x[3, :8] = 0
    x[3, 8:16] = torch.randn(8, device="cuda")
    x[300, :16] = x[3, :16]
    x = x.to(dtype)
    m = {"heads": H, "kv_heads": G, "dim": dk, "vdim": dv, "conv": taps}
    want = P.gated_delta(x.double().cpu().numpy(), w, "m.", m, 1e-5)
    lost = P.gated_delta(x[4:].double().cpu().numpy(), w, "m.", m, 1e-5)
    assert np.abs(want[-1] - lost[-1]).max() > 0.1 * np.abs(want[-1]).max()
    hs = Harness(part, prec, dtype, {"a": x})
    for steps in ([[("a", T)]], [[("a", 290)]] + [[("a", 1)]] * 11, [[("a", 2)], [("a", 150)], [("a", 147)], [("a", 2)]]):
        close(hs.run(steps)["a"][-3:], want[-3:], dtype, "far key")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("taps", [2, 4, 6])
def test_short_convolution_across_the_edges_of_portions(dtype, taps):
    """Only the OLDEST tap has a weight: a row's output is the input taps - 1 rows back, which for the first rows of a
    portion lies in the portion before (or, with portions of one and two rows, several portions back), and is zero at
    the start of a request.  A second request in the same steps must not see the first one's rows."""
    from hk_b200.csrc import ops
    C, n_a, n_b = 70, 23, 11
    wt = torch.zeros(C, taps, device="cuda")
    wt[:, 0] = torch.linspace(0.5, 2.0, C, device="cuda")
    xa, xb = torch.randn(n_a, C + 5, device="cuda"), torch.randn(n_b, C + 5, device="cuda")
    tail = torch.zeros(4, taps - 1, C, device="cuda")
    tail[2].fill_(7.0)                             # a slot nobody uses must stay as it is
    cuts_a, cuts_b = [1, 2, 1, 5, 2, 12], [2, 1, 1, 3, 2, 2]
    got_a, got_b, pa, pb = [], [], 0, 0
    for ca, cb in zip(cuts_a, cuts_b):
        x = torch.cat([xa[pa:pa + ca], xb[pb:pb + cb]])
        y = torch.full((ca + cb, C), float("nan"), device="cuda")
        segs = torch.tensor([[3, 0, ca], [1, ca, cb]], dtype=torch.int32, device="cuda")
        ops.short_conv(x[:, 2:2 + C], wt, segs, tail, y)
        got_a.append(y[:ca]); got_b.append(y[ca:])
        pa, pb = pa + ca, pb + cb
    for got, x in ((torch.cat(got_a), xa), (torch.cat(got_b), xb)):
        z = torch.zeros(x.shape[0], C, device="cuda")
        z[taps - 1:] = x[:x.shape[0] - (taps - 1), 2:2 + C] * wt[:, 0]
        want = z * torch.sigmoid(z)
        assert torch.allclose(got, want, rtol=1e-6, atol=1e-6)
    assert torch.all(tail[2] == 7.0) and torch.all(tail[0] == 0.0)
    assert torch.equal(tail[3], xa[n_a - (taps - 1):, 2:2 + C]) and torch.equal(tail[1], xb[n_b - (taps - 1):, 2:2 + C])


# ------------------------------------------------------------------------------------ mLSTM


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,dk,dv,cap", [(40, 2, 16, 8, 8.0), (24, 3, 8, 11, 15.0), (72, 1, 64, 64, 10.0), (48, 2, 40, 23, 3.0),
                                           (32, 1, 136, 4, 12.0), (32, 4, 32, 63, 20.0)])
def test_mlstm_under_every_cut(dtype, d, H, dk, dv, cap):
    from hk_b200.parts import MLSTM
    part = MLSTM(d, H, dk, dv, cap, "m.", norm_eps=1e-5)
    prec, w = bind_random(part, dtype, std=0.3)
    m = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 64}, lambda x: P.mlstm(x, w, "m.", m, 1e-5), std_in=2.0)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_mlstm_gates_at_their_cap_and_a_maximum_that_starts_at_zero(dtype):
    """Large gate logits of either sign: the cap bounds them, and with strongly negative input gates the running maximum
    stays where it started (0, not minus infinity), which the normaliser's floor exp(-m) then shows.  Long decoding:
    the maximum and the state are carried through 200 single tokens."""
    from hk_b200.parts import MLSTM
    d, H, dk, dv, cap = 24, 2, 8, 12, 6.0
    part = MLSTM(d, H, dk, dv, cap, "m.", norm_eps=1e-5)
    prec, w = bind_random(part, dtype, std=0.3)
    K, V = H * dk, H * dv
    with torch.no_grad():
        part.i_bias.copy_(torch.tensor([-40.0, 40.0]))
        part.f_bias.copy_(torch.tensor([40.0, -2.0]))
    w["m.i.b"], w["m.f.b"] = np.array([-40.0, 40.0]), np.array([40.0, -2.0])
    m = {"heads": H, "dim": dk, "vdim": dv, "gate_cap": cap}
    x = torch.randn(230, d, device="cuda").to(dtype)
    want = P.mlstm(x.double().cpu().numpy(), w, "m.", m, 1e-5)
    other = dict(w)
    other["m.i.b"] = np.array([-40.0 + 3.0, 40.0])
    assert np.abs(P.mlstm(x.double().cpu().numpy()[:5], other, "m.", m, 1e-5) - want[:5]).max() < 1e-3 * np.abs(want[:5]).max()   # the cap holds
    hs = Harness(part, prec, dtype, {"a": x})
    for steps in ([[("a", 230)]], [[("a", 30)]] + [[("a", 1)]] * 200, [[("a", 1)]] * 3 + [[("a", 2)]] * 4 + [[("a", 219)]]):
        close(hs.run(steps)["a"], want, dtype, "capped gates")


# ------------------------------------------------------------------------------------ attention beside a delta rule


def left_part(d, m, eps, positions=600):
    from hk_b200.parts import GQAAttention, RopeScaling, RotaryEmbedding
    rope = None
    if m.get("rot"):
        r = m["rot"]
        s = r.get("scaling")
        sc = RopeScaling("yarn", factor=s["factor"], orig_ctx=s["original"], beta_fast=s["fast"], beta_slow=s["slow"]) if s else None
        rope = RotaryEmbedding(r["base"], r["dims"], positions, pairing="half", scaling=sc)
    return GQAAttention(d, m["heads"], m["kv_heads"], m["dim"], "m.left.", qk_norm_eps=eps, position=rope, scale=m["scale"],
                        qkv_bias=True, v_head_dim=m["vdim"], softcap=m.get("softcap"), gate=True,
                        names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g",
                               "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"})


YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
LEFTS = [
    {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "softcap": 20.0, "rot": {"base": 900.0, "dims": 8, "scaling": YARN}},
    {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 24, "scale": 0.2, "rot": {"base": 10000.0, "dims": 32}},
    {"heads": 3, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.125, "softcap": 5.0, "rot": {"base": 20000.0, "dims": 32, "scaling": YARN}},
    {"heads": 6, "kv_heads": 3, "dim": 40, "vdim": 48, "scale": 0.16},
]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("left", LEFTS, ids=["capped16", "narrow_values", "tensor64", "plain40"])
def test_attention_with_biases_cap_and_gate_under_every_cut(dtype, left):
    d = 48
    part = left_part(d, left, 1e-5)
    prec, w = bind_random(part, dtype, std=0.3)
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 64}, lambda x: P.softmax_attention(x, w, "m.left.", left, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("far", [0, 15, 16, 17, 255, 256])
def test_attention_finds_one_key_among_hundreds(dtype, far):
    """Query and key share weights (which read the first half of the input; the values read the second half) and have no
    bias, and the last token repeats the first half of the input of position `far`: that key's score stands out among 400,
    at the first positions and on either side of page borders, in a prompt, decoded alone and in a portion of two.  The
    result is half the far token's value, which a key that is lost, or read from the wrong place, does not give."""
    left = {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.5}
    d, T = 32, 400
    part = left_part(d, left, 1e-5)
    prec, w = bind_random(part, dtype, std=0.25)
    K = left["kv_heads"] * left["dim"]
    with torch.no_grad():
        part.w_qkv[2 * K:3 * K, d // 2:] = 0
        part.w_qkv[:K] = part.w_qkv[2 * K:3 * K]
        part.w_qkv[K:2 * K] = part.w_qkv[2 * K:3 * K]
        part.w_qkv[3 * K:4 * K, :d // 2] = 0
        part.b_qkv[:3 * K] = 0
    w["m.left.k"][:, d // 2:] = 0
    w["m.left.q"] = np.concatenate([w["m.left.k"], w["m.left.k"]])
    w["m.left.v"][:, :d // 2] = 0
    for b in ("q.b", "k.b"):
        w["m.left." + b] = np.zeros_like(w["m.left." + b])
    x = torch.randn(T, d, device="cuda")
    x[:, :d // 2] *= 0.3
    x[far, :d // 2] = torch.randn(d // 2, device="cuda") * 3.0
    x[T - 1, :d // 2] = x[far, :d // 2]
    x = x.to(dtype)
    want = P.softmax_attention(x.double().cpu().numpy(), w, "m.left.", left, 1e-5)
    moved = x.clone()
    moved[far] = x[far - 1 if far else 1]
    assert np.abs(P.softmax_attention(moved.double().cpu().numpy(), w, "m.left.", left, 1e-5)[-1] - want[-1]).max() \
        > 0.2 * np.abs(want[-1]).max()
    hs = Harness(part, prec, dtype, {"a": x}, page_tokens=16)
    for steps in ([[("a", T)]], [[("a", T - 1)], [("a", 1)]], [[("a", 100)], [("a", T - 102)], [("a", 2)]]):
        close(hs.run(steps)["a"][-1:], want[-1:], dtype, f"far key at {far}")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("which", [0, 1, 2])
def test_parallel_mixer_under_every_cut(dtype, which):
    from hk_b200.parts import GatedDeltaRule, ParallelMixer
    d = 48
    left = LEFTS[which]
    right = [{"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 12, "conv": 3}, {"heads": 1, "kv_heads": 1, "dim": 64, "vdim": 16, "conv": 4},
             {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "conv": 4}][which]
    scales = [(0.7, 1.3), (1.0, 0.5), (-0.9, 2.0)][which]
    m = {"left": left, "right": right, "left_scale": scales[0], "right_scale": scales[1]}
    part = ParallelMixer(left_part(d, left, 1e-5),
                         GatedDeltaRule(d, right["heads"], right["kv_heads"], right["dim"], right["vdim"], right["conv"], "m.right.",
                                        norm_eps=1e-5), scales[0], scales[1])
    prec, w = bind_random(part, dtype, std=0.3)
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 64}, lambda x: P.parallel(x, w, "m.", m, 1e-5))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_parallel_mixer_whose_sides_carry_no_factor(dtype):
    """A matrix memory on the right has no place for a factor on its result: both sides then write buffers of their
    own and one kernel sums them with the factors."""
    from hk_b200.parts import MLSTM, ParallelMixer
    d, left = 48, LEFTS[0]
    right = {"heads": 2, "dim": 16, "vdim": 8, "gate_cap": 8.0}
    part = ParallelMixer(left_part(d, left, 1e-5), MLSTM(d, 2, 16, 8, 8.0, "m.right.", norm_eps=1e-5), 0.6, -1.4)
    assert part.left.out_scale == 1.0
    prec, w = bind_random(part, dtype, std=0.3)
    under_every_cut(part, prec, dtype, {"a": 37, "b": 9, "c": 64},
                    lambda x: 0.6 * P.softmax_attention(x, w, "m.left.", left, 1e-5) - 1.4 * P.mlstm(x, w, "m.right.", right, 1e-5))


# ------------------------------------------------------------------------------------ per-layer token input, sums


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,dim,layers,i", [(48, 6, 4, 2), (64, 16, 3, 0), (40, 5, 2, 1), (128, 32, 1, 0)])
def test_token_side_input(dtype, d, dim, layers, i):
    from hk_b200.parts import TokenSideInput
    from types import SimpleNamespace
    vocab, n = 57, 21
    part = TokenSideInput(d, vocab, "side.embed", layers * dim, i * dim, dim, f"l{i}.side.", 1e-5)
    prec, w = bind_random(part, dtype, std=0.3)
    ids = torch.randint(0, vocab, (n,), dtype=torch.int32, device="cuda")
    x = torch.randn(n, d, device="cuda") * 2
    want = x.double().cpu().numpy()
    xin = want if dtype == torch.float32 else x.to(dtype).double().cpu().numpy()
    want = want + P.token_side_input(xin, ids.cpu().numpy(), w, i, dim, 1e-5)
    part.forward(x, SimpleNamespace(token_ids=ids))
    close(x.double().cpu().numpy(), want, dtype, "token side input")


def test_scaled_sum_and_narrow():
    from hk_b200.csrc import ops
    for n in (1, 3, 4, 1000, 4099):
        a, b, out = (torch.randn(n, device="cuda") for _ in range(3))
        want = out + 0.7 * a - 1.5 * b
        ops.scaled_sum(out, a, 0.7, b, -1.5)
        assert torch.allclose(out, want, rtol=1e-6, atol=1e-6)
        ops.scaled_sum(out, a, 2.0, accumulate=False)
        assert torch.allclose(out, 2.0 * a)
        sl = torch.randn(n + 1, device="cuda")[1:]            # not 16-byte aligned
        ops.scaled_sum(out, sl, 1.0)
        assert torch.allclose(out, 2.0 * a + sl, rtol=1e-6, atol=1e-6)
        nb = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        ops.narrow(a, nb)
        assert torch.equal(nb, a.to(torch.bfloat16))
