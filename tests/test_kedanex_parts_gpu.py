"""The mechanisms of the Kedanex decoder one by one: each part alone against its function of the plain
implementation (`plain_kedanex`), whole, cut into portions down to two tokens, token by token, in batches of
unequal requests, and after a slot was freed and taken again.  Where random weights would hide a fault, the
weights or inputs are made so that it shows."""
import math

import numpy as np
import pytest
import torch

import plain_kedanex as K
from test_parts_gpu import DTYPES, IDS, bind_random, make_ctx

pytestmark = pytest.mark.gpu


def close(got, want, dtype, what=""):
    """max |difference| relative to the largest |value|: float32 by accumulated rounding, bfloat16 by 8-bit inputs."""
    scale = max(float(np.abs(want).max()), 1e-6)
    worst = float(np.abs(got - want).max()) / scale
    limit = 3e-5 if dtype == torch.float32 else 3e-2
    assert np.isfinite(got).all() and worst <= limit, f"{what}: {worst:.3g} of the largest value, allowed {limit:.3g}"


class MixerHarness:
    """Runs a mixer part over several requests under a schedule of steps; every step is one batch."""

    def __init__(self, part, prec, dtype, inputs, page_tokens=4, slots=3, pages=64):
        from hk_b200.cache.device import PagedCache
        self.part, self.prec, self.dtype, self.inputs = part, prec, dtype, inputs
        self.cache = PagedCache([[part.cache_spec()]], prec, page_tokens, pages, slots, 1024)
        self.d_out = part.hidden

    def run(self, steps, names=None):
        """steps: [[(request, count), ...], ...]; returns {request: rows [T, d]} (float64)."""
        names = names or sorted({r for st in steps for r, _ in st})
        slot = {r: self.cache.open() for r in names}
        fed = {r: 0 for r in names}
        got = {r: [] for r in names}
        for st in steps:
            spans = [(slot[r], fed[r], c) for r, c in st]
            ctx = make_ctx(self.prec, spans, self.cache, page_tokens=self.cache.page_tokens, part=self.part)
            xb = torch.cat([self.inputs[r][fed[r]:fed[r] + c] for r, c in st])
            y = torch.full((xb.shape[0], self.d_out), float("nan"), device="cuda")
            self.part.forward(xb, y, ctx, self.cache.layers[0][0], accumulate=False)
            at = 0
            for r, c in st:
                got[r].append(y[at:at + c].double().cpu().numpy())
                at += c
                fed[r] += c
        self.last_slots = slot
        states = {r: self.cache.layers[0][0].state[slot[r]].double().cpu().numpy() for r in names} \
            if self.cache.layers[0][0].kind == "state" else {}
        for r in names:
            self.cache.close(slot[r])
        return {r: np.concatenate(v) for r, v in got.items()}, states


def schedules(lengths):
    """Whole; token by token; portions of changing size down to two tokens; a batch of all requests with unequal
    portions."""
    names = sorted(lengths)
    whole = [[(r, lengths[r])] for r in names]
    single = [[(r, 1)] for r in names for _ in range(lengths[r])]
    sizes = (5, 2, 3, 1, 7, 2, 11, 4)
    portions = []
    for r in names:
        p, k = 0, 0
        while p < lengths[r]:
            c = min(sizes[k % len(sizes)], lengths[r] - p)
            portions.append([(r, c)])
            p, k = p + c, k + 1
    left = dict(lengths)
    batch, k = [], 0
    while any(left.values()):
        st = []
        for i, r in enumerate(names):
            if left[r]:
                c = min(left[r], (1, 6, 2, 9)[(k + i) % 4])
                st.append((r, c))
                left[r] -= c
        batch.append(st)
        k += 1
    return {"whole": whole, "single": single, "portions": portions, "batch": batch}


# ------------------------------------------------------------------------------------ delta rule


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,dk,rank", [(40, 2, 16, 6), (24, 3, 8, 4), (72, 1, 64, 8), (48, 2, 40, 5), (32, 1, 136, 3),
                                         (24, 2, 6, 2), (16, 1, 260, 2), (32, 4, 32, 7)])
def test_general_delta_rule_under_every_cut(dtype, d, H, dk, rank):
    from hk_b200.parts import GeneralDeltaRule
    part = GeneralDeltaRule(d, H, dk, "m.", norm_eps=1e-5, decay_rank=rank)
    prec, w = bind_random(part, dtype, std=0.3)
    lengths = {"a": 37, "b": 9, "c": 64}
    inputs = {r: torch.randn(n, d, device="cuda").to(dtype) for r, n in lengths.items()}
    want, want_state = {}, {}
    for r, x in inputs.items():
        want[r], want_state[r] = K.general_delta(x.double().cpu().numpy(), w, "m.", H, dk, 1e-5)
    hs = MixerHarness(part, prec, dtype, inputs)
    first = None
    for name, steps in schedules(lengths).items():
        got, states = hs.run(steps)           # the slots of the run before are taken again, with their old contents zeroed
        for r in lengths:
            close(got[r], want[r], dtype, f"{name} {r}")
            close(states[r], want_state[r], dtype, f"state after {name} {r}")
        if first is None:
            first = got
        elif dtype == torch.float32:
            for r in lengths:                 # the scan walks the tokens in the same order however they were cut
                np.testing.assert_allclose(got[r], first[r], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_general_delta_rule_keeps_a_key_from_far_back(dtype):
    """With decay 1 and removal 0 the state is the sum of k v^T; receptance and key share their weight, so a token
    whose input is the sum of the inputs of positions 3 and 7 reads those positions' values back, beside its own.
    A state that is lost, cleared or decayed on the way gives another mixture."""
    from hk_b200.parts import GeneralDeltaRule
    d, H, dk, T = 32, 2, 16, 301
    part = GeneralDeltaRule(d, H, dk, "m.", norm_eps=1e-5, decay_rank=4)
    prec, w = bind_random(part, dtype, std=0.2)
    K_ = H * dk
    with torch.no_grad():
        part.w_in[:K_] = part.w_in[K_:2 * K_]                 # r = k
        part.a_bias.fill_(-30.0)
        part.w_bias.fill_(-30.0)
    w["m.r"], w["m.a.b"], w["m.w0"] = w["m.k"], np.full(K_, -30.0), np.full(K_, -30.0)
    x = torch.randn(T, d, device="cuda") * 0.1
    x[3] = torch.randn(d, device="cuda") * 3.0
    x[7] = torch.randn(d, device="cuda") * 6.0
    x[300] = x[3] + x[7]          # two far keys of unequal size: the head's norm cannot hide their loss
    x = x.to(dtype)
    want, _ = K.general_delta(x.double().cpu().numpy(), w, "m.", H, dk, 1e-5)
    lost, _ = K.general_delta(x[8:].double().cpu().numpy(), w, "m.", H, dk, 1e-5)
    assert np.abs(want[-1] - lost[-1]).max() > 0.05 * np.abs(want[-1]).max()       # the far key does show
    hs = MixerHarness(part, prec, dtype, {"a": x})
    for steps in ([[("a", T)]], [[("a", 290)]] + [[("a", 1)]] * 11, [[("a", 2)], [("a", 150)], [("a", 147)], [("a", 2)]]):
        got, _ = hs.run(steps)
        close(got["a"][-1:], want[-1:], dtype, "the far key's value")
        close(got["a"], want, dtype)


# ------------------------------------------------------------------------------------ minGRU


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,width", [(40, 24), (24, 200), (64, 1)])
def test_mingru_under_every_cut(dtype, d, width):
    from hk_b200.parts import MinGRU
    part = MinGRU(d, width, "m.")
    prec, w = bind_random(part, dtype, std=0.4)
    lengths = {"a": 50, "b": 3, "c": 21}
    inputs = {r: torch.randn(n, d, device="cuda").to(dtype) for r, n in lengths.items()}
    want, want_state = {}, {}
    for r, x in inputs.items():
        want[r], want_state[r] = K.mingru(x.double().cpu().numpy(), w, "m.")
    hs = MixerHarness(part, prec, dtype, inputs)
    for name, steps in schedules(lengths).items():
        got, states = hs.run(steps)
        for r in lengths:
            close(got[r], want[r], dtype, f"{name} {r}")
            close(states[r], want_state[r], dtype, f"state after {name} {r}")


def test_mingru_candidate_has_both_branches():
    """Inputs of both signs reach the candidate: x + 1/2 above zero, sigmoid(x) below."""
    from hk_b200.parts import MinGRU
    part = MinGRU(8, 8, "m.")
    prec, w = bind_random(part, torch.float32, std=1.0)
    x = torch.randn(40, 8, device="cuda")
    c = K.linear(x.double().cpu().numpy(), w["m.x"], w["m.x.b"])
    assert (c > 0.5).any() and (c < -0.5).any()
    hs = MixerHarness(part, prec, torch.float32, {"a": x})
    got, _ = hs.run([[("a", 40)]])
    close(got["a"], K.mingru(x.double().cpu().numpy(), w, "m.")[0], torch.float32)


# ------------------------------------------------------------------------------------ attention


def attention_part(d, H, G, hd, vd, window, rot_dims, scale, positions=512, base=700.0):
    from hk_b200.parts import GQAAttention, RotaryEmbedding
    rope = RotaryEmbedding(base, rot_dims, positions, pairing="half") if rot_dims else None
    part = GQAAttention(d, H, G, hd, "m.", qk_norm_eps=1e-5, position=rope, window=window, scale=scale, qk_norm_after=True,
                        qk_norm_weight=False, value_from_key=True, v_head_dim=vd, sink=True, names={"q": "q", "k": "k", "o": "o"})
    mixer = dict(heads=H, kv_heads=G, dim=hd, vdim=vd, mask={"size": window}, scale=scale)
    if rot_dims:
        mixer["rot"] = {"base": base, "dims": rot_dims}
    return part, mixer


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,G,hd,vd,window,rot", [(40, 4, 2, 16, 16, 7, 8), (24, 3, 3, 8, 4, 1000, 8), (48, 6, 1, 32, 32, 33, 0),
                                                    (64, 2, 1, 64, 64, 20, 64), (40, 2, 2, 40, 24, 5, 12),
                                                    # every head size of the flash kernels, which take the bfloat16 steps
                                                    (64, 2, 1, 128, 128, 40, 128), (48, 4, 1, 96, 96, 50, 96), (40, 4, 2, 48, 48, 9, 16),
                                                    (64, 2, 2, 80, 80, 1000, 40), (64, 2, 1, 112, 112, 30, 112), (32, 8, 1, 16, 16, 1, 16)])
def test_window_sink_attention_under_every_cut(dtype, d, H, G, hd, vd, window, rot):
    part, mixer = attention_part(d, H, G, hd, vd, window, rot, scale=0.4)
    prec, w = bind_random(part, dtype, std=0.3)
    lengths = {"a": 45, "b": 6, "c": 70}
    inputs = {r: torch.randn(n, d, device="cuda").to(dtype) for r, n in lengths.items()}
    want = {r: K.window_sink_attention(x.double().cpu().numpy(), w, "m.", mixer, 1e-5) for r, x in inputs.items()}
    hs = MixerHarness(part, prec, dtype, inputs, page_tokens=4, pages=96)
    for name, steps in schedules(lengths).items():
        got, _ = hs.run(steps)
        for r in lengths:
            close(got[r], want[r], dtype, f"{name} {r}")
        hs.cache.books.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hd", [16, 64])
def test_window_edge_and_sink_stand_out(dtype, hd):
    """Queries and keys share their weight and nothing is rotated, so a token that repeats the input of position j
    meets that key with the largest score there is and takes nearly all of its output from it, as long as j is inside
    its window: at i = j + window - 1 it is, at i = j + window it is not.  The marked key's input is large, so its
    value is.  A window that is one token off in either direction changes one of the two rows completely, in a prompt
    portion and in a decoded token alike.  Negated queries push every score far below zero: then the sink takes the
    weight and the output is nearly zero; without a sink it would be a mean of values."""
    d, H, G, window, j, T = 32, 2, 1, 11, 5, 40
    part, mixer = attention_part(d, H, G, hd, hd, window, 0, scale=12.0 / hd)
    prec, w = bind_random(part, dtype, std=0.3)
    with torch.no_grad():
        part.w_qkv[:H * hd] = part.w_qkv[H * hd:].repeat(H, 1)            # q of every head = k
    w["m.q"] = np.concatenate([w["m.k"]] * H)
    x = torch.randn(T, d, device="cuda")
    x[j] = torch.randn(d, device="cuda") * 4.0
    x[j + window - 1] = x[j] / 4.0
    x[j + window] = x[j] / 4.0
    x = x.to(dtype)
    xn = x.double().cpu().numpy()
    want = K.window_sink_attention(xn, w, "m.", mixer, 1e-5)
    for off in (-1, 1):                                # the oracle itself tells the neighbours apart
        other = K.window_sink_attention(xn, w, "m.", dict(mixer, mask={"size": window + off}), 1e-5)
        row = j + window - 1 if off < 0 else j + window
        assert np.abs(other[row] - want[row]).max() > 0.3 * np.abs(want[row]).max()
    hs = MixerHarness(part, prec, dtype, {"a": x}, page_tokens=4)
    for steps in ([[("a", T)]], [[("a", j + window - 2)]] + [[("a", 1)]] * (T - j - window + 2), [[("a", j + 2)], [("a", window - 3)], [("a", 2)], [("a", T - j - window - 1)]]):
        got, _ = hs.run(steps)
        close(got["a"], want, dtype)
    # the sink: q = -k
    with torch.no_grad():
        part.w_qkv[:H * hd] = -part.w_qkv[:H * hd]
    w["m.q"] = -w["m.q"]
    want = K.window_sink_attention(xn[:1], w, "m.", mixer, 1e-5)
    no_sink = K.linear(np.concatenate([K.linear(xn[:1], w["m.k"])] * H, axis=1), w["m.o"])
    assert np.abs(want).max() < 1e-3 * np.abs(no_sink).max()
    got, _ = hs.run([[("a", 1)]])
    assert np.abs(got["a"] - want).max() <= (1e-5 if dtype == torch.float32 else 1e-2) * np.abs(no_sink).max()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_attention_reads_a_key_from_far_back_and_across_page_borders(dtype):
    """One key among hundreds, on the first slot of a page, is the one that the last token repeats."""
    d, H, G, hd, T = 32, 2, 2, 16, 400
    part, mixer = attention_part(d, H, G, hd, hd, 1000, 0, scale=1.0)
    prec, w = bind_random(part, dtype, std=0.3)
    with torch.no_grad():
        part.w_qkv[:H * hd] = part.w_qkv[H * hd:]
    w["m.q"] = w["m.k"]
    for j in (0, 15, 16, 17, 250):
        x = torch.randn(T, d, device="cuda")
        x[j] = torch.randn(d, device="cuda") * 4.0
        x[T - 1] = x[j] / 4.0
        x = x.to(dtype)
        xn = x.double().cpu().numpy()
        want = K.window_sink_attention(xn, w, "m.", mixer, 1e-5)
        without = K.window_sink_attention(np.delete(xn, j, axis=0), w, "m.", mixer, 1e-5)
        assert np.abs(want[-1] - without[-1]).max() > 0.3 * np.abs(want[-1]).max()
        hs = MixerHarness(part, prec, dtype, {"a": x}, page_tokens=16, pages=32)
        for steps in ([[("a", T)]], [[("a", T - 3)]] + [[("a", 1)]] * 3):
            got, _ = hs.run(steps)
            close(got["a"][-4:], want[-4:], dtype, f"key at {j}")


# ------------------------------------------------------------------------------------ feed-forwards, block


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,F", [(40, 72), (24, 9), (128, 640)])
def test_polynorm_feed_forward(dtype, d, F):
    from hk_b200.parts import PolyNormFeedForward
    part = PolyNormFeedForward(d, F, "f.", eps=1e-5)
    prec, w = bind_random(part, dtype, std=0.3, norm_std=0.5)
    x = torch.randn(19, d, device="cuda").to(dtype)
    y = torch.full((19, d), float("nan"), device="cuda")
    part.forward(x, y, None, accumulate=False)
    want = K.polynorm_ff(x.double().cpu().numpy(), w, "f.", 1e-5)
    close(y.double().cpu().numpy(), want, dtype)
    base = torch.randn(19, d, device="cuda")
    z = base.clone()
    part.forward(x, z, None)                        # the default adds onto what is there
    close((z - base).double().cpu().numpy(), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,F,E,top,n", [(40, 24, 3, 1, 50), (32, 16, 8, 2, 150), (24, 8, 5, 5, 7), (64, 40, 4, 3, 1), (48, 72, 6, 2, 300),
                                         (40, 12, 3, 2, 33), (36, 20, 40, 4, 90), (128, 96, 1, 1, 70),
                                         # prompt-sized steps: in bfloat16 the tcgen05 grouped product takes them
                                         (64, 48, 6, 2, 700), (128, 96, 4, 3, 400), (256, 64, 8, 2, 1120), (72, 40, 3, 1, 1500)])
def test_routed_feed_forward(dtype, d, F, E, top, n):
    from hk_b200.parts import RoutedFeedForward
    part = RoutedFeedForward(d, F, E, top, "f.")
    prec, w = bind_random(part, dtype, std=0.3)
    x = torch.randn(n, d, device="cuda").to(dtype)
    xn = x.double().cpu().numpy()
    logits = np.sort(K.linear(xn, w["f.router"]), axis=1)
    gap = logits[:, E - top] - logits[:, E - top - 1] if top < E else np.ones(n)
    assert gap.min() > 1e-4                          # no row rests on a close call
    y = torch.full((n, d), float("nan"), device="cuda")
    from hk_b200.csrc import gemm_fast
    taken, plain_run = [], gemm_fast.run_grouped
    gemm_fast.run_grouped = lambda *a, **k: taken.append(plain_run(*a, **k)) or taken[-1]
    try:
        part.forward(x, y, None, accumulate=False)
    finally:
        gemm_fast.run_grouped = plain_run
    # a prompt-sized bfloat16 step took the tcgen05 grouped product for both of its products, nothing else did
    assert taken == ([True, True] if dtype == torch.bfloat16 and n * top >= part.TC_MIN_PAIRS else [])
    close(y.double().cpu().numpy(), K.routed_ff(xn, w, "f.", E, top), dtype)
    # a row's result does not depend on which rows share the batch
    some = [0, n // 2, n - 1]
    y2 = torch.empty((len(some), d), device="cuda")
    part.forward(x[some].contiguous(), y2, None, accumulate=False)
    if dtype == torch.float32 or n * top < part.TC_MIN_PAIRS:
        assert torch.equal(y2, y[some])
    else:                       # a few rows take another kernel than a prompt does: equal to rounding
        close(y2.double().cpu().numpy(), y[some].double().cpu().numpy(), dtype)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("with_ffn", [True, False])
def test_sandwich_norm_block(dtype, with_ffn):
    from hk_b200.cache.device import PagedCache
    from hk_b200.parts import MinGRU, PolyNormFeedForward, RMSNorm, SandwichNormBlock
    d, eps = 40, 2e-5
    ffn = (RMSNorm(d, eps, "n2"), PolyNormFeedForward(d, 56, "f.", eps), RMSNorm(d, eps, "n2b")) if with_ffn else (None, None, None)
    block = SandwichNormBlock(RMSNorm(d, eps, "n1"), MinGRU(d, 24, "m."), RMSNorm(d, eps, "n1b"), *ffn)
    prec, w = bind_random(block, dtype, std=0.3, norm_std=0.3)
    cache = PagedCache([block.cache_specs()], prec, 4, 16, 2, 64)
    slot = cache.open()
    x0 = torch.randn(17, d, device="cuda")
    x = x0.clone()
    ctx = make_ctx(prec, [(slot, 0, 17)], cache, part=block)
    block.forward(x, ctx, cache.layers[0])
    xn = x0.double().cpu().numpy()
    h = K.rms_norm(xn, w["n1"], eps)
    if dtype == torch.bfloat16:
        h = torch.from_numpy(h).to(torch.bfloat16).double().numpy()
    want = xn + K.rms_norm(K.mingru(h, w, "m.")[0], w["n1b"], eps)
    if with_ffn:
        h = K.rms_norm(want, w["n2"], eps)
        want = want + K.rms_norm(K.polynorm_ff(h, w, "f.", eps), w["n2b"], eps)
    close(x.double().cpu().numpy(), want, dtype)


@pytest.mark.parametrize("d", [40, 512, 1000, 4096, 5000, 8200])
def test_rms_norm_add_kernel_over_widths(d):
    """Narrow rows, rows that stay in registers (one to eight 16-byte loads a thread) and rows too wide for that."""
    from hk_b200.csrc import ops
    y = torch.randn(5, d, device="cuda") * 3.0
    w = 1.0 + 0.2 * torch.randn(d, device="cuda")
    res = torch.randn(5, d, device="cuda")
    want = res.double() + y.double() / torch.sqrt((y.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    ops.rms_norm_add(y, w, 1e-5, res)
    close(res.double().cpu().numpy(), want.cpu().numpy(), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("F", [36, 512, 3000, 12288, 16384, 20000])
def test_polynorm_kernel_over_widths(dtype, F):
    from hk_b200.csrc import ops
    z = torch.randn(3, F, device="cuda") * 1.5
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1], device="cuda")
    out = torch.empty(3, F, dtype=dtype, device="cuda")
    ops.polynorm(z, coef, 1e-5, out)
    zd = z.double().cpu().numpy()
    want = 0.7 * K.unit_rms(zd, 1e-5) - 0.4 * K.unit_rms(zd ** 2, 1e-5) + 0.25 * K.unit_rms(zd ** 3, 1e-5) + 0.1
    close(out.double().cpu().numpy(), want, dtype)


@pytest.mark.parametrize("d,E,top", [(4096, 8, 2), (1000, 20, 3), (72, 5, 5)])
def test_router_over_widths(d, E, top):
    from hk_b200.csrc import ops
    x = torch.randn(9, d, device="cuda").to(torch.bfloat16)
    w = torch.randn(E, d, device="cuda") * 0.1
    ids = torch.empty(9, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(9, top, device="cuda")
    ops.route_topk(x, w, ids, wts)
    z = x.double() @ w.double().T
    best = torch.topk(z, top, dim=1)
    assert torch.equal(ids.long().cpu(), best.indices.cpu())
    np.testing.assert_allclose(wts.double().cpu().numpy(), torch.softmax(best.values, dim=1).cpu().numpy(), rtol=1e-4, atol=1e-6)
