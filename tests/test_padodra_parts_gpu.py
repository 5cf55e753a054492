"""The mechanisms of the Padodra decoder one by one: each part alone against its function of the plain implementation
(`plain_padodra`), whole, cut into portions down to two tokens, token by token, in batches of unequal requests, and after
a slot and its pages were freed and taken again.  Where random weights would hide a fault (a key far back, the edge of
a block of the mask, the sink), the weights or inputs are made so that it shows."""
import numpy as np
import pytest
import torch

import padodra_models as M
import plain_padodra as K
from test_kedanex_parts_gpu import MixerHarness, close, schedules
from test_parts_gpu import DTYPES, IDS, bind_random

pytestmark = pytest.mark.gpu
EPS = 1e-5
K_sigmoid = K.sigmoid


def attention_part(d, H, G, dk, dv, scale, block=None, cap=None, rot=None, positions=1024):
    from hk_b200.parts import GQAAttention, RopeScaling, RotaryEmbedding
    entry = M.attention(H, G, dk, dv, scale, block, cap, rot)["mixer"]
    rope = None
    if rot:
        s = rot.get("scaling")
        scaling = RopeScaling("llama3", factor=s["factor"], orig_ctx=s["original"], low_freq_factor=s["low"],
                              high_freq_factor=s["high"]) if s else None
        rope = RotaryEmbedding(rot["base"], rot["dims"], positions, pairing="adjacent", scaling=scaling)
    part = GQAAttention(d, H, G, dk, "m.", qk_norm_eps=EPS, position=rope, scale=scale, v_head_dim=dv, sink=True, sink_weights=True,
                        softcap=cap, chunk=block, gate=True,
                        names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink", "gate": "g"})
    return part, entry


def latent_part(d, H, dn, dr, dv, r, scale, rot=None, positions=1024):
    from hk_b200.parts import LatentAttention, RopeScaling, RotaryEmbedding
    entry = M.latent(H, dn, dr, dv, r, scale, rot)["mixer"]
    rope = None
    if rot:
        s = rot.get("scaling")
        scaling = RopeScaling("yarn", factor=s["factor"], orig_ctx=s["original"], beta_fast=s["fast"], beta_slow=s["slow"]) if s else None
        rope = RotaryEmbedding(rot["base"], rot["dims"], positions, pairing="half", scaling=scaling)
    return LatentAttention(d, H, dn, dr, dv, r, "m.", norm_eps=EPS, scale=scale, position=rope, gate=True), entry


def under_every_cut(part, entry, plain, dtype, d, std=0.3, page_tokens=4, lengths=None):
    prec, w = bind_random(part, dtype, std=std)
    lengths = lengths or {"a": 37, "b": 9, "c": 64}
    inputs = {r: torch.randn(n, d, device="cuda").to(dtype) for r, n in lengths.items()}
    want = {r: plain(x.double().cpu().numpy(), w, "m.", entry, EPS) for r, x in inputs.items()}
    hs = MixerHarness(part, prec, dtype, inputs, page_tokens=page_tokens)
    first = None
    for name, steps in schedules(lengths).items():
        got, _ = hs.run(steps)          # the slots and pages of the run before are taken again, with their old contents
        for r in lengths:
            close(got[r], want[r], dtype, f"{name} {r}")
        if first is None:
            first = got
        elif dtype == torch.float32:
            for r in lengths:
                np.testing.assert_allclose(got[r], first[r], rtol=2e-4, atol=2e-5)
    return w


# ------------------------------------------------------------------------------------ grouped-query attention


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,G,dk,dv,scale,block,cap,rot", [
    (40, 4, 2, 16, 16, 0.3, 7, 4.0, M.banded(900.0, 8, 2.5, original=24)),       # blocks shorter than two pages
    (24, 3, 1, 12, 20, 0.4, 16, None, M.banded(10000.0, 12)),                    # values wider than keys, no cap
    (48, 2, 2, 34, 10, 0.2, None, 9.0, None),                                    # no mask, no rotation, sizes no multiple of 4
    (64, 6, 2, 64, 64, 0.125, 23, 15.0, M.banded(60000.0, 64, 8.0, low=0.5, high=3.0, original=48)),
    (32, 1, 1, 136, 72, 0.1, 5, 2.0, M.banded(300.0, 30, 4.0, original=16)),     # one wide head
    (40, 5, 5, 8, 8, 0.5, 1000, 50.0, M.banded(100.0, 8)),                       # a block no request reaches
])
def test_grouped_attention_under_every_cut(dtype, d, H, G, dk, dv, scale, block, cap, rot):
    part, entry = attention_part(d, H, G, dk, dv, scale, block, cap, rot)
    under_every_cut(part, entry, K.grouped_attention, dtype, d)


def tie_queries_to_keys(part, w, H, G, dk):
    """W_q of every head becomes W_k of its group and both norms share a weight: a token whose input is a multiple of an
    earlier token's scores scale * dk against it (the norms take the factor out; before any rotation), far above every
    other key, while its own value is that multiple of the earlier token's."""
    with torch.no_grad():
        for h in range(H):
            g = h // (H // G)
            part.w_qkv[h * dk:(h + 1) * dk] = part.w_qkv[(H + g) * dk:(H + g + 1) * dk]
        part.q_norm.copy_(part.k_norm)
    w["m.q"] = np.concatenate([w["m.k"][(h // (H // G)) * dk:(h // (H // G) + 1) * dk] for h in range(H)])
    w["m.q.norm"] = w["m.k.norm"]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_attention_sees_the_first_key_of_its_block_and_not_the_last_of_the_block_before(dtype):
    """A token repeats the input of the key just inside, or just outside, the edge of its block: in a prompt, and
    decoded alone, with the edge in the middle of a page."""
    d, H, G, dk, block, T = 32, 4, 2, 16, 20, 75
    part, entry = attention_part(d, H, G, dk, dk, 1.0, block=block)
    prec, w = bind_random(part, dtype, std=0.3)
    tie_queries_to_keys(part, w, H, G, dk)
    for t in (20, 39, 47, 59, 60, 74):                   # first and last positions of blocks, and inside
        start = (t // block) * block
        for j, inside in ((start, True), (start - 1, False)):
            if j < 0 or j == t:
                continue
            x = torch.randn(T, d, device="cuda")
            x[j] *= 4.0
            x[t] = x[j] / 4.0
            x = x.to(dtype)
            xn = x.double().cpu().numpy()
            want = K.grouped_attention(xn, w, "m.", entry, EPS)
            other = xn.copy()
            other[j] = np.random.default_rng(j).standard_normal(d)
            moved = np.abs(K.grouped_attention(other, w, "m.", entry, EPS)[t] - want[t]).max()
            if inside:
                assert moved > 0.2 * np.abs(want[t]).max(), (t, j)          # the key matters
            else:
                assert moved == 0.0, (t, j)                                  # nothing of it reaches the token
            hs = MixerHarness(part, prec, dtype, {"a": x}, page_tokens=8, pages=16)
            for steps in ([[("a", T)]], [[("a", t)], [("a", 1)], [("a", T - t - 1)]], [[("a", j + 1)], [("a", t - j - 1)], [("a", 1)], [("a", T - t - 1)]]):
                steps = [st for st in steps if st[0][1] > 0]
                got, _ = hs.run(steps)
                close(got["a"][max(0, t - 2):t + 2], want[max(0, t - 2):t + 2], dtype, f"token {t}, key {j}")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_attention_reads_a_key_from_far_back_and_across_page_borders(dtype):
    """One key among hundreds, on the first or last place of a page, is the one that the last token repeats."""
    d, H, G, dk, T = 32, 2, 2, 16, 400
    part, entry = attention_part(d, H, G, dk, dk, 1.0, cap=30.0)
    prec, w = bind_random(part, dtype, std=0.3)
    tie_queries_to_keys(part, w, H, G, dk)
    for j in (0, 15, 16, 17, 250):
        x = torch.randn(T, d, device="cuda")
        x[j] *= 4.0
        x[T - 1] = x[j] / 4.0
        x = x.to(dtype)
        xn = x.double().cpu().numpy()
        want = K.grouped_attention(xn, w, "m.", entry, EPS)
        without = K.grouped_attention(np.delete(xn, j, axis=0), w, "m.", entry, EPS)
        assert np.abs(want[-1] - without[-1]).max() > 0.3 * np.abs(want[-1]).max()
        hs = MixerHarness(part, prec, dtype, {"a": x}, page_tokens=16, pages=32)
        for steps in ([[("a", T)]], [[("a", T - 3)]] + [[("a", 1)]] * 3):
            got, _ = hs.run(steps)
            close(got["a"][-4:], want[-4:], dtype, f"key at {j}")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_the_sink_takes_its_share_per_head(dtype):
    """A large sink score on one head empties that head's output, a very negative one leaves a plain softmax; the first
    token of a sequence, which sees only itself, shows it most plainly."""
    d, H, G, dk, dv = 24, 4, 2, 8, 12
    part, entry = attention_part(d, H, G, dk, dv, 0.5, block=9)
    prec, w = bind_random(part, dtype, std=0.3)
    sinks = np.array([6.0, -20.0, 0.0, 2.5])
    with torch.no_grad():
        part.sinks.copy_(torch.from_numpy(sinks))
    w["m.sink"] = sinks
    x = torch.randn(30, d, device="cuda").to(dtype)
    xn = x.double().cpu().numpy()
    want = K.grouped_attention(xn, w, "m.", entry, EPS)
    w0 = dict(w)
    w0["m.sink"] = np.full(4, -50.0)
    assert np.abs(K.grouped_attention(xn, w0, "m.", entry, EPS) - want).max() > 0.3 * np.abs(want).max()
    hs = MixerHarness(part, prec, dtype, {"a": x}, page_tokens=4)
    for steps in ([[("a", 30)]], [[("a", 1)]] * 30, [[("a", 2)]] * 15):
        got, _ = hs.run(steps)
        close(got["a"], want, dtype)


# ------------------------------------------------------------------------------------ latent attention


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,H,dn,dr,dv,r,scale,rot", [
    (40, 3, 8, 12, 10, 20, 0.3, M.ramped(700.0, 12, 3.0, fast=8.0, slow=0.5, original=16)),    # rotated part wider than the plain one
    (24, 2, 16, 4, 6, 36, 0.4, M.ramped(5000.0, 4)),                                           # latent wider than the width
    (64, 4, 32, 32, 32, 96, 0.15, M.ramped(100000.0, 32, 6.0, original=96)),                   # a cache row of 128
    (48, 5, 6, 6, 14, 22, 0.35, M.ramped(300.0, 6, 5.0, original=32)),                         # nothing a multiple of 4
    (32, 1, 24, 8, 40, 300, 0.1, M.ramped(10000.0, 8, 2.0, original=8)),                       # one head, a cache row above 256
    (32, 2, 10, 16, 10, 12, 0.3, None),                                                        # no rotation at all
    (40, 3, 8, 16, 10, 64, 0.2, M.ramped(2000.0, 16, 2.0, original=24)),                       # a cache row of 80: the flash kernels' sizes
    (32, 2, 16, 16, 8, 32, 0.25, M.ramped(2000.0, 8)),                                         # a cache row of 48, part of the rotated dims turned
    # cache rows wider than a flash head (multiples of 16): the kernel with the query tile in shared memory
    (64, 4, 16, 16, 24, 176, 0.1, M.ramped(10000.0, 16, 4.0, original=32)),                   # values over 2 x 128 columns
    (48, 3, 32, 64, 16, 512, 0.05, M.ramped(10000.0, 64, 8.0, original=64)),                  # the widest row: 576, values 512
    (32, 20, 8, 16, 8, 144, 0.15, M.ramped(500.0, 16)),                                        # 20 heads: three tokens a tile
    (32, 64, 8, 16, 8, 128, 0.15, M.ramped(500.0, 16)),                                        # 64 heads: one token a tile
])
def test_latent_attention_under_every_cut(dtype, d, H, dn, dr, dv, r, scale, rot):
    part, entry = latent_part(d, H, dn, dr, dv, r, scale, rot)
    under_every_cut(part, entry, K.latent_attention, dtype, d)
    assert part.cache_spec().v_dim == 0 and part.cache_spec().k_dim == r + dr and part.cache_spec().n_kv_heads == 1
    if dtype == torch.bfloat16 and (r + dr) % 16 == 0 and r % 16 == 0:       # a tensor-core kernel took it, not the generic one
        assert part.step_tables_key() is not None and part._wide == (r + dr > 128)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_latent_attention_reads_keys_from_far_back(dtype):
    """Scores so sharp that nearly all of a token's weight lies on one key, wherever among 300 it is: a key that is lost,
    misplaced in its page or read from another request's page changes the token's output."""
    d, H, dn, dr, dv, r, T = 32, 2, 16, 8, 12, 24, 300
    part, entry = latent_part(d, H, dn, dr, dv, r, 1.0, M.ramped(10000.0, 8, 4.0, original=64))
    prec, w = bind_random(part, dtype, std=0.3)
    inputs = {"a": torch.randn(T, d, device="cuda").to(dtype), "b": torch.randn(40, d, device="cuda").to(dtype)}
    want = {k: K.latent_attention(v.double().cpu().numpy(), w, "m.", entry, EPS) for k, v in inputs.items()}
    xn = inputs["a"].double().cpu().numpy()
    moved = 0
    for j in (0, 15, 16, 130):
        without = K.latent_attention(np.delete(xn, j, axis=0), w, "m.", entry, EPS)
        moved += int((np.abs(without[j:] - want["a"][j + 1:]).max(axis=1) > 0.2 * np.abs(want["a"]).max()).sum())
    assert moved >= 4                                    # some later token hangs on each of these keys
    # scores this sharp magnify the rounding of queries and cache rows: in bfloat16 the limit is four times what rounding
    # alone does to the plain result (a lost key moves a token by 0.2 and more of the largest value, see above)
    limit = {k: 0.0 for k in inputs}
    if dtype == torch.bfloat16:
        K.round_inputs = lambda v: torch.from_numpy(np.ascontiguousarray(v)).to(torch.bfloat16).double().numpy()
        try:
            for k, v in inputs.items():
                rounded = K.latent_attention(v.double().cpu().numpy(), w, "m.", entry, EPS)
                limit[k] = 4 * float(np.abs(rounded - want[k]).max())
        finally:
            K.round_inputs = None
        assert max(limit.values()) < 0.2 * np.abs(want["a"]).max()
    hs = MixerHarness(part, prec, dtype, inputs, page_tokens=16, pages=32)
    for steps in ([[("a", T)], [("b", 40)]], [[("a", 100), ("b", 7)], [("a", 1), ("b", 1)], [("a", 180), ("b", 2)], [("a", 19), ("b", 30)]],
                  [[("a", T - 5)]] + [[("a", 1)]] * 5 + [[("b", 40)]]):
        got, _ = hs.run(steps)
        for k in inputs:
            if np.abs(got[k] - want[k]).max() > limit[k]:
                close(got[k], want[k], dtype, k)


# ------------------------------------------------------------------------------------ feed-forward, block, embedding, head


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d,F,n", [(40, 72, 19), (24, 9, 5), (128, 640, 19), (128, 640, 300), (256, 1024, 3), (64, 96, 1)])
def test_gelu_gated_feed_forward(dtype, d, F, n):
    from hk_b200.parts import SwiGLUFeedForward
    part = SwiGLUFeedForward(d, F, "f.", act="gelu_tanh", names={"gate": "gate", "up": "up", "down": "down"})
    prec, w = bind_random(part, dtype, std=0.3)
    x = (2.0 * torch.randn(n, d, device="cuda")).to(dtype)
    y = torch.full((n, d), float("nan"), device="cuda")
    part.forward(x, y, None, accumulate=False)
    want = K.feed_forward(x.double().cpu().numpy(), w, "f.")
    close(y.double().cpu().numpy(), want, dtype)
    silu = SwiGLUFeedForward(d, F, "f.", names={"gate": "gate", "up": "up", "down": "down"})
    silu.bind({k: torch.from_numpy(v).cuda().to(dtype) for k, v in w.items()}, prec)
    z = torch.zeros((n, d), device="cuda")
    silu.forward(x, z, None, accumulate=False)
    assert np.abs(z.double().cpu().numpy() - want).max() > 0.005 * np.abs(want).max()       # the activation is not silu


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("d", [48, 512, 1000])
def test_post_norm_block_embedding_scale_and_logit_scale(dtype, d):
    """A model of one layer whose sublayers read the residual stream itself, with factors on the embedding and the
    logits that are no powers of two."""
    from hk_b200.config import config_from_dict, resolve_architecture
    from hk_b200.cache.device import PagedCache
    from test_parts_gpu import make_ctx
    raw = M.config(d, 77, 1e-5, 2.7, 0.37, [dict(M.attention(2, 1, 8, 12, 0.3, block=6, cap=7.0, rot=M.banded(500.0, 4)), mlp=M.dense(40)),
                                            dict(M.latent(2, 4, 4, 6, 10, 0.3, M.ramped(500.0, 4)), mlp=None)], 0.1)
    model = resolve_architecture("Padodra")[1](config_from_dict(raw), 64)
    prec, w = bind_random(model, dtype, std=0.2)
    ids = np.random.default_rng(3).integers(0, 77, 21)
    want = K.forward(raw, w, ids)
    cache = PagedCache(model.cache_specs(), prec, 4, 32, 2, 64)
    slot = cache.open()
    got = []
    for lo, hi in ((0, 9), (9, 11), (11, 12), (12, 21)):
        ctx = make_ctx(prec, [(slot, lo, hi - lo)], cache, page_tokens=4, part=model)
        ctx.token_ids.copy_(torch.from_numpy(ids[lo:hi].astype(np.int32)))
        x = model.forward(ctx, cache.layers)
        rows = torch.arange(hi - lo, dtype=torch.int32, device="cuda")
        got.append(model.head.forward(x, rows, hi - lo, ctx).double().cpu().numpy())
    close(np.concatenate(got), want, dtype)
    plain = dict(raw, embedding={"scale": 1.0})
    assert np.abs(K.forward(plain, w, ids) - want).max() > 0.05 * np.abs(want).max()


# ------------------------------------------------------------------------------------ the kernels underneath


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n,H,K,N", [(1, 3, 16, 24), (70, 2, 128, 512), (9, 5, 40, 12), (130, 4, 512, 128), (64, 1, 8, 8), (33, 6, 6, 10)])
def test_a_product_per_head_over_slices_of_wider_rows(dtype, n, H, K, N):
    """out[t, h] = a[t, h] W_h^T where a and out are the first columns of wider heads, in the type's tensor-core kernel
    (bfloat16, sizes it takes) and in the plain one."""
    from hk_b200.csrc import ops
    g = torch.Generator().manual_seed(n * 7 + K)
    a_wide = torch.randn(n, H, K + 8, generator=g).to(dtype).cuda()
    w = (torch.randn(H, N, K, generator=g) * 0.2).to(dtype).cuda()
    want = np.einsum("thk,hnk->thn", a_wide[:, :, :K].double().cpu().numpy(), w.double().cpu().numpy())
    for out_dtype in ({dtype, torch.float32}):
        out_wide = torch.full((n, H, N + 6), 7.0, dtype=out_dtype, device="cuda")
        ops.gemm_heads(a_wide[:, :, :K], w, out_wide[:, :, :N], H)
        close(out_wide[:, :, :N].double().cpu().numpy(), want, dtype)
        assert (out_wide[:, :, N:] == 7.0).all()                   # nothing beside the slice was touched
        with ops.force(gemm="generic"):
            again = torch.zeros((n, H, N), dtype=out_dtype, device="cuda")
            ops.gemm_heads(a_wide[:, :, :K], w, again, H)
        close(again.double().cpu().numpy(), want, dtype)
        # with a gate in the epilogue: logits as a column slice of wider float32 rows
        logits = torch.randn(n, H * N + 5, generator=g).cuda()
        gated = want * K_sigmoid(logits[:, 5:].double().cpu().numpy()).reshape(n, H, N)
        for kernel in (None, "generic"):
            got = torch.zeros((n, H, N), dtype=out_dtype, device="cuda")
            with ops.force(gemm=kernel):
                ops.gemm_heads(a_wide[:, :, :K], w, got, H, gate=logits[:, 5:])
            close(got.double().cpu().numpy(), gated, dtype)


@pytest.mark.parametrize("d", [48, 512, 1000, 4096])
def test_rows_written_with_their_narrowed_copy(d):
    """The embedding (with its factor) and the norm + residual sum also leave the new rows rounded to bfloat16."""
    from hk_b200.csrc import ops
    table = torch.randn(50, d, device="cuda").to(torch.bfloat16)
    ids = torch.tensor([3, 49, 0, 3, 17], dtype=torch.int32, device="cuda")
    x = torch.empty(5, d, device="cuda")
    xb = torch.empty(5, d, dtype=torch.bfloat16, device="cuda")
    ops.embedding(table, ids, x, 2.7, xb)
    want = table[ids.long()].float() * 2.7
    assert torch.equal(x, want) and torch.equal(xb, want.to(torch.bfloat16))
    y, w = torch.randn(5, d, device="cuda"), torch.rand(d, device="cuda") + 0.5
    res = x.clone()
    ops.rms_norm_add(y, w, 1e-5, res, xb)
    want = x.double() + y.double() / torch.sqrt((y.double() ** 2).mean(-1, keepdim=True) + 1e-5) * w.double()
    assert torch.allclose(res.double(), want, rtol=1e-5, atol=1e-5) and torch.equal(xb, res.to(torch.bfloat16))
