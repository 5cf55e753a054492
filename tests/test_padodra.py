"""The Padodra decoder without a GPU: its configuration, its model description, and the plain implementation's own
consistency (the identities that the engine's form of the latent attention rests on, masks, sinks, frequencies)."""
import copy
import math

import numpy as np
import pytest

import padodra_models as M
import plain_padodra as K


def test_configuration_reads_every_key_and_writes_it_back():
    from hk_b200.config import ConfigError, PadodraConfig, config_from_dict
    for which, raw in M.CONFIGS.items():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, PadodraConfig) and config_from_dict(cfg.to_dict()) == cfg
        assert cfg.width == raw["width"] and cfg.vocab == raw["vocab"] and cfg.norm_eps == raw["norm"]["eps"]
        assert cfg.embedding_scale == raw["embedding"]["scale"] and cfg.logit_scale == raw["logit_scale"]
        for layer, e in zip(cfg.layers, raw["layers"]):
            m = e["mixer"]
            assert (layer.mixer.kind, layer.mixer.heads, layer.mixer.dim, layer.mixer.vdim) == (e["type"], m["heads"], m["dim"], m["vdim"])
            assert (layer.mlp is None) == (e["mlp"] is None)
            if e["type"] == "attention":
                assert layer.mixer.chunk == (m.get("mask") or {}).get("size", 0) and layer.mixer.softcap == m.get("softcap", 0.0)
            else:
                assert (layer.mixer.kv_rank, layer.mixer.rot_dim) == (m["kv_rank"], m["rot_dim"])
    p = M.CONFIGS["P"]
    cfg = config_from_dict(p)
    assert cfg.layers[1].mixer.rot.scaling == {"factor": 2.5, "low": 1.0, "high": 4.0, "original": 24.0}
    assert cfg.layers[3].mixer.rot.scaling == {}
    for path, value, word in ((("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mixer", "rot", "dims"), 18, "dims"), (("layers", 0, "mlp", "kind"), "moe", "kind"),
                              (("layers", 0, "mixer", "rot", "scaling", "factor"), -1, "factor")):
        bad = copy.deepcopy(p)
        at = bad
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            config_from_dict(bad)
    bad = copy.deepcopy(p)
    del bad["layers"][0]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        config_from_dict(bad)


def test_model_description_names_the_tensors_and_their_shapes():
    from hk_b200.config import config_from_dict, resolve_architecture
    from hk_b200.parts import GQAAttention, KVCacheSpec, LatentAttention, PostNormBlock
    cfg = config_from_dict(M.CONFIGS["P"])
    model = resolve_architecture("Padodra")[1](cfg, 64)
    specs = {k: v.shape for k, v in model.param_specs().items()}
    assert specs["embed"] == (131, 48) and specs["head"] == (131, 48) and specs["final.norm"] == (48,)
    assert specs["l0.mix.q"] == (3 * 20, 48) and specs["l0.mix.dkv"] == (32, 48) and specs["l0.mix.dkv.norm"] == (20,)
    assert specs["l0.mix.uk"] == (24, 20) and specs["l0.mix.uv"] == (30, 20) and specs["l0.mix.g"] == (30, 48) and specs["l0.mix.o"] == (48, 30)
    assert specs["l1.mix.q"] == (64, 48) and specs["l1.mix.k"] == (32, 48) and specs["l1.mix.v"] == (48, 48)
    assert specs["l1.mix.q.norm"] == (16,) and specs["l1.mix.sink"] == (4,) and specs["l1.mix.g"] == (96, 48) and specs["l1.mix.o"] == (48, 96)
    assert "l1.mlp.gate" not in specs and "l1.norm2" not in specs and specs["l2.mlp.gate"] == (56, 48) and specs["l2.mlp.down"] == (48, 56)
    assert all(isinstance(b, PostNormBlock) for b in model.layers)
    assert isinstance(model.layers[0].mixer, LatentAttention) and isinstance(model.layers[1].mixer, GQAAttention)
    # the latent layers cache one row per token and nothing else; the two attention layers share a page pool
    assert model.cache_specs()[0] == [KVCacheSpec(1, 32, None, 0)] and model.cache_specs()[1] == [KVCacheSpec(2, 16, None, 24)]
    assert model.layers[1].mixer.position is model.layers[2].mixer.position and model.layers[1].mixer.position.pairing == "adjacent"
    assert model.layers[0].mixer.position.pairing == "half" and model.layers[0].mixer.position.scaling.kind == "yarn"
    assert model.layers[3].mixer.position.scaling.kind == "none"


def test_rotation_tables_of_the_package_equal_the_plain_frequencies():
    from hk_b200.config import config_from_dict, resolve_architecture
    for which in M.CONFIGS:
        raw = M.CONFIGS[which]
        model = resolve_architecture("Padodra")[1](config_from_dict(raw), 64)
        for block, e in zip(model.layers, raw["layers"]):
            rot = e["mixer"].get("rot")
            if not rot:
                assert block.mixer.position is None
                continue
            f, mag = (K.banded_frequencies if e["type"] == "attention" else K.ramped_frequencies)(rot)
            assert np.allclose(block.mixer.position.inv_freq().numpy(), f, rtol=1e-6, atol=0)
            assert math.isclose(block.mixer.position.mscale(), mag, rel_tol=1e-6)
    # the numbers move: a scaled table differs from the plain one, and the ramp has all three regimes in "R"
    rot = M.CONFIGS["R"]["layers"][1]["mixer"]["rot"]
    f, mag = K.ramped_frequencies(rot)
    base = K.base_frequencies(rot)
    ratio = f / base
    assert mag > 1.0 and np.isclose(ratio[0], 1.0) and np.isclose(ratio[-1], 1.0 / 6.0) and ((ratio < 0.99) & (ratio > 0.17)).any()
    rot = M.CONFIGS["R"]["layers"][0]["mixer"]["rot"]
    ratio = K.banded_frequencies(rot)[0] / K.base_frequencies(rot)
    assert np.isclose(ratio[0], 1.0) and np.isclose(ratio[-1], 0.25) and ((ratio < 0.99) & (ratio > 0.26)).any()


def _weights(which, seed=0):
    from hk_b200.config import config_from_dict, resolve_architecture
    rng = np.random.default_rng(seed)
    specs = resolve_architecture("Padodra")[1](config_from_dict(M.CONFIGS[which]), 8).param_specs()
    return {k: (1.0 + 0.1 * rng.standard_normal(s.shape)) if s.init == "one_plus_normal" else 0.2 * rng.standard_normal(s.shape)
            for k, s in specs.items()}


def test_latent_attention_equals_its_form_over_the_cached_rows():
    """The engine never forms per-head keys and values: it carries the query into the latent space and applies the
    values' up-projection to the attention's result.  Both forms, plainly."""
    raw = M.CONFIGS["P"]
    w = _weights("P")
    m, p, eps = raw["layers"][0]["mixer"], "l0.mix.", raw["norm"]["eps"]
    T = 9
    x = np.random.default_rng(1).standard_normal((T, raw["width"]))
    want = K.latent_attention(x, w, p, m, eps)
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    q = (x @ w[p + "q"].T).reshape(T, H, dn + dr)
    down = x @ w[p + "dkv"].T
    f, mag = K.ramped_frequencies(m["rot"])
    row = np.concatenate([K.rms(down[:, :r], eps) * w[p + "dkv.norm"],
                          K.turn(down[:, None, r:], pos, f, mag, m["rot"]["dims"], "halves")[:, 0]], axis=1)     # what is cached
    q_rot = K.turn(q[..., dn:], pos, f, mag, m["rot"]["dims"], "halves")
    heads = np.zeros((T, H, dv))
    for h in range(H):
        uk, uv = w[p + "uk"][h * dn:(h + 1) * dn], w[p + "uv"][h * dv:(h + 1) * dv]
        q_row = np.concatenate([q[:, h, :dn] @ uk, q_rot[:, h]], axis=1)
        pr = K.softmax_with_sink(q_row @ row.T * m["scale"], K.visible(T))
        heads[:, h] = (pr @ row[:, :r]) @ uv.T
    got = (heads.reshape(T, H * dv) * K.sigmoid(x @ w[p + "g"].T)) @ w[p + "o"].T
    assert np.allclose(got, want, rtol=1e-9, atol=1e-12)


def test_block_mask_sink_and_cap_do_what_they_say():
    assert K.visible(7, 3).astype(int).tolist() == [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0],
                                                    [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0], [0, 0, 0, 0, 0, 0, 1]]
    s = np.array([[0.5, 1.5, -0.3]])
    see = np.array([[True, True, False]])
    pr = K.softmax_with_sink(s, see, sink=0.7)
    den = math.exp(0.5) + math.exp(1.5) + math.exp(0.7)
    assert np.allclose(pr, [[math.exp(0.5) / den, math.exp(1.5) / den, 0.0]]) and pr.sum() < 1.0
    assert np.allclose(K.softmax_with_sink(s, see).sum(), 1.0)
    # a cap bounds a huge score; the whole attention moves when cap, block or sink change
    raw = M.CONFIGS["P"]
    w = _weights("P", 3)
    m, p, eps = raw["layers"][1]["mixer"], "l1.mix.", raw["norm"]["eps"]
    x = 3.0 * np.random.default_rng(2).standard_normal((30, raw["width"]))
    base = K.grouped_attention(x, w, p, m, eps)
    for change in ({"softcap": None}, {"mask": None}, {"mask": {"size": 12}}, {"rot": None}):
        assert np.abs(K.grouped_attention(x, w, p, {**m, **change}, eps) - base).max() > 1e-3, change
    w2 = dict(w)
    w2[p + "sink"] = w[p + "sink"] + 1.0
    assert np.abs(K.grouped_attention(x, w2, p, m, eps) - base).max() > 1e-3
    # rows up to the first block's end do not depend on the block size when it is larger
    assert np.allclose(K.grouped_attention(x, w, p, {**m, "mask": {"size": 12}}, eps)[:11], base[:11])


def test_layer_norms_only_what_the_sublayers_give_back():
    raw = M.CONFIGS["Q"]
    w = _weights("Q", 4)
    x = np.random.default_rng(5).standard_normal((6, raw["width"]))
    eps = raw["norm"]["eps"]
    y = K.layer(x, w, 0, raw["layers"][0], eps)
    mid = x + K.rms(K.grouped_attention(x, w, "l0.mix.", raw["layers"][0]["mixer"], eps), eps) * w["l0.norm1"]
    assert np.allclose(y, mid + K.rms(K.feed_forward(mid, w, "l0.mlp."), eps) * w["l0.norm2"])
    assert np.allclose(K.gelu_tanh(np.array([0.0, 1.0, -2.0])), [0.0, 0.8411919906082768, -0.04540230591222977])


def test_work_items_of_a_block_mask_begin_at_the_block_of_their_first_token():
    """The flash kernels' work items: with blocks of 10 positions a prompt portion's items start their keys at the block of
    their first token (the kernel masks row by row where an item crosses an edge), a decoded token's at its own block."""
    from hk_b200.csrc import attention_fast as af
    items, merge, info = af.plan_arrays([0, 1], [0, 40], [40, 1], [5, 37], 41, 0, 4, 2, 148, prefill_rows=64, chunk=10)
    recs = {(int(r[0]), int(r[1])): (int(r[4]), int(r[5])) for r in items}
    assert recs[(0, 32)] == (0, 37) and recs[(32, 8)] == (30, 45) and recs[(40, 1)] == (30, 38)
    items, merge, info = af.plan_arrays([0, 1, 2], [0, 1, 2], [1, 1, 1], [9, 10, 300], 3, 0, 4, 2, 148, fixed_splits=2, max_context=512, chunk=10)
    full = [q for q in items if q[5] > q[4]]                 # a split past the token's keys is an empty range
    lo = {int(r[3]): min(int(q[4]) for q in full if q[3] == r[3]) for r in full}
    hi = {int(r[3]): max(int(q[5]) for q in full if q[3] == r[3]) for r in full}
    assert lo == {9: 0, 10: 10, 300: 300} and hi == {9: 10, 10: 11, 300: 301}
