"""What needs no GPU of the Kedanex decoder: its configuration, the model description built from it, and the plain
implementation's own consistency (a recurrence continued from a carried state equals the whole)."""
import copy

import numpy as np
import pytest

import kedanex_models as M
import plain_kedanex as K


def test_config_reads_its_own_keys_and_round_trips():
    from hk_b200.config import ConfigError, KedanexConfig, config_from_dict
    for which, raw in M.CONFIGS.items():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, KedanexConfig) and cfg.width == raw["width"] and cfg.vocab == raw["vocab"]
        assert cfg.norm_eps == raw["norm"]["eps"] and len(cfg.layers) == len(raw["layers"])
        assert config_from_dict(cfg.to_dict()) == cfg
    cfg = config_from_dict(M.CONFIGS["Y"])
    att = cfg.layers[1].mixer
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.window, att.rot_dims, att.rot_base, att.scale) == (2, 2, 32, 24, 300, 32, 10000.0, 0.2)
    assert cfg.layers[3].weights_of == 2 and cfg.layers[2].mlp is None and cfg.layers[1].mlp.top == 2
    raw = copy.deepcopy(M.CONFIGS["Y"])
    del raw["layers"][1]["mixer"]["mask"], raw["layers"][1]["mixer"]["rot"], raw["layers"][1]["mixer"]["vdim"]
    free = config_from_dict(raw).layers[1].mixer
    assert (free.window, free.rot_dims, free.vdim) == (0, 0, 32) and config_from_dict(config_from_dict(raw).to_dict()).layers[1].mixer == free
    for breaker, text in [
        (lambda r: r["layers"][1]["mixer"].pop("scale"), "scale"),
        (lambda r: r["layers"][1].update(type="conv"), "type"),
        (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), "top"),
        (lambda r: r["layers"][3].update(weights_of=3), "weights_of"),
        (lambda r: r["layers"][1]["mixer"].update(vdim=40), "vdim"),
        (lambda r: r.pop("norm"), "norm"),
    ]:
        raw = copy.deepcopy(M.CONFIGS["Y"])
        breaker(raw)
        with pytest.raises(ConfigError, match=text):
            config_from_dict(raw)


def test_model_description_names_the_tensors_and_shares_layers():
    from hk_b200.config import config_from_dict, resolve_architecture
    from hk_b200.parts import KVCacheSpec, StateSpec
    cfg = config_from_dict(M.CONFIGS["Z"])
    _, build = resolve_architecture("Kedanex")
    model = build(cfg, 64)
    specs = model.param_specs()
    assert not any(n.startswith("l0.") for n in specs)          # layer 0 runs with layer 2's tensors
    assert specs["l2.mix.w1"].shape == (5, 128) and specs["l2.mix.w2"].shape == (64, 5) and specs["l2.mix.a.b"].shape == (64,)
    assert specs["l1.mix.q"].shape == (192, 128) and specs["l1.mix.k"].shape == (64, 128) and "l1.mix.v" not in specs
    assert specs["l1.mlp.act"].shape == (4,) and specs["l3.mlp.e1.down"].shape == (128, 24) and specs["l3.mlp.router"].shape == (2, 128)
    assert [c.layer for c in model.schedule] == [1, 0, 1, 2]    # blocks are numbered in the order of their tensors
    caches = model.cache_specs()
    assert caches[0] == [StateSpec((2, 32, 32))] and caches[2] == caches[0] and caches[1] == [KVCacheSpec(1, 64, 70)]
    # a width that only the file knows: the decay's low-rank size is absent from a file's configuration
    raw = copy.deepcopy(M.CONFIGS["Z"])
    del raw["layers"][2]["mixer"]["decay_rank"], raw["layers"][0]["mixer"]["decay_rank"]
    assert build(config_from_dict(raw), 64).param_specs()["l2.mix.w1"].shape == (-1, 128)


def test_loader_takes_the_low_rank_width_from_the_file(tmp_path):
    import torch
    from hk_b200.parts import Precision
    from hk_b200.parts.base import MATRIX, ParamSpec
    from hk_b200.weights.loader import WeightError, load_tensors
    from hk_b200.weights.safetensors_io import save_file
    save_file({"a": torch.zeros(7, 4), "b": torch.zeros(3, 7)}, str(tmp_path / "model.safetensors"))
    prec = Precision(torch.float32, torch.device("cpu"))
    got = load_tensors(str(tmp_path), {"a": ParamSpec((-1, 4), MATRIX), "b": ParamSpec((3, -1), MATRIX)}, prec)
    assert got["a"].shape == (7, 4) and got["b"].shape == (3, 7)
    with pytest.raises(WeightError):
        load_tensors(str(tmp_path), {"a": ParamSpec((-1, 5), MATRIX), "b": ParamSpec((3, -1), MATRIX)}, prec)


def random_weights(specs, rng, std=0.3):
    return {n: (1.0 if s.init == "one_plus_normal" else 0.0) + std * rng.standard_normal(s.shape) for n, s in specs.items()}


def test_plain_recurrences_continue_from_a_carried_state():
    from hk_b200.parts import GeneralDeltaRule, MinGRU
    rng = np.random.default_rng(0)
    h = rng.standard_normal((23, 12))
    w = random_weights(GeneralDeltaRule(12, 2, 4, "m.", 1e-5, decay_rank=3).param_specs(), rng)
    whole, s_whole = K.general_delta(h, w, "m.", 2, 4, 1e-5)
    first, s = K.general_delta(h[:9], w, "m.", 2, 4, 1e-5)
    second, s2 = K.general_delta(h[9:], w, "m.", 2, 4, 1e-5, state=s)
    np.testing.assert_allclose(np.concatenate([first, second]), whole, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(s2, s_whole, rtol=1e-12, atol=1e-12)
    w = random_weights(MinGRU(12, 5, "m.").param_specs(), rng)
    whole, s_whole = K.mingru(h, w, "m.")
    first, s = K.mingru(h[:9], w, "m.")
    second, s2 = K.mingru(h[9:], w, "m.", state=s)
    np.testing.assert_allclose(np.concatenate([first, second]), whole, rtol=1e-12, atol=1e-12)


def test_plain_delta_rule_is_the_written_recurrence():
    """One step by hand: S1 = k v^T (from zero), S2 = diag(d) S1 - (a u)(u^T S1) + k2 v2^T, o = S^T r."""
    rng = np.random.default_rng(1)
    from hk_b200.parts import GeneralDeltaRule
    w = random_weights(GeneralDeltaRule(6, 1, 3, "m.", 1e-5, decay_rank=2).param_specs(), rng)
    h = rng.standard_normal((2, 6))
    r, k, v = h @ w["m.r"].T, h @ w["m.k"].T, h @ w["m.v"].T
    d = np.exp(-np.exp(-0.5) / (1 + np.exp(-(np.tanh(h @ w["m.w1"].T) @ w["m.w2"].T + w["m.w0"]))))
    a = 1 / (1 + np.exp(-(h @ w["m.a"].T + w["m.a.b"])))
    u = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    S1 = np.outer(k[0], v[0])
    S2 = d[1][:, None] * S1 - np.outer(a[1] * u[1], u[1] @ S1) + np.outer(k[1], v[1])
    o = np.stack([S1.T @ r[0], S2.T @ r[1]])
    o = o / np.sqrt((o * o).mean(-1, keepdims=True) + 1e-5) * w["m.norm"] / (1 + np.exp(-(h @ w["m.g"].T)))
    np.testing.assert_allclose(K.general_delta(h, w, "m.", 1, 3, 1e-5)[0], o @ w["m.o"].T, rtol=1e-12, atol=1e-12)


def test_plain_attention_window_and_sink():
    m = dict(heads=1, kv_heads=1, dim=2, vdim=2, mask={"size": 2}, scale=1.0)
    w = {"m.q": np.eye(2), "m.k": np.eye(2), "m.o": np.eye(2)}
    h = np.array([[3.0, 0.0], [0.0, 5.0], [0.0, 1.0]])
    out = K.window_sink_attention(h, w, "m.", m, 0.0)
    # position 2 sees positions 1 and 2 only; both unit keys are (0, sqrt 2), scores 2; the values are the raw keys
    p = np.exp(2.0) / (1 + 2 * np.exp(2.0))
    np.testing.assert_allclose(out[2], p * h[1] + p * h[2], rtol=1e-12)
    np.testing.assert_allclose(out[0], np.exp(2.0) / (1 + np.exp(2.0)) * h[0], rtol=1e-12)
