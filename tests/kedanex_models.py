"""Tiny Kedanex configurations for the tests: every mixer, both feed-forwards and none, a shared layer, and
sizes chosen so that nothing that could be confused is equal (heads and key/value heads, key and value size,
rotated and whole head size, experts and top) or happens to be 1 by accident."""
from __future__ import annotations

import os

import numpy as np
import torch

import helpers


def attention(heads, kv_heads, dim, vdim, window, rot_dims, scale, base=900.0):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": window}, "scale": scale, "vdim": vdim}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": m}


def delta(heads, dim, rank):
    return {"type": "general_delta", "mixer": {"dim": dim, "heads": heads, "decay_rank": rank}}


def mingru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, eps, layers, std):
    return {"architecture": "Kedanex", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers,
            "initializer_range": std}


CONFIGS = {
    # a window shorter than a page run, one expert of three, a shared attention layer, a layer without feed-forward
    "X": config(48, 131, 1e-6, [
        dict(attention(4, 2, 16, 16, 9, 8, 0.3), mlp=moe(24, 3, 1)),
        dict(delta(2, 16, 6), mlp=dense(40)),
        dict(mingru(20), mlp=None),
        dict(attention(4, 2, 16, 16, 9, 8, 0.3), mlp=moe(24, 3, 1), weights_of=0),
        dict(delta(3, 8, 4), mlp=moe(16, 5, 3)),
    ], 0.12),
    # a window no request reaches (every key stays), values narrower than keys, one wide delta head used twice
    "Y": config(64, 200, 1e-5, [
        dict(mingru(96), mlp=dense(72)),
        dict(attention(2, 2, 32, 24, 300, 32, 0.2, base=10000.0), mlp=moe(32, 4, 2)),
        dict(delta(1, 64, 8), mlp=None),
        dict(delta(1, 64, 8), mlp=None, weights_of=2),
    ], 0.1),
    # head size 64 with three query heads per key head (the tensor-core attention's shapes), a window of 70, a shared
    # layer that comes BEFORE the layer whose tensors it uses
    "Z": config(128, 300, 1e-5, [
        dict(delta(2, 32, 5), mlp=moe(48, 4, 2), weights_of=2),
        dict(attention(3, 1, 64, 64, 70, 64, 0.125, base=20000.0), mlp=dense(160)),
        dict(delta(2, 32, 5), mlp=moe(48, 4, 2)),
        dict(mingru(40), mlp=moe(24, 2, 2)),
    ], 0.08),
}
SEEDS = {"X": 21, "Y": 22, "Z": 23}


def make_model_dir(tmpdir, which: str, dtype=torch.float32) -> str:
    from hk_b200.config import config_from_dict
    from hk_b200.weights import write_random_model
    raw = CONFIGS[which]
    d = os.path.join(str(tmpdir), f"kedanex_{which}_{str(dtype).split('.')[-1]}")
    write_random_model(d, config_from_dict(raw), SEEDS[which], std=raw["initializer_range"], norm_std=0.1, dtype=dtype)
    return d


def prompts(which: str, rng: np.random.Generator, lengths):
    return [rng.integers(0, CONFIGS[which]["vocab"], n).tolist() for n in lengths]


load_plain = helpers.load_plain
