"""Tiny Padodra configurations for the tests: both mixers in several orders, layers with and without a feed-forward,
and sizes chosen so that nothing that could be confused is equal (heads and key/value heads, key and value size,
rotated and whole head size, plain and rotated query part, latent size and head sizes) or happens to be 1 by accident."""
from __future__ import annotations

import os

import numpy as np
import torch

import helpers


def attention(heads, kv_heads, dim, vdim, scale, block=None, cap=None, rot=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if block:
        m["mask"] = {"size": block}
    if cap:
        m["softcap"] = cap
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, rank, scale, rot=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if rot:
        m["rot"] = rot
    return {"type": "latent_attention", "mixer": m}


def banded(base, dims, factor=None, low=1.0, high=4.0, original=64):
    r = {"base": base, "dims": dims}
    if factor:
        r["scaling"] = {"factor": factor, "high": high, "low": low, "original": original}
    return r


def ramped(base, dims, factor=None, fast=32.0, slow=1.0, original=64):
    r = {"base": base, "dims": dims}
    if factor:
        r["scaling"] = {"factor": factor, "fast": fast, "original": original, "slow": slow}
    return r


def dense(ff):
    return {"kind": "dense", "ff": ff}


def config(width, vocab, eps, emb_scale, logit_scale, layers, std):
    return {"architecture": "Padodra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": emb_scale},
            "logit_scale": logit_scale, "layers": layers, "initializer_range": std}


CONFIGS = {
    # blocks of 11 positions (no multiple of a page), values wider than keys, part of the head turned, a latent layer whose
    # rotated part is wider than its plain part, a layer without a feed-forward, a latent layer first
    "P": config(48, 131, 1e-6, 3.0, 0.7, [
        dict(latent(3, 8, 12, 10, 20, 0.21, ramped(700.0, 12, 3.0, fast=8.0, slow=0.5, original=16)), mlp=dense(40)),
        dict(attention(4, 2, 16, 24, 0.3, block=11, cap=5.0, rot=banded(900.0, 8, 2.5, original=24)), mlp=None),
        dict(attention(4, 2, 16, 24, 0.3, block=11, cap=5.0, rot=banded(900.0, 8, 2.5, original=24)), mlp=dense(56)),
        dict(latent(2, 16, 4, 6, 36, 0.4, ramped(5000.0, 4)), mlp=dense(24)),
    ], 0.12),
    # one key/value head, values narrower than keys, no cap on the scores, a block mask no request reaches, no scaling of
    # the frequencies, scales of 1 on embedding and logits, sizes that are no multiple of 4
    "Q": config(62, 200, 1e-5, 1.0, 1.0, [
        dict(attention(3, 1, 18, 10, 0.25, block=400, rot=banded(10000.0, 18)), mlp=dense(50)),
        dict(latent(5, 6, 6, 14, 22, 0.35, ramped(300.0, 6, 5.0, original=32)), mlp=None),
        dict(attention(2, 2, 30, 34, 0.15, cap=30.0), mlp=dense(70)),
    ], 0.1),
    # head size 64 with three query heads per key head and a latent row of 128 (the shapes the tensor-core kernels take),
    # blocks of 70 positions, multiples of 16 everywhere
    "R": config(128, 300, 1e-5, 8.0, 0.25, [
        dict(attention(6, 2, 64, 64, 0.125, block=70, cap=12.0, rot=banded(20000.0, 64, 4.0, original=128)), mlp=dense(160)),
        dict(latent(4, 32, 32, 32, 96, 0.11, ramped(100000.0, 32, 6.0, original=96)), mlp=dense(96)),
        dict(latent(4, 32, 32, 32, 96, 0.11, ramped(100000.0, 32, 6.0, original=96)), mlp=dense(96)),
        dict(attention(6, 2, 64, 64, 0.125, block=70, cap=12.0, rot=banded(20000.0, 64, 4.0, original=128)), mlp=dense(160)),
    ], 0.08),
    # a latent row of 160 numbers (wider than a flash head), heads of 128 with four query heads per key head
    "S": config(96, 180, 1e-6, 4.0, 0.5, [
        dict(latent(5, 24, 16, 16, 144, 0.09, ramped(40000.0, 16, 3.0, original=48)), mlp=dense(112)),
        dict(attention(4, 1, 128, 128, 0.09, block=48, cap=25.0, rot=banded(30000.0, 128, 6.0, original=96)), mlp=dense(80)),
        dict(latent(5, 24, 16, 16, 144, 0.09, ramped(40000.0, 16, 3.0, original=48)), mlp=None),
    ], 0.08),
}
SEEDS = {"P": 31, "Q": 32, "R": 33, "S": 34}


def make_model_dir(tmpdir, which: str, dtype=torch.float32) -> str:
    from hk_b200.config import config_from_dict
    from hk_b200.weights import write_random_model
    raw = CONFIGS[which]
    d = os.path.join(str(tmpdir), f"padodra_{which}_{str(dtype).split('.')[-1]}")
    write_random_model(d, config_from_dict(raw), SEEDS[which], std=raw["initializer_range"], norm_std=0.1, dtype=dtype)
    return d


def prompts(which: str, rng: np.random.Generator, lengths):
    return [rng.integers(0, CONFIGS[which]["vocab"], n).tolist() for n in lengths]


load_plain = helpers.load_plain
