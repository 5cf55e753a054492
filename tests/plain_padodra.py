"""The Padodra decoder, plainly: numpy, float64, whole sequences, one function per mechanism, no code shared with the
package.  `cfg` is config.json as a dict, `w` the tensors by name as float64 arrays.

Notation: T tokens at positions 0..T-1, a linear map y = x W^T for a weight stored [out, in].
  layer          x <- x + N1(mixer(x));  x <- x + N2(ff(x))            (the sublayers read x itself)
  N(y)           y / sqrt(mean(y^2) + eps) * weight
  attention      q, k normed per head with a weight, then turned in adjacent pairs; s = scale q.k; s <- c tanh(s / c);
                 position t sees j <= t with floor(j / B) = floor(t / B); p_j = exp(s_j) / (exp(sink_h) + sum exp(s_j));
                 out = concat_h(sum p_j v_j) * sigmoid(W_g x), then W_o
  latent         c = N(first r of W_dkv x), k_rot = turn(last dr of W_dkv x) shared by the heads; head h has the key
                 [W_uk,h c | k_rot] and the value W_uv,h c; q_h = [plain | turned]; plain causal softmax; gate; W_o
  feed-forward   W_down (gelu_tanh(W_gate x) * W_up x)
`round_inputs`, when set, is applied to the inputs of every matrix product and to what a cache would hold: a coarse
model of what bfloat16 serving rounds.
"""
from __future__ import annotations

import math

import numpy as np

round_inputs = None


def _r(x):
    return x if round_inputs is None else round_inputs(x)


def linear(x, weight):
    return _r(x) @ _r(weight).T


def rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def base_frequencies(rot):
    n = rot["dims"]
    return np.array([rot["base"] ** (-2.0 * i / n) for i in range(n // 2)])


def banded_frequencies(rot):
    """Frequencies whose wavelength is long against the original context are divided by `factor`, short ones kept, the
    band between blended linearly in original / wavelength.  Returns (frequencies, magnitude of cos and sin)."""
    f = base_frequencies(rot)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    out = []
    for fi in f:
        wavelength = 2.0 * math.pi / fi
        if wavelength < s["original"] / s["high"]:
            out.append(fi)
        elif wavelength > s["original"] / s["low"]:
            out.append(fi / s["factor"])
        else:
            t = (s["original"] / wavelength - s["low"]) / (s["high"] - s["low"])
            out.append((1.0 - t) * fi / s["factor"] + t * fi)
    return np.array(out), 1.0


def ramped_frequencies(rot):
    """A ramp over the pair index between the pairs that make `fast` and `slow` turns within the original context
    blends f (below the ramp) into f / factor (above it); cos and sin grow by 0.1 ln(factor) + 1."""
    f = base_frequencies(rot)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    n = rot["dims"]

    def pair_with_turns(turns):
        return n * math.log(s["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(rot["base"]))
    lo = max(math.floor(pair_with_turns(s["fast"])), 0)
    hi = min(math.ceil(pair_with_turns(s["slow"])), n - 1)
    ramp = np.clip((np.arange(n // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / s["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(s["factor"]) + 1.0


def turn(x, positions, freqs, magnitude, dims, pairs):
    """x [T, heads, size]: the first `dims` dims are turned by angle position * freq; pairs 'adjacent' = (2i, 2i + 1),
    'halves' = (i, i + dims / 2)."""
    angle = positions[:, None].astype(np.float64) * freqs[None, :]
    c, s = np.cos(angle)[:, None, :] * magnitude, np.sin(angle)[:, None, :] * magnitude
    y = x.copy()
    if pairs == "adjacent":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        y[..., 0:dims:2], y[..., 1:dims:2] = a * c - b * s, b * c + a * s
    else:
        h = dims // 2
        a, b = x[..., :h], x[..., h:dims]
        y[..., :h], y[..., h:dims] = a * c - b * s, b * c + a * s
    return y


def visible(T, block=None):
    """[T, T] True where position t (row) sees position j (column)."""
    t, j = np.arange(T)[:, None], np.arange(T)[None, :]
    see = j <= t
    if block:
        see &= (j // block) == (t // block)
    return see


def softmax_with_sink(scores, see, sink=None):
    """Rows of `scores` over the visible columns; `sink` (a number) adds exp(sink) to the denominator."""
    s = np.where(see, scores, -np.inf)
    top = s.max(axis=-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink)
    e = np.exp(s - top)
    den = e.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink - top)
    return e / den


def grouped_attention(x, w, p, m, eps):
    T = x.shape[0]
    H, G = m["heads"], m.get("kv_heads", m["heads"])
    dk, dv = m["dim"], m.get("vdim", m["dim"])
    pos = np.arange(T)
    q = linear(x, w[p + "q"]).reshape(T, H, dk)
    k = linear(x, w[p + "k"]).reshape(T, G, dk)
    v = linear(x, w[p + "v"]).reshape(T, G, dv)
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    if m.get("rot"):
        f, mag = banded_frequencies(m["rot"])
        q = turn(q, pos, f, mag, m["rot"]["dims"], "adjacent")
        k = turn(k, pos, f, mag, m["rot"]["dims"], "adjacent")
    q, k, v = _r(q), _r(k), _r(v)
    see = visible(T, (m.get("mask") or {}).get("size"))
    cap = m.get("softcap")
    heads = np.zeros((T, H, dv))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        heads[:, h] = softmax_with_sink(s, see, w[p + "sink"][h]) @ v[:, g]
    gated = heads.reshape(T, H * dv) * sigmoid(linear(x, w[p + "g"]))
    return linear(gated, w[p + "o"])


def latent_attention(x, w, p, m, eps):
    T = x.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T)
    q = linear(x, w[p + "q"]).reshape(T, H, dn + dr)
    down = linear(x, w[p + "dkv"])
    c = _r(rms(down[:, :r], eps) * w[p + "dkv.norm"])
    shared = down[:, None, r:]
    q_plain, q_rot = q[..., :dn], q[..., dn:]
    if m.get("rot"):
        f, mag = ramped_frequencies(m["rot"])
        q_rot = turn(q_rot, pos, f, mag, m["rot"]["dims"], "halves")
        shared = turn(shared, pos, f, mag, m["rot"]["dims"], "halves")
    shared = _r(shared[:, 0])
    k_plain = (c @ _r(w[p + "uk"]).T).reshape(T, H, dn)
    v = (c @ _r(w[p + "uv"]).T).reshape(T, H, dv)
    see = visible(T)
    heads = np.zeros((T, H, dv))
    for h in range(H):
        s = (_r(q_plain[:, h]) @ k_plain[:, h].T + _r(q_rot[:, h]) @ shared.T) * m["scale"]
        heads[:, h] = softmax_with_sink(s, see) @ v[:, h]
    gated = heads.reshape(T, H * dv) * sigmoid(linear(x, w[p + "g"]))
    return linear(gated, w[p + "o"])


def feed_forward(x, w, p):
    return linear(gelu_tanh(linear(x, w[p + "gate"])) * linear(x, w[p + "up"]), w[p + "down"])


def layer(x, w, i, entry, eps):
    p = f"l{i}."
    mixer = grouped_attention if entry["type"] == "attention" else latent_attention
    x = x + rms(mixer(x, w, p + "mix.", entry["mixer"], eps), eps) * w[p + "norm1"]
    if entry.get("mlp"):
        x = x + rms(feed_forward(x, w, p + "mlp."), eps) * w[p + "norm2"]
    return x


def forward(cfg, w, token_ids, residuals=None):
    """Logits [T, vocab] of a whole sequence; `residuals` (a list) receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(token_ids)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    for i, entry in enumerate(cfg["layers"]):
        x = layer(x, w, i, entry, eps)
        if residuals is not None:
            residuals.append(x.copy())
    return linear(rms(x, eps) * w["final.norm"], w["head"]) * cfg.get("logit_scale", 1.0)
