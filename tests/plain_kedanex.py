"""The Kedanex decoder written plainly: numpy, float64, whole sequences, one function per mechanism.

It shares no code with the package and is slow on purpose: every recurrence is a Python loop over
the tokens, attention is a loop over the queries.  `forward(cfg, w, ids)` takes the raw
config.json dictionary, a {tensor name: array} dictionary and the token ids of one sequence, and
returns the logits at every position (and, if asked, the residual stream after every layer run).

Notation.  h: a mixer's or feed-forward's input [T, d] (already normed).  W x means x @ W.T for a
weight stored [out, in].  rms(x) = x / sqrt(mean(x^2) + eps) over the last axis.
"""
from __future__ import annotations

import math

import numpy as np


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


round_inputs = None      # a function, to model an implementation that narrows the inputs of its matrix products


def linear(x, w, b=None):
    if round_inputs is not None:
        x = round_inputs(x)
    y = x @ w.T
    return y if b is None else y + b


def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
    return unit_rms(x, eps) * w


# ---------------------------------------------------------------------------- mixers


def general_delta(h, w, p, heads, dim, eps, state=None):
    """Generalised delta rule.  Per head, with a state S [dim keys, dim values] that starts at zero:
         decay   d_t = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h_t) + w0))      per key channel
         removal a_t = sigmoid(W_a h_t + b_a)                                   per key channel
         unit key u_t = k_t / sqrt(sum(k_t^2) + 1e-6)
         S_t = diag(d_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T
         o_t = S_t^T r_t
       then each head's o over its rms, all heads times the weight `norm`, times sigmoid(W_g h), then W_o.
       Returns (output [T, d], final state)."""
    T = h.shape[0]
    r = linear(h, w[p + "r"]).reshape(T, heads, dim)
    k = linear(h, w[p + "k"]).reshape(T, heads, dim)
    v = linear(h, w[p + "v"]).reshape(T, heads, dim)
    g = sigmoid(linear(h, w[p + "g"]))
    decay = np.exp(-math.exp(-0.5) * sigmoid(linear(np.tanh(linear(h, w[p + "w1"])), w[p + "w2"]) + w[p + "w0"]))
    decay = decay.reshape(T, heads, dim)
    a = sigmoid(linear(h, w[p + "a"], w[p + "a.b"])).reshape(T, heads, dim)
    u = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    S = np.zeros((heads, dim, dim)) if state is None else state.copy()
    o = np.zeros((T, heads, dim))
    for t in range(T):
        for hd in range(heads):
            old = S[hd]
            S[hd] = decay[t, hd][:, None] * old - np.outer(a[t, hd] * u[t, hd], u[t, hd] @ old) + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ r[t, hd]
    o = unit_rms(o, eps).reshape(T, heads * dim) * w[p + "norm"] * g
    return linear(o, w[p + "o"]), S


def mingru(h, w, p, eps=None, state=None):
    """minGRU: gates that read only the current token.
         z_t = sigmoid(W_z h_t + b_z);  c_t = W_x h_t + b_x;  candidate = c + 1/2 (c >= 0), sigmoid(c) (c < 0)
         S_t = (1 - z_t) S_(t-1) + z_t * candidate      element by element, S_(-1) = 0
         out_t = W_o (S_t * silu(W_g h_t))"""
    T = h.shape[0]
    z = sigmoid(linear(h, w[p + "z"], w[p + "z.b"]))
    c = linear(h, w[p + "x"], w[p + "x.b"])
    cand = np.where(c >= 0, c + 0.5, sigmoid(c))
    gate = silu(linear(h, w[p + "g"]))
    S = np.zeros(z.shape[1]) if state is None else state.copy()
    out = np.zeros_like(z)
    for t in range(T):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        out[t] = S * gate[t]
    return linear(out, w[p + "o"]), S


def rotate_half(x, positions, base, dims):
    """x [T, heads, dim]: the first `dims` dimensions of every head are rotated, dimension i paired with
    i + dims/2, by the angle position * base^(-2i/dims)."""
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    lo, hi = x[..., :half], x[..., half:dims]
    out[..., :half] = lo * c - hi * s
    out[..., half:dims] = hi * c + lo * s
    return out


def window_sink_attention(h, w, p, m, eps, first_position=0):
    """Grouped-query attention whose values are its keys as projected, with a sliding window and a sink.
         q = W_q h, k = W_k h, v = k (before rotation and norm, its first `vdim` dimensions)
         q, k rotated, then each head divided by its rms (no weight)
         position i sees j with 0 <= i - j < window
         p_ij = exp(s_ij) / (1 + sum_j exp(s_ij)),  s_ij = scale * q_i . k_j"""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w[p + "q"]).reshape(T, H, dim)
    k = linear(h, w[p + "k"]).reshape(T, G, dim)
    v = k[..., :vdim].copy()
    pos = np.arange(first_position, first_position + T)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, pos, rot["base"], rot["dims"])
        k = rotate_half(k, pos, rot["base"], rot["dims"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    if round_inputs is not None:       # a cache that stores narrowed keys and values, and narrowed queries
        q, k, v = round_inputs(q), round_inputs(k), round_inputs(v)
    window = m["mask"]["size"]
    out = np.zeros((T, H, vdim))
    for i in range(T):
        lo = max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * m["scale"]
            mx = max(0.0, s.max())
            e = np.exp(s - mx)
            out[i, hh] = (e / (math.exp(-mx) + e.sum())) @ v[lo:i + 1, g]
    return linear(out.reshape(T, H * vdim), w[p + "o"])


# ---------------------------------------------------------------------------- feed-forwards


def polynorm_ff(h, w, p, eps):
    """W_down act(W_up h), act(z) = a rms(z) + b rms(z^2) + c rms(z^3) + e with (a, b, c, e) = `act`."""
    z = linear(h, w[p + "up"])
    a, b, c, e = w[p + "act"]
    act = a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e
    return linear(act, w[p + "down"])


def routed_ff(h, w, p, experts, top, routes=None):
    """Each token goes to the `top` experts with the largest router logits (the lower index wins a tie); their
    weights are the softmax over the chosen logits; expert: W_down (silu(W_gate h) * (W_up h)).
    `routes` [T, top], when given, replaces the choice (not the weights): to follow an implementation whose
    rounding fell the other way in a close call."""
    logits = linear(h, w[p + "router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = np.argsort(-logits[t], kind="stable")[:top] if routes is None else np.asarray(routes[t])
        z = logits[t, chosen]
        pw = np.exp(z - z.max())
        pw /= pw.sum()
        for e, pe in zip(chosen, pw):
            q = f"{p}e{e}."
            out[t] += pe * linear(silu(linear(h[t], w[q + "gate"])) * linear(h[t], w[q + "up"]), w[q + "down"])
    return out


def router_margin(h, w, p, top):
    """Per token: by how much the last chosen router logit exceeds the best one not chosen, relative to the largest
    |logit| of the token (infinite when every expert is chosen).  A small margin is a close call: rounding may choose
    otherwise, and then the output is another one altogether."""
    z = np.sort(linear(h, w[p + "router"]), axis=1)[:, ::-1]
    if top >= z.shape[1]:
        return np.full(z.shape[0], np.inf)
    return (z[:, top - 1] - z[:, top]) / np.maximum(np.abs(z).max(axis=1), 1e-30)


# ---------------------------------------------------------------------------- the model


def layer_prefix(layers, i):
    """Layer i's tensors are named after layer `weights_of` when it has that key."""
    j = layers[i].get("weights_of")
    return f"l{i if j is None else j}."


def forward(cfg, w, ids, with_layers=False, with_margins=False, routes=None):
    """Logits [T, vocab]; with_layers: also the residual stream after every layer run; with_margins: also, per
    position, the smallest `router_margin` over the layers.  `routes`: for every routed feed-forward in running
    order, the experts [T, top] to use instead of its own choice."""
    routes = list(routes) if routes is not None else None
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(ids)]
    seen = []
    margins = np.full(len(ids), np.inf)
    for i, layer in enumerate(cfg["layers"]):
        p = layer_prefix(cfg["layers"], i)
        m = layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "general_delta":
            y, _ = general_delta(h, w, p + "mix.", m["heads"], m["dim"], eps)
        elif layer["type"] == "mingru":
            y, _ = mingru(h, w, p + "mix.")
        elif layer["type"] == "attention":
            y = window_sink_attention(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = polynorm_ff(h, w, p + "mlp.", eps)
            else:
                y = routed_ff(h, w, p + "mlp.", mlp["router"]["experts"], mlp["router"]["top"],
                              routes.pop(0) if routes is not None else None)
                margins = np.minimum(margins, router_margin(h, w, p + "mlp.", mlp["router"]["top"]))
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        seen.append(x.copy())
    logits = linear(rms_norm(x, w["final.norm"], eps), w["head"])
    out = (logits,) + ((np.stack(seen),) if with_layers else ()) + ((margins,) if with_margins else ())
    return out if len(out) > 1 else logits
