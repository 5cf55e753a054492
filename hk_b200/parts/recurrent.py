"""Recurrent mixers: a state of fixed size per request, advanced token by token.

Both keep their state in float32 in the request's state slot (`StateSpec`) and find the rows of every request
of a step through one host-built table, `segments` int32 [requests of the step, 3] = (slot, first row, rows),
shared by all recurrent mixers of a model.  The scans (`csrc/recurrent.cu`) walk a request's rows in order, so
what a position computes does not depend on how the prompt was cut, on the batch or on the slot.  Projections
are products in the compute type with float32 results; everything from there to the state and the scan's
output is float32.

`GeneralDeltaRule` (per head a matrix state S [key_dim, value_dim], zero at the start):
      r, k, v, g = W_r h, W_k h, W_v h, W_g h;   decay logits wl = W_w2 tanh(W_w1 h) + w0;   al = W_a h + a0
      d = exp(-decay_scale * sigmoid(wl)),  a = sigmoid(al),  u = k / sqrt(sum(k^2) + key_eps)        per head
      S <- diag(d) S - (a * u) (u^T S) + k v^T        (both terms read the old S);    o = S^T r
      y = W_o ((o / rms(o) per head) * norm_weight * sigmoid(g))
  `decay_scale` and `key_eps` are parameters (exp(-1/2) and 1e-6 by default); the width of W_w1 is read from the
  configuration or, at binding, from the tensor.

`MinGRU` (one scalar state per channel, zero at the start; the gates read only the current token):
      z = sigmoid(W_z h + b_z);  x = W_x h + b_x;  c = x + 1/2 for x >= 0, sigmoid(x) below
      S <- (1 - z) S + z c;   y = W_o (S * silu(W_g h))
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from ..csrc import ops
from .base import MATRIX, VECTOR, ParamSpec, Part, Precision, StateSpec, StepTables, register_part

SEGMENTS_KEY = ("request_segments",)


def segment_tables(ctx) -> StepTables:
    """(slot, first row, rows) of every request of the step.  Its shape depends on the number of requests alone."""
    seg = np.stack([np.asarray(ctx.slots, dtype=np.int32), np.asarray(ctx.q_starts, dtype=np.int32),
                    np.asarray(ctx.q_lens, dtype=np.int32)], axis=1)
    return StepTables({"segments": seg})


class _SegmentScan(Part):
    graph_safe = True           # the batch is read from device tensors and the segment table only
    kernel_libraries = ("recurrent",)

    def step_tables_key(self):
        return SEGMENTS_KEY

    def step_tables(self, ctx):
        return segment_tables(ctx)

    @staticmethod
    def _segments(ctx) -> torch.Tensor:
        return ctx.tables[SEGMENTS_KEY][0]["segments"]


class GeneralDeltaRule(_SegmentScan):
    def __init__(self, hidden: int, n_heads: int, key_dim: int, prefix: str, norm_eps: float,
                 value_dim: Optional[int] = None, decay_rank: Optional[int] = None,
                 decay_scale: float = math.exp(-0.5), key_eps: float = 1e-6, names: Optional[Dict[str, str]] = None):
        self.hidden, self.H, self.dk = hidden, n_heads, key_dim
        self.dv = key_dim if value_dim is None else int(value_dim)
        self.prefix, self.norm_eps = prefix, float(norm_eps)
        self.decay_rank = decay_rank         # None: whatever the file's tensor has (known at binding)
        self.decay_scale, self.key_eps = float(decay_scale), float(key_eps)
        self.names = {"r": "r", "k": "k", "v": "v", "g": "g", "a": "a", "a_bias": "a.b", "w1": "w1", "w2": "w2",
                      "w_bias": "w0", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_w2 = self.w_o = self.a_bias = self.w_bias = self.norm_weight = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, d = self.prefix, self.names, self.hidden
        K, V = self.H * self.dk, self.H * self.dv
        R = self.decay_rank if self.decay_rank is not None else -1      # -1: any size along that axis
        return {
            p + nm["r"]: ParamSpec((K, d), MATRIX), p + nm["k"]: ParamSpec((K, d), MATRIX),
            p + nm["v"]: ParamSpec((V, d), MATRIX), p + nm["g"]: ParamSpec((V, d), MATRIX),
            p + nm["a"]: ParamSpec((K, d), MATRIX), p + nm["a_bias"]: ParamSpec((K,), VECTOR),
            p + nm["w1"]: ParamSpec((R, d), MATRIX), p + nm["w2"]: ParamSpec((K, R), MATRIX),
            p + nm["w_bias"]: ParamSpec((K,), VECTOR), p + nm["norm"]: ParamSpec((V,), VECTOR, "one_plus_normal"),
            p + nm["o"]: ParamSpec((d, V), MATRIX),
        }

    def cache_spec(self):
        return StateSpec((self.H, self.dk, self.dv), torch.float32)

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("r", "k", "v", "g", "a", "w1")]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        # one product gives r, k, v, g, the removal logits and the hidden layer of the decay's low-rank projection
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()
        self.rank = int(tensors[p + nm["w1"]].shape[0])
        self.w_w2 = tensors[p + nm["w2"]]
        if int(self.w_w2.shape[1]) != self.rank:
            raise ValueError(f"'{p + nm['w2']}' takes {int(self.w_w2.shape[1])} inputs, '{p + nm['w1']}' gives {self.rank}")
        self.w_o = tensors[p + nm["o"]]
        self.a_bias, self.w_bias = tensors[p + nm["a_bias"]], tensors[p + nm["w_bias"]]
        self.norm_weight = tensors[p + nm["norm"]]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n = xb.shape[0]
        K, V = self.H * self.dk, self.H * self.dv
        proj = torch.empty((n, self.w_in.shape[0]), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_in, proj)
        r, k, v = proj[:, :K], proj[:, K:2 * K], proj[:, 2 * K:2 * K + V]
        g, al = proj[:, 2 * K + V:2 * K + 2 * V], proj[:, 2 * K + 2 * V:3 * K + 2 * V]
        hid = torch.empty((n, self.rank), dtype=xb.dtype, device=xb.device)
        ops.tanh_cols(proj[:, 3 * K + 2 * V:], hid)
        wl = torch.empty((n, K), dtype=torch.float32, device=xb.device)
        ops.gemm(hid, self.w_w2, wl)
        o = torch.empty((n, V), dtype=torch.float32, device=xb.device)
        ops.delta_rule_scan(r, k, v, al, wl, self.a_bias, self.w_bias, self._segments(ctx), cache.state, o,
                            self.H, self.dk, self.dv, self.decay_scale, self.key_eps)
        og = torch.empty((n, V), dtype=xb.dtype, device=xb.device)
        ops.head_norm_gate(o, g, self.norm_weight, self.norm_eps, og, self.H, self.dv)
        ops.gemm(og, self.w_o, residual, accumulate=accumulate)


class MinGRU(_SegmentScan):
    def __init__(self, hidden: int, width: int, prefix: str, names: Optional[Dict[str, str]] = None):
        self.hidden, self.width, self.prefix = hidden, width, prefix
        self.names = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "g": "g", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_o = self.z_bias = self.x_bias = None

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, d, W = self.prefix, self.names, self.hidden, self.width
        return {
            p + nm["z"]: ParamSpec((W, d), MATRIX), p + nm["z_bias"]: ParamSpec((W,), VECTOR),
            p + nm["x"]: ParamSpec((W, d), MATRIX), p + nm["x_bias"]: ParamSpec((W,), VECTOR),
            p + nm["g"]: ParamSpec((W, d), MATRIX), p + nm["o"]: ParamSpec((d, W), MATRIX),
        }

    def cache_spec(self):
        return StateSpec((self.width,), torch.float32)

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm = self.prefix, self.names
        mats = [tensors[p + nm[c]] for c in ("z", "x", "g")]
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()
        self.w_o = tensors[p + nm["o"]]
        self.z_bias, self.x_bias = tensors[p + nm["z_bias"]], tensors[p + nm["x_bias"]]

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n = xb.shape[0]
        proj = torch.empty((n, 3 * self.width), dtype=torch.float32, device=xb.device)
        ops.gemm(xb, self.w_in, proj)
        out = torch.empty((n, self.width), dtype=xb.dtype, device=xb.device)
        ops.mingru_scan(proj, self.z_bias, self.x_bias, self._segments(ctx), cache.state, out)
        ops.gemm(out, self.w_o, residual, accumulate=accumulate)


register_part("mixer", "general_delta_rule", GeneralDeltaRule)
register_part("mixer", "mingru", MinGRU)
