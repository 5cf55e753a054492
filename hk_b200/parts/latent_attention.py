"""Attention over a compressed cache ("latent attention"), as a mixer part.

Per token the mixer keeps ONE vector of `kv_rank + rot_dim` numbers instead of keys and values for every head:
    q = W_q x                      per head [plain_dim plain | rot_dim rotated by position]
    W_dkv x                        kv_rank + rot_dim numbers: the first kv_rank, RMS-normed with a weight, are the
                                   latent c; the last rot_dim, rotated by position, are a key part all heads share
    head h:  key = [W_uk,h c | shared rotated part],  value = W_uv,h c
    score = scale * (q_plain . W_uk,h c + q_rot . k_rot),  causal softmax,  y = W_o (concat_h(sum_j p_j W_uv,h c_j) [* sigmoid(W_g x)])
Nothing but c and the rotated part is cached, and the per-head keys and values are never formed: because the score
is linear in c, the query is carried into the latent space instead (q_lat,h = W_uk,h^T q_plain,h, one small product
per head), the attention runs as H query heads over one shared key/value head whose key is the cache row
[c | k_rot] and whose value is the row's first kv_rank dims, and W_uv,h is applied to the attention's result
(sum_j p_j c_j).  A decode step therefore reads kv_rank + rot_dim numbers per cached token, whatever the number of
heads.  Sizes, the norm's eps, the position encoding (its pairing, scaling and magnitude), the scale, a window and
the output gate are parameters; `names` renames the tensors (keys q, dkv, dkv_norm, uk, uv, gate, o).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import KVCacheSpec, MATRIX, VECTOR, ParamSpec, Part, Precision, register_part
from .position import RotaryEmbedding


class LatentAttention(Part):
    graph_safe = True   # reads the batch from device tensors only

    def __init__(self, hidden: int, n_heads: int, plain_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int, prefix: str,
                 norm_eps: float, scale: float, position: Optional[RotaryEmbedding] = None, gate: bool = False,
                 window: Optional[int] = None, names: Optional[Dict[str, str]] = None):
        if min(n_heads, plain_dim, v_head_dim, kv_rank) < 1 or rot_dim < 0:
            raise ValueError("heads, plain_dim, v_head_dim and kv_rank must be positive, rot_dim not negative")
        if kv_rank + rot_dim > 640:
            raise ValueError(f"a cache row of {kv_rank + rot_dim} numbers is above 640")
        if position is not None and position.rotary_dim > rot_dim:
            raise ValueError("the rotary width exceeds rot_dim")
        self.hidden, self.H, self.dn, self.dr, self.vd, self.r = hidden, n_heads, plain_dim, rot_dim, v_head_dim, kv_rank
        self.prefix, self.norm_eps, self.scale = prefix, float(norm_eps), float(scale)
        self.position, self.gate, self.window = position, bool(gate), window
        self.names = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g", "o": "o"}
        self.names.update(names or {})
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.c_norm = None
        self._tables_key = None        # set at bind: the flash kernels' work items, when they take a row of this size
        self._sm_count = 0
        self._wide = False             # set at bind: the row is too wide for the flash kernels, the latent kernel takes it

    def _flash_takes(self) -> bool:
        """The flash kernels run H query heads over ONE key/value head whose keys and values are both the cache row
        (the last rot_dim dims of their result are not used), when the row has a head size they know."""
        from ..csrc import attention_fast
        return attention_fast.supported(self.r + self.dr, self.H)

    def _latent_kernel_takes(self) -> bool:
        """Wider rows: the kernel that keeps the query tile in shared memory and splits the value columns among warps."""
        from ..csrc import attention_fast
        return attention_fast.latent_supported(self.H, self.r + self.dr, self.r)

    def kernel_libraries(self, bfloat16: bool):
        from ..csrc import attention_fast
        if not bfloat16:
            return ()
        if not self._flash_takes():
            return ("gemm_heads", "attention_latent") if self._latent_kernel_takes() else ("gemm_heads",)
        return ("gemm_heads", "attention_flash", "attention_prefill_tc") if attention_fast.tc_prefill_supported(self.r + self.dr, self.H) \
            else ("gemm_heads", "attention_flash")

    def step_tables_key(self):
        return self._tables_key

    def step_tables(self, ctx):
        from .attention import flash_step_tables
        if self._wide:
            # items of at most 64 / H tokens, all heads of a token in one item; never the tcgen05 prompt kernels' tiles
            return flash_step_tables(ctx, self.H, 1, self.r + self.dr, self.window or 0, 0, self._sm_count, tensor_prompt=False)
        return flash_step_tables(ctx, self.H, 1, self.r + self.dr, self.window or 0, 0, self._sm_count)

    def children(self):
        return (self.position,) if self.position is not None else ()

    def own_param_specs(self) -> Dict[str, ParamSpec]:
        p, nm, H, d = self.prefix, self.names, self.H, self.hidden
        specs = {
            p + nm["q"]: ParamSpec((H * (self.dn + self.dr), d), MATRIX),
            p + nm["dkv"]: ParamSpec((self.r + self.dr, d), MATRIX),
            p + nm["dkv_norm"]: ParamSpec((self.r,), VECTOR, "one_plus_normal"),
            p + nm["uk"]: ParamSpec((H * self.dn, self.r), MATRIX),
            p + nm["uv"]: ParamSpec((H * self.vd, self.r), MATRIX),
            p + nm["o"]: ParamSpec((d, H * self.vd), MATRIX),
        }
        if self.gate:
            specs[p + nm["gate"]] = ParamSpec((H * self.vd, d), MATRIX)
        return specs

    def cache_spec(self):
        """One shared head whose row is [latent | rotated key part]; no value tensor."""
        return KVCacheSpec(1, self.r + self.dr, self.window, 0)

    def own_bind(self, tensors, precision: Precision) -> None:
        p, nm, H = self.prefix, self.names, self.H
        mats = [tensors[p + nm["q"]], tensors[p + nm["dkv"]]] + ([tensors[p + nm["gate"]]] if self.gate else [])
        wide = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.w_in = torch.cat([t.to(wide) for t in mats], dim=0).contiguous()       # one product: q, compressed row, gate
        dt = precision.compute
        # q_lat,h = W_uk,h^T q_plain,h: as a product with weights [out = kv_rank, in = plain_dim] per head
        self.w_uk_t = tensors[p + nm["uk"]].to(dt).view(H, self.dn, self.r).transpose(1, 2).contiguous()
        self.w_uv = tensors[p + nm["uv"]].to(dt).view(H, self.vd, self.r).contiguous()
        self.w_o = tensors[p + nm["o"]]
        self.c_norm = tensors[p + nm["dkv_norm"]]
        if precision.compute == torch.bfloat16 and self._flash_takes():
            self._tables_key = ("paged_attention_items", self.window or 0, self.H, 1, self.r + self.dr, False, 0, False)
            self._sm_count = torch.cuda.get_device_properties(precision.device).multi_processor_count
        elif precision.compute == torch.bfloat16 and self._latent_kernel_takes():
            self._wide = True
            self._tables_key = ("latent_attention_items", self.window or 0, self.H, self.r + self.dr)
            self._sm_count = torch.cuda.get_device_properties(precision.device).multi_processor_count

    def _attend(self, q_full: torch.Tensor, ctx, cache) -> torch.Tensor:
        """The attention over the cache rows: a view [n, H, kv_rank] of the heads' latent sums.  In bfloat16 a tensor-core
        kernel takes it where one knows the row's size; else (and in 32-bit) the generic kernel."""
        from .attention import flash_plan
        n, dev, dt = q_full.shape[0], q_full.device, q_full.dtype
        H, dr, r = self.H, self.dr, self.r
        plan = flash_plan(ctx, self._tables_key) if dt == torch.bfloat16 and ops.forced("attention") != "generic" else None
        if plan is not None and self._wide:
            from ..csrc import attention_fast
            lat = torch.empty((n, H * r), dtype=dt, device=dev)
            # which variant runs depends on the batch's shape alone (single tokens or not), as a captured step's launches must
            if attention_fast.run_latent(q_full, cache.k_pages, cache.block_table, lat, H, r + dr, r, cache.page_tokens,
                                         self.window or 0, self.scale, plan,
                                         single_tokens=all(int(c) == 1 for c in ctx.q_lens)):
                return lat.view(n, H, r)
        elif plan is not None:
            # the flash kernels, with the cache rows as keys AND values: the first r dims of a head's result are its latent sums
            wide = torch.empty((n, H * (r + dr)), dtype=dt, device=dev)
            ops.paged_attention(q_full, cache.k_pages, cache.k_pages, cache.block_table, ctx.positions, ctx.slot_of_token, wide,
                                H, 1, r + dr, cache.page_tokens, self.window or 0, self.scale, plan=plan)
            return wide.view(n, H, r + dr)[:, :, :r]
        lat = torch.empty((n, H * r), dtype=dt, device=dev)
        ops.paged_attention(q_full, cache.k_pages, None, cache.block_table, ctx.positions, ctx.slot_of_token, lat,
                            H, 1, r + dr, cache.page_tokens, self.window or 0, self.scale)
        return lat.view(n, H, r)

    def forward(self, xb: torch.Tensor, residual: torch.Tensor, ctx, cache, write_cache: bool = True,
                accumulate: bool = True) -> None:
        n, dev, dt = xb.shape[0], xb.device, xb.dtype
        H, dn, dr, r, vd = self.H, self.dn, self.dr, self.r, self.vd
        proj = torch.empty((n, self.w_in.shape[0]), dtype=torch.float32, device=dev)
        ops.gemm(xb, self.w_in, proj)
        q_plain = torch.empty((n, H * dn), dtype=dt, device=dev)
        q_full = torch.empty((n, H * (r + dr)), dtype=dt, device=dev)
        cos = sin = None
        rot, pairing = 0, "half"
        if self.position is not None:
            cos, sin, rot = self.position.tables()
            pairing = self.position.pairing
        ops.latent_prep(proj, q_plain, q_full, self.c_norm, self.norm_eps, cos, sin, rot, pairing, ctx.positions,
                        ctx.slot_of_token, cache.block_table, cache.k_pages, H, dn, dr, r, cache.page_tokens,
                        write_kv=write_cache)
        ops.gemm_heads(q_plain.view(n, H, dn), self.w_uk_t, q_full.view(n, H, r + dr)[:, :, :r], H)
        lat = self._attend(q_full, ctx, cache)                  # [n, H, r]: sum_j p_j c_j per head
        att = torch.empty((n, H * vd), dtype=dt, device=dev)
        # the values' up-projection per head, with the output gate in its epilogue
        ops.gemm_heads(lat, self.w_uv, att.view(n, H, vd), H, gate=proj[:, H * (dn + dr) + r + dr:] if self.gate else None)
        ops.gemm(att, self.w_o, residual, accumulate=accumulate)


register_part("mixer", "latent_attention", LatentAttention)
