"""The Padodra decoder put together from parts, by its configuration.

A layer norms only what its sublayers give back and the sublayers read the residual stream itself
(`PostNormBlock`): x <- x + N1(mixer(x)), x <- x + N2(ff(x)).  The mixer is, layer by layer,

  * `attention`: grouped-query attention (`GQAAttention`) with a weighted per-head norm of q and k before the
    rotation, a rotation of the first `rot.dims` dims in adjacent pairs (2i, 2i + 1) with Llama-3 frequency scaling,
    scores bounded by a soft cap, a mask of blocks of `mask.size` positions, a learned sink score per head, values of
    their own width and an output gate;
  * `latent_attention`: attention over a compressed cache (`LatentAttention`): per head `dim` plain and `rot_dim`
    rotated query/key dims, the rotation in halves (i, i + dims/2) with YaRN frequency scaling and magnitude, plain
    causal softmax and an output gate.

The feed-forward is a GeGLU (`SwiGLUFeedForward` with the tanh form of gelu) or absent.  The embedding is multiplied
by `embedding.scale`, and `logit_scale` multiplies the logits: the final norm's weight carries it.  Tensor names:
`embed`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config import PadodraConfig, register_architecture
from ..parts import (GQAAttention, LatentAttention, OutputHead, PostNormBlock, RMSNorm, RopeScaling, RotaryEmbedding,
                     SwiGLUFeedForward, TokenEmbedding)
from .spec import ModelSpec


def _rotation(rot, kind: str, pairing: str, positions: int, made: dict):
    """The position encoding of a mixer's `rot` (shared by the mixers whose numbers agree), or None."""
    if rot is None:
        return None
    s = rot.scaling
    key = (kind, pairing, rot.base, rot.dims, tuple(sorted(s.items())))
    if key not in made:
        scaling = None
        if s and kind == "llama3":
            scaling = RopeScaling("llama3", factor=s["factor"], orig_ctx=s["original"], low_freq_factor=s["low"],
                                  high_freq_factor=s["high"])
        elif s:
            scaling = RopeScaling("yarn", factor=s["factor"], orig_ctx=s["original"], beta_fast=s["fast"], beta_slow=s["slow"])
        made[key] = RotaryEmbedding(rot.base, rot.dims, positions, pairing=pairing, scaling=scaling)
    return made[key]


def build_padodra(cfg: PadodraConfig, max_positions: int = 0) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    positions = max(int(max_positions), 1)
    ropes: dict = {}
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if m.kind == "attention":
            mixer = GQAAttention(d, m.heads, m.kv_heads, m.dim, p + "mix.", qk_norm_eps=eps,
                                 position=_rotation(m.rot, "llama3", "adjacent", positions, ropes), scale=m.scale,
                                 v_head_dim=m.vdim, sink=True, sink_weights=True, softcap=m.softcap or None,
                                 chunk=m.chunk or None, gate=True,
                                 names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                                        "sink": "sink", "gate": "g"})
        else:
            mixer = LatentAttention(d, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, p + "mix.", norm_eps=eps, scale=m.scale,
                                    position=_rotation(m.rot, "yarn", "half", positions, ropes), gate=True)
        ffn = ffn_norm = None
        if layer.mlp is not None:
            ffn = SwiGLUFeedForward(d, layer.mlp.ff, p + "mlp.", act="gelu_tanh",
                                    names={"gate": "gate", "up": "up", "down": "down"})
            ffn_norm = RMSNorm(d, eps, p + "norm2")
        blocks.append(PostNormBlock(mixer, RMSNorm(d, eps, p + "norm1"), ffn, ffn_norm))
    embedding = TokenEmbedding(cfg.vocab, d, "embed", scale=cfg.embedding_scale)
    # logits = head(norm(x)) * logit_scale, computed as head(norm(x) * logit_scale)
    head = OutputHead(d, cfg.vocab, RMSNorm(d, eps, "final.norm", weight_scale=cfg.logit_scale), "head")
    return ModelSpec(cfg, embedding, blocks, head)


register_architecture("Padodra", PadodraConfig, build_padodra, "padodra")
