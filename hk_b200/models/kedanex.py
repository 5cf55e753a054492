"""The Kedanex decoder put together from parts, by its configuration.

A layer norms both sides of its mixer and of its feed-forward (`SandwichNormBlock`).  The mixer is, layer by
layer, a generalised delta rule (`GeneralDeltaRule`), a minGRU (`MinGRU`) or a sliding-window attention whose
values are its keys as projected, with rotation before a weightless per-head norm and a sink in the softmax
(`GQAAttention` with those options).  The feed-forward is dense with the polynomial activation
(`PolyNormFeedForward`), a mixture of experts (`RoutedFeedForward`), or absent.  A layer with `weights_of`: j is
one more call of layer j's block in the schedule, with a cache or state of its own.  Tensor names: `embed`,
`l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config import KedanexConfig, register_architecture
from ..parts import (GQAAttention, GeneralDeltaRule, MinGRU, OutputHead, PolyNormFeedForward, RMSNorm, RotaryEmbedding,
                     RoutedFeedForward, SandwichNormBlock, TokenEmbedding)
from .spec import LayerCall, ModelSpec


def build_kedanex(cfg: KedanexConfig, max_positions: int = 0) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    positions = max(int(max_positions), 1)
    ropes = {}
    blocks, block_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p, m = f"l{i}.", layer.mixer
        if m.kind == "general_delta":
            mixer = GeneralDeltaRule(d, m.heads, m.dim, p + "mix.", norm_eps=eps, decay_rank=m.decay_rank or None)
        elif m.kind == "mingru":
            mixer = MinGRU(d, m.width, p + "mix.")
        else:
            rope = None
            if m.rot_dims:
                key = (m.rot_base, m.rot_dims)
                if key not in ropes:
                    ropes[key] = RotaryEmbedding(m.rot_base, m.rot_dims, positions, pairing="half")
                rope = ropes[key]
            mixer = GQAAttention(d, m.heads, m.kv_heads, m.dim, p + "mix.", qk_norm_eps=eps, position=rope,
                                 window=m.window or None, scale=m.scale, qk_norm_after=True, qk_norm_weight=False,
                                 value_from_key=True, v_head_dim=m.vdim, sink=True,
                                 names={"q": "q", "k": "k", "o": "o"})
        ffn = ffn_norm = post_ffn = None
        if layer.mlp is not None:
            if layer.mlp.kind == "dense":
                ffn = PolyNormFeedForward(d, layer.mlp.ff, p + "mlp.", eps)
            else:
                ffn = RoutedFeedForward(d, layer.mlp.ff, layer.mlp.experts, layer.mlp.top, p + "mlp.")
            ffn_norm, post_ffn = RMSNorm(d, eps, p + "norm2"), RMSNorm(d, eps, p + "norm2b")
        block_of[i] = len(blocks)
        blocks.append(SandwichNormBlock(RMSNorm(d, eps, p + "norm1"), mixer, RMSNorm(d, eps, p + "norm1b"),
                                        ffn_norm, ffn, post_ffn))
    schedule = [LayerCall(block_of[i if layer.weights_of is None else layer.weights_of]) for i, layer in enumerate(cfg.layers)]
    embedding = TokenEmbedding(cfg.vocab, d, "embed")
    head = OutputHead(d, cfg.vocab, RMSNorm(d, eps, "final.norm"), "head")
    return ModelSpec(cfg, embedding, blocks, head, schedule)


register_architecture("Kedanex", KedanexConfig, build_kedanex, "kedanex")
