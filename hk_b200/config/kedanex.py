"""Typed configuration of the Kedanex decoder, read from its own config.json keys.

config.json of this design is nested: `width`, `vocab`, `norm.eps` and a list `layers`, one entry per
layer in running order.  An entry has `type` (which mixer: general_delta, mingru or attention), `mixer`
(that mixer's sizes and constants), `mlp` (null for none; `kind` dense with `ff`, or moe with `expert.ff`,
`router.experts` and `router.top`) and optionally `weights_of`: j, which says that the layer has no tensors
of its own and runs with those of layer j (its cache or state is still its own).  Every size and constant
of a model stands here and nowhere else in the package; what the design fixes for all of its models (the
decay's factor, the eps of the unit key, the activation's exponents) stands in the parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .base import ConfigError, ModelConfig, need_int, opt_float, opt_int

MIXERS = ("general_delta", "mingru", "attention")


def _need_dict(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json {where}'{key}' must be an object")
    return v


def _need_float(raw: dict, key: str, where: str) -> float:
    v = raw.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json {where}'{key}' = {v!r} is not a number")
    return float(v)


@dataclass
class KedanexMixer:
    """One layer's mixer: `kind` and the sizes that kind reads."""
    kind: str
    heads: int = 0          # general_delta, attention
    dim: int = 0            # general_delta: key and value size of a head; attention: query/key size
    width: int = 0          # mingru: size of the recurrent state
    kv_heads: int = 0       # attention
    vdim: int = 0           # attention: value size (the first vdim dimensions of the projected key)
    window: int = 0         # attention: mask.size (0: no window)
    rot_dims: int = 0       # attention: rot.dims (0: no rotation)
    rot_base: float = 10000.0
    scale: float = 1.0      # attention
    decay_rank: int = 0     # general_delta: width of the decay's low-rank projection; 0: as the file's tensor has it

    @classmethod
    def from_dict(cls, kind: str, raw: dict, where: str) -> "KedanexMixer":
        if kind == "general_delta":
            return cls(kind, heads=need_int(raw, "heads"), dim=need_int(raw, "dim"), decay_rank=opt_int(raw, "decay_rank", 0))
        if kind == "mingru":
            return cls(kind, width=need_int(raw, "width"))
        heads, dim = need_int(raw, "heads"), need_int(raw, "dim")
        kv_heads = opt_int(raw, "kv_heads", heads)
        if heads % kv_heads:
            raise ConfigError(f"config.json {where}'heads' = {heads} is not a multiple of 'kv_heads' = {kv_heads}")
        vdim = opt_int(raw, "vdim", dim)
        if vdim > dim:
            raise ConfigError(f"config.json {where}'vdim' = {vdim} exceeds 'dim' = {dim}: the values are the projected keys")
        window = 0                                   # no mask: every earlier position stays visible
        if raw.get("mask") is not None:
            window = need_int(_need_dict(raw, "mask", where), "size")
        rot = raw.get("rot")
        rot_dims, rot_base = 0, 10000.0
        if rot is not None:
            if not isinstance(rot, dict):
                raise ConfigError(f"config.json {where}'rot' must be an object or null")
            rot_dims = need_int(rot, "dims")
            rot_base = _need_float(rot, "base", where + "rot.")
            if rot_dims % 2 or rot_dims > dim:
                raise ConfigError(f"config.json {where}'rot.dims' = {rot_dims} must be even and at most 'dim' = {dim}")
            if not rot_base > 0:
                raise ConfigError(f"config.json {where}'rot.base' = {rot_base} must be positive")
        return cls(kind, heads=heads, dim=dim, kv_heads=kv_heads, vdim=vdim, window=window, rot_dims=rot_dims,
                   rot_base=rot_base, scale=_need_float(raw, "scale", where))

    def to_dict(self) -> dict:
        if self.kind == "general_delta":
            return {"dim": self.dim, "heads": self.heads, **({"decay_rank": self.decay_rank} if self.decay_rank else {})}
        if self.kind == "mingru":
            return {"width": self.width}
        d = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass
class KedanexMlp:
    kind: str               # "dense" or "moe"
    ff: int = 0             # dense: the hidden size; moe: one expert's
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "KedanexMlp":
        kind = raw.get("kind")
        if kind == "dense":
            return cls("dense", ff=need_int(raw, "ff"))
        if kind == "moe":
            router = _need_dict(raw, "router", where)
            experts, top = need_int(router, "experts"), need_int(router, "top")
            if top > experts:
                raise ConfigError(f"config.json {where}'router.top' = {top} exceeds 'router.experts' = {experts}")
            return cls("moe", ff=need_int(_need_dict(raw, "expert", where), "ff"), experts=experts, top=top)
        raise ConfigError(f"config.json {where}'kind' = {kind!r} is neither 'dense' nor 'moe'")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        return {"expert": {"ff": self.ff}, "kind": "moe", "router": {"experts": self.experts, "top": self.top}}


@dataclass
class KedanexLayer:
    mixer: KedanexMixer
    mlp: Optional[KedanexMlp]
    weights_of: Optional[int] = None


@dataclass
class KedanexConfig(ModelConfig):
    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-5
    layers: List[KedanexLayer] = field(default_factory=list)
    initializer_range: float = 0.05

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: dict) -> "KedanexConfig":
        width, vocab = need_int(raw, "width"), need_int(raw, "vocab")
        eps = _need_float(_need_dict(raw, "norm", ""), "eps", "norm.")
        if not eps > 0:
            raise ConfigError(f"config.json 'norm.eps' = {eps} must be positive")
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json 'layers' must be a list with at least one layer")
        layers: List[KedanexLayer] = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json layers[{i}] must be an object")
            kind = e.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"config.json {where}'type' = {kind!r} is not supported (supported: {', '.join(MIXERS)})")
            mixer = KedanexMixer.from_dict(kind, _need_dict(e, "mixer", where), where + "mixer.")
            mlp = None if e.get("mlp") is None else KedanexMlp.from_dict(_need_dict(e, "mlp", where), where + "mlp.")
            layers.append(KedanexLayer(mixer, mlp, opt_int(e, "weights_of", None, minimum=0)))
        for i, layer in enumerate(layers):
            of = layer.weights_of
            if of is None:
                continue
            if of >= len(layers) or of == i or layers[of].weights_of is not None:
                raise ConfigError(f"config.json layers[{i}].'weights_of' = {of} must name another layer that has tensors of its own")
            if layers[of].mixer.kind != layer.mixer.kind:
                raise ConfigError(f"config.json layers[{i}]: a layer with 'weights_of' = {of} must have that layer's type")
        return cls(architecture="Kedanex", width=width, vocab=vocab, norm_eps=eps, layers=layers,
                   initializer_range=opt_float(raw, "initializer_range", 0.05))

    def to_dict(self) -> dict:
        out = []
        for layer in self.layers:
            e = {"mixer": layer.mixer.to_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict(),
                 "type": layer.mixer.kind}
            if layer.weights_of is not None:
                e["weights_of"] = layer.weights_of
            out.append(e)
        return {"architecture": self.architecture, "layers": out, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
                "width": self.width, "initializer_range": self.initializer_range}
