"""Typed configuration of the Padodra decoder, read from its own config.json keys.

config.json of this design is nested: `width`, `vocab`, `norm.eps`, `embedding.scale`, `logit_scale` and a list
`layers`, one entry per layer in running order.  An entry has `type` (which mixer: attention or latent_attention),
`mixer` (that mixer's sizes and constants) and `mlp` (null for none; `kind` dense with `ff`).  Every size and constant
of a model stands here and nowhere else in the package; what the design fixes for all of its models (the pairing of
the rotated dims per mixer type, the kind of frequency scaling per mixer type, the feed-forward's activation) stands in
the model's builder.  A key that a mixer may go without (`mask`, `softcap`, `rot`, `rot.scaling`) is read as absent.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .base import ConfigError, ModelConfig, need_int, opt_float, opt_int

MIXERS = ("attention", "latent_attention")


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


def _opt_positive(raw: dict, key: str, where: str) -> float:
    """A positive number, or 0 when the key is absent or null."""
    if raw.get(key) is None:
        return 0.0
    v = _need_float(raw, key, where)
    if not v > 0:
        raise ConfigError(f"config.json {where}'{key}' = {v} must be positive")
    return v


@dataclass
class PadodraRotation:
    """`rot` of a mixer: base, how many dims turn, and the scaling's numbers by their config.json names (`factor`,
    `original`, and `low`, `high` or `fast`, `slow`); an empty dict: no scaling."""
    base: float
    dims: int
    scaling: Dict[str, float] = field(default_factory=dict)

    @classmethod
    def from_dict(cls, raw: dict, where: str, limit: int, scaling_keys) -> "PadodraRotation":
        dims = need_int(raw, "dims")
        base = _need_float(raw, "base", where)
        if dims % 2 or dims > limit:
            raise ConfigError(f"config.json {where}'dims' = {dims} must be even and at most {limit}")
        if not base > 0 or base == 1.0:
            raise ConfigError(f"config.json {where}'base' = {base} must be positive and not 1")
        scaling: Dict[str, float] = {}
        if raw.get("scaling") is not None:
            sc = _need_dict(raw, "scaling", where)
            for key in scaling_keys:
                scaling[key] = _need_float(sc, key, where + "scaling.")
                if not scaling[key] > 0:
                    raise ConfigError(f"config.json {where}scaling.'{key}' = {scaling[key]} must be positive")
        return cls(base, dims, scaling)

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.scaling:
            d["scaling"] = {k: (int(v) if k == "original" and float(v).is_integer() else v) for k, v in self.scaling.items()}
        return d


@dataclass
class PadodraMixer:
    """One layer's mixer: `kind` and the sizes that kind reads."""
    kind: str
    heads: int = 0
    dim: int = 0                    # attention: query/key size of a head; latent_attention: its part that is not rotated
    vdim: int = 0                   # value size of a head
    scale: float = 1.0              # factor on the scores
    rot: Optional[PadodraRotation] = None
    kv_heads: int = 0               # attention
    chunk: int = 0                  # attention: mask.size (0: plain causal)
    softcap: float = 0.0            # attention (0: none)
    rot_dim: int = 0                # latent_attention: the rotated part of a query or key
    kv_rank: int = 0                # latent_attention: size of the cached latent

    @classmethod
    def from_dict(cls, kind: str, raw: dict, where: str) -> "PadodraMixer":
        heads, dim = need_int(raw, "heads"), need_int(raw, "dim")
        vdim = opt_int(raw, "vdim", dim)
        scale = _need_float(raw, "scale", where)
        if kind == "attention":
            kv_heads = opt_int(raw, "kv_heads", heads)
            if heads % kv_heads:
                raise ConfigError(f"config.json {where}'heads' = {heads} is not a multiple of 'kv_heads' = {kv_heads}")
            chunk = 0
            if raw.get("mask") is not None:
                chunk = need_int(_need_dict(raw, "mask", where), "size")
            rot = None
            if raw.get("rot") is not None:
                rot = PadodraRotation.from_dict(_need_dict(raw, "rot", where), where + "rot.", dim,
                                                ("factor", "low", "high", "original"))
                s = rot.scaling
                if s and not s["low"] < s["high"]:
                    raise ConfigError(f"config.json {where}rot.scaling needs 'low' < 'high'")
            return cls(kind, heads=heads, dim=dim, vdim=vdim, scale=scale, rot=rot, kv_heads=kv_heads, chunk=chunk,
                       softcap=_opt_positive(raw, "softcap", where))
        rot_dim, kv_rank = need_int(raw, "rot_dim"), need_int(raw, "kv_rank")
        rot = None
        if raw.get("rot") is not None:
            rot = PadodraRotation.from_dict(_need_dict(raw, "rot", where), where + "rot.", rot_dim,
                                            ("factor", "original", "fast", "slow"))
        return cls(kind, heads=heads, dim=dim, vdim=vdim, scale=scale, rot=rot, rot_dim=rot_dim, kv_rank=kv_rank)

    def to_dict(self) -> dict:
        d = {"dim": self.dim, "heads": self.heads, "scale": self.scale, "vdim": self.vdim}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.kind == "attention":
            d["kv_heads"] = self.kv_heads
            if self.chunk:
                d["mask"] = {"size": self.chunk}
            if self.softcap:
                d["softcap"] = self.softcap
        else:
            d["kv_rank"], d["rot_dim"] = self.kv_rank, self.rot_dim
        return d


@dataclass
class PadodraMlp:
    kind: str               # "dense"
    ff: int = 0

    @classmethod
    def from_dict(cls, raw: dict, where: str) -> "PadodraMlp":
        kind = raw.get("kind")
        if kind != "dense":
            raise ConfigError(f"config.json {where}'kind' = {kind!r} is not supported (supported: dense)")
        return cls("dense", ff=need_int(raw, "ff"))

    def to_dict(self) -> dict:
        return {"ff": self.ff, "kind": self.kind}


@dataclass
class PadodraLayer:
    mixer: PadodraMixer
    mlp: Optional[PadodraMlp]


@dataclass
class PadodraConfig(ModelConfig):
    width: int = 0
    vocab: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    layers: List[PadodraLayer] = field(default_factory=list)
    initializer_range: float = 0.05

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: dict) -> "PadodraConfig":
        width, vocab = need_int(raw, "width"), need_int(raw, "vocab")
        eps = _need_float(_need_dict(raw, "norm", ""), "eps", "norm.")
        if not eps > 0:
            raise ConfigError(f"config.json 'norm.eps' = {eps} must be positive")
        emb_scale = 1.0
        if raw.get("embedding") is not None:
            emb_scale = opt_float(_need_dict(raw, "embedding", ""), "scale", 1.0)
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json 'layers' must be a list with at least one layer")
        layers: List[PadodraLayer] = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]."
            if not isinstance(e, dict):
                raise ConfigError(f"config.json layers[{i}] must be an object")
            kind = e.get("type")
            if kind not in MIXERS:
                raise ConfigError(f"config.json {where}'type' = {kind!r} is not supported (supported: {', '.join(MIXERS)})")
            mixer = PadodraMixer.from_dict(kind, _need_dict(e, "mixer", where), where + "mixer.")
            mlp = None if e.get("mlp") is None else PadodraMlp.from_dict(_need_dict(e, "mlp", where), where + "mlp.")
            layers.append(PadodraLayer(mixer, mlp))
        return cls(architecture="Padodra", width=width, vocab=vocab, norm_eps=eps, embedding_scale=emb_scale,
                   logit_scale=opt_float(raw, "logit_scale", 1.0), layers=layers,
                   initializer_range=opt_float(raw, "initializer_range", 0.05))

    def to_dict(self) -> dict:
        out = [{"mixer": layer.mixer.to_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict(),
                "type": layer.mixer.kind} for layer in self.layers]
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale}, "layers": out,
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width,
                "initializer_range": self.initializer_range}
