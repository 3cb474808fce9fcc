"""Typed configuration of the Nusudra decoder, read from config.json.

The file is nested.  Top level: ``architecture`` ("Nusudra"), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``,
``streams`` (how many residual streams a token has; absent: one plain residual row) and ``layers``, a list in which
every entry gives ``type`` (its mixer), the sizes and constants of its ``mixer`` and its ``mlp`` (``kind`` "dense"
with ``ff``, or null for a layer without a feed-forward).

  latent_attention:  heads, dim, rot_dim, vdim, kv_rank, scale, rot.base, rot.dims
  delta:             heads, kv_heads, dim, vdim, conv (taps)
  parallel:          left  = heads, kv_heads, dim, vdim, scale        (attention with a distance penalty and a sink)
                     right = heads, vdim, state, groups, norm_groups, conv (taps)   (a state-space layer)

Every size and constant that can differ between two models of the design is read from here and from nowhere else;
what the design fixes (the unit norms' eps, the activations) is written where it is computed.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

from ..errors import ConfigError, UnsupportedError
from .json_file import read_config_json
from .kugilix import _of

MIXER_TYPES = ("latent_attention", "delta", "parallel")


@dataclass(frozen=True)
class LatentAttentionSizes:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}

    def validate(self, where: str) -> None:
        for name in ("heads", "dim", "vdim", "kv_rank"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {where}.{name} must be > 0")
        if self.rot_dim < 0 or self.rot_dims < 0 or self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ConfigError(f"config.json: {where}: {self.rot_dims} of {self.rot_dim} rotated dimensions rotate")
        if self.rot_dims and not self.rot_base > 0:
            raise ConfigError(f"config.json: {where}.rot.base must be > 0")


@dataclass(frozen=True)
class DeltaSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}

    def validate(self, where: str) -> None:
        for name in ("heads", "kv_heads", "dim", "vdim", "conv"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {where}.{name} must be > 0")
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}: {self.heads} heads cannot share {self.kv_heads} q/k heads")


@dataclass(frozen=True)
class SinkAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}

    def validate(self, where: str) -> None:
        for name in ("heads", "kv_heads", "dim", "vdim"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {where}.{name} must be > 0")
        if self.heads % self.kv_heads:
            raise ConfigError(f"config.json: {where}: {self.heads} heads cannot share {self.kv_heads} kv heads")


@dataclass(frozen=True)
class StateSpaceSizes:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int

    def to_dict(self) -> dict:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "norm_groups": self.norm_groups, "conv": self.conv}

    def validate(self, where: str) -> None:
        for name in ("heads", "vdim", "state", "groups", "norm_groups", "conv"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {where}.{name} must be > 0")
        if self.heads % self.groups:
            raise ConfigError(f"config.json: {where}: {self.heads} heads cannot share {self.groups} groups")
        if (self.heads * self.vdim) % self.norm_groups:
            raise ConfigError(f"config.json: {where}: {self.heads * self.vdim} columns cannot be normed in "
                              f"{self.norm_groups} equal parts")


@dataclass(frozen=True)
class ParallelSizes:
    left: SinkAttentionSizes
    right: StateSpaceSizes

    def to_dict(self) -> dict:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}

    def validate(self, where: str) -> None:
        self.left.validate(where + ".left")
        self.right.validate(where + ".right")


@dataclass(frozen=True)
class NusudraLayer:
    type: str  # one of MIXER_TYPES
    mixer: Any  # the sizes class of its type
    ff: Optional[int]  # None: no feed-forward

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


def _read_mixer(kind: str, m: dict, where: str):
    if kind == "latent_attention":
        rot = _of(m, "rot", dict, where, required=False)
        rot_dim = _of(m, "rot_dim", int, where, default=0, required=False)
        return LatentAttentionSizes(
            heads=_of(m, "heads", int, where), dim=_of(m, "dim", int, where), rot_dim=rot_dim,
            vdim=_of(m, "vdim", int, where), kv_rank=_of(m, "kv_rank", int, where), scale=_of(m, "scale", float, where),
            rot_base=10000.0 if rot is None else _of(rot, "base", float, where + ".rot"),
            rot_dims=0 if rot is None else _of(rot, "dims", int, where + ".rot", default=rot_dim, required=False))
    if kind == "delta":
        heads = _of(m, "heads", int, where)
        return DeltaSizes(heads=heads, kv_heads=_of(m, "kv_heads", int, where, default=heads, required=False),
                          dim=_of(m, "dim", int, where), vdim=_of(m, "vdim", int, where), conv=_of(m, "conv", int, where))
    if kind == "parallel":
        left, right = _of(m, "left", dict, where), _of(m, "right", dict, where)
        lw, rw = where + ".left", where + ".right"
        heads = _of(left, "heads", int, lw)
        return ParallelSizes(
            SinkAttentionSizes(heads=heads, kv_heads=_of(left, "kv_heads", int, lw, default=heads, required=False),
                               dim=_of(left, "dim", int, lw), vdim=_of(left, "vdim", int, lw),
                               scale=_of(left, "scale", float, lw)),
            StateSpaceSizes(heads=_of(right, "heads", int, rw), vdim=_of(right, "vdim", int, rw),
                            state=_of(right, "state", int, rw), groups=_of(right, "groups", int, rw, default=1, required=False),
                            norm_groups=_of(right, "norm_groups", int, rw, default=1, required=False),
                            conv=_of(right, "conv", int, rw)))
    raise UnsupportedError(f"config.json: {where}: '{kind}' is not a mixer of this design ({', '.join(MIXER_TYPES)})")


@dataclass(frozen=True)
class NusudraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    streams: Optional[int]  # None: one plain residual row
    layers: tuple = field(default_factory=tuple)  # of NusudraLayer
    architecture: str = "Nusudra"

    def validate(self) -> None:
        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be > 0, found {getattr(self, name)}")
        if not (self.norm_eps >= 0.0):
            raise ConfigError(f"config.json: norm.eps must be >= 0, found {self.norm_eps}")
        if self.streams is not None and not (1 <= self.streams <= 8):
            raise ConfigError(f"config.json: streams must be 1..8, found {self.streams}")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        for i, layer in enumerate(self.layers):
            layer.mixer.validate(f"layers[{i}].mixer")
            if layer.ff is not None and layer.ff <= 0:
                raise ConfigError(f"config.json: layers[{i}].mlp.ff must be > 0")

    @classmethod
    def from_dict(cls, d: dict) -> "NusudraConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != "Nusudra":
            raise UnsupportedError(f"architecture {name!r} is not read by NusudraConfig")
        raw = d.get("layers")
        if not isinstance(raw, list):
            raise ConfigError("config.json: 'layers' must be a list")
        layers = []
        for i, e in enumerate(raw):
            where = f"layers[{i}]"
            if not isinstance(e, dict) or not isinstance(e.get("type"), str):
                raise ConfigError(f"config.json: {where} must be an object with a 'type'")
            mixer = _read_mixer(e["type"], _of(e, "mixer", dict, where), where + ".mixer")
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise UnsupportedError(f"config.json: {where}.mlp must be null or of kind 'dense'")
                ff = _of(mlp, "ff", int, where + ".mlp")
            layers.append(NusudraLayer(e["type"], mixer, ff))
        norm = _of(d, "norm", dict, "the top level")
        emb = _of(d, "embedding", dict, "the top level", required=False)
        cfg = cls(
            vocab=_of(d, "vocab", int, "the top level"),
            width=_of(d, "width", int, "the top level"),
            embedding_scale=1.0 if emb is None else _of(emb, "scale", float, "embedding", default=1.0, required=False),
            norm_eps=_of(norm, "eps", float, "norm"),
            streams=_of(d, "streams", int, "the top level", required=False),
            layers=tuple(layers),
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d: dict = {
            "architecture": self.architecture,
            "vocab": self.vocab,
            "width": self.width,
            "embedding": {"scale": self.embedding_scale},
            "norm": {"eps": self.norm_eps},
            "layers": [layer.to_dict() for layer in self.layers],
        }
        if self.streams is not None:
            d["streams"] = self.streams
        return d

    @classmethod
    def from_json(cls, path: str) -> "NusudraConfig":
        return cls.from_dict(read_config_json(path))
