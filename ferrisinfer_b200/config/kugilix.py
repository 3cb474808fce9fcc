"""Typed configuration of the Kugilix decoder, read from config.json.

The file is nested.  Top level: ``architecture`` ("Kugilix"), ``vocab``, ``width``, ``embedding.scale``,
``norm.eps`` and ``norm.groups`` (every norm of the model but the two inside its mixers is an RMS norm in that
many groups), ``canon.taps`` (a causal convolution of that many taps in front of every mixer), ``loop``
(``start``, ``stop``, ``times``: layers start .. stop - 1 run that many times in a row) and ``layers``, a list in
which every entry gives ``type`` ("attention" or "lightning"), the sizes and constants of its ``mixer`` and its
``mlp`` (``kind`` "dense" with ``ff``, or null for a layer without a feed-forward).

  attention mixer:  heads, kv_heads, dim, vdim, scale, mask.size (the window), q_temp.coef and q_temp.every
  lightning mixer:  heads, dim, vdim, decay (one per head)

Every size and constant that can differ between two models of the design is read from here and from nowhere
else; what the design fixes (the base of the position frequencies, the span of the distance slopes, the
activations) is written where it is computed.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Optional

from ..errors import ConfigError, UnsupportedError
from .json_file import read_config_json


def _of(d, key, kind, where, default=None, required=True):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    v = d.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: {where} lacks '{key}'")
        return default
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"config.json: {where}.{key} must be an integer, found {v!r}")
        return int(v)
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
            raise ConfigError(f"config.json: {where}.{key} must be a finite number, found {v!r}")
        return float(v)
    if kind is dict:
        if not isinstance(v, dict):
            raise ConfigError(f"config.json: {where}.{key} must be an object")
        return v
    raise AssertionError(kind)


@dataclass(frozen=True)
class KugilixMixer:
    type: str  # "attention" or "lightning"
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0  # attention
    scale: float = 0.0  # attention
    window: Optional[int] = None  # attention: mask.size
    temp_coef: float = 0.0  # attention: q_temp.coef
    temp_every: int = 0  # attention: q_temp.every (0: no temperature)
    decay: tuple = ()  # lightning, one per head

    def to_dict(self) -> dict:
        if self.type == "lightning":
            return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        d: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.temp_every:
            d["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
        return d


@dataclass(frozen=True)
class KugilixLayer:
    mixer: KugilixMixer
    ff: Optional[int]  # None: no feed-forward

    def to_dict(self) -> dict:
        return {"type": self.mixer.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class KugilixConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    canon_taps: Optional[int]  # None: no convolution in front of the mixers
    layers: tuple  # of KugilixLayer
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    architecture: str = "Kugilix"

    # ------------------------------------------------------------------ derived
    def run_order(self) -> list:
        """(layer, whether the embedding output is added right before it) in the order in which layers run."""
        order = [(i, False) for i in range(self.loop_start)]
        for r in range(self.loop_times):
            order += [(i, r > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        order += [(i, False) for i in range(self.loop_stop, len(self.layers))]
        return order

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        for name in ("vocab", "width", "norm_groups"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"config.json: {name} must be > 0, found {getattr(self, name)}")
        if self.width % self.norm_groups:
            raise ConfigError(f"config.json: width {self.width} cannot be normed in {self.norm_groups} equal groups")
        if not (self.norm_eps >= 0.0):
            raise ConfigError(f"config.json: norm.eps must be >= 0, found {self.norm_eps}")
        if self.canon_taps is not None and self.canon_taps < 1:
            raise ConfigError(f"config.json: canon.taps must be >= 1, found {self.canon_taps}")
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        n = len(self.layers)
        if not (0 <= self.loop_start <= self.loop_stop <= n) or self.loop_times < 1:
            raise ConfigError(f"config.json: loop start={self.loop_start} stop={self.loop_stop} times={self.loop_times} "
                              f"does not fit {n} layers")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            if m.heads <= 0 or m.dim <= 0 or m.vdim <= 0:
                raise ConfigError(f"config.json: layers[{i}].mixer sizes must be > 0")
            if m.type == "attention":
                if m.kv_heads <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"config.json: layers[{i}]: {m.heads} heads cannot share {m.kv_heads} kv heads")
                if m.window is not None and m.window <= 0:
                    raise ConfigError(f"config.json: layers[{i}].mixer.mask.size must be > 0")
                if m.temp_every < 0:
                    raise ConfigError(f"config.json: layers[{i}].mixer.q_temp.every must be > 0")
            elif m.type == "lightning":
                if len(m.decay) != m.heads:
                    raise ConfigError(f"config.json: layers[{i}]: {len(m.decay)} decays for {m.heads} heads")
            if layer.ff is not None and layer.ff <= 0:
                raise ConfigError(f"config.json: layers[{i}].mlp.ff must be > 0")

    # --------------------------------------------------------------------- I/O
    @classmethod
    def from_dict(cls, d: dict) -> "KugilixConfig":
        name = d.get("architecture") or (d.get("architectures") or [None])[0]
        if name != "Kugilix":
            raise UnsupportedError(f"architecture {name!r} is not read by KugilixConfig")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, list):
            raise ConfigError("config.json: 'layers' must be a list")
        layers = []
        for i, e in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(e, dict) or not isinstance(e.get("type"), str):
                raise ConfigError(f"config.json: {where} must be an object with a 'type'")
            kind = e["type"]
            m = _of(e, "mixer", dict, where)
            mw = where + ".mixer"
            if kind == "attention":
                mask = _of(m, "mask", dict, mw, required=False)
                temp = _of(m, "q_temp", dict, mw, required=False)
                heads = _of(m, "heads", int, mw)
                mixer = KugilixMixer(
                    "attention", heads, _of(m, "dim", int, mw), _of(m, "vdim", int, mw),
                    kv_heads=_of(m, "kv_heads", int, mw, default=heads, required=False),
                    scale=_of(m, "scale", float, mw),
                    window=None if mask is None else _of(mask, "size", int, mw + ".mask"),
                    temp_coef=0.0 if temp is None else _of(temp, "coef", float, mw + ".q_temp"),
                    temp_every=0 if temp is None else _of(temp, "every", int, mw + ".q_temp"))
            elif kind == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, list) or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
                    raise ConfigError(f"config.json: {mw}.decay must be a list of numbers")
                mixer = KugilixMixer("lightning", _of(m, "heads", int, mw), _of(m, "dim", int, mw), _of(m, "vdim", int, mw),
                                     decay=tuple(float(x) for x in decay))
            else:
                raise UnsupportedError(f"config.json: {where}.type '{kind}' is not a mixer of this design")
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise UnsupportedError(f"config.json: {where}.mlp must be null or of kind 'dense'")
                ff = _of(mlp, "ff", int, where + ".mlp")
            layers.append(KugilixLayer(mixer, ff))
        loop = _of(d, "loop", dict, "the top level", required=False)
        canon = _of(d, "canon", dict, "the top level", required=False)
        norm = _of(d, "norm", dict, "the top level")
        emb = _of(d, "embedding", dict, "the top level", required=False)
        cfg = cls(
            vocab=_of(d, "vocab", int, "the top level"),
            width=_of(d, "width", int, "the top level"),
            embedding_scale=1.0 if emb is None else _of(emb, "scale", float, "embedding", default=1.0, required=False),
            norm_eps=_of(norm, "eps", float, "norm"),
            norm_groups=_of(norm, "groups", int, "norm", default=1, required=False),
            canon_taps=None if canon is None else _of(canon, "taps", int, "canon"),
            layers=tuple(layers),
            loop_start=0 if loop is None else _of(loop, "start", int, "loop"),
            loop_stop=0 if loop is None else _of(loop, "stop", int, "loop"),
            loop_times=1 if loop is None else _of(loop, "times", int, "loop"),
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        d: dict = {
            "architecture": self.architecture,
            "vocab": self.vocab,
            "width": self.width,
            "embedding": {"scale": self.embedding_scale},
            "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
            "layers": [layer.to_dict() for layer in self.layers],
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
        }
        if self.canon_taps is not None:
            d["canon"] = {"taps": self.canon_taps}
        return d

    @classmethod
    def from_json(cls, path: str) -> "KugilixConfig":
        return cls.from_dict(read_config_json(path))
