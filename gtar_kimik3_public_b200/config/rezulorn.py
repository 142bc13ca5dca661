"""Configuration of the Rezulorn decoder (config.json key ``"architecture": "Rezulorn"``).

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``canon.taps`` (taps of the convolutions in front of every
sublayer; absent or 0: none), ``residual_mult`` (the constant on every branch), ``logit_scale`` and a list ``layers``
whose entries give the layer's ``type`` (which mixer: ``lightning``, ``attention`` or ``parallel``), the mixer's sizes
under ``mixer`` and the feed-forward under ``mlp`` (null: none).  Every size and every constant that the file gives is
read from it; what the design fixes (the norms' form, SiLU, the pairing of the rotation, which mixer norms what) is in
the parts and in the builder.
"""

from __future__ import annotations

import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("lightning", "attention", "parallel")
FEED_FORWARDS = ("dense",)
_NAME = "RezulornConfig"


def _need(where: str, table: Any, keys: tuple[str, ...], optional: tuple[str, ...] = ()) -> dict:
    if not isinstance(table, dict):
        raise ConfigError(f"{_NAME}: {where} must be an object")
    missing = [k for k in keys if k not in table]
    unknown = [k for k in table if k not in keys and k not in optional]
    if missing or unknown:
        parts = ([f"missing keys {sorted(missing)}"] if missing else []) + ([f"unknown keys {sorted(unknown)}"] if unknown else [])
        raise ConfigError(f"{_NAME}: {where}: " + "; ".join(parts))
    return table


def _int(where: str, value: Any, least: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or value < least:
        raise ConfigError(f"{_NAME}: {where} must be an integer of at least {least}, got {value!r}")
    return int(value)


def _number(where: str, value: Any, positive: bool = True) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or (positive and not value > 0):
        raise ConfigError(f"{_NAME}: {where} must be a {'positive ' if positive else ''}number, got {value!r}")
    return float(value)


def _check_rot(where: str, rot: Any, dim: int) -> None:
    if rot is None:
        return
    _need(where, rot, ("base", "dims"), ("scaling",))
    dims = _int(where + ".dims", rot["dims"])
    _number(where + ".base", rot["base"])
    if dims % 2 or dims > dim:
        raise ConfigError(f"{_NAME}: {where}.dims ({dims}) must be even and at most dim ({dim})")
    if rot.get("scaling") is not None:
        _number(where + ".scaling.factor", _need(where + ".scaling", rot["scaling"], ("factor",))["factor"])


def _check_softmax_kind(where: str, m: Any) -> None:
    """An attention mixer's sizes (both the plain one and the left of a pair)."""
    _need(where, m, ("heads", "kv_heads", "dim", "vdim", "scale"), ("rot", "mask"))
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _int(f"{where}.{key}", m[key])
    _number(where + ".scale", m["scale"])
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"{_NAME}: {where}.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
    _check_rot(where + ".rot", m.get("rot"), m["dim"])
    if m.get("mask") is not None:
        mask = _need(where + ".mask", m["mask"], ("size",), ("keep_first",))
        _int(where + ".mask.size", mask["size"])
        if mask.get("keep_first") is not None:
            _int(where + ".mask.keep_first", mask["keep_first"], least=0)


def _check_decay_kind(where: str, m: Any) -> None:
    """A linear-attention mixer's sizes (the lightning one and the right of a pair)."""
    _need(where, m, ("heads", "dim", "vdim", "decay"), ("rot",))
    for key in ("heads", "dim", "vdim"):
        _int(f"{where}.{key}", m[key])
    if m["dim"] > 256:
        raise ConfigError(f"{_NAME}: {where}.dim ({m['dim']}) must be at most 256 (a state's rows are held by eight lanes)")
    decay = m["decay"]
    if not isinstance(decay, list) or len(decay) != m["heads"]:
        raise ConfigError(f"{_NAME}: {where}.decay must list one number per head ({m['heads']})")
    for i, g in enumerate(decay):
        _number(f"{where}.decay[{i}]", g, positive=False)
    _check_rot(where + ".rot", m.get("rot"), m["dim"])


@dataclasses.dataclass(frozen=True)
class RezulornConfig(ModelConfig):
    vocab: int
    width: int
    layers: list
    norm: dict
    canon: dict | None = None  # absent: no convolution in front of the sublayers
    residual_mult: float = 1.0
    logit_scale: float = 1.0
    initializer_range: float | None = None  # only read by the random-weights mode
    max_position_embeddings: int | None = None  # longest sequence a request may reach (optional)

    ARCH_NAMES: ClassVar[tuple[str, ...]] = ("Rezulorn",)
    IGNORED_KEYS: ClassVar[frozenset[str]] = frozenset({"architecture", "torch_dtype", "dtype"})

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def taps(self) -> int:
        return int(self.canon["taps"]) if self.canon else 0

    def to_dict(self) -> dict[str, Any]:
        out = {k: v for k, v in dataclasses.asdict(self).items() if v is not None}
        out["architecture"] = self.ARCH_NAMES[0]
        return out

    def validate(self) -> None:
        _int("vocab", self.vocab)
        _int("width", self.width)
        _number("norm.eps", _need("norm", self.norm, ("eps",))["eps"])
        if self.canon is not None:
            _int("canon.taps", _need("canon", self.canon, ("taps",))["taps"], least=0)
        _number("residual_mult", self.residual_mult, positive=False)
        _number("logit_scale", self.logit_scale, positive=False)
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError(f"{_NAME}: layers must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(where, layer, ("type", "mixer"), ("mlp",))
            kind = layer["type"]
            if kind not in MIXERS:
                raise ConfigError(f"{_NAME}: {where}.type {kind!r} is not a mixer of this design (known: {list(MIXERS)})")
            m = layer["mixer"]
            if kind == "lightning":
                _check_decay_kind(where + ".mixer", m)
            elif kind == "attention":
                _check_softmax_kind(where + ".mixer", m)
            else:
                _need(where + ".mixer", m, ("left", "right"), ("left_scale", "right_scale"))
                _check_softmax_kind(where + ".mixer.left", m["left"])
                _check_decay_kind(where + ".mixer.right", m["right"])
                for key in ("left_scale", "right_scale"):
                    if m.get(key) is not None:
                        _number(f"{where}.mixer.{key}", m[key], positive=False)
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(where + ".mlp", mlp, ("kind", "ff"))
                if mlp["kind"] not in FEED_FORWARDS:
                    raise ConfigError(f"{_NAME}: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design "
                                      f"(known: {list(FEED_FORWARDS)})")
                _int(where + ".mlp.ff", mlp["ff"])
        if self.max_position_embeddings is not None:
            _int("max_position_embeddings", self.max_position_embeddings)
