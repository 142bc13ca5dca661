"""Configuration of the Zasorax decoder (config.json key ``"architecture": "Zasorax"``).

The file is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and a list ``layers`` whose entries give the
layer's ``type`` (which mixer: ``attention`` or ``attention_2``), the mixer's sizes under ``mixer`` and the feed-forward
under ``mlp`` (null: none; ``kind`` ``dense`` with ``ff``, or ``moe`` with ``expert.ff``, ``router.experts`` and
``router.top``).  Every size and every constant that the file gives is read from it; what the design fixes (norms on the
sublayers' results only, the forms of the activations, the pairing of rotated entries, the sinks) is in the parts.  The
number of rows of a layer's distance table is a tensor's shape (``rel``); a file may name it (``bias_rows``) for the
random-weights mode.  A mixer with ``kv_from: j`` has no keys and values of its own and reads those of layer ``j``.
"""

from __future__ import annotations

import dataclasses
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig

MIXERS = ("attention", "attention_2")
FEED_FORWARDS = ("dense", "moe")
DEFAULT_BIAS_ROWS = 32  # what the random-weights mode writes where the file does not say


def _need(where: str, table: Any, keys: tuple[str, ...], optional: tuple[str, ...] = ()) -> dict:
    if not isinstance(table, dict):
        raise ConfigError(f"ZasoraxConfig: {where} must be an object")
    missing = [k for k in keys if k not in table]
    unknown = [k for k in table if k not in keys and k not in optional]
    if missing or unknown:
        parts = ([f"missing keys {sorted(missing)}"] if missing else []) + ([f"unknown keys {sorted(unknown)}"] if unknown else [])
        raise ConfigError(f"ZasoraxConfig: {where}: " + "; ".join(parts))
    return table


def _positive_int(where: str, value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or value <= 0:
        raise ConfigError(f"ZasoraxConfig: {where} must be a positive integer, got {value!r}")
    return int(value)


def _positive(where: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not value > 0:
        raise ConfigError(f"ZasoraxConfig: {where} must be a positive number, got {value!r}")
    return float(value)


@dataclasses.dataclass(frozen=True)
class ZasoraxConfig(ModelConfig):
    vocab: int
    width: int
    layers: list
    norm: dict
    embedding: dict | None = None  # absent: the table's rows enter the stream as they are
    initializer_range: float | None = None  # only read by the random-weights mode
    max_position_embeddings: int | None = None  # longest sequence a request may reach (optional)

    ARCH_NAMES: ClassVar[tuple[str, ...]] = ("Zasorax",)
    IGNORED_KEYS: ClassVar[frozenset[str]] = frozenset({"architecture", "torch_dtype", "dtype"})

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"]) if self.embedding else 1.0

    def to_dict(self) -> dict[str, Any]:
        out = {k: v for k, v in dataclasses.asdict(self).items() if v is not None}
        out["architecture"] = self.ARCH_NAMES[0]
        return out

    def validate(self) -> None:
        _positive_int("vocab", self.vocab)
        _positive_int("width", self.width)
        _positive("norm.eps", _need("norm", self.norm, ("eps",))["eps"])
        if self.embedding is not None:
            _positive("embedding.scale", _need("embedding", self.embedding, ("scale",))["scale"])
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("ZasoraxConfig: layers must be a list with at least one layer")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _need(where, layer, ("type", "mixer"), ("mlp",))
            kind = layer["type"]
            if kind not in MIXERS:
                raise ConfigError(f"ZasoraxConfig: {where}.type {kind!r} is not a mixer of this design (known: {list(MIXERS)})")
            if kind == "attention":
                m = _need(where + ".mixer", layer["mixer"], ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max"),
                          ("kv_from", "bias_rows", "mask"))
                _positive(f"{where}.mixer.bias_max", m["bias_max"])
                if m.get("mask") is not None:  # absent: every earlier key is seen
                    _positive_int(f"{where}.mixer.mask.size", _need(where + ".mixer.mask", m["mask"], ("size",))["size"])
                if m.get("bias_rows") is not None and _positive_int(f"{where}.mixer.bias_rows", m["bias_rows"]) < 2:
                    raise ConfigError(f"ZasoraxConfig: {where}.mixer.bias_rows must be at least 2")
            else:
                m = _need(where + ".mixer", layer["mixer"], ("heads", "kv_heads", "dim", "vdim", "scale", "rot"), ("kv_from",))
                rot = _need(where + ".mixer.rot", m["rot"], ("base", "dims"))
                dims = _positive_int(f"{where}.mixer.rot.dims", rot["dims"])
                _positive(f"{where}.mixer.rot.base", rot["base"])
                if dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"ZasoraxConfig: {where}.mixer.rot.dims ({dims}) must be even and at most dim ({m['dim']})")
                if m["vdim"] % 2:
                    raise ConfigError(f"ZasoraxConfig: {where}.mixer.vdim ({m['vdim']}) must be even: the values turn in pairs")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _positive_int(f"{where}.mixer.{key}", m[key])
            _positive(f"{where}.mixer.scale", m["scale"])
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"ZasoraxConfig: {where}.mixer.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
            source = m.get("kv_from")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                    raise ConfigError(f"ZasoraxConfig: {where}.mixer.kv_from ({source!r}) must name an earlier layer")
                other = self.layers[source]
                if other["mixer"].get("kv_from") is not None:
                    raise ConfigError(f"ZasoraxConfig: {where}.mixer.kv_from names layer {source}, which has no keys and values of its own")
                same = other["type"] == kind and all(other["mixer"][k] == m[k] for k in ("kv_heads", "dim", "vdim"))
                if same and kind == "attention_2":
                    same = other["mixer"]["rot"] == m["rot"]
                if not same:
                    raise ConfigError(f"ZasoraxConfig: {where}.mixer reads the keys and values of layer {source}: type, kv_heads, dim, vdim "
                                      "and rotation must be that layer's")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in FEED_FORWARDS:
                    raise ConfigError(f"ZasoraxConfig: {where}.mlp.kind must be one of {list(FEED_FORWARDS)}")
                if mlp["kind"] == "dense":
                    _positive_int(f"{where}.mlp.ff", _need(where + ".mlp", mlp, ("kind", "ff"))["ff"])
                else:
                    _need(where + ".mlp", mlp, ("kind", "expert", "router"))
                    _positive_int(f"{where}.mlp.expert.ff", _need(where + ".mlp.expert", mlp["expert"], ("ff",))["ff"])
                    r = _need(where + ".mlp.router", mlp["router"], ("experts", "top"))
                    if _positive_int(f"{where}.mlp.router.top", r["top"]) > _positive_int(f"{where}.mlp.router.experts", r["experts"]):
                        raise ConfigError(f"ZasoraxConfig: {where}.mlp.router: {r['top']} of {r['experts']} experts cannot be chosen")
        if self.max_position_embeddings is not None:
            _positive_int("max_position_embeddings", self.max_position_embeddings)
