"""Configuration of the Fanidra design: a decoder whose layers are listed one by one.

``config.json`` is nested: ``layers`` is a list of objects, each with ``type`` (which mixer), ``mixer`` (its
sizes and constants) and ``mlp`` (the feed-forward, or null); the model-wide keys are ``vocab``, ``width``,
``norm.eps``, ``residual_mult``, ``embedding.scale`` and ``canon.taps`` (the taps of the convolution in front of
every mixer).  The file names the design with the single string ``architecture``.  Every size and constant is
read from the file; nothing about a particular model is assumed here.
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar, Dict, Tuple

from .base import ConfigError, ModelConfig, register_config

MIXER_KEYS = {
    "attention": {"required": ("heads", "dim", "vdim", "conv", "scale", "diff"),
                  "optional": ("kv_heads", "mask", "rot", "softcap")},
    "hgrn2": {"required": ("heads", "dim", "vdim"), "optional": ()},
}


def _need(obj: Any, key: str, where: str, kinds=(int, float)) -> Any:
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"Fanidra: config.json lacks '{where}{key}'")
    v = obj[key]
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"Fanidra: '{where}{key}' has the wrong type ({v!r})")
    return v


@register_config
@dataclasses.dataclass(frozen=True)
class FanidraConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "Fanidra"

    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    residual_mult: float = 1.0
    embedding_scale: float = 1.0
    canon_taps: int = 0          # 0: no convolution in front of the mixers

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FanidraConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Fanidra: config.json lacks 'layers' (a list with one object per layer)")
        cfg = cls(vocab=_need(raw, "vocab", "", int), width=_need(raw, "width", "", int),
                  layers=tuple(copy.deepcopy(layers)),
                  norm_eps=float(_need(raw.get("norm"), "eps", "norm.")),
                  residual_mult=float(raw.get("residual_mult", 1.0)),
                  embedding_scale=float(_need(raw["embedding"], "scale", "embedding.")) if "embedding" in raw else 1.0,
                  canon_taps=_need(raw["canon"], "taps", "canon.", int) if raw.get("canon") else 0)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
                               "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale}}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        return out

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Fanidra: 'vocab' and 'width' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("Fanidra: 'norm.eps' must be positive")
        if self.canon_taps < 0:
            raise ConfigError("Fanidra: 'canon.taps' must not be negative")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in MIXER_KEYS:
                raise ConfigError(f"Fanidra: '{where}type' = {kind!r} is not a known mixer "
                                  f"({', '.join(sorted(MIXER_KEYS))})")
            mx = layer.get("mixer")
            for key in MIXER_KEYS[kind]["required"]:
                _need(mx, key, where + "mixer.")
            for key in ("heads", "dim", "vdim"):
                if not isinstance(mx[key], int) or mx[key] <= 0:
                    raise ConfigError(f"Fanidra: '{where}mixer.{key}' must be a positive integer")
            if kind == "attention":
                g = mx.get("kv_heads", mx["heads"])
                if not isinstance(g, int) or g <= 0 or mx["heads"] % g:
                    raise ConfigError(f"Fanidra: '{where}mixer.kv_heads' must divide 'heads'")
                if not isinstance(mx["conv"], int) or mx["conv"] < 1:
                    raise ConfigError(f"Fanidra: '{where}mixer.conv' must be a positive integer")
                if mx.get("rot"):
                    dims = _need(mx["rot"], "dims", where + "mixer.rot.", int)
                    _need(mx["rot"], "base", where + "mixer.rot.")
                    if dims < 0 or dims % 2 or dims > mx["dim"]:
                        raise ConfigError(f"Fanidra: '{where}mixer.rot.dims' must be even and at most 'dim'")
                if mx.get("mask"):
                    if _need(mx["mask"], "size", where + "mixer.mask.", int) <= 0:
                        raise ConfigError(f"Fanidra: '{where}mixer.mask.size' must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"Fanidra: '{where}mlp.kind' = {mlp.get('kind')!r} is not known (dense)")
                if _need(mlp, "ff", where + "mlp.", int) <= 0:
                    raise ConfigError(f"Fanidra: '{where}mlp.ff' must be positive")
