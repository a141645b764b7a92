"""Configuration of the Pikadra design: latent attention, parallel sub-layers, a looped stretch of layers.

``config.json`` is nested: ``layers`` is a list of objects, each with ``type`` (which mixer), ``mixer`` (its sizes
and constants) and ``mlp`` (the feed-forward: ``kind`` "dense" with ``ff``, or "moe" with ``expert.ff``,
``router.experts`` / ``router.top`` and optionally ``shared.ff``; or null).  Model-wide keys: ``vocab``, ``width``,
``norm.eps``, ``embedding.scale``, ``logit_scale``, ``logit_softcap`` and ``loop`` (``start``, ``stop``, ``times``:
the layers start..stop-1 run ``times`` times in a row with the same weights).  The file names the design with the
single string ``architecture``.  Every size and constant is read from the file; what the file does not mention
does not exist (no loop, no scale, no cap).
"""
from __future__ import annotations

import copy
import dataclasses
from typing import Any, ClassVar, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig, register_config

MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale"),
}


def _need(obj: Any, key: str, where: str, kinds=(int, float)) -> Any:
    if not isinstance(obj, dict) or key not in obj:
        raise ConfigError(f"Pikadra: config.json lacks '{where}{key}'")
    v = obj[key]
    if isinstance(v, bool) or not isinstance(v, kinds):
        raise ConfigError(f"Pikadra: '{where}{key}' has the wrong type ({v!r})")
    return v


def _positive_int(obj: Any, key: str, where: str) -> int:
    v = _need(obj, key, where, int)
    if v <= 0:
        raise ConfigError(f"Pikadra: '{where}{key}' must be a positive integer")
    return v


@register_config
@dataclasses.dataclass(frozen=True)
class PikadraConfig(ModelConfig):
    ARCHITECTURE: ClassVar[str] = "Pikadra"

    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm_eps: float
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: float = 0.0                      # 0: the logits are not capped
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "PikadraConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("Pikadra: config.json lacks 'layers' (a list with one object per layer)")
        loop = None
        if raw.get("loop"):
            lp = raw["loop"]
            loop = (_need(lp, "start", "loop.", int), _need(lp, "stop", "loop.", int), _need(lp, "times", "loop.", int))
        cfg = cls(vocab=_need(raw, "vocab", "", int), width=_need(raw, "width", "", int),
                  layers=tuple(copy.deepcopy(layers)),
                  norm_eps=float(_need(raw.get("norm"), "eps", "norm.")),
                  embedding_scale=float(_need(raw["embedding"], "scale", "embedding.")) if raw.get("embedding") else 1.0,
                  logit_scale=float(_need(raw, "logit_scale", "")) if raw.get("logit_scale") is not None else 1.0,
                  logit_softcap=float(_need(raw, "logit_softcap", "")) if raw.get("logit_softcap") is not None else 0.0,
                  loop=loop)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                               "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def layer_runs(self):
        """The order in which layers run: [(layer index, pass number or None, whether a pass opens here)]."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, None, False) for i in range(start)]
        for t in range(times):
            runs += [(i, t, i == start) for i in range(start, stop)]
        return runs + [(i, None, False) for i in range(stop, n)]

    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("Pikadra: 'vocab' and 'width' must be positive")
        if self.norm_eps <= 0:
            raise ConfigError("Pikadra: 'norm.eps' must be positive")
        if self.logit_softcap < 0:
            raise ConfigError("Pikadra: 'logit_softcap' must not be negative")
        if self.loop is not None:
            start, stop, times = self.loop
            if not (0 <= start < stop <= len(self.layers)) or times < 1:
                raise ConfigError("Pikadra: 'loop' needs 0 <= start < stop <= number of layers and times >= 1")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in MIXER_KEYS:
                raise ConfigError(f"Pikadra: '{where}type' = {kind!r} is not a known mixer "
                                  f"({', '.join(sorted(MIXER_KEYS))})")
            mx = layer.get("mixer")
            for key in MIXER_KEYS[kind]:
                _need(mx, key, where + "mixer.")
            for key in ("heads", "dim", "vdim", "kv_rank", "q_rank"):
                _positive_int(mx, key, where + "mixer.")
            if _need(mx, "rot_dim", where + "mixer.", int) < 0:
                raise ConfigError(f"Pikadra: '{where}mixer.rot_dim' must not be negative")
            if mx["rot_dim"]:
                rot = mx.get("rot")
                dims = _need(rot, "dims", where + "mixer.rot.", int)
                _need(rot, "base", where + "mixer.rot.")
                if dims < 0 or dims % 2 or dims > mx["rot_dim"]:
                    raise ConfigError(f"Pikadra: '{where}mixer.rot.dims' must be even and at most 'rot_dim'")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _positive_int(mlp, "ff", where + "mlp.")
            elif mlp.get("kind") == "moe":
                _positive_int(mlp.get("expert"), "ff", where + "mlp.expert.")
                n = _positive_int(mlp.get("router"), "experts", where + "mlp.router.")
                if _positive_int(mlp.get("router"), "top", where + "mlp.router.") > n:
                    raise ConfigError(f"Pikadra: '{where}mlp.router.top' exceeds the number of experts")
                if mlp.get("shared"):
                    _positive_int(mlp["shared"], "ff", where + "mlp.shared.")
            else:
                raise ConfigError(f"Pikadra: '{where}mlp.kind' = {mlp.get('kind')!r} is not known (dense, moe)")
