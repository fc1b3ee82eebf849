"""Configuration of the Zetizen design: a list of layers, each an attention mixer beside an optional routed feed-forward.

``config.json`` of this design is nested::

    {"architecture": "Zetizen", "vocab": V, "width": D, "logit_scale": s, "norm": {"eps": e},
     "layers": [{"type": "attention" | "attention_2" | "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

Mixer sizes and constants:

``attention``         ``heads, kv_heads, dim, vdim, scale``; optional ``softcap`` and ``bias_max`` (with it the layer has a
                      table of biases by distance whose row count is the checkpoint's; the optional key ``bias_rows``
                      exists only so that random weights can be drawn from a configuration alone).
``attention_2``       ``heads, kv_heads, dim, vdim, scale`` (``vdim = dim``: the values are the keys); optional ``softcap``,
                      ``mask: {"size"}`` (chunks of visible keys) and ``rot: {"dims", "base", "scaling": {"factor",
                      "original", "fast", "slow"}}`` (``scaling`` optional).
``latent_attention``  ``heads, dim, rot_dim, vdim, kv_rank, q_rank, scale`` and ``rot: {"dims" (= rot_dim), "base", "scaling"}``.

Feed-forward: ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}, "shared": {"ff"}}``; ``shared`` may be
absent (no shared expert). The design has no position limit and no end-of-sequence token.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .model_config import ConfigError, ModelConfig, _take

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim"),
    "attention_2": ("heads", "kv_heads", "dim", "vdim"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"),
}


@dataclass(frozen=True)
class ZetizenConfig(ModelConfig):
    norm_eps: float = 0.0
    logit_scale: float = 1.0
    layers: tuple[dict[str, Any], ...] = field(default_factory=tuple)

    ARCHITECTURE: ClassVar[str] = "Zetizen"
    MODEL_TYPE: ClassVar[str] = "zetizen"

    @classmethod
    def from_json_dict(cls, raw: dict[str, Any]) -> "ZetizenConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json key 'norm' must be an object")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        config = cls(
            architecture=cls.ARCHITECTURE,
            vocab_size=_take(raw, "vocab", int),
            hidden_size=_take(raw, "width", int),
            num_hidden_layers=len(layers),
            max_position_embeddings=cls.MAX_POSITIONS,
            eos_token_ids=(),
            norm_eps=_take(norm, "eps", float),
            logit_scale=_take(raw, "logit_scale", float, 1.0),
            layers=tuple(copy.deepcopy(layer) for layer in layers),
        )
        config.validate()
        return config

    def validate(self) -> None:
        super().validate()
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0):
            raise ConfigError(f"norm.eps={self.norm_eps} must be finite and positive")
        if not (math.isfinite(self.logit_scale) and self.logit_scale > 0):
            raise ConfigError(f"logit_scale={self.logit_scale} must be finite and positive")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_KEYS:
                raise ConfigError(f"{where}.type must be one of {sorted(MIXER_KEYS)}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            for key in MIXER_KEYS[layer["type"]]:
                if _take(mixer, key, int) <= 0:
                    raise ConfigError(f"{where}.mixer.{key} must be positive")
            if not _take(mixer, "scale", float) > 0:
                raise ConfigError(f"{where}.mixer.scale must be positive")
            softcap = _take(mixer, "softcap", float, None)
            if softcap is not None and not softcap > 0:
                raise ConfigError(f"{where}.mixer.softcap must be positive")
            kind = layer["type"]
            if kind != "latent_attention" and mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"{where}.mixer: heads={mixer['heads']} is not a multiple of kv_heads={mixer['kv_heads']}")
            if kind == "attention":
                reach = _take(mixer, "bias_max", int, None)
                rows = _take(mixer, "bias_rows", int, None)
                if reach is not None and reach < 2:
                    raise ConfigError(f"{where}.mixer.bias_max must be at least 2")
                if rows is not None and (reach is None or rows < 2 or reach <= rows // 2):
                    raise ConfigError(f"{where}.mixer.bias_rows={rows} does not fit bias_max={reach}")
            if kind == "attention_2":
                if mixer["vdim"] != mixer["dim"]:
                    raise ConfigError(f"{where}.mixer: the values are the keys, so vdim={mixer['vdim']} must equal dim={mixer['dim']}")
                mask = mixer.get("mask")
                if mask is not None and (not isinstance(mask, dict) or _take(mask, "size", int) <= 0):
                    raise ConfigError(f"{where}.mixer.mask.size must be positive")
                if mixer.get("rot") is not None:
                    self._validate_rot(mixer["rot"], mixer["dim"], where + ".mixer.rot")
            if kind == "latent_attention":
                if softcap is not None:
                    raise ConfigError(f"{where}.mixer.softcap: attention over latents has no soft cap")
                self._validate_rot(mixer.get("rot"), mixer["rot_dim"], where + ".mixer.rot")
                if mixer["rot"]["dims"] != mixer["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must equal rot_dim: the whole shared key part is rotated")
            mlp = layer.get("mlp")
            if mlp is not None:
                self._validate_mlp(mlp, where + ".mlp")

    @staticmethod
    def _validate_rot(rot: Any, limit: int, where: str) -> None:
        if not isinstance(rot, dict):
            raise ConfigError(f"{where} must be an object")
        dims = _take(rot, "dims", int)
        if dims % 2 or not 0 <= dims <= limit or not _take(rot, "base", float) > 1:
            raise ConfigError(f"{where}: dims must be even and at most {limit}, base above 1")
        scaling = rot.get("scaling")
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{where}.scaling must be an object")
            for key in ("factor", "original", "fast", "slow"):
                if not _take(scaling, key, float) > 0:
                    raise ConfigError(f"{where}.scaling.{key} must be positive")

    def _validate_mlp(self, mlp: Any, where: str) -> None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
            raise ConfigError(f"{where}.kind must be 'moe' (or mlp null)")
        for name in ("expert", "shared"):
            part = mlp.get(name)
            if part is None and name == "shared":
                continue
            if not isinstance(part, dict) or not 0 < _take(part, "ff", int) <= self.MAX_INTERMEDIATE:
                raise ConfigError(f"{where}.{name}.ff is missing or out of range")
        router = mlp.get("router")
        if not isinstance(router, dict):
            raise ConfigError(f"{where}.router must be an object")
        experts, top = _take(router, "experts", int), _take(router, "top", int)
        if not 0 < top <= experts:
            raise ConfigError(f"{where}.router: top={top} of {experts} experts")

    def to_json_dict(self) -> dict[str, Any]:
        return {
            "architecture": self.architecture,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
