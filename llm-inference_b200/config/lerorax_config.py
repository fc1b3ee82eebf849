"""Configuration of the Lerorax design: a list of layers, each with a mixer and a feed-forward.

``config.json`` of this design is nested::

    {"architecture": "Lerorax", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "mingru" | "parallel", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F, "limit": c} | null,
                 "weights_of": j (optional)}, ...]}

Mixer sizes: ``mingru``: ``width``; ``parallel``: ``left`` (attention: ``heads, kv_heads, dim, vdim,
conv, scale`` and optionally ``rot: {base, dims, scaling: {factor, low, high, original} (optional)}``)
and ``right`` (delta rule: ``heads, dim``). A layer with ``weights_of: j`` runs layer ``j``'s tensors
against a cache and state of its own. Absent keys mean absent mechanisms: no ``embedding.bigram`` is a
plain table, no ``rot`` (or ``dims`` 0) no rotation, no ``scaling`` plain frequencies, ``mlp: null`` no
feed-forward. The inner size of the delta rule's decay pair is the checkpoint's tensor shape; the
optional key ``right.decay_rank`` exists only so that random weights can be drawn from a configuration
alone. The design has no position limit and no end-of-sequence token.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .model_config import ConfigError, ModelConfig, _take

MIXER_TYPES = ("mingru", "parallel")


@dataclass(frozen=True)
class LeroraxConfig(ModelConfig):
    norm_eps: float = 0.0
    bigram: dict[str, int] | None = None
    layers: tuple[dict[str, Any], ...] = field(default_factory=tuple)

    ARCHITECTURE: ClassVar[str] = "Lerorax"
    MODEL_TYPE: ClassVar[str] = "lerorax"

    @classmethod
    def from_json_dict(cls, raw: dict[str, Any]) -> "LeroraxConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json key 'layers' must be a non-empty list")
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json key 'norm' must be an object")
        embedding = raw.get("embedding") or {}
        if not isinstance(embedding, dict):
            raise ConfigError("config.json key 'embedding' must be an object")
        bigram = embedding.get("bigram")
        if bigram is not None:
            if not isinstance(bigram, dict):
                raise ConfigError("config.json key 'embedding.bigram' must be an object")
            bigram = {key: _take(bigram, key, int) for key in ("buckets", "mul_prev", "mul_cur")}
        config = cls(
            architecture=cls.ARCHITECTURE,
            vocab_size=_take(raw, "vocab", int),
            hidden_size=_take(raw, "width", int),
            num_hidden_layers=len(layers),
            max_position_embeddings=cls.MAX_POSITIONS,
            eos_token_ids=(),
            norm_eps=_take(norm, "eps", float),
            bigram=bigram,
            layers=tuple(copy.deepcopy(layer) for layer in layers),
        )
        config.validate()
        return config

    def owner(self, index: int) -> int:
        """The layer whose tensors layer ``index`` runs (itself unless it names another)."""
        seen = set()
        while self.layers[index].get("weights_of") is not None:
            if index in seen:
                raise ConfigError(f"layers[{index}].weights_of runs in a circle")
            seen.add(index)
            index = int(self.layers[index]["weights_of"])
        return index

    def validate(self) -> None:
        super().validate()
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0):
            raise ConfigError(f"norm.eps={self.norm_eps} must be finite and positive")
        if self.bigram is not None:
            if self.bigram["buckets"] <= 0 or self.bigram["mul_prev"] < 0 or self.bigram["mul_cur"] < 0:
                raise ConfigError("embedding.bigram: buckets must be positive and the multipliers not negative")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"{where}.type must be one of {sorted(MIXER_TYPES)}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            if layer["type"] == "mingru":
                if _take(mixer, "width", int) <= 0:
                    raise ConfigError(f"{where}.mixer.width must be positive")
            else:
                left, right = mixer.get("left"), mixer.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    raise ConfigError(f"{where}.mixer needs the objects 'left' and 'right'")
                for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    if _take(left, key, int) <= 0:
                        raise ConfigError(f"{where}.mixer.left.{key} must be positive")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.left: heads={left['heads']} is not a multiple of kv_heads={left['kv_heads']}")
                _take(left, "scale", float)
                rot = left.get("rot")
                if rot is not None:
                    if not isinstance(rot, dict):
                        raise ConfigError(f"{where}.mixer.left.rot must be an object")
                    dims = _take(rot, "dims", int)
                    if dims % 2 or not 0 <= dims <= left["dim"] or _take(rot, "base", float) <= 0:
                        raise ConfigError(f"{where}.mixer.left.rot: dims must be even and at most dim, base positive")
                    scaling = rot.get("scaling")
                    if scaling is not None:
                        if not isinstance(scaling, dict):
                            raise ConfigError(f"{where}.mixer.left.rot.scaling must be an object")
                        values = [_take(scaling, key, float) for key in ("factor", "low", "high", "original")]
                        if min(values) <= 0 or scaling["high"] == scaling["low"]:
                            raise ConfigError(f"{where}.mixer.left.rot.scaling: positive numbers with high != low")
                for key in ("heads", "dim"):
                    if _take(right, key, int) <= 0:
                        raise ConfigError(f"{where}.mixer.right.{key} must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"{where}.mlp.kind must be 'dense' (or mlp null)")
                if not 0 < _take(mlp, "ff", int) <= self.MAX_INTERMEDIATE:
                    raise ConfigError(f"{where}.mlp.ff is out of range")
                if not _take(mlp, "limit", float) > 0:
                    raise ConfigError(f"{where}.mlp.limit must be positive")
            other = layer.get("weights_of")
            if other is not None:
                if isinstance(other, bool) or not isinstance(other, int) or not 0 <= other < len(self.layers) or other == index:
                    raise ConfigError(f"{where}.weights_of must name another layer")
                target = self.layers[other]
                if not isinstance(target, dict) or target.get("type") != layer["type"] or target.get("mixer") != mixer or target.get("mlp") != mlp:
                    raise ConfigError(f"{where} runs layer {other}'s tensors, so its type, mixer and mlp must equal that layer's")
        for index in range(len(self.layers)):
            self.owner(index)

    def to_json_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture,
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "norm": {"eps": self.norm_eps},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
        }
        if self.bigram is not None:
            out["embedding"] = {"bigram": dict(self.bigram)}
        return out
