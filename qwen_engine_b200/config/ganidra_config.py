"""Configuration of the Ganidra design, from the keys of its ``config.json``.

A Ganidra model is a list of layers, each with one of two mixers and an
optional gated feed-forward, of which a run of layers may be passed several
times with the same weights:

    {"architecture": "Ganidra", "vocab": V, "width": W,
     "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "gla" | "parallel", "mixer": {...}, "mlp": null | {"kind": "dense", "ff": F}}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

``gla`` mixer sizes: heads, dim (keys), vdim (values), tau (the decay's root).
``parallel`` mixer: ``left`` (softmax attention: heads, kv_heads, dim, vdim,
scale, mask.size), ``right`` (as ``gla``), ``left_scale``, ``right_scale``.
Every size and constant is read from here; the rank of a decay's low-rank pair
is no key and comes from the stored tensor's shape (``rank``, if a mixer gives
it, is what random weights are drawn with).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .model_config import ConfigError, ModelConfig, _require_int

_MIXERS = ("gla", "parallel")


def _number(name: str, value: Any, positive: bool = True) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {name} must be a number, got {value!r}")
    if positive and not value > 0:
        raise ConfigError(f"config.json: {name} must be positive, got {value}")
    return float(value)


def _check_gla(where: str, m: Any) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    for key in ("heads", "dim", "vdim"):
        _require_int(f"{where}.{key}", m.get(key))
    _number(f"{where}.tau", m.get("tau"))
    if "rank" in m:
        _require_int(f"{where}.rank", m["rank"])


def _check_softmax(where: str, m: Any) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _require_int(f"{where}.{key}", m.get(key))
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
    _number(f"{where}.scale", m.get("scale"))
    mask = m.get("mask")
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}.mask must be an object with 'size'")
    _require_int(f"{where}.mask.size", mask.get("size"))


@dataclass
class GanidraConfig(ModelConfig):
    architecture: ClassVar[str] = "Ganidra"

    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 1e-6
    layers: tuple = ()                  # the config.json entries, checked
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_ids: tuple = field(default_factory=tuple)

    # what the engine asks of every configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "GanidraConfig":
        for key in ("vocab", "width", "layers", "norm", "embedding"):
            if key not in raw:
                raise ConfigError(f"config.json: '{key}' is missing")
        norm, emb = raw["norm"], raw["embedding"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("config.json: norm.eps is missing")
        if not isinstance(emb, dict) or "scale" not in emb:
            raise ConfigError("config.json: embedding.scale is missing")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        loop = raw.get("loop") or {}
        if not isinstance(loop, dict):
            raise ConfigError("config.json: 'loop' must be an object")
        eos = raw.get("eos_token_id")
        eos_all = tuple(int(t) for t in eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))
        cfg = cls(vocab=_require_int("vocab", raw["vocab"]), width=_require_int("width", raw["width"]),
                  embedding_scale=_number("embedding.scale", emb["scale"], positive=False),
                  norm_eps=_number("norm.eps", norm["eps"]),
                  layers=tuple(copy.deepcopy(raw["layers"])),
                  loop_start=_require_int("loop.start", loop.get("start", 0), 0),
                  loop_stop=_require_int("loop.stop", loop.get("stop", 0), 0),
                  loop_times=_require_int("loop.times", loop.get("times", 1), 1),
                  eos_token_ids=eos_all)
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": copy.deepcopy(list(self.layers)),
            "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    def validate(self) -> None:
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: {where} must be an object")
            kind = layer.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design; known: {list(_MIXERS)}")
            m = layer.get("mixer")
            if kind == "gla":
                _check_gla(f"{where}.mixer", m)
            else:
                if not isinstance(m, dict):
                    raise ConfigError(f"config.json: {where}.mixer must be an object")
                _check_softmax(f"{where}.mixer.left", m.get("left"))
                _check_gla(f"{where}.mixer.right", m.get("right"))
                _number(f"{where}.mixer.left_scale", m.get("left_scale"), positive=False)
                _number(f"{where}.mixer.right_scale", m.get("right_scale"), positive=False)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp must be null or a 'dense' feed-forward, got {mlp!r}")
                _require_int(f"{where}.mlp.ff", mlp.get("ff"))
        n = len(self.layers)
        if not (0 <= self.loop_start <= self.loop_stop <= n) and (self.loop_start or self.loop_stop):
            raise ConfigError(f"config.json: loop {self.loop_start}..{self.loop_stop} does not lie within the {n} layers")

    def layer_runs(self) -> list[tuple[int, bool]]:
        """(layer, whether the embedding output is added before it) in the order of running: the layers
        loop_start .. loop_stop-1 run loop_times times in a row; every pass but the first starts from the
        stream plus the embedding output."""
        n = len(self.layers)
        a, b, times = self.loop_start, self.loop_stop, self.loop_times
        if times <= 1 or b <= a:
            return [(i, False) for i in range(n)]
        runs = [(i, False) for i in range(a)]
        for t in range(times):
            runs += [(i, t > 0 and i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, n)]
