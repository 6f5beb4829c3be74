"""Configuration of the Besavik design, from the keys of its ``config.json``.

A Besavik model is a list of layers, each with one of three mixers and an
optional feed-forward that is dense or a mixture of routed experts:

    {"architecture": "Besavik", "vocab": V, "width": W, "logit_scale": s, "norm": {"eps": e},
     "layers": [{"type": "latent_attention" | "lightning" | "channel_delta", "mixer": {...},
                 "mlp": null | {"kind": "dense", "ff": F, "limit": L}
                             | {"kind": "moe", "expert": {"ff": F, "limit": L}, "router": {"experts": E, "top": k}}}, ...]}

Mixer sizes:
``latent_attention``: heads, dim (unrotated query/key channels per head), rot_dim (rotated ones), vdim, kv_rank,
q_rank, scale, rot {base, dims}.
``lightning``: heads, dim, vdim, decay (one number per head).
``channel_delta``: heads, kv_heads, dim, vdim, conv (taps of the short convolution).
Every size and constant is read from here; the ranks of the delta mixer's low-rank pairs are no keys and come from the
stored tensors' shapes (``rank``, if a mixer gives it, is what random weights are drawn with).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .ganidra_config import _number
from .model_config import ConfigError, ModelConfig, _require_int

_MIXERS = ("latent_attention", "lightning", "channel_delta")


def _check_mixer(where: str, kind: str, m: Any) -> None:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    if kind == "latent_attention":
        for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
            _require_int(f"{where}.{key}", m.get(key))
        _number(f"{where}.scale", m.get("scale"))
        rot = m.get("rot")
        if not isinstance(rot, dict):
            raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims'")
        _number(f"{where}.rot.base", rot.get("base"))
        dims = _require_int(f"{where}.rot.dims", rot.get("dims"), 0)
        if dims % 2 or dims > m["rot_dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims ({dims}) must be even and at most rot_dim ({m['rot_dim']})")
    elif kind == "lightning":
        for key in ("heads", "dim", "vdim"):
            _require_int(f"{where}.{key}", m.get(key))
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != m["heads"]:
            raise ConfigError(f"config.json: {where}.decay must list one number per head")
        for i, d in enumerate(decay):
            _number(f"{where}.decay[{i}]", d, positive=False)
    else:
        for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
            _require_int(f"{where}.{key}", m.get(key))
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"config.json: {where}.heads ({m['heads']}) must be a multiple of kv_heads ({m['kv_heads']})")
        if "rank" in m:
            _require_int(f"{where}.rank", m["rank"])


def _check_mlp(where: str, mlp: Any) -> None:
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where} must be null, a 'dense' feed-forward or a 'moe' one, got {mlp!r}")
    if mlp["kind"] == "dense":
        _require_int(f"{where}.ff", mlp.get("ff"))
        _number(f"{where}.limit", mlp.get("limit"))
        return
    expert, router = mlp.get("expert"), mlp.get("router")
    if not isinstance(expert, dict) or not isinstance(router, dict):
        raise ConfigError(f"config.json: {where} needs 'expert' and 'router' objects")
    _require_int(f"{where}.expert.ff", expert.get("ff"))
    _number(f"{where}.expert.limit", expert.get("limit"))
    experts = _require_int(f"{where}.router.experts", router.get("experts"))
    top = _require_int(f"{where}.router.top", router.get("top"))
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top ({top}) exceeds its experts ({experts})")


@dataclass
class BesavikConfig(ModelConfig):
    architecture: ClassVar[str] = "Besavik"

    vocab: int = 0
    width: int = 0
    logit_scale: float = 1.0
    norm_eps: float = 1e-6
    layers: tuple = ()                  # the config.json entries, checked
    eos_token_ids: tuple = field(default_factory=tuple)

    # what the engine asks of every configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "BesavikConfig":
        for key in ("vocab", "width", "layers", "norm", "logit_scale"):
            if key not in raw:
                raise ConfigError(f"config.json: '{key}' is missing")
        norm = raw["norm"]
        if not isinstance(norm, dict) or "eps" not in norm:
            raise ConfigError("config.json: norm.eps is missing")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        eos = raw.get("eos_token_id")
        eos_all = tuple(int(t) for t in eos) if isinstance(eos, list) else (() if eos is None else (int(eos),))
        cfg = cls(vocab=_require_int("vocab", raw["vocab"]), width=_require_int("width", raw["width"]),
                  logit_scale=_number("logit_scale", raw["logit_scale"], positive=False),
                  norm_eps=_number("norm.eps", norm["eps"]), layers=tuple(copy.deepcopy(raw["layers"])),
                  eos_token_ids=eos_all)
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
                               "layers": copy.deepcopy(list(self.layers))}
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
            _check_mixer(f"{where}.mixer", kind, layer.get("mixer"))
            _check_mlp(f"{where}.mlp", layer.get("mlp"))
