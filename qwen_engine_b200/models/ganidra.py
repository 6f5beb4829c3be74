"""Ganidra as a layout of parts.

Layers of two kinds, in the order config.json gives: ``gla`` (a gated-linear-
attention mixer) and ``parallel`` (windowed softmax attention with a distance
bias and an output gate beside a gated-linear-attention mixer, their outputs
weighted and summed); each with an optional gated feed-forward with the tanh
form of gelu.  Norms are RMS norms whose stored weight sits around zero (the
scale is 1 + w).  The embedding output is the table's row times a scale; the
head is the table itself.  A run of layers may be passed several times with
the same weights: every pass has cache slots of its own, and every pass but
the first starts from the stream plus the embedding output.

Tensor names: ``embed``, ``final.norm``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.*`` (``.left.*`` / ``.right.*`` in a parallel layer), ``l<i>.mlp.*``.
"""
from __future__ import annotations

from ..config.ganidra_config import GanidraConfig
from ..parts.base import PartSpec
from .decoder import LayerSpec, ModelLayout, PlanEntry

_SOFTMAX_NAMES = dict(q="q", k="k", v="v", out="o", gate="g", q_norm="q.norm", k_norm="k.norm")


def distance_slopes(num_heads: int) -> tuple:
    """The design's distance bias: head h of H takes 2^(-8 (h + 1) / H) per token of distance."""
    return tuple(2.0 ** (-8.0 * (h + 1) / num_heads) for h in range(num_heads))


def _gla(cfg: GanidraConfig, m: dict) -> PartSpec:
    return PartSpec("gated_linear_attention", dict(
        hidden_size=cfg.width, num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
        decay_tau=m["tau"], norm_eps=cfg.norm_eps, decay_rank=m.get("rank")))


def _softmax(cfg: GanidraConfig, m: dict) -> PartSpec:
    return PartSpec("gqa_attention", dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
        value_dim=m["vdim"], scale=m["scale"], qk_norm_eps=cfg.norm_eps, position_encoding=None,
        window=m["mask"]["size"], distance_slopes=distance_slopes(m["heads"]), output_gate="sigmoid",
        names=_SOFTMAX_NAMES))


def _mixer(cfg: GanidraConfig, layer: dict) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "gla":
        return _gla(cfg, m)
    return PartSpec("parallel_mixers", dict(
        branches=(_softmax(cfg, m["left"]), _gla(cfg, m["right"])),
        scales=(m["left_scale"], m["right_scale"]), prefixes=("left.", "right.")))


def ganidra_layout(cfg: GanidraConfig) -> ModelLayout:
    norm = PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name="", weight_offset=1.0))
    layers = []
    for i, layer in enumerate(cfg.layers):
        mlp = layer.get("mlp")
        ffn = None if mlp is None else PartSpec("swiglu", dict(
            hidden_size=cfg.width, intermediate_size=mlp["ff"], activation="gelu_tanh", names=("gate", "up", "down")))
        block = PartSpec("pre_norm", dict(hidden_size=cfg.width, mixer=_mixer(cfg, layer), feed_forward=ffn, norm=norm,
                                          mixer_prefix="mix.", ffn_prefix="mlp.", norm1_prefix="norm1", norm2_prefix="norm2"))
        layers.append(LayerSpec(block, f"l{i}."))
    # every run of a layer has caches of its own: a parallel layer takes two slots (pages, state), the others one
    plan, slot = [], 0
    for i, again in cfg.layer_runs():
        if cfg.layers[i]["type"] == "parallel":
            plan.append(PlanEntry(i, (slot, slot + 1), True, add_embedding=again))
            slot += 2
        else:
            plan.append(PlanEntry(i, slot, True, add_embedding=again))
            slot += 1
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), plan=tuple(plan), final_norm=norm,
        embed_name="embed", final_norm_prefix="final.norm", head_name=None, tie_head=True,
        max_positions=None, embed_scale=cfg.embedding_scale)
