"""Besavik as a layout of parts.

Layers in the order config.json gives, each a pre-norm block with one of three
mixers: ``latent_attention`` (softmax attention whose keys and values are read
out of one small latent per token, with a rotated key part shared by all heads
and a sigmoid output gate), ``lightning`` (linear attention with one constant
decay per head, the joined heads normed together) and ``channel_delta`` (the
gated delta rule with a decay per head and key channel, behind short causal
convolutions); and a feed-forward that is absent, dense, or a mixture of
routed experts, all of the limited gated form.  The embedding output passes a
norm of its own; the head is the embedding table, its logits times a scale.

Tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*`` (experts ``l<i>.mlp.e<j>.*``).
"""
from __future__ import annotations

from ..config.besavik_config import BesavikConfig
from ..parts.base import PartSpec
from .decoder import LayerSpec, ModelLayout, PlanEntry

GLU_FORM = "swish_limit"


def _mixer(cfg: BesavikConfig, layer: dict) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    if kind == "latent_attention":
        return PartSpec("latent_attention", dict(
            hidden_size=cfg.width, num_heads=m["heads"], plain_dim=m["dim"], rot_dim=m["rot_dim"], value_dim=m["vdim"],
            latent_dim=m["kv_rank"], query_rank=m["q_rank"], scale=m["scale"], norm_eps=cfg.norm_eps,
            rope_base=m["rot"]["base"], rope_dims=m["rot"]["dims"], output_gate="sigmoid"))
    if kind == "lightning":
        return PartSpec("decayed_linear_attention", dict(
            hidden_size=cfg.width, num_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
            head_decays=tuple(float(d) for d in m["decay"]), norm_eps=cfg.norm_eps))
    return PartSpec("gated_delta_rule", dict(
        hidden_size=cfg.width, num_heads=m["heads"], num_key_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
        conv_taps=m["conv"], norm_eps=cfg.norm_eps, low_rank=m.get("rank")))


def _feed_forward(cfg: BesavikConfig, mlp):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(hidden_size=cfg.width, intermediate_size=mlp["ff"],
                                       activation=(GLU_FORM, float(mlp["limit"])), names=("gate", "up", "down")))
    return PartSpec("routed_experts", dict(
        hidden_size=cfg.width, intermediate_size=mlp["expert"]["ff"], num_experts=mlp["router"]["experts"],
        top=mlp["router"]["top"], activation=(GLU_FORM, float(mlp["expert"]["limit"]))))


def besavik_layout(cfg: BesavikConfig) -> ModelLayout:
    norm = PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name=""))
    layers, plan, slot = [], [], 0
    for i, layer in enumerate(cfg.layers):
        block = PartSpec("pre_norm", dict(hidden_size=cfg.width, mixer=_mixer(cfg, layer),
                                          feed_forward=_feed_forward(cfg, layer.get("mlp")), norm=norm,
                                          mixer_prefix="mix.", ffn_prefix="mlp.", norm1_prefix="norm1", norm2_prefix="norm2"))
        layers.append(LayerSpec(block, f"l{i}."))
        # the delta mixer keeps two states (the recurrence's and the convolutions' last inputs), the others one cache
        if layer["type"] == "channel_delta":
            plan.append(PlanEntry(i, (slot, slot + 1), True))
            slot += 2
        else:
            plan.append(PlanEntry(i, slot, True))
            slot += 1
    # the logits' scale rides on the final norm's weight
    final = PartSpec("rmsnorm", dict(width=cfg.width, eps=cfg.norm_eps, weight_name="", output_scale=cfg.logit_scale))
    return ModelLayout(
        vocab_size=cfg.vocab, hidden_size=cfg.width, layers=tuple(layers), plan=tuple(plan), final_norm=final,
        embed_name="embed", final_norm_prefix="final.norm", head_name=None, tie_head=True, max_positions=None,
        embed_norm=norm, embed_norm_prefix="embed.norm")
