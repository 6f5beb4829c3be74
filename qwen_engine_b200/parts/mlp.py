"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases
(reference src/models/qwen3/model.py:227-237; silu(g) = g / (1 + exp(-g)) in
float32, src/layers/fused_ops/silumul.py:50-53).  gate and up are one product
over the stacked weights.

The same part serves other gated feed-forwards: ``activation`` names the
function on the gate ("silu", or "gelu_tanh": 0.5 z (1 + tanh(sqrt(2/pi) (z +
0.044715 z^3)))), or the limited form ("swish_limit", L): g' = min(g, L), u' =
clamp(u, -L, L), g' sigmoid(1.702 g') (u' + 1); ``names`` the three tensors.  The gate/up products that form
the activation in their own epilogue take either; the down product that forms
SiLU-mul while it loads (some tens of rows) is SiLU's alone, so another
activation runs there as product, activation kernel, product."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.spec import MATRIX, WeightSpec
from .base import FeedForward, StepContext, register, step_hint


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    takes_lazy_input = True       # x goes to one product only
    writes_through_linear = True  # out is the out of the last product
    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        if not ops.gate_activation_known(activation):
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(ops.GATE_ACTIVATIONS)} and ({ops.LIMITED_GLU!r}, limit)")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation = tuple(activation) if isinstance(activation, (tuple, list)) else activation
        self.names = tuple(names)
        self.w_gate_up = self.w_down = None

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        I, H = self.intermediate_size, self.hidden_size
        gate, up, down = self.names
        return [WeightSpec(prefix + gate, (I, H), MATRIX),
                WeightSpec(prefix + up, (I, H), MATRIX),
                WeightSpec(prefix + down, (H, I), MATRIX)]

    def load(self, prefix, source, dtype, device) -> None:
        gate, up, down = self.names
        stacked = torch.cat([source.get(prefix + gate), source.get(prefix + up)], dim=0)
        self.w_gate_up = ops.prepare_matrix(stacked.to(dtype).to(device))
        self.w_down = ops.prepare_matrix(source.get(prefix + down).to(dtype).to(device))

    def first_weights(self):
        return self.w_gate_up

    def forward(self, ctx: StepContext, x, out) -> None:
        T, I = ctx.num_tokens, self.intermediate_size
        if ops.swiglu_fused_applies(T, I, self.hidden_size, ctx.dtype):
            # many rows: the activation comes out of the gate/up product's epilogue
            if isinstance(x, ops.NormedInput):
                x = x.materialize()
            act = ctx.arena.alloc((T, I), ctx.dtype)
            ops.linear_swiglu(x, self.w_gate_up, act, self.activation)
            ops.linear(act, self.w_down, out)
            return
        if ops.swiglu_small_applies(T, I, self.hidden_size, ctx.dtype):
            # a few rows: the product that streams the gate and up weights forms the activation itself
            act = ctx.arena.alloc((T, I), ctx.dtype)
            ops.prefetch_next(self.w_down)
            ops.linear_swiglu_small(x, self.w_gate_up, act, self.activation)
            ops.prefetch_next(step_hint(ctx, "weights_after_ffn"))
            ops.linear(act, self.w_down, out)
            ops.prefetch_next(None)
            return
        gate_up = ctx.arena.alloc((T, 2 * I), ctx.dtype)
        ops.prefetch_next(self.w_down)
        ops.linear(x, self.w_gate_up, gate_up)
        ops.prefetch_next(step_hint(ctx, "weights_after_ffn"))
        if self.activation == "silu":
            ops.linear_silu_mul(gate_up, self.w_down, out, ctx.arena.alloc)
        else:
            act = ctx.arena.alloc((T, I), ctx.dtype)
            ops.act_mul(gate_up, act, self.activation)
            ops.linear(act, self.w_down, out)
        ops.prefetch_next(None)
