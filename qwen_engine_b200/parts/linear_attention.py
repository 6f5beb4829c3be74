"""Gated linear attention: a recurrent mixer whose state is one matrix per head.

For a head with dk key channels and dv value channels, and the mixer's input h:

    q = W_q h * dk^-1/2,  k = W_k h,  v = W_v h
    alpha = sigmoid(W_a2 (W_a1 h) + b) ^ (1 / tau)         one decay per key channel, in (0, 1)
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T                  S: dk x dv, float32, zero before the first token
    o_t = S_t^T q_t

Each head's o is RMS-normed over its dv channels (one weight of size dv for all
heads), the heads are joined and multiplied by silu(W_g h), and W_o projects
back.  The state is of fixed size: it lives in the request's state slot and is
carried from step to step, so a prompt may be cut anywhere.

q, k, v, the gate and the first half of the decay's low-rank pair are one
product over stacked weights (in the compute type); everything else that
enters the recurrence (the second half of the pair with its bias, the
log-sigmoid, alpha, the state, o and its norm) is float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.spec import FixedStateSpec
from ..weights.spec import MATRIX, NORM, VECTOR, WeightSpec
from .base import Mixer, StepContext, register

_NAMES = dict(q="q", k="k", v="v", gate="g", out="o", norm="norm", decay_in="a1", decay_out="a2", decay_bias="a2.b")


@register("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    takes_lazy_input = True       # x goes to one product only
    writes_through_linear = True  # out is the out of the last product

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay_tau: float,
                 norm_eps: float, decay_rank: Optional[int] = None, random_decay_rank: int = 16,
                 names: Optional[dict] = None):
        """``decay_rank`` None: the rank of the decay's low-rank pair is whatever the checkpoint stores
        (random weights are drawn with ``random_decay_rank``)."""
        if decay_tau <= 0:
            raise ValueError("decay_tau must be positive")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.key_dim = key_dim
        self.value_dim = value_dim
        self.decay_tau = float(decay_tau)
        self.norm_eps = float(norm_eps)
        self.decay_rank = decay_rank
        self.random_decay_rank = decay_rank or random_decay_rank
        self.names = dict(_NAMES, **(names or {}))
        self.k_width = num_heads * key_dim
        self.v_width = num_heads * value_dim
        self.inner_width = self.v_width
        self.q_scale = float(key_dim) ** -0.5
        self.w_in = self.w_decay = self.decay_bias = self.norm_w = self.w_o = None
        self.rank = decay_rank
        self.input_width = None if decay_rank is None else 2 * self.k_width + 2 * self.v_width + decay_rank    # (known at load otherwise)

    def cache_spec(self):
        # a head's state is kept with the key channels of a value channel side by side (the scan's threads
        # own value channels)
        return FixedStateSpec((self.num_heads, self.value_dim, self.key_dim), torch.float32)

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        n, W, r = self.names, self.hidden_size, self.decay_rank
        fill_in = None if r is not None else (self.random_decay_rank, W)
        fill_out = None if r is not None else (self.k_width, self.random_decay_rank)
        return [
            WeightSpec(prefix + n["q"], (self.k_width, W), MATRIX),
            WeightSpec(prefix + n["k"], (self.k_width, W), MATRIX),
            WeightSpec(prefix + n["v"], (self.v_width, W), MATRIX),
            WeightSpec(prefix + n["gate"], (self.v_width, W), MATRIX),
            WeightSpec(prefix + n["out"], (W, self.v_width), MATRIX),
            WeightSpec(prefix + n["norm"], (self.value_dim,), NORM),
            WeightSpec(prefix + n["decay_in"], (r, W), MATRIX, fill=fill_in),
            WeightSpec(prefix + n["decay_out"], (self.k_width, r), MATRIX, fill=fill_out),
            WeightSpec(prefix + n["decay_bias"], (self.k_width,), VECTOR),
        ]

    def load(self, prefix, source, dtype, device) -> None:
        n = self.names
        a1, a2 = source.get(prefix + n["decay_in"]), source.get(prefix + n["decay_out"])
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{prefix}: the decay's pair does not fit: {tuple(a1.shape)} and {tuple(a2.shape)}")
        self.rank = int(a1.shape[0])
        self.input_width = 2 * self.k_width + 2 * self.v_width + self.rank
        # q, k, v, the gate and the first half of the pair as rows of one matrix: one product gives them all
        stacked = torch.cat([source.get(prefix + n[x]) for x in ("q", "k", "v", "gate")] + [a1], dim=0)
        self.w_in = ops.prepare_matrix(stacked.to(dtype).to(device))
        self.w_decay = a2.to(dtype).to(device).contiguous()
        self.decay_bias = source.get(prefix + n["decay_bias"]).to(torch.float32).to(device).contiguous()
        self.norm_w = source.get(prefix + n["norm"]).to(torch.float32).to(device).contiguous()
        self.w_o = ops.prepare_matrix(source.get(prefix + n["out"]).to(dtype).to(device))

    def first_weights(self):
        return self.w_in

    def output_weight(self):
        return self.w_o

    def input_weight(self):
        return self.w_in

    def mix_into(self, ctx: StepContext, x, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        proj = ctx.arena.alloc((ctx.num_tokens, self.input_width), ctx.dtype)
        ops.linear(x, self.w_in, proj)
        self.mix_projected(ctx, proj, cache, group, inner, write_cache, scale)

    def mix_projected(self, ctx: StepContext, proj, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        T, H, dk, dv = ctx.num_tokens, self.num_heads, self.key_dim, self.value_dim
        kw, vw = self.k_width, self.v_width
        q, k = proj[:, :kw], proj[:, kw:2 * kw]
        v, gate = proj[:, 2 * kw:2 * kw + vw], proj[:, 2 * kw + vw:2 * kw + 2 * vw]
        o = ctx.arena.alloc((T, vw), torch.float32)
        if ops.SCAN_FORMS_DECAY and ctx.max_q_len <= 1:
            # single tokens: the scan's CTAs form their head's decay themselves (one launch less in a chain of launches)
            ops.linear_attention_scan(q, k, v, None, cache, ctx, o, self.q_scale, H, dk, dv, write_state=write_cache,
                                      decay=(proj[:, 2 * kw + 2 * vw:], self.w_decay, self.decay_bias, self.decay_tau))
        else:
            alpha = ctx.arena.alloc((T, kw), torch.float32)
            ops.channel_decay(proj[:, 2 * kw + 2 * vw:], self.w_decay, self.decay_bias, self.decay_tau, alpha)
            ops.linear_attention_scan(q, k, v, alpha, cache, ctx, o, self.q_scale, H, dk, dv, write_state=write_cache)
        ops.head_norm_gate(o, gate, self.norm_w, self.norm_eps, inner, H, dv, gate_kind="silu", scale=scale)

    def forward(self, ctx: StepContext, x, cache, group, out, write_cache: bool = True) -> None:
        inner = ctx.arena.alloc((ctx.num_tokens, self.inner_width), ctx.dtype)
        self.mix_into(ctx, x, cache, group, inner, write_cache)
        ops.linear(inner, self.w_o, out)


_DECAYED_NAMES = dict(q="q", k="k", v="v", gate="g", out="o", norm="norm")


@register("mixer", "decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    """Linear attention with ONE constant decay per head:

        q = silu(W_q h),  k = silu(W_k h),  v = silu(W_v h)
        S_t = decay_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t           (no other scale)

    The joined heads are RMS-normed together (one weight of heads x dv), multiplied by sigmoid(W_g h) and projected by
    W_o.  The state is float32 in the request's state slot; the scan is the one of gated linear attention with the
    head's constant in the place of the decays per channel."""

    takes_lazy_input = True       # x goes to one product only
    writes_through_linear = True  # out is the out of the last product

    def __init__(self, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, head_decays, norm_eps: float,
                 names: Optional[dict] = None):
        if len(head_decays) != num_heads:
            raise ValueError("one decay per head")
        self.hidden_size, self.num_heads, self.key_dim, self.value_dim = hidden_size, num_heads, key_dim, value_dim
        self.head_decays = tuple(float(d) for d in head_decays)
        self.norm_eps = float(norm_eps)
        self.names = dict(_DECAYED_NAMES, **(names or {}))
        self.k_width, self.v_width = num_heads * key_dim, num_heads * value_dim
        self.inner_width = self.v_width
        self.input_width = 2 * self.k_width + 2 * self.v_width
        self.w_in = self.w_o = self.norm_w = self.decays = None

    def cache_spec(self):
        return FixedStateSpec((self.num_heads, self.value_dim, self.key_dim), torch.float32)

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        n, W = self.names, self.hidden_size
        return [WeightSpec(prefix + n["q"], (self.k_width, W), MATRIX),
                WeightSpec(prefix + n["k"], (self.k_width, W), MATRIX),
                WeightSpec(prefix + n["v"], (self.v_width, W), MATRIX),
                WeightSpec(prefix + n["gate"], (self.v_width, W), MATRIX),
                WeightSpec(prefix + n["out"], (W, self.v_width), MATRIX),
                WeightSpec(prefix + n["norm"], (self.v_width,), NORM)]

    def load(self, prefix, source, dtype, device) -> None:
        n = self.names
        stacked = torch.cat([source.get(prefix + n[x]) for x in ("q", "k", "v", "gate")], dim=0)
        self.w_in = ops.prepare_matrix(stacked.to(dtype).to(device))
        self.w_o = ops.prepare_matrix(source.get(prefix + n["out"]).to(dtype).to(device))
        self.norm_w = source.get(prefix + n["norm"]).to(torch.float32).to(device).contiguous()
        self.decays = torch.tensor(self.head_decays, dtype=torch.float32).to(device)

    def first_weights(self):
        return self.w_in

    def output_weight(self):
        return self.w_o

    def mix_into(self, ctx: StepContext, x, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        T, H, dk, dv = ctx.num_tokens, self.num_heads, self.key_dim, self.value_dim
        kw, vw = self.k_width, self.v_width
        proj = ctx.arena.alloc((T, self.input_width), ctx.dtype)
        ops.linear(x, self.w_in, proj)
        # silu of q, k and v in one pass: x sigmoid(x), rounded once
        qkv = ctx.arena.alloc((T, 2 * kw + vw), ctx.dtype)
        ops.head_norm_gate(proj[:, :2 * kw + vw], proj[:, :2 * kw + vw], None, 0.0, qkv, 1, 2 * kw + vw, gate_kind="sigmoid")
        o = ctx.arena.alloc((T, vw), torch.float32)
        ops.linear_attention_scan(qkv[:, :kw], qkv[:, kw:2 * kw], qkv[:, 2 * kw:], None, cache, ctx, o, 1.0, H, dk, dv,
                                  write_state=write_cache, head_decay=self.decays)
        ops.head_norm_gate(o, proj[:, 2 * kw + vw:], self.norm_w, self.norm_eps, inner, 1, vw, gate_kind="sigmoid", scale=scale)

    def forward(self, ctx: StepContext, x, cache, group, out, write_cache: bool = True) -> None:
        inner = ctx.arena.alloc((ctx.num_tokens, self.inner_width), ctx.dtype)
        self.mix_into(ctx, x, cache, group, inner, write_cache)
        ops.linear(inner, self.w_o, out)
