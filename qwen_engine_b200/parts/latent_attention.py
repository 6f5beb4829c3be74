"""Latent attention: softmax attention whose keys and values are read out of one small latent per token.

For the mixer's input h, H heads with dn unrotated and dr rotated query/key channels and dv value channels, a latent
of R channels:

    c_q = rmsnorm(W_dq h),  q_h = W_uq,h c_q = [q_plain (dn) | q_rot (dr)]
    [c' | k_rot] = W_dkv h,  c = rmsnorm(c') (R channels),  k_rot (dr channels) is one key part for all heads
    k_plain,h = W_uk,h c,  v_h = W_uv,h c
    score_h(i, j) = scale (q_plain,h,i . k_plain,h,j + rot(q_rot,h,i) . rot(k_rot,j)),  j <= i,  softmax over j

The rotation turns the pairs (x[i], x[i + dims/2]) of the first ``dims`` rotated channels by position x base^(-2i/dims).
The joined heads are multiplied by sigmoid(W_g h) and projected by W_o.

The cache holds c and the rotated k_rot, one plane of R + dr channels per token and nothing per head.  W_uk is folded into the query
(q_lat,h = W_uk,h^T q_plain,h) and W_uv applied after the softmax, so the paged attention kernels see ONE key/value
head of R + dr channels whose values are the keys' first R channels, for prompt portions and decoded tokens alike.
Norms, angles, scores and softmax are float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.spec import PagedKVSpec
from ..weights.spec import MATRIX, NORM, WeightSpec
from .base import Mixer, StepContext, register

_NAMES = dict(q_down="dq", q_norm="dq.norm", q_up="uq", kv_down="dkv", kv_norm="dkv.norm", k_up="uk", v_up="uv",
              gate="g", out="o")


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    takes_lazy_input = True       # x goes to one product only
    writes_through_linear = True  # out is the out of the last product

    def __init__(self, hidden_size: int, num_heads: int, plain_dim: int, rot_dim: int, value_dim: int, latent_dim: int,
                 query_rank: int, scale: float, norm_eps: float, rope_base: float, rope_dims: Optional[int] = None,
                 output_gate: Optional[str] = "sigmoid", names: Optional[dict] = None):
        if output_gate not in (None, "sigmoid"):
            raise ValueError(f"unknown output gate {output_gate!r}")
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.plain_dim, self.rot_dim, self.value_dim = plain_dim, rot_dim, value_dim
        self.latent_dim, self.query_rank = latent_dim, query_rank
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.rope_base = float(rope_base)
        self.rope_dims = rot_dim if rope_dims is None else int(rope_dims)
        if self.rope_dims % 2 or not (0 <= self.rope_dims <= rot_dim):
            raise ValueError(f"rope_dims {self.rope_dims} must be even and within rot_dim {rot_dim}")
        self.output_gate = output_gate
        self.names = dict(_NAMES, **(names or {}))
        self.cache_dim = latent_dim + rot_dim                     # channels of a token's cache row
        self.q_width = num_heads * (plain_dim + rot_dim)
        self.inner_width = num_heads * value_dim
        self.input_width = query_rank + self.cache_dim + (self.inner_width if output_gate else 0)
        self.w_in = self.w_uq = self.w_uk_t = self.w_uv = self.w_o = None
        self.q_norm_w = self.kv_norm_w = self.inv_freq = None

    def cache_spec(self):
        return PagedKVSpec(1, self.cache_dim, None, planes=1)

    def attention_geometry(self):
        return (self.num_heads, 1, self.cache_dim, 0, False, 1)

    def weight_specs(self, prefix: str) -> list[WeightSpec]:
        n, H, W = self.names, self.num_heads, self.hidden_size
        specs = [
            WeightSpec(prefix + n["q_down"], (self.query_rank, W), MATRIX),
            WeightSpec(prefix + n["q_norm"], (self.query_rank,), NORM),
            WeightSpec(prefix + n["q_up"], (self.q_width, self.query_rank), MATRIX),
            WeightSpec(prefix + n["kv_down"], (self.cache_dim, W), MATRIX),
            WeightSpec(prefix + n["kv_norm"], (self.latent_dim,), NORM),
            WeightSpec(prefix + n["k_up"], (H * self.plain_dim, self.latent_dim), MATRIX),
            WeightSpec(prefix + n["v_up"], (H * self.value_dim, self.latent_dim), MATRIX),
            WeightSpec(prefix + n["out"], (W, H * self.value_dim), MATRIX),
        ]
        if self.output_gate:
            specs.append(WeightSpec(prefix + n["gate"], (H * self.value_dim, W), MATRIX))
        return specs

    def load(self, prefix, source, dtype, device) -> None:
        n, H = self.names, self.num_heads
        rows = [source.get(prefix + n["q_down"]), source.get(prefix + n["kv_down"])]
        if self.output_gate:
            rows.append(source.get(prefix + n["gate"]))
        self.w_in = ops.prepare_matrix(torch.cat(rows, dim=0).to(dtype).to(device))
        self.w_uq = ops.prepare_matrix(source.get(prefix + n["q_up"]).to(dtype).to(device))
        # W_uk per head, transposed: the fold of a head's plain query into the latent's channels is a product with it
        uk = source.get(prefix + n["k_up"]).reshape(H, self.plain_dim, self.latent_dim)
        self.w_uk_t = uk.transpose(1, 2).contiguous().to(dtype).to(device)
        self.w_uv = source.get(prefix + n["v_up"]).reshape(H, self.value_dim, self.latent_dim).contiguous().to(dtype).to(device)
        self.w_o = ops.prepare_matrix(source.get(prefix + n["out"]).to(dtype).to(device))
        self.q_norm_w = source.get(prefix + n["q_norm"]).to(torch.float32).to(device).contiguous()
        self.kv_norm_w = source.get(prefix + n["kv_norm"]).to(torch.float32).to(device).contiguous()
        i = torch.arange(max(self.rope_dims // 2, 1), dtype=torch.float64)
        self.inv_freq = (self.rope_base ** (-2.0 * i / max(self.rope_dims, 1))).to(torch.float32).to(device).contiguous()

    def first_weights(self):
        return self.w_in

    def output_weight(self):
        return self.w_o

    def mix_into(self, ctx: StepContext, x, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        T, H = ctx.num_tokens, self.num_heads
        dn, dr, dv, R, D = self.plain_dim, self.rot_dim, self.value_dim, self.latent_dim, self.cache_dim
        view = ctx.groups[group]
        proj = ctx.arena.alloc((T, self.input_width), ctx.dtype)
        ops.linear(x, self.w_in, proj)
        cq = ctx.arena.alloc((T, self.query_rank), ctx.dtype)
        ops.head_norm_gate(proj[:, :self.query_rank], None, self.q_norm_w, self.norm_eps, cq, 1, self.query_rank, gate_kind=None)
        q = ctx.arena.alloc((T, self.q_width), ctx.dtype)
        ops.linear(cq, self.w_uq, q)
        qlat = ctx.arena.alloc((T, H * D), ctx.dtype)
        ops.latent_prepare(proj[:, self.query_rank:self.query_rank + D], q, self.kv_norm_w, self.norm_eps, ctx.positions,
                           self.inv_freq, self.rope_dims, cache, view.slot_mapping, qlat, H, dn, R, dr, write_kv=write_cache)
        ops.head_linear(q, self.w_uk_t, qlat, dn + dr, D)
        olat = ctx.arena.alloc((T, H * D), ctx.dtype)
        ops.paged_attention(qlat, cache, view.block_tables, ctx, olat, self.scale, 0, H, 1, D)
        gated = bool(self.output_gate) or scale != 1.0
        attn = ctx.arena.alloc((T, H * dv), ctx.dtype) if gated or not inner.is_contiguous() else inner
        ops.head_linear(olat, self.w_uv, attn, D, dv)
        if attn is not inner:
            gate = proj[:, self.query_rank + D:] if self.output_gate else None
            ops.head_norm_gate(attn, gate, None, 0.0, inner, H, dv, gate_kind=self.output_gate, scale=scale)

    def forward(self, ctx: StepContext, x, cache, group, out, write_cache: bool = True) -> None:
        inner = ctx.arena.alloc((ctx.num_tokens, self.inner_width), ctx.dtype)
        self.mix_into(ctx, x, cache, group, inner, write_cache)
        ops.linear(inner, self.w_o, out)
