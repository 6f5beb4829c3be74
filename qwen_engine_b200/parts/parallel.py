"""Several mixers side by side: all read the same input, and the layer's mixer
output is the weighted sum of theirs.

    out = sum_b scale_b * mixer_b(x)

Each branch keeps its own cache (pages of keys and values, a state slot, or
nothing); the plan names one cache slot per cache description, in the order of
the branches.  When every branch ends in an output projection and offers its
two halves apart (``Mixer.mix_into`` / ``output_weight``), the branches write
their inner rows, already multiplied by their scale in float32, side by side
into one buffer and ONE product over the output matrices joined along K gives
the sum: no product per branch, no add kernel, and each value is rounded once.
Otherwise the branches run whole and their outputs are added.  In the same
way, branches that begin with one product of the input over stacked weights
(``Mixer.input_weight`` / ``mix_projected``) share ONE product over all their
stacked weights: the input is read once and the weights stream in one launch.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from .base import Mixer, PartSpec, StepContext, register


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    takes_lazy_input = False      # every branch reads x: it is formed once (and goes to ops.linear as a tensor)
    writes_through_linear = True  # out is the out of the one joined product (or of the first branch's last product)

    def __init__(self, branches: Sequence[PartSpec], scales: Sequence[float], prefixes: Sequence[str]):
        if not (len(branches) == len(scales) == len(prefixes)) or not branches:
            raise ValueError("one scale and one tensor prefix per branch")
        self.branches: list[Mixer] = [b.build("mixer") for b in branches]
        self.scales = [float(s) for s in scales]
        self.prefixes = list(prefixes)
        self.joined = all(b.inner_width is not None for b in self.branches)
        self.inner_width = sum(b.inner_width for b in self.branches) if self.joined else None
        self.w_o: Optional[torch.Tensor] = None
        self.w_in: Optional[torch.Tensor] = None      # the branches' stacked input weights, stacked once more (if all offer them)
        self._n_caches = [len(b.cache_specs()) for b in self.branches]

    @property
    def capturable(self) -> bool:
        return all(getattr(b, "capturable", True) for b in self.branches)

    def cache_specs(self) -> list:
        return [s for b in self.branches for s in b.cache_specs()]

    def attention_geometries(self) -> list:
        return [g for b in self.branches for g in b.attention_geometries()]

    def weight_specs(self, prefix: str):
        return [s for b, p in zip(self.branches, self.prefixes) for s in b.weight_specs(prefix + p)]

    def load(self, prefix, source, dtype, device) -> None:
        for b, p in zip(self.branches, self.prefixes):
            b.load(prefix + p, source, dtype, device)
        if self.joined:
            # [hidden, inner_1 + inner_2 + ...]: the sum over branches happens inside the product
            self.w_o = ops.prepare_matrix(torch.cat([b.output_weight() for b in self.branches], dim=1))
            # (every branch's columns then begin on a 16-byte boundary of a row whose stride is a multiple of 16 bytes,
            # which the attention kernels ask of their queries; widths that do not allow it keep a product per branch)
            if all(b.input_width is not None and b.input_width % 8 == 0 for b in self.branches):
                self.w_in = ops.prepare_matrix(torch.cat([b.input_weight() for b in self.branches], dim=0))

    def first_weights(self):
        return self.w_in if self.w_in is not None else self.branches[0].first_weights()

    def output_weight(self):
        return self.w_o

    def _caches(self, cache, group):
        """The branches' shares of the tuples of caches and groups the plan handed over."""
        caches = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        groups = group if isinstance(group, tuple) else (() if group is None else (group,))
        out, at = [], 0
        for n in self._n_caches:
            if n == 0:
                out.append((None, None))
            elif n == 1:
                out.append((caches[at], groups[at]))
            else:
                out.append((tuple(caches[at:at + n]), tuple(groups[at:at + n])))
            at += n
        return out

    def mix_into(self, ctx: StepContext, x, cache, group, inner, write_cache: bool = True, scale: float = 1.0) -> None:
        at = col = 0
        proj = None
        if self.w_in is not None:
            proj = ctx.arena.alloc((ctx.num_tokens, self.w_in.shape[0]), ctx.dtype)
            ops.linear(x, self.w_in, proj)
        for b, s, (c, g) in zip(self.branches, self.scales, self._caches(cache, group)):
            mark = ctx.arena.mark()
            if proj is not None:
                b.mix_projected(ctx, proj[:, col:col + b.input_width], c, g, inner[:, at:at + b.inner_width], write_cache, scale * s)
                col += b.input_width
            else:
                b.mix_into(ctx, x, c, g, inner[:, at:at + b.inner_width], write_cache, scale * s)
            ctx.arena.release(mark)
            at += b.inner_width

    def forward(self, ctx: StepContext, x, cache, group, out, write_cache: bool = True) -> None:
        T = ctx.num_tokens
        if self.joined:
            inner = ctx.arena.alloc((T, self.inner_width), ctx.dtype)
            self.mix_into(ctx, x, cache, group, inner, write_cache)
            ops.linear(inner, self.w_o, out)
            return
        # branches that cannot be joined: each runs whole, the outputs are added in float32
        if isinstance(out, ops.ResidualSink):
            out = out.as_delta()
        total = ctx.arena.alloc(tuple(out.shape), torch.float32)
        part = ctx.arena.alloc(tuple(out.shape), ctx.dtype)
        for i, (b, s, (c, g)) in enumerate(zip(self.branches, self.scales, self._caches(cache, group))):
            b.forward(ctx, x, c, g, part, write_cache)
            ops.scaled_add(total, part, s, first=i == 0)
        ops.scaled_add(out, total, 1.0, first=True)
