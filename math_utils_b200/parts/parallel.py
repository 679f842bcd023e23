"""Two mixers side by side: both read the layer's input, and their results join with a weight each.

Parameters: ``left`` and ``right`` (the two mixers' ``PartSpec``), ``left_scale``, ``right_scale``.  The layer's
cache entry is a pair: each member's own kind of cache (pages, state, or nothing).
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import CompositeCacheSpec, Mixer, build_part, register_part


class ParallelMixers(Mixer):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        left, right = self.param("left"), self.param("right")
        if not isinstance(left, PartSpec) or not isinstance(right, PartSpec):
            raise ConfigError("parallel mixers: 'left' and 'right' are part specs")
        self.members = (build_part("mixer", left), build_part("mixer", right))
        self.scales = (float(self.param("left_scale")), float(self.param("right_scale")))
        self.hidden_size = int(self.param("hidden_size"))
        self.graph_safe = all(m.graph_safe for m in self.members)

    def tensor_specs(self):
        return tuple(s for m in self.members for s in m.tensor_specs())

    def cache_spec(self):
        return CompositeCacheSpec(tuple(m.cache_spec() for m in self.members))

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        for m in self.members:
            m.bind(tensors, runtime)

    def forward(self, h, residual, ctx, cache, owns_cache: bool, accumulate: bool = True) -> None:
        outs = self.forward_pair(h, ctx, cache, owns_cache)
        self.runtime.ops.scaled_sum(outs[0], self.scales[0], outs[1], self.scales[1], residual, add=accumulate)

    def forward_pair(self, h, ctx, cache, owns_cache: bool):
        """The two members' results, float32, not yet joined: for an arrangement whose next step (a norm of the
        sum) can take them with their weights (``self.scales``) and save the pass that adds them."""
        tag = ctx.tag
        outs = []
        for name, member, view in zip(("left", "right"), self.members, cache or (None, None)):
            y = ctx.buffer("parallel." + name, (ctx.n_tokens, self.hidden_size), torch.float32)
            ctx.tag = f"{tag}{name}."
            if member.can_overwrite:
                member.forward(h, y, ctx, view, owns_cache, accumulate=False)
            else:
                y.zero_()
                member.forward(h, y, ctx, view, owns_cache)
            outs.append(y)
        ctx.tag = tag
        return outs


register_part("mixer", "parallel", ParallelMixers, replace=True)
