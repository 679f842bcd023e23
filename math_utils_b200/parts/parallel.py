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
        self._side = None
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

    # Steps of up to this many tokens (single-token steps above all) run the second member on a stream of its own
    # beside the first: both are short chains of dependent launches, and side by side the layer's chain is as long
    # as the longer of the two.  (At this size every product is a kernel that keeps no workspace in device memory
    # that two launches could share.)  Larger steps fill the device a member at a time and run one after the other.
    SIDE_BY_SIDE_TOKENS = 32

    def forward_pair(self, h, ctx, cache, owns_cache: bool):
        """The two members' results, float32, not yet joined: for an arrangement whose next step (a norm of the
        sum) can take them with their weights (``self.scales``) and save the pass that adds them."""
        tag = ctx.tag
        views = cache or (None, None)
        outs = [ctx.buffer("parallel." + name, (ctx.n_tokens, self.hidden_size), torch.float32) for name in ("left", "right")]

        def run(i, name):
            ctx.tag = f"{tag}{name}."
            member = self.members[i]
            if member.can_overwrite:
                member.forward(h, outs[i], ctx, views[i], owns_cache, accumulate=False)
            else:
                outs[i].zero_()
                member.forward(h, outs[i], ctx, views[i], owns_cache)

        # (two members of one kind would share that kind's scratch memory: they run one after the other)
        apart = type(self.members[0]) is not type(self.members[1])
        if apart and ctx.trace is None and ctx.n_tokens <= self.SIDE_BY_SIDE_TOKENS and h.is_cuda:
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream(device=h.device)
                self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
            self._fork.record(main)
            self._side.wait_event(self._fork)               # the input is ready
            with torch.cuda.stream(self._side):
                run(1, "right")
                self._join.record(self._side)
            run(0, "left")
            main.wait_event(self._join)                     # both results are there for what comes next
        else:
            run(0, "left")
            run(1, "right")
        ctx.tag = tag
        return outs


register_part("mixer", "parallel", ParallelMixers, replace=True)
