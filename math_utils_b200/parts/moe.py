"""A feed-forward of routed experts.

Parameters: ``hidden_size, inner_size`` (of one expert), ``n_experts, top``, ``router_scale``,
``score`` (``sigmoid`` | ``softmax``), ``renormalize`` (divide the chosen weights by their sum) and
``correction`` (a per-expert term added to the scores for the CHOICE only).  Tensors: ``router``
[experts, hidden], ``correction`` [experts], and per expert ``gate``, ``up`` [inner, hidden] and ``down``
[hidden, inner] whose names carry ``{e}``.  An expert is down(silu(gate h) * (up h)), without biases.

Router logits, scores and weights are float32.  The (token, expert) pairs are grouped by expert on the
device, each expert's products run over its own rows only, and the results are summed per token in the
order of the token's choices: no host round trip, so single-token steps can be replayed from a graph.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import FeedForward, TensorSpec, register_part


class RoutedExperts(FeedForward):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.inner_size = int(p("hidden_size")), int(p("inner_size"))
        self.n_experts, self.top = int(p("n_experts")), int(p("top"))
        self.router_scale = float(p("router_scale", 1.0))
        self.score = p("score", "sigmoid")
        self.renormalize = bool(p("renormalize", False))
        self.has_correction = bool(p("correction", False))
        if self.score not in ("sigmoid", "softmax"):
            raise ConfigError(f"routed_experts: score '{self.score}' is not sigmoid or softmax")
        if not 1 <= self.top <= self.n_experts:
            raise ConfigError(f"routed_experts: top {self.top} of {self.n_experts} experts")

    def tensor_specs(self):
        D, F, name = self.hidden_size, self.inner_size, self.tensor_name
        specs = [TensorSpec(name("router"), (self.n_experts, D), role="matrix32")]
        if self.has_correction:
            specs.append(TensorSpec(name("correction"), (self.n_experts,), role="vector", init="bias"))
        for e in range(self.n_experts):
            specs += [TensorSpec(name("gate").format(e=e), (F, D)), TensorSpec(name("up").format(e=e), (F, D)),
                      TensorSpec(name("down").format(e=e), (D, F), init="residual_projection")]
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        name = self.tensor_name
        self.router = tensors[name("router")]
        self.correction = tensors[name("correction")] if self.has_correction else None
        stack = lambda role: torch.stack([tensors[name(role).format(e=e)] for e in range(self.n_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        self.tile_rows = runtime.ops.moe_tile_rows()

    fuses_output_norm = True           # forward(..., output_norm=): the norm of the result, added into the stream

    def forward(self, h, residual, ctx, accumulate: bool = True, output_norm=None) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T, top, E = ctx.n_tokens, self.top, self.n_experts
        P = T * top
        # tiles of 64 slots where the tensor cores take the products and an expert has the rows to fill them
        tile_rows = self.tile_rows
        if ops.moe_tc_ok(dt, self.hidden_size, self.inner_size) and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0:
            tile_rows = 64 if P >= 48 * E else 32
        max_tiles = P // tile_rows + E                     # every grouping of P pairs into E experts fits
        index = ctx.buffer("moe.index", (3 * P + 3 * max_tiles + 4,), torch.int32)
        expert_of, slot_of, pair_of = index[:P], index[P:2 * P], index[2 * P:3 * P]
        tile_info, n_tiles = index[3 * P: 3 * P + 3 * max_tiles], index[3 * P + 3 * max_tiles:]
        weight_of = ctx.buffer("moe.weight", (P,), torch.float32)
        ops.moe_route(h, self.router, self.correction, top, self.router_scale, expert_of, weight_of,
                      softmax=self.score == "softmax", renormalize=self.renormalize)
        ops.moe_group(expert_of, E, slot_of, pair_of, tile_info, n_tiles, tile_rows)
        ctx.note("route", weight_of)
        hidden = ctx.buffer("moe.hidden", (P, self.inner_size), dt)
        ops.moe_gemm(h, pair_of, top, self.w_gate, self.w_up, tile_info, n_tiles, max_tiles, hidden, tile_rows=tile_rows)
        ctx.note("act", hidden)
        y = ctx.buffer("moe.out", (P, self.hidden_size), torch.float32)
        ops.moe_gemm(hidden, None, top, self.w_down, None, tile_info, n_tiles, max_tiles, y, tile_rows=tile_rows)
        if output_norm is not None:
            # residual += norm(sum of the token's experts); Dynamic Tanh in the same launch as the sum
            from .norm import DynamicTanh
            if type(output_norm) is DynamicTanh:
                ops.moe_combine_tanh(y, slot_of, weight_of, top, output_norm.weight, output_norm.bias, output_norm.alpha,
                                     residual)
            else:
                mixed = ctx.buffer("moe.mixed", (T, self.hidden_size), torch.float32)
                ops.moe_combine(y, slot_of, weight_of, top, mixed)
                output_norm.add_into(mixed, residual)
        elif accumulate:
            mixed = ctx.buffer("moe.mixed", (T, self.hidden_size), torch.float32)
            ops.moe_combine(y, slot_of, weight_of, top, mixed)
            residual += mixed
        else:
            ops.moe_combine(y, slot_of, weight_of, top, residual)


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
