"""A state-space mixer with a matrix state per head (the state-space-duality form of a selective scan).

Parameters: ``hidden_size, n_heads, head_dim`` (P), ``state`` (N), ``groups`` (heads share B and C within a group:
head h reads group h // (n_heads / groups)), ``conv`` (taps of the short convolution), ``norm_groups``, ``eps``.

One input product gives, per token, [z: inner | x: inner | B: groups * N | C: groups * N | dt: n_heads] with
inner = n_heads * P.  x, B and C pass a causal convolution per channel (zeros before a sequence's start; the last
tap is the current token's) and silu.  dt = softplus(dt + dt_bias).  Per head, with S [N, P] starting at zero:
    S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,      y_t = S_t^T C_t + D x_t.
The heads' y, side by side, is multiplied by silu(z), brought to unit rms in ``norm_groups`` equal parts, multiplied
by a weight, and goes through the output matrix.  A sequence's state (the convolution's last taps - 1 inputs and
every head's S) is float32 and lives in the sequence's cache slot; decays, step sizes and the recurrence are
float32 whatever the compute dtype.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import Mixer, StateCacheSpec, TensorSpec, register_part
from .linear import Linear


class StateSpaceMixer(Mixer):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.n_heads, self.head_dim = int(p("hidden_size")), int(p("n_heads")), int(p("head_dim"))
        self.state, self.groups, self.taps = int(p("state")), int(p("groups")), int(p("conv"))
        self.norm_groups, self.eps = int(p("norm_groups", 1)), float(p("eps"))
        if self.n_heads % self.groups:
            raise ConfigError(f"state-space mixer: {self.n_heads} heads do not split over {self.groups} groups")
        self.inner = self.n_heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ConfigError(f"state-space mixer: {self.inner} channels do not split into {self.norm_groups} norm groups")
        self.channels = self.inner + 2 * self.groups * self.state           # what the convolution sees: x | B | C
        self.tail_values = (self.taps - 1) * self.channels

    def tensor_specs(self):
        name, H = self.tensor_name, self.n_heads
        return (TensorSpec(name("in"), (2 * self.inner + 2 * self.groups * self.state + H, self.hidden_size)),
                TensorSpec(name("conv"), (self.channels, self.taps), role="vector"),
                TensorSpec(name("conv_bias"), (self.channels,), role="vector", init="bias"),
                TensorSpec(name("dt_bias"), (H,), role="vector", init="bias"),
                TensorSpec(name("A_log"), (H,), role="vector", init="bias"),
                TensorSpec(name("D"), (H,), role="vector", init="norm_weight"),
                TensorSpec(name("norm"), (self.inner,), role="vector", init="norm_weight"),
                TensorSpec(name("out"), (self.hidden_size, self.inner), init="residual_projection"))

    def cache_spec(self):
        return StateCacheSpec(self.tail_values + self.n_heads * self.state * self.head_dim)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        t = lambda role: tensors[self.tensor_name(role)]
        self.proj = Linear(t("in"), None, runtime)
        self.out = Linear(t("out"), None, runtime)
        self.conv_weight, self.conv_bias = t("conv"), t("conv_bias")
        self.dt_bias, self.a_log, self.skip, self.norm_weight = t("dt_bias"), t("A_log"), t("D"), t("norm")

    def forward(self, h, residual, ctx, cache, owns_cache: bool, accumulate: bool = True) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T, inner = ctx.n_tokens, self.inner
        if not owns_cache:
            raise ConfigError("a state-space mixer keeps its own state: it cannot read another layer's")
        u = ctx.buffer("ssd.proj", (T, 2 * inner + 2 * self.groups * self.state + self.n_heads), dt)
        self.proj(h, out=u)
        z, conv_in, dt_raw = u[:, :inner], u[:, inner:inner + self.channels], u[:, inner + self.channels:]
        xbc = ctx.buffer("ssd.xbc", (T, self.channels), torch.float32)
        ops.ssd_conv(conv_in, self.conv_weight, self.conv_bias, ctx.tok_seq, ctx.seq_first, ctx.seq_slots, cache.values,
                     ctx.is_decode, xbc)
        y = ctx.buffer("ssd.y", (T, inner), torch.float32)
        ops.ssd_scan(xbc, dt_raw, self.dt_bias, self.a_log, self.skip, self.n_heads, self.head_dim, self.state,
                     self.groups, ctx.seq_first, ctx.seq_slots, cache.values, self.tail_values, y)
        ctx.note("scan", y)
        gated = ctx.buffer("ssd.gated", (T, inner), dt)
        ops.gated_group_norm(y, z, self.norm_weight, self.norm_groups, self.eps, gated)
        ctx.note("attn", gated)
        self.out(gated, residual=residual if accumulate else None, out=residual)


register_part("mixer", "state_space", StateSpaceMixer, replace=True)
