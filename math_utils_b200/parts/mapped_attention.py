"""Attention with normed, rotated queries and keys, one or two score maps per head, and values of their own size.

Parameters: ``hidden_size, n_heads, n_kv_heads`` (query head h reads key/value head h // (n_heads / n_kv_heads)),
``dim`` (query/key entries of ONE score map), ``vdim`` (value entries per head), ``maps`` (1, or 2 for differential
attention), ``softmax_scale``, ``window`` (0: every earlier position; w: a token sees itself and the w - 1 before
it), ``cache_window`` (what the cache must keep: the largest window of the layers that read it, 0 for all), ``eps``,
``rot`` = {base, dims, scaling?}, ``bias`` (the four projections have biases), ``own_kv`` (false for a layer that
reads the cached keys and values of an earlier layer and has no key/value tensors of its own) and, with two maps,
``diff``.

Per head and map the queries and keys are brought to unit rms over ``dim`` and multiplied by a weight shared by
all heads and maps, then their first ``rot.dims`` entries are rotated (entry i with entry i + dims/2).  With two
maps each map is a softmax attention of its own over the SAME values, and the head's result is
a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number for the layer; that result is
brought to unit rms over its vdim entries (no weight) and multiplied by 1 - diff.  The cache keeps one row per
position: the kv heads' keys (after norm and rotation), then their values.
"""
from __future__ import annotations

import torch

from ..config.base import ConfigError, PartSpec
from .base import Mixer, RowCacheSpec, TensorSpec, register_part
from .linear import Linear
from .position import rotary_frequencies


class MappedAttention(Mixer):
    can_overwrite = True

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = self.param
        self.hidden_size, self.n_heads = int(p("hidden_size")), int(p("n_heads"))
        self.n_kv_heads = int(p("n_kv_heads", self.n_heads))
        self.dim, self.vdim, self.maps = int(p("dim")), int(p("vdim")), int(p("maps", 1))
        self.scale, self.eps = float(p("softmax_scale")), float(p("eps"))
        self.window = int(p("window", 0))
        self.cache_window = int(p("cache_window", self.window))
        self.own_kv = bool(p("own_kv", True))
        self.bias = bool(p("bias", False))
        self.diff = float(p("diff", 0.0))
        if self.maps not in (1, 2):
            raise ConfigError(f"mapped attention has one or two score maps, got {self.maps}")
        if self.n_heads % self.n_kv_heads:
            raise ConfigError(f"mapped attention: {self.n_heads} heads do not split over {self.n_kv_heads} kv heads")
        if self.window and self.cache_window and self.cache_window < self.window:
            raise ConfigError("mapped attention: the cache keeps fewer positions than the window sees")
        rot = p("rot")
        self.rot_dims = int(rot["dims"])
        if self.rot_dims > self.dim or self.rot_dims % 2:
            raise ConfigError(f"mapped attention: {self.rot_dims} rotated entries do not fit a map of {self.dim}")
        self.freqs, self.magnitude = rotary_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
        self.q_width = self.n_heads * self.maps * self.dim
        self.k_width = self.n_kv_heads * self.maps * self.dim
        self.v_width = self.n_kv_heads * self.vdim

    def tensor_specs(self):
        D, name = self.hidden_size, self.tensor_name
        specs = [TensorSpec(name("q"), (self.q_width, D)), TensorSpec(name("q_norm"), (self.dim,), role="vector", init="norm_weight")]
        widths = [("q_bias", self.q_width)]
        if self.own_kv:
            specs += [TensorSpec(name("k"), (self.k_width, D)), TensorSpec(name("v"), (self.v_width, D)),
                      TensorSpec(name("k_norm"), (self.dim,), role="vector", init="norm_weight")]
            widths += [("k_bias", self.k_width), ("v_bias", self.v_width)]
        specs.append(TensorSpec(name("out"), (D, self.n_heads * self.vdim), init="residual_projection"))
        widths.append(("out_bias", D))
        if self.bias:
            specs += [TensorSpec(name(role), (n,), role="vector", init="bias") for role, n in widths]
        if self.maps == 2:
            specs += [TensorSpec(name(role), (self.dim,), role="vector", init="bias") for role in ("lq1", "lk1", "lq2", "lk2")]
        return specs

    def cache_spec(self):
        return RowCacheSpec(self.k_width + self.v_width, self.cache_window)

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        t = lambda role: tensors[self.tensor_name(role)]
        roles = ["q"] + (["k", "v"] if self.own_kv else [])
        weight = torch.cat([t(r) for r in roles], dim=0).contiguous() if len(roles) > 1 else t("q")
        bias = torch.cat([t(r + "_bias") for r in roles]).contiguous() if self.bias else None
        self.widths = tuple(t(r).shape[0] for r in roles)
        self.proj = Linear(weight, bias, runtime)
        self.out = Linear(t("out"), t("out_bias") if self.bias else None, runtime)
        self.q_norm = t("q_norm")
        self.k_norm = t("k_norm") if self.own_kv else None
        self.freq_table = torch.tensor(self.freqs or [0.0], dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.lam, self.out_scale = 0.0, 1.0
        if self.maps == 2:
            # one number for the layer, in float32 like everything around the softmax
            dot = lambda a, b: (t(a).float() * t(b).float()).sum(dtype=torch.float32)
            self.lam = float(torch.exp(dot("lq1", "lk1")) - torch.exp(dot("lq2", "lk2")) + self.diff)
            self.out_scale = 1.0 - self.diff

    def forward(self, h, residual, ctx, cache, owns_cache: bool, accumulate: bool = True) -> None:
        ops, dt = self.runtime.ops, self.runtime.dtype
        T = ctx.n_tokens
        if owns_cache and not self.own_kv:
            raise ConfigError("an attention layer without key and value projections cannot own a cache")
        views = ctx.buffer("mapped.proj" if self.own_kv else "mapped.proj_q", (T, sum(self.widths)), dt, columns=self.widths)
        self.proj(h, out=views[0])
        q = views[1]
        k, v = (views[2], views[3]) if owns_cache else (None, None)
        table = ctx.block_tables[cache.group]
        ops.qk_prepare(q, k, v, self.q_norm, self.k_norm, self.freq_table, self.magnitude, self.rot_dims, self.eps,
                       self.n_heads, self.n_kv_heads, self.maps, self.dim, self.vdim, ctx.tok_pos, ctx.tok_seq,
                       table if owns_cache else None, cache.page_tokens, cache.pages if owns_cache else None)
        ctx.note("q", q)
        heads = ctx.buffer("mapped.heads", (T, self.n_heads * self.vdim), dt)
        ops.mapped_attention(q, cache.pages, table, cache.page_tokens, ctx.tok_pos, ctx.tok_seq, self.n_heads,
                             self.n_kv_heads, self.maps, self.dim, self.vdim, self.scale, self.window, heads,
                             lam=self.lam, out_scale=self.out_scale, eps=self.eps, unit_rms=self.maps == 2,
                             tiles=None if ctx.is_decode else ctx.q_tiles, single_tokens=ctx.is_decode)
        ctx.note("attn", heads)
        self.out(heads, residual=residual if accumulate else None, out=residual)


register_part("mixer", "mapped_attention", MappedAttention, replace=True)
