"""Lusalorn's configuration: its nested config.json, typed, and its plan.

Keys read: ``vocab``, ``width``, ``residual_mult``, ``norm.eps``, ``embedding.bigram`` = {``buckets, mul_prev,
mul_cur``} and the list ``layers``; an entry of that list has ``type`` (the kind of mixer), ``mixer`` (its sizes)
and ``mlp`` (the feed-forward, or null).
Mixer ``attention`` (differential, windowed): ``heads, kv_heads, dim, vdim, scale, diff``, ``mask.size``,
``rot`` = {``base, dims``, optional ``scaling``} and optionally ``kv_from`` (the layer whose cached keys and values
this layer reads instead of making its own).
Mixer ``parallel``: ``left`` (causal attention: ``heads, kv_heads, dim, vdim, scale, rot``), ``right`` (state-space:
``heads, vdim, state, groups, conv, norm_groups``), ``left_scale, right_scale``.
Feed-forward ``dense``: ``ff`` (gated, SiLU).

The design: x = token row + a hashed row of (token before, token).  Every layer reads the residual stream itself and
norms each sublayer's OUTPUT: x += m * norm1(mixer(x)); x += m * norm2(ff(x)), with m = ``residual_mult`` and norms
x / rms(x) * (1 + w).  At the end the same kind of norm and an output matrix.  Nothing limits the positions;
``max_positions`` (an optional key of this library's, 131,072 if absent) only sizes the page lists.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, KeyReader, LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("attention", "parallel")
DEFAULT_MAX_POSITIONS = 1 << 17


def _sub(reader: KeyReader, key: str) -> KeyReader:
    value = reader.raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{reader.where}: key '{key}' must be an object")
    return KeyReader(value, f"{reader.where}: {key}")


def _check_rot(m: KeyReader, where: str) -> None:
    rot = _sub(m, "rot")
    rot.number("base")
    dims = rot.integer("dims", minimum=0)
    if dims % 2 or dims > m.integer("dim"):
        raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim")
    if rot.raw.get("scaling") is not None:
        sc = _sub(rot, "scaling")
        for key in ("factor", "original", "fast", "slow"):
            sc.number(key)


def _check_heads(m: KeyReader, where: str) -> None:
    heads, kv = m.integer("heads"), m.integer("kv_heads")
    if heads % kv:
        raise ConfigError(f"{where}: heads {heads} must be a multiple of kv_heads {kv}")
    for key in ("dim", "vdim"):
        m.integer(key)
    m.number("scale")
    _check_rot(m, where)


@dataclass(frozen=True)
class LusalornConfig:
    vocab: int
    width: int
    residual_mult: float
    norm_eps: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: tuple                     # the checked raw entries
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Lusalorn"

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "LusalornConfig":
        r = KeyReader(raw)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: key 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            cls._check_layer(i, layer, layers)
        big = _sub(_sub(r, "embedding"), "bigram")
        return cls(vocab=r.integer("vocab"), width=r.integer("width"),
                   residual_mult=r.number("residual_mult", positive=False), norm_eps=_sub(r, "norm").number("eps"),
                   buckets=big.integer("buckets"), mul_prev=big.integer("mul_prev", minimum=0),
                   mul_cur=big.integer("mul_cur", minimum=0), layers=tuple(layers),
                   max_positions=r.integer("max_positions", default=DEFAULT_MAX_POSITIONS))

    @staticmethod
    def _check_layer(i: int, layer, layers) -> None:
        where = f"config.json: layers[{i}]"
        lr = KeyReader(layer, where)
        kind = lr.string("type", choices=MIXERS)
        m = _sub(lr, "mixer")
        if kind == "attention":
            _check_heads(m, where)
            m.number("diff", positive=False)
            _sub(m, "mask").integer("size")
            src = m.raw.get("kv_from")
            if src is not None:
                src = m.integer("kv_from", minimum=0)
                other = layers[src] if src < i else None
                if (other is None or other.get("type") != "attention"
                        or other.get("mixer", {}).get("kv_from") is not None):
                    raise ConfigError(f"{where}: kv_from {src} must name an earlier attention layer that keeps its own keys")
                if any(other["mixer"].get(k) != m.raw.get(k) for k in ("kv_heads", "dim", "vdim", "rot")):
                    raise ConfigError(f"{where}: kv_from {src} differs in kv_heads, dim, vdim or rot")
        else:
            left, right = _sub(m, "left"), _sub(m, "right")
            _check_heads(left, where + ": left")
            for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                right.integer(key)
            if right.integer("heads") % right.integer("groups"):
                raise ConfigError(f"{where}: right.heads must be a multiple of right.groups")
            if (right.integer("heads") * right.integer("vdim")) % right.integer("norm_groups"):
                raise ConfigError(f"{where}: right.norm_groups must divide heads * vdim")
            m.number("left_scale", positive=False)
            m.number("right_scale", positive=False)
        mlp = layer.get("mlp")
        if mlp is not None:
            f = KeyReader(mlp, where + ": mlp")
            f.string("kind", choices=("dense",))
            f.integer("ff")

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps},
               "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
               "layers": [dict(layer) for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    def init_distribution(self, rule: str):
        """(mean, standard deviation) of a random-weights rule: matrices N(0, 1/width); the output norms' weights are
        stored around zero."""
        r = 1.0 / math.sqrt(self.width)
        rules = {"normal": (0.0, r), "residual_projection": (0.0, r), "bias": (0.0, 0.05),
                 "norm_weight": (1.0, 0.05), "norm_bias": (0.0, 0.05), "norm_offset_weight": (0.0, 0.05)}
        if rule not in rules:
            raise ConfigError(f"no random-weights rule '{rule}'")
        return rules[rule]

    # ------------------------------------------------------------------ plan
    def _output_norm(self, name: str, scale: float) -> PartSpec:
        return PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps, "weight_offset": 1.0, "scale": scale,
                                     "init": "norm_offset_weight"}, {"weight": name})

    def _attention(self, m, prefix: str, maps: int, window: int, cache_window: int, own_kv: bool, bias: bool) -> PartSpec:
        names = {"q": prefix + "q", "q_norm": prefix + "q.norm", "out": prefix + "o"}
        if own_kv:
            names.update({"k": prefix + "k", "v": prefix + "v", "k_norm": prefix + "k.norm"})
        if bias:
            names.update({"q_bias": prefix + "q.b", "out_bias": prefix + "o.b"})
            if own_kv:
                names.update({"k_bias": prefix + "k.b", "v_bias": prefix + "v.b"})
        params = {"hidden_size": self.width, "n_heads": int(m["heads"]), "n_kv_heads": int(m["kv_heads"]),
                  "dim": int(m["dim"]), "vdim": int(m["vdim"]), "maps": maps, "softmax_scale": float(m["scale"]),
                  "window": window, "cache_window": cache_window, "eps": self.norm_eps, "rot": m["rot"],
                  "bias": bias, "own_kv": own_kv}
        if maps == 2:
            params["diff"] = float(m["diff"])
            names.update({n: prefix + n for n in ("lq1", "lk1", "lq2", "lk2")})
        return PartSpec("mapped_attention", params, names)

    def plan(self) -> ModelPlan:
        D = self.width
        # a layer's cache keeps what the widest window among its readers sees
        kept = {}
        for i, layer in enumerate(self.layers):
            if layer["type"] == "attention":
                owner = layer["mixer"].get("kv_from")
                owner = i if owner is None else int(owner)
                kept[owner] = max(kept.get(owner, 0), int(layer["mixer"]["mask"]["size"]))
        layers, schedule = [], []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer["mixer"]
            owner = i
            if layer["type"] == "attention":
                src = m.get("kv_from")
                owner = i if src is None else int(src)
                mixer = self._attention(m, p + "mix.", 2, int(m["mask"]["size"]), kept[owner], src is None, True)
            else:
                right = m["right"]
                q = p + "mix.right."
                state = PartSpec(
                    "state_space",
                    {"hidden_size": D, "n_heads": int(right["heads"]), "head_dim": int(right["vdim"]),
                     "state": int(right["state"]), "groups": int(right["groups"]), "conv": int(right["conv"]),
                     "norm_groups": int(right["norm_groups"]), "eps": self.norm_eps},
                    {"in": q + "in", "conv": q + "conv", "conv_bias": q + "conv.b", "dt_bias": q + "dt_bias",
                     "A_log": q + "A_log", "D": q + "D", "norm": q + "norm", "out": q + "o"})
                mixer = PartSpec("parallel", {"hidden_size": D, "left": self._attention(m["left"], p + "mix.left.", 1, 0, 0, True, False),
                                              "right": state, "left_scale": float(m["left_scale"]),
                                              "right_scale": float(m["right_scale"])})
            mlp = layer.get("mlp")
            extra = [("norm1b", "norm", self._output_norm(p + "norm1", self.residual_mult))]
            if mlp is None:
                ffn = PartSpec("none")
            else:
                ffn = PartSpec("gated_ffn", {"hidden_size": D, "inner_size": int(mlp["ff"]), "activation": "silu"},
                               {"gate_weight": p + "mlp.gate", "up_weight": p + "mlp.up", "down_weight": p + "mlp.down"})
                extra.append(("norm2b", "norm", self._output_norm(p + "norm2", self.residual_mult)))
            # the sublayers read the stream itself: the input norms are identities
            layers.append(LayerSpec("sandwich_norm", PartSpec("identity"), mixer, PartSpec("identity"), ffn,
                                    extra=tuple(extra)))
            schedule.append(ScheduleEntry(layer=i, cache_of=owner))
        plan = ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_pair_embedding",
                               {"vocab_size": self.vocab, "hidden_size": D, "buckets": self.buckets,
                                "mul_prev": self.mul_prev, "mul_cur": self.mul_cur},
                               {"weight": "embed", "pair_weight": "bigram"}),
            position=PartSpec("none"), layers=tuple(layers), schedule=tuple(schedule),
            final_norm=self._output_norm("final.norm", 1.0),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D}, {"weight": "head"}))
        plan.validate()
        return plan
