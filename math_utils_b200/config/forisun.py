"""Forisun's configuration: its nested config.json, typed, and its plan.

Keys read: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and the list ``layers``; an entry of
that list has ``type`` (the kind of mixer), ``mixer`` (its sizes) and ``mlp`` (the feed-forward, or null).
Mixer ``latent_attention``: ``heads, dim, rot_dim, vdim, kv_rank, scale``, ``rot`` = {``base, dims``,
optional ``scaling`` = {``factor, original, fast, slow``}} and optionally ``kv_from`` (the layer whose
latent cache this layer reads instead of keeping its own).  Feed-forward ``dense``: ``ff``; ``moe``:
``expert.ff`` and ``router`` = {``experts, top, scale``}.

The design: token embedding times a constant, then a Dynamic-Tanh norm on the residual stream; every
layer norms each sublayer's input AND its output with Dynamic Tanh; latent attention with a decoupled
rotary key part and an output gate; feed-forwards either dense (erf GELU, two matrices) or routed
experts (sigmoid scores, a correction term for the choice only, gated SiLU experts); a Dynamic-Tanh norm
and an output matrix of its own at the end.  Nothing limits the positions; ``max_positions`` (an
optional key of this library's, 131,072 if absent) only sizes the page lists.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, KeyReader, LayerSpec, ModelPlan, PartSpec, ScheduleEntry

MIXERS = ("latent_attention",)
DEFAULT_MAX_POSITIONS = 1 << 17


def _sub(reader: KeyReader, key: str) -> KeyReader:
    value = reader.raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{reader.where}: key '{key}' must be an object")
    return KeyReader(value, f"{reader.where}: {key}")


@dataclass(frozen=True)
class ForisunConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: tuple                     # the checked raw entries
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = "Forisun"

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "ForisunConfig":
        r = KeyReader(raw)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: key 'layers' must be a list with at least one layer")
        for i, layer in enumerate(layers):
            cls._check_layer(i, layer, layers)
        return cls(vocab=r.integer("vocab"), width=r.integer("width"),
                   embedding_scale=_sub(r, "embedding").number("scale", positive=False),
                   norm_eps=_sub(r, "norm").number("eps"), layers=tuple(layers),
                   max_positions=r.integer("max_positions", default=DEFAULT_MAX_POSITIONS))

    @staticmethod
    def _check_layer(i: int, layer, layers) -> None:
        where = f"config.json: layers[{i}]"
        lr = KeyReader(layer, where)
        lr.string("type", choices=MIXERS)
        m = _sub(lr, "mixer")
        for key in ("heads", "dim", "vdim", "kv_rank"):
            m.integer(key)
        m.integer("rot_dim", minimum=0)
        m.number("scale")
        rot = _sub(m, "rot")
        rot.number("base")
        dims = rot.integer("dims", minimum=0)
        if dims % 2 or dims > m.integer("rot_dim", minimum=0):
            raise ConfigError(f"{where}: rot.dims {dims} must be even and at most rot_dim")
        if rot.raw.get("scaling") is not None:
            sc = _sub(rot, "scaling")
            for key in ("factor", "original", "fast", "slow"):
                sc.number(key)
        src = m.raw.get("kv_from")
        if src is not None:
            src = m.integer("kv_from", minimum=0)
            if src >= i or layers[src].get("mixer", {}).get("kv_from") is not None:
                raise ConfigError(f"{where}: kv_from {src} must name an earlier layer that keeps its own cache")
            other = layers[src]["mixer"]
            if any(other.get(k) != m.raw.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                raise ConfigError(f"{where}: kv_from {src} differs in kv_rank, rot_dim or rot")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        f = KeyReader(mlp, where + ": mlp")
        if f.string("kind", choices=("dense", "moe")) == "dense":
            f.integer("ff")
        else:
            _sub(f, "expert").integer("ff")
            router = _sub(f, "router")
            n, top = router.integer("experts"), router.integer("top")
            router.number("scale")
            if top > n:
                raise ConfigError(f"{where}: mlp.router.top {top} exceeds its {n} experts")

    def to_json(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": [dict(layer) for layer in self.layers]}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    def init_distribution(self, rule: str):
        """(mean, standard deviation) of a random-weights rule: matrices N(0, 1/width), Dynamic Tanh's
        alpha near one half, other norm parameters near 1 and 0."""
        r = 1.0 / math.sqrt(self.width)
        rules = {"normal": (0.0, r), "residual_projection": (0.0, r), "bias": (0.0, 0.05),
                 "norm_weight": (1.0, 0.05), "norm_bias": (0.0, 0.05), "norm_alpha": (0.5, 0.02)}
        if rule not in rules:
            raise ConfigError(f"no random-weights rule '{rule}'")
        return rules[rule]

    # ------------------------------------------------------------------ plan
    def _norm(self, name: str) -> PartSpec:
        return PartSpec("dynamic_tanh", {"size": self.width},
                        {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})

    def plan(self) -> ModelPlan:
        D = self.width
        layers, schedule, ignored = [], [], []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer["mixer"]
            src = m.get("kv_from")
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": D, "n_heads": int(m["heads"]), "dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
                 "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "softmax_scale": float(m["scale"]),
                 "eps": self.norm_eps, "rot": m["rot"], "own_kv": src is None},
                {"q": p + "mix.q", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk",
                 "uv": p + "mix.uv", "gate": p + "mix.g", "out": p + "mix.o"})
            extra = [("norm1b", "norm", self._norm(p + "norm1b"))]
            mlp = layer.get("mlp")
            if mlp is None:
                norm2, ffn = PartSpec("identity"), PartSpec("none")
                ignored.append(rf"l{i}\.norm2b?(\.b|\.alpha)?")       # a file may carry them all the same
            else:
                norm2 = self._norm(p + "norm2")
                extra.append(("norm2b", "norm", self._norm(p + "norm2b")))
                if mlp["kind"] == "dense":
                    ffn = PartSpec("dense_ffn", {"hidden_size": D, "inner_size": int(mlp["ff"]), "activation": "gelu",
                                                 "bias": False},
                                   {"up_weight": p + "mlp.up", "down_weight": p + "mlp.down"})
                else:
                    router = mlp["router"]
                    ffn = PartSpec("routed_experts",
                                   {"hidden_size": D, "inner_size": int(mlp["expert"]["ff"]),
                                    "n_experts": int(router["experts"]), "top": int(router["top"]),
                                    "router_scale": float(router["scale"]), "score": "sigmoid", "renormalize": False,
                                    "correction": True},
                                   {"router": p + "mlp.router", "correction": p + "mlp.correction",
                                    "gate": p + "mlp.e{e}.gate", "up": p + "mlp.e{e}.up", "down": p + "mlp.e{e}.down"})
            layers.append(LayerSpec("sandwich_norm", self._norm(p + "norm1"), mixer, norm2, ffn, extra=tuple(extra)))
            schedule.append(ScheduleEntry(layer=i, cache_of=i if src is None else int(src)))
        plan = ModelPlan(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=D, max_positions=self.max_positions,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": D,
                                                   "scale": self.embedding_scale}, {"weight": "embed"}),
            position=PartSpec("none"), layers=tuple(layers), schedule=tuple(schedule),
            final_norm=self._norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": D}, {"weight": "head"}),
            embedding_norm=self._norm("embed.norm"), ignored_tensors=tuple(ignored))
        plan.validate()
        return plan
