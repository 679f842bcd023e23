"""A plain, slow statement of the Forisun design in NumPy float64, one function per mechanism.

It shares no code with the package: the tests hold the package's kernels, cache and scheduler to
these functions.  A model is a dict ``config`` (the JSON of config.json) and a dict ``w`` of arrays by
tensor name.  Everything works on one whole sequence (positions 0..T-1); what a cache would hold is
simply recomputed.

Notation: x the residual stream [T, D]; h a sublayer's input; H heads; per head d_n unrotated and d_r
rotated query/key dimensions, d_v value dimensions; r the latent size.
"""
import math

import numpy as np

F = np.float64


# ------------------------------------------------------------------ elementwise
def dynamic_tanh(x, weight, bias, alpha):
    """y = tanh(alpha x) * weight + bias (no statistics of the row)."""
    return np.tanh(F(alpha) * x) * weight + bias


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# ------------------------------------------------------------------ rotary positions
def rotary_frequencies(rot):
    """(frequencies [dims/2], magnitude) of a rotary block ``rot`` = {base, dims, scaling?}.

    Plain: f_i = base^(-2i/dims), magnitude 1.  With ``scaling`` = {factor, original, fast, slow}
    (YaRN): dimensions that turn often within the original length keep f_i, those that turn
    rarely get f_i / factor, a linear ramp in between, and cos and sin grow by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=F) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v, positions, rot):
    """Rotates the first ``rot.dims`` entries of the last axis of v [T, ..., n]; entry i is paired with
    entry i + dims/2.  The rest of the axis passes unchanged."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=F)[:, None] * f[None, :]            # [T, half]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (half,)
    cos, sin = (np.cos(ang) * mag).reshape(shape), (np.sin(ang) * mag).reshape(shape)
    out = np.array(v, dtype=F, copy=True)
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


# ------------------------------------------------------------------ latent attention
def latent_kv(h, positions, m, w, p):
    """What a latent-attention layer keeps per position: the normed latent c [T, r] and the rotated
    shared key part [T, d_r]."""
    r = int(m["kv_rank"])
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :r], w[p + "dkv.norm"], w["__eps__"])
    return c, rotate(down[:, r:], positions, m["rot"])


def latent_attention(h, positions, m, w, p, kv):
    """The mixer's output [T, D] for the whole sequence; ``kv`` = (c, rotated key part) of this layer
    or of the layer it borrows them from."""
    T = h.shape[0]
    H, dn, dr, dv, r = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    c, k_rot = kv
    q = (h @ w[p + "q"].T).reshape(T, H, dn + dr)
    q_n, q_r = q[..., :dn], rotate(q[..., dn:], positions, m["rot"])
    k_n = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    s = (np.einsum("ihd,jhd->hij", q_n, k_n) + np.einsum("ihd,jd->hij", q_r, k_rot)) * float(m["scale"])
    pos = np.asarray(positions)
    s = np.where(pos[None, :, None] >= pos[None, None, :], s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    a = e / e.sum(axis=-1, keepdims=True)
    o = np.einsum("hij,jhd->ihd", a, v).reshape(T, H * dv)
    o = o * sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward
def dense_ff(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def routed_ff(h, mlp, w, p):
    """Every token goes to the ``top`` experts with the largest sigmoid(router) + correction; their
    outputs are weighted by sigmoid(router) * scale, not renormalised."""
    n, top, scale = int(mlp["router"]["experts"]), int(mlp["router"]["top"]), float(mlp["router"]["scale"])
    s = sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    out = np.zeros((h.shape[0], w[p + "e0.down"].shape[0]), dtype=F)
    for t in range(h.shape[0]):
        for e in np.argsort(-choice[t], kind="stable")[:top]:
            q = f"{p}e{e}."
            y = (silu(h[t] @ w[q + "gate"].T) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T
            out[t] += s[t, e] * scale * y
    return out


def feed_forward(h, mlp, w, p):
    if mlp["kind"] == "dense":
        return dense_ff(h, w, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, mlp, w, p)
    raise ValueError(mlp["kind"])


# ------------------------------------------------------------------ the model
def norm(x, w, name):
    return dynamic_tanh(x, w[name], w[name + ".b"], w[name + ".alpha"])


def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the residual stream
    after every layer."""
    w = {k: np.asarray(v, dtype=F) for k, v in w.items()}
    w["__eps__"] = float(config["norm"]["eps"])
    positions = np.arange(len(tokens))
    x = w["embed"][np.asarray(tokens)] * float(config["embedding"]["scale"])
    x = norm(x, w, "embed.norm")
    kept = {}
    for i, layer in enumerate(config["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        m, p = layer["mixer"], f"l{i}."
        h = norm(x, w, p + "norm1")
        if m.get("kv_from") is None:
            kept[i] = latent_kv(h, positions, m, w, p + "mix.")
        y = latent_attention(h, positions, m, w, p + "mix.", kept[i if m.get("kv_from") is None else int(m["kv_from"])])
        x = x + norm(y, w, p + "norm1b")
        if layer.get("mlp") is not None:
            y = feed_forward(norm(x, w, p + "norm2"), layer["mlp"], w, p + "mlp.")
            x = x + norm(y, w, p + "norm2b")
        if layers_out is not None:
            layers_out.append(x.copy())
    return norm(x, w, "final.norm") @ w["head"].T


# ------------------------------------------------------------------ random models for tests
def tensor_shapes(config):
    """name -> shape of every tensor a model of this configuration has."""
    D, V = int(config["width"]), int(config["vocab"])
    out = {"embed": (V, D), "head": (V, D)}

    def add_norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (D,), (D,), ()

    add_norm("embed.norm")
    add_norm("final.norm")
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, dn, dr, dv, r = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.get("mlp") is not None else ()):
            add_norm(p + n)
        out[p + "mix.q"] = (H * (dn + dr), D)
        if m.get("kv_from") is None:
            out[p + "mix.dkv"] = (r + dr, D)
            out[p + "mix.dkv.norm"] = (r,)
        out[p + "mix.uk"], out[p + "mix.uv"] = (H * dn, r), (H * dv, r)
        out[p + "mix.g"], out[p + "mix.o"] = (H * dv, D), (D, H * dv)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            out[p + "mlp.up"], out[p + "mlp.down"] = (int(mlp["ff"]), D), (D, int(mlp["ff"]))
        else:
            n, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
            out[p + "mlp.router"], out[p + "mlp.correction"] = (n, D), (n,)
            for e in range(n):
                out[f"{p}mlp.e{e}.gate"], out[f"{p}mlp.e{e}.up"], out[f"{p}mlp.e{e}.down"] = (ff, D), (ff, D), (D, ff)
    return out


def random_weights(config, seed, bf16=True):
    """Random weights scaled so that activations stay of order one through the layers; rounded to
    bfloat16 values (kept as float32 arrays) so that a bfloat16 file holds exactly these numbers."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        if name.endswith(".alpha"):
            v = np.asarray(rng.uniform(0.4, 0.9))
        elif name.endswith(".correction"):
            v = rng.normal(0.0, 0.1, shape)
        elif len(shape) == 1:
            v = rng.normal(0.0, 0.1, shape) if name.endswith(".b") else 1.0 + rng.normal(0.0, 0.2, shape)
        elif name == "embed":
            v = rng.normal(0.0, 0.5, shape)
        else:
            v = rng.normal(0.0, 1.0 / math.sqrt(shape[1]), shape) * (1.5 if name.endswith((".q", ".dkv", ".uk")) else 1.0)
        v = np.asarray(v, dtype=np.float32)
        if bf16:
            bits = v.view(np.uint32).astype(np.uint64)
            bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
            v = bits.astype(np.uint32).view(np.float32).reshape(v.shape)
        w[name] = v
    return w
