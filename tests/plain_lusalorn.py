"""A plain, slow statement of the Lusalorn design in NumPy float64, one function per mechanism.

It shares no code with the package: the tests hold the package's kernels, cache and scheduler to
these functions.  A model is a dict ``config`` (the JSON of config.json) and a dict ``w`` of arrays by
tensor name.  Everything works on one whole sequence (positions 0..T-1); what a cache or a state
would hold is simply recomputed.

Notation: x the residual stream [T, D]; h a sublayer's input (x itself: the design norms outputs,
not inputs); H query heads, G key/value heads; d the query/key size of one score map, d_v the value
size; for the state-space mixer P the head size, N the state size.
"""
import math

import numpy as np

F = np.float64


# ------------------------------------------------------------------ elementwise
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


# ------------------------------------------------------------------ embedding
def embedding(tokens, w, big):
    """Token rows plus hashed rows of the pair (token before, token); the first token of a sequence
    takes the table's last row."""
    tokens = np.asarray(tokens, dtype=np.int64)
    buckets = int(big["buckets"])
    rows = np.empty(len(tokens), dtype=np.int64)
    rows[0] = buckets
    rows[1:] = (tokens[:-1] * int(big["mul_prev"]) + tokens[1:] * int(big["mul_cur"])) % buckets
    return w["embed"][tokens] + w["bigram"][rows]


# ------------------------------------------------------------------ rotary positions
def rotary_frequencies(rot):
    """(frequencies [dims/2], magnitude).  Plain: f_i = base^(-2i/dims), magnitude 1.  With ``scaling``
    = {factor, original, fast, slow}: dimensions that turn often within the original length keep f_i,
    those that turn rarely get f_i / factor, a linear ramp in between; cos and sin grow by
    0.1 ln(factor) + 1."""
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
    """Rotates the first ``rot.dims`` entries of the last axis of v [T, ..., n]; entry i turns with
    entry i + dims/2; the rest of the axis passes unchanged."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=F)[:, None] * f[None, :]
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (half,)
    cos, sin = (np.cos(ang) * mag).reshape(shape), (np.sin(ang) * mag).reshape(shape)
    out = np.array(v, dtype=F, copy=True)
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


# ------------------------------------------------------------------ attention
def softmax_attention(q, k, v, scale, window):
    """q [T, H, d], k [T, G, d], v [T, G, d_v] -> [T, H, d_v]; query i sees key j with 0 <= i - j
    (and i - j < window when there is one)."""
    T, H, _ = q.shape
    G = k.shape[1]
    kv_of = np.arange(H) // (H // G)
    s = np.einsum("ihd,jhd->hij", q, k[:, kv_of]) * scale
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (j <= i) if not window else ((j <= i) & (i - j < window))
    s = np.where(seen[None], s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    a = e / e.sum(axis=-1, keepdims=True)
    return np.einsum("hij,jhd->ihd", a, v[:, kv_of])


def normed_rotated(y, weight, positions, rot, eps):
    """Per head (and map): unit rms over the last axis times ``weight``, then the rotation."""
    return rotate(unit_rms(y, eps) * weight, positions, rot)


def attention_kv(h, positions, m, w, p, eps, maps, bias):
    """What an attention layer keeps per position: keys after norm and rotation [T, G, maps, d] and
    values [T, G, d_v]."""
    T = h.shape[0]
    G, d, dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = h @ w[p + "k"].T + (w[p + "k.b"] if bias else 0.0)
    v = h @ w[p + "v"].T + (w[p + "v.b"] if bias else 0.0)
    k = normed_rotated(k.reshape(T, G, maps, d), w[p + "k.norm"], positions, m["rot"], eps)
    return k, v.reshape(T, G, dv)


def differential_attention(h, positions, m, w, p, eps, kv):
    """Two score maps per head over the same values, a2 taken off a1 with one factor per layer, then
    each head's output brought to unit rms and scaled by 1 - diff."""
    T = h.shape[0]
    H, d, dv, diff = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["diff"])
    k, v = kv
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, 2, d)
    q = normed_rotated(q, w[p + "q.norm"], positions, m["rot"], eps)
    window = int(m["mask"]["size"])
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, float(m["scale"]), window)
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, float(m["scale"]), window)
    lam = math.exp(float(np.sum(w[p + "lq1"] * w[p + "lk1"]))) - math.exp(float(np.sum(w[p + "lq2"] * w[p + "lk2"]))) + diff
    o = unit_rms(a1 - lam * a2, eps) * (1.0 - diff)
    return o.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def causal_attention(h, positions, m, w, p, eps):
    """Grouped-query attention with normed, rotated queries and keys; every earlier position is seen."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    k, v = attention_kv(h, positions, m, w, p, eps, 1, False)
    q = normed_rotated((h @ w[p + "q"].T).reshape(T, H, d), w[p + "q.norm"], positions, m["rot"], eps)
    o = softmax_attention(q, k[:, :, 0], v, float(m["scale"]), 0)
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------------ state-space mixer
def short_convolution(u, weight, bias):
    """Per channel over time, zeros before the start: out_t = bias + sum_j weight[:, j] u_(t - taps + 1 + j)."""
    T, taps = u.shape[0], weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1]), dtype=F), u], axis=0)
    out = np.tile(bias, (T, 1)).astype(F)
    for j in range(taps):
        out += padded[j:j + T] * weight[:, j]
    return out


def state_space(h, m, w, p, eps):
    """Per head a matrix state S [N, P]: S_t = exp(-exp(A) dt_t) S_(t-1) + dt_t B_t x_t^T,
    y_t = S_t^T C_t + D x_t; then the gate, a unit rms per group of channels, a weight, the output matrix."""
    T = h.shape[0]
    Hs, P, N, G = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"])
    inner = Hs * P
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hs, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    rate = np.exp(w[p + "A_log"])
    y = np.zeros((T, Hs, P), dtype=F)
    for hd in range(Hs):
        g = hd // (Hs // G)
        S = np.zeros((N, P), dtype=F)
        for t in range(T):
            S = math.exp(-rate[hd] * dt[t, hd]) * S + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward, layers, model
def gated_ff(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def output_norm(y, w, name, eps):
    """The norm of a sublayer's output: unit rms times (1 + weight)."""
    return unit_rms(y, eps) * (1.0 + w[name])


def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the residual stream
    after every layer."""
    w = {k: np.asarray(v, dtype=F) for k, v in w.items()}
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    positions = np.arange(len(tokens))
    x = embedding(tokens, w, config["embedding"]["bigram"])
    kept = {}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = attention_kv(x, positions, m, w, p, eps, 2, True)
            y = differential_attention(x, positions, m, w, p, eps, kept[i if src is None else int(src)])
        elif layer["type"] == "parallel":
            y = (float(m["left_scale"]) * causal_attention(x, positions, m["left"], w, p + "left.", eps)
                 + float(m["right_scale"]) * state_space(x, m["right"], w, p + "right.", eps))
        else:
            raise ValueError(layer["type"])
        x = x + mult * output_norm(y, w, f"l{i}.norm1", eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            x = x + mult * output_norm(gated_ff(x, w, f"l{i}.mlp."), w, f"l{i}.norm2", eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return output_norm(x, w, "final.norm", eps) @ w["head"].T


# ------------------------------------------------------------------ random models for tests
def tensor_shapes(config):
    """name -> shape of every tensor a model of this configuration has."""
    D, V = int(config["width"]), int(config["vocab"])
    out = {"embed": (V, D), "bigram": (int(config["embedding"]["bigram"]["buckets"]) + 1, D),
           "final.norm": (D,), "head": (V, D)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (D,)
        if layer["type"] == "attention":
            H, G, d, dv = (int(m[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            q = p + "mix."
            out[q + "q"], out[q + "q.b"], out[q + "q.norm"] = (H * 2 * d, D), (H * 2 * d,), (d,)
            if m.get("kv_from") is None:
                out[q + "k"], out[q + "k.b"], out[q + "k.norm"] = (G * 2 * d, D), (G * 2 * d,), (d,)
                out[q + "v"], out[q + "v.b"] = (G * dv, D), (G * dv,)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[q + n] = (d,)
            out[q + "o"], out[q + "o.b"] = (D, H * dv), (D,)
        else:
            a, s = m["left"], m["right"]
            H, G, d, dv = (int(a[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            q = p + "mix.left."
            out[q + "q"], out[q + "k"], out[q + "v"] = (H * d, D), (G * d, D), (G * dv, D)
            out[q + "q.norm"], out[q + "k.norm"], out[q + "o"] = (d,), (d,), (D, H * dv)
            Hs, P, N, Gs, taps = (int(s[k]) for k in ("heads", "vdim", "state", "groups", "conv"))
            q = p + "mix.right."
            inner, ch = Hs * P, Hs * P + 2 * Gs * N
            out[q + "in"] = (2 * inner + 2 * Gs * N + Hs, D)
            out[q + "conv"], out[q + "conv.b"] = (ch, taps), (ch,)
            out[q + "dt_bias"], out[q + "A_log"], out[q + "D"] = (Hs,), (Hs,), (Hs,)
            out[q + "norm"], out[q + "o"] = (inner,), (D, inner)
        if layer.get("mlp") is not None:
            ff = int(layer["mlp"]["ff"])
            out[p + "norm2"] = (D,)
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (ff, D), (ff, D), (D, ff)
    return out


def round_bf16(v):
    v = np.ascontiguousarray(v, dtype=np.float32)
    bits = v.view(np.uint32).astype(np.uint64)
    bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return bits.astype(np.uint32).view(np.float32).reshape(v.shape)


def random_weights(config, seed, bf16=True):
    """Random weights scaled so that activations stay of order one through the layers; rounded to
    bfloat16 values (kept as float32 arrays) so that a bfloat16 file holds exactly these numbers."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        last = name.rsplit(".", 1)[-1]
        if name in ("embed", "bigram"):
            v = rng.normal(0.0, 0.5, shape)
        elif name.endswith(("q.norm", "k.norm")) or name.endswith("right.norm"):
            v = 1.0 + rng.normal(0.0, 0.2, shape)
        elif last in ("norm1", "norm2") or name == "final.norm":
            v = rng.normal(0.0, 0.2, shape)                   # stored around zero
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            v = rng.normal(0.0, 0.3, shape)
        elif last == "b":
            v = rng.normal(0.0, 0.1, shape)
        elif last == "dt_bias":
            v = rng.uniform(-3.0, 0.5, shape)
        elif last == "A_log":
            v = rng.uniform(-1.0, 1.5, shape)
        elif last == "D":
            v = rng.normal(1.0, 0.3, shape)
        elif last == "conv":
            v = rng.normal(0.0, 0.5, shape)
        else:
            v = rng.normal(0.0, 1.0 / math.sqrt(shape[1]), shape) * (2.0 if last in ("q", "k") else 1.0)
        w[name] = round_bf16(v) if bf16 else np.asarray(v, dtype=np.float32)
    return w
