"""The Roritar design once more, plain and slow: NumPy float64, whole sequences, no cache, no state carried between
calls, one function per mechanism.  It shares no code with the library; the tests compare the engine with it.  A model
is a dict ``cfg`` (the parsed config.json) and a dict ``w`` of float64 arrays by tensor name.

``round16`` rounds the operands of the large matrix products to bfloat16, as the bfloat16 engine does; everything
else stays in float64.
"""
from __future__ import annotations

import math

import numpy as np

GATE_SHARPNESS = 8.0          # log a = -GATE_SHARPNESS * r * softplus(lam)


# ----------------------------------------------------------------------------- small pieces
def round_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def product(x, W, round16=False):
    """Rows of x times W [out, in] transposed."""
    x = round_bf16(x) if round16 else np.asarray(x, dtype=np.float64)
    return x @ np.asarray(W, dtype=np.float64).T


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2."""
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (np.expm1(np.minimum(z, 0.0)) - z) + 0.5 * z
    return np.where(z > 0, pos, neg)


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight over the last axis; var is the mean squared deviation; no bias."""
    mu = x.mean(axis=-1, keepdims=True)
    d = x - mu
    return d / np.sqrt((d * d).mean(axis=-1, keepdims=True) + eps) * weight


def rms_norm(x, weight, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * weight


def causal_conv(x, taps_w, bias):
    """x [T, C]; taps_w [C, taps], the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    n = taps_w.shape[1]
    padded = np.concatenate([np.zeros((n - 1, C)), x], axis=0)
    out = np.zeros((T, C))
    for j in range(n):
        out += padded[j:j + T] * taps_w[:, j][None, :]
    return out + bias[None, :]


# ----------------------------------------------------------------------------- rotation
def turn(x, positions, base, dims, layout="halves", sign=1.0):
    """x [T, heads, n]: the first ``dims`` values of each head turned by sign * position * base^(-2i/dims) for pair i.
    halves: i with i + dims/2; interleaved: 2i with 2i + 1.  The rest passes unchanged."""
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    ang = sign * np.asarray(positions, dtype=np.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = np.array(x, dtype=np.float64, copy=True)
    if layout == "halves":
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    else:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- mixers
def rglru_scan(u, r, i, lam, sharpness=GATE_SHARPNESS):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0, a_t = exp(-sharpness r_t softplus(lam)).  All [T, C]."""
    a = np.exp(-sharpness * r * softplus(lam)[None, :])
    S = np.zeros(u.shape[1])
    out = np.zeros_like(u)
    for t in range(u.shape[0]):
        S = a[t] * S + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return out


def block_gate(u, mats, bias):
    """u [T, C] cut into len(mats) equal parts; part b goes through mats[b] [out, in] plus bias[b]; sigmoid."""
    nb, n = mats.shape[0], mats.shape[1]
    parts = u.reshape(u.shape[0], nb, n)
    z = np.einsum("tbi,boi->tbo", parts, mats) + bias[None]
    return sigmoid(z).reshape(u.shape)


def rglru_mixer(h, w, px, m, round16=False):
    y = gelu_tanh(product(h, w[px + "y"], round16) + w[px + "y.b"][None, :])
    u = causal_conv(product(h, w[px + "x"], round16) + w[px + "x.b"][None, :], w[px + "conv"], w[px + "conv.b"])
    r = block_gate(u, w[px + "ra"], w[px + "ra.b"])
    i = block_gate(u, w[px + "ri"], w[px + "ri.b"])
    S = rglru_scan(u, r, i, w[px + "lam"])
    return product(S * y, w[px + "o"], round16)


def visible(i, size, pool):
    """(first token of the window, number of pooled blocks) that position i sees."""
    first = max(0, i - size + 1)
    blocks = 0 if not pool else max(0, (i - size + 1) // pool)
    return first, blocks


def pooled_window_attention(h, w, px, m, eps, round16=False, layout="halves"):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size = m["mask"]["size"] if m.get("mask") else 0
    pool = m["mask"].get("pool", 0) if m.get("mask") else 0
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    pos = np.arange(T)
    q = product(h, w[px + "q"], round16).reshape(T, H, dim)
    k = product(h, w[px + "k"], round16).reshape(T, G, dim)
    v = product(h, w[px + "v"], round16).reshape(T, G, vdim)
    q = turn(rms_norm(q, w[px + "q.norm"], eps), pos, base, dims, layout)
    k = turn(rms_norm(k, w[px + "k.norm"], eps), pos, base, dims, layout)
    v = turn(v, pos, base, vdim, layout)
    if round16:
        q, k, v = round_bf16(q), round_bf16(k), round_bf16(v)
    nb = T // pool if pool else 0                  # a block's key and value: the means of its cached keys and values
    kb = k[:nb * pool].reshape(nb, pool, G, dim).mean(axis=1) if nb else np.zeros((0, G, dim))
    vb = v[:nb * pool].reshape(nb, pool, G, vdim).mean(axis=1) if nb else np.zeros((0, G, vdim))
    if round16:
        kb, vb = round_bf16(kb), round_bf16(vb)
    out = np.zeros((T, H, vdim))
    for i in range(T):
        first, blocks = visible(i, size, pool) if size else (0, 0)
        for hh in range(H):
            g = hh // (H // G)
            keys = np.concatenate([kb[:blocks, g], k[first:i + 1, g]])
            vals = np.concatenate([vb[:blocks, g], v[first:i + 1, g]])
            s = keys @ q[i, hh] * m["scale"]
            p = np.exp(s - s.max())
            out[i, hh] = (p / p.sum()) @ vals
    out = turn(out, pos, base, vdim, layout, sign=-1.0)
    return product(out.reshape(T, H * vdim), w[px + "o"], round16)


def dense_ff(h, w, px, round16=False):
    p, q = w[px + "act"]
    return product(xielu(product(h, w[px + "up"], round16), p, q), w[px + "down"], round16)


# ----------------------------------------------------------------------------- the model
def schedule(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(tokens, w, cfg, round16=False, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that gets the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    for li in schedule(cfg):
        layer, px = cfg["layers"][li], f"l{li}."
        hin = layer_norm(x, w[px + "norm1"], eps)
        if layer["type"] == "rglru":
            y = rglru_mixer(hin, w, px + "mix.", layer["mixer"], round16)
        else:
            y = pooled_window_attention(hin, w, px + "mix.", layer["mixer"], eps, round16)
        x = x + layer_norm(y, w[px + "norm1b"], eps)
        if layer.get("mlp"):
            y = dense_ff(layer_norm(x, w[px + "norm2"], eps), w, px + "mlp.", round16)
            x = x + layer_norm(y, w[px + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    z = product(layer_norm(x, w["final.norm"], eps), w["embed"], round16) * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(z / cap) if cap else z
