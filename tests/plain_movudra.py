"""The Movudra design once more, plain and slow: NumPy float64, whole sequences, no cache, no state carried
between calls, one function per mechanism.  It shares no code with the library; the tests compare the engine
with it.  A model is a dict ``cfg`` (the parsed config.json) and a dict ``w`` of float64 arrays by tensor name.

``round16`` (None or "bf16") rounds the operands of matrix products to bfloat16, as the bfloat16 engine does;
everything else stays in float64.
"""
from __future__ import annotations

import math

import numpy as np


# ----------------------------------------------------------------------------- small pieces
def round_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(a.shape)


def rounder(round16):
    return round_bf16 if round16 else (lambda a: np.asarray(a, dtype=np.float64))


def matvec_rows(x, W, round16=None):
    """Rows of x times W [out, in] transposed."""
    r = rounder(round16)
    return r(x) @ np.asarray(W, dtype=np.float64).T


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def causal_conv(x, taps_w, bias=None):
    """x [T, C]; taps_w [C, taps], the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    n = taps_w.shape[1]
    padded = np.concatenate([np.zeros((n - 1, C)), x], axis=0)
    out = np.zeros((T, C))
    for j in range(n):
        out += padded[j:j + T] * taps_w[:, j][None, :]
    if bias is not None:
        out = out + bias[None, :]
    return out


# ----------------------------------------------------------------------------- rotation
def yarn_frequencies(dims, base, scaling=None):
    """Per pair i: the angle per position, and the factor on cos and sin."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, freqs, mult):
    """x [T, ..., R]: the first 2 * len(freqs) values of the last axis are pairs (2i, 2i + 1)."""
    out = np.array(x, dtype=np.float64, copy=True)
    n = len(freqs)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (n,)
    c, s = (np.cos(ang) * mult).reshape(shape), (np.sin(ang) * mult).reshape(shape)
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- mixers
def mamba2(h, w, px, m, eps, round16=None):
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = H * P, h.shape[0]
    proj = matvec_rows(h, w[px + "in"], round16)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[px + "conv"], w[px + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    Bm = xbc[:, inner:inner + G * N].reshape(T, G, N)
    Cm = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[px + "dt_bias"][None, :])
    A = -np.exp(w[px + "A_log"])
    y = np.zeros((T, H, P))
    for hd in range(H):
        g = hd // (H // G)
        S = np.zeros((N, P))
        for t in range(T):
            S = math.exp(A[hd] * dt[t, hd]) * S + dt[t, hd] * np.outer(Bm[t, g], x[t, hd])
            y[t, hd] = S.T @ Cm[t, g] + w[px + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[px + "norm"][None, :]
    return matvec_rows(y, w[px + "o"], round16)


def channel_delta(h, w, px, m, eps, round16=None):
    H, Hk, K, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(matvec_rows(h, w[px + "q"], round16), w[px + "q.conv"])).reshape(T, Hk, K)
    k = silu(causal_conv(matvec_rows(h, w[px + "k"], round16), w[px + "k.conv"])).reshape(T, Hk, K)
    v = silu(causal_conv(matvec_rows(h, w[px + "v"], round16), w[px + "v.conv"])).reshape(T, H, P)
    q = q / np.sqrt(np.sum(q * q, -1, keepdims=True) + 1e-6) * K ** -0.5
    k = k / np.sqrt(np.sum(k * k, -1, keepdims=True) + 1e-6)
    beta = sigmoid(matvec_rows(h, w[px + "b"], round16))                               # [T, H]
    a = matvec_rows(matvec_rows(h, w[px + "a1"], round16), w[px + "a2"], round16)       # [T, H * K]
    decay = np.exp(-np.exp(w[px + "A_log"])[None, :, None] * softplus(a + w[px + "dt_bias"][None, :]).reshape(T, H, K))
    gate = sigmoid(matvec_rows(matvec_rows(h, w[px + "g1"], round16), w[px + "g2"], round16)).reshape(T, H, P)
    o = np.zeros((T, H, P))
    for hd in range(H):
        kh = hd // (H // Hk)
        S = np.zeros((K, P))
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + np.outer(k[t, kh], u)
            o[t, hd] = S.T @ q[t, kh]
    o = rms_unit(o, eps) * w[px + "norm"][None, None, :] * gate
    return matvec_rows(o.reshape(T, H * P), w[px + "o"], round16)


def latent_attention(h, w, px, m, eps, round16=None):
    H, K, R, P, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    rot = m["rot"]
    freqs, mult = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    pos = np.arange(T)
    cq = rms_unit(matvec_rows(h, w[px + "dq"], round16), eps) * w[px + "dq.norm"][None, :]
    q = matvec_rows(cq, w[px + "uq"], round16).reshape(T, H, K + R)
    q_plain, q_rot = q[..., :K], rotate_interleaved(q[..., K:], pos, freqs, mult)
    dkv = matvec_rows(h, w[px + "dkv"], round16)
    c = rms_unit(dkv[:, :L], eps) * w[px + "dkv.norm"][None, :]
    k_rot = rotate_interleaved(dkv[:, L:], pos, freqs, mult)                              # [T, R], shared by heads
    k_plain = matvec_rows(c, w[px + "uk"], round16).reshape(T, H, K)
    val = matvec_rows(c, w[px + "uv"], round16).reshape(T, H, P)
    window = m["mask"]["size"] if m.get("mask") else None
    out = np.zeros((T, H, P))
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (j <= i) & ((i - j < window) if window else True)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        s = np.where(seen, s, -np.inf)
        sink = w[px + "sink"][hd]
        mx = np.maximum(s.max(-1, keepdims=True), sink)
        e = np.exp(s - mx)
        out[:, hd] = (e / (e.sum(-1, keepdims=True) + np.exp(sink - mx))) @ val[:, hd]
    return matvec_rows(out.reshape(T, H * P), w[px + "o"], round16)


MIXERS = {"mamba2": mamba2, "channel_delta": channel_delta, "latent_attention": latent_attention}


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(h, w, px, round16=None):
    a = np.maximum(matvec_rows(h, w[px + "up"], round16) + w[px + "up.b"][None, :], 0.0) ** 2
    return matvec_rows(a, w[px + "down"], round16) + w[px + "down.b"][None, :]


def moe_ff(h, w, px, mlp, round16=None):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = matvec_rows(h, w[px + "router"], round16)
    s = np.exp(z - z.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    out = np.zeros((h.shape[0], w[px + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for e in np.argsort(-s[t], kind="stable")[:top]:
            ex = f"{px}e{e}."
            a = silu(matvec_rows(h[t:t + 1], w[ex + "gate"], round16)) * matvec_rows(h[t:t + 1], w[ex + "up"], round16)
            out[t] += s[t, e] * matvec_rows(a, w[ex + "down"], round16)[0]
    return out


# ----------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, round16=None, layers_out=None):
    """Logits [T, vocab] for one sequence; ``layers_out`` (a list) gets the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = np.asarray(w["embed"], dtype=np.float64)[np.asarray(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        px = f"l{i}."
        y = MIXERS[layer["type"]](x, w, px + "mix.", layer["mixer"], eps, round16)
        x = x + rms_unit(y, eps) * w[px + "norm1"][None, :]
        mlp = layer.get("mlp")
        if mlp:
            y = dense_ff(x, w, px + "mlp.", round16) if mlp["kind"] == "dense" else moe_ff(x, w, px + "mlp.", mlp, round16)
            x = x + rms_unit(y, eps) * w[px + "norm2"][None, :]
        if layers_out is not None:
            layers_out.append(x.copy())
    x = rms_unit(x, eps) * w["final.norm"][None, :]
    return matvec_rows(x, w["head"], round16)
