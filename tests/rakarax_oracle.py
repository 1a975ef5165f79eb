"""Plain, slow restatement of the Rakarax design for the tests: one function per mechanism, numpy only, whole sequences at once
(no cache, no state carried between calls), nothing shared with the code under nano_b200/.

Notation: x [T, E] is the residual stream of one sequence, W matrices are [out, in] and act as h @ W.T.  `dt` is the numpy float
type everything is computed in (float64 gives a reference that rounding does not touch).
"""
import math

import numpy as np


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps under the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose stored gain sits around zero: the unit vector times (1 + w)."""
    return rms_unit(x, eps) * (1.0 + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def causal_conv(v, taps, bias=None):
    """Per-channel causal convolution: taps [C, K], the last column multiplies the current token, zeros before the start."""
    T, C = v.shape
    K = taps.shape[1]
    out = np.zeros_like(v) if bias is None else np.tile(bias, (T, 1)).astype(v.dtype)
    for j in range(K):                      # column j looks K-1-j tokens back
        back = K - 1 - j
        if back < T:
            out[back:] += v[: T - back] * taps[:, j]
    return out


def rotate_half(x, dims, base):
    """x [T, H, D]: the first `dims` coordinates of every head turn by angle p * base^(-2i/dims), coordinate i paired with
    i + dims/2; the remaining coordinates pass."""
    T = x.shape[0]
    half = dims // 2
    freq = np.asarray(base, np.float64) ** (-2.0 * np.arange(half) / dims)
    ang = np.arange(T)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :].astype(x.dtype), np.sin(ang)[:, None, :].astype(x.dtype)
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def retention_mixer(h, w, m, eps):
    """Linear attention with one fixed decay per head, no softmax and no denominator; rotary positions on q and k; per-head
    unit-RMS output times a silu gate."""
    T = h.shape[0]
    H, D, VD = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, D)
    k = (h @ w["k"].T).reshape(T, H, D)
    v = (h @ w["v"].T).reshape(T, H, VD)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, rot["dims"], rot["base"])
        k = rotate_half(k, rot["dims"], rot["base"])
    k = k * D ** -0.5
    decay = np.asarray(m["decay"], h.dtype)
    S = np.zeros((H, D, VD), h.dtype)
    o = np.empty((T, H, VD), h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * VD)
    return (o * silu(h @ w["g"].T)) @ w["o"].T


def window_attention(h, w, m, eps):
    """Grouped-query softmax attention inside a sliding window.  q and k pass a short causal convolution; the value IS the
    convolved key (before its norm); q and k are unit-RMS per head; the score is scaled, given a per-head temperature, soft-capped,
    lowered by a per-head slope times the distance, and then mixed ACROSS heads by a square matrix before the softmax; the
    concatenated heads are gated by sigmoid(W_g h)."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = causal_conv(h @ w["q"].T, w["q.conv"]).reshape(T, H, D)
    k = causal_conv(h @ w["k"].T, w["k.conv"]).reshape(T, G, D)
    v = k
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    rep = H // G
    kk = np.repeat(k, rep, axis=1)                      # query head h reads key/value head h // rep
    s = np.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    s = s * w["temp"][:, None, None]
    cap = m.get("softcap")
    if cap:
        s = cap * np.tanh(s / cap)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    slope = 2.0 ** (-8.0 * (np.arange(H) + 1) / H)
    s = s - slope[:, None, None] * (i - j)[None]
    s = np.einsum("hg,gij->hij", w["talk"], s)
    seen = (j <= i)
    if m.get("mask"):
        seen = seen & (i - j < m["mask"]["size"])
    s = np.where(seen[None], s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(-1, keepdims=True)
    o = np.einsum("hij,jhd->ihd", p, np.repeat(v, rep, axis=1)).reshape(T, H * D)
    return (o * sigmoid(h @ w["g"].T)) @ w["o"].T


def selective_scan_mixer(h, w, m):
    """Mamba: x and z from one projection; x through a causal convolution with bias and silu; step size, B and C from x; a
    diagonal state per channel that decays by exp(dt A) and is driven by dt x B; read out by C, plus D x; gated by silu(z)."""
    T = h.shape[0]
    C, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w["in"].T
    x, z = xz[:, :C], xz[:, C:]
    x = silu(causal_conv(x, w["conv"], w["conv.b"]))
    dbc = x @ w["x"].T
    dt = softplus(dbc[:, :R] @ w["dt"].T + w["dt.b"])
    B, Cm = dbc[:, R:R + N], dbc[:, R + N:]
    A = -np.exp(w["A_log"])
    S = np.zeros((C, N), h.dtype)
    y = np.empty((T, C), h.dtype)
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + w["D"] * x[t]
    return (y * silu(z)) @ w["o"].T


def parallel_mixer(h, w, m, eps):
    """Two mixers on the same input, their outputs added with fixed scales."""
    left = window_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps)
    right = selective_scan_mixer(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"])
    return m["left_scale"] * left + m["right_scale"] * right


def polynorm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, N = unit RMS over the feed-forward width."""
    a, b, c, e = coef
    return a * rms_unit(z, eps) + b * rms_unit(z * z, eps) + c * rms_unit(z * z * z, eps) + e


def dense_ff(h, w, eps):
    return polynorm(h @ w["up"].T, w["act"], eps) @ w["down"].T


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, dt=np.float64, trace=None):
    """Logits [T, vocab] of one sequence.  trace (a list) receives the residual stream after every layer."""
    W = {k: np.asarray(v).astype(dt) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    T = len(tokens)
    x = W["embed"][np.asarray(tokens, np.int64)] + W["pos"][:T]
    for i, L in enumerate(config["layers"]):
        p = "l%d." % L.get("weights_of", i)
        lw = sub(W, p)
        h = offset_norm(x, lw["norm1"], eps)
        mw = sub(lw, "mix.")
        if L["type"] == "retention":
            d = retention_mixer(h, mw, L["mixer"], eps)
        elif L["type"] == "parallel":
            d = parallel_mixer(h, mw, L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + offset_norm(d, lw["norm1b"], eps)
        if L.get("mlp"):
            d = dense_ff(offset_norm(x, lw["norm2"], eps), sub(lw, "mlp."), eps)
            x = x + offset_norm(d, lw["norm2b"], eps)
        if trace is not None:
            trace.append(x.copy())
    return offset_norm(x, W["final.norm"], eps) @ W["head"].T
