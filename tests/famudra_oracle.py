"""Plain, slow restatement of the Famudra design for the tests: one function per mechanism, numpy only, whole sequences
at once (no cache, no state carried between calls), nothing shared with the code under nano_b200/.

Notation: x [T, E] is the residual stream of one sequence, W matrices are [out, in] and act as h @ W.T.  `dt` is the numpy
float type everything is computed in (float64 gives a reference that rounding does not touch).
"""
import math

import numpy as np


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis (eps under the root)."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is one number for all coordinates."""
    return rms_unit(x, eps) * g


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu per coordinate, h_{-1} = 0; the previous h is the one before this replacement."""
    prev = np.zeros_like(h)
    prev[1:] = h[:-1]
    return h + (prev - h) * mu


def causal_conv(v, taps, bias):
    """Per-channel causal convolution: taps [C, K], the last column multiplies the current token, zeros before the start."""
    T, C = v.shape
    K = taps.shape[1]
    out = np.tile(bias, (T, 1)).astype(v.dtype)
    for j in range(K):                      # column j looks K-1-j tokens back
        back = K - 1 - j
        if back < T:
            out[back:] += v[: T - back] * taps[:, j]
    return out


def rglru_mixer(h, w, blocks):
    """Recurrent block with a real-gated linear recurrent unit.  w: dict of the mixer's tensors by their short names."""
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    u = causal_conv(h @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    T, C = u.shape
    bs = C // blocks
    r = np.empty_like(u)
    i = np.empty_like(u)
    for b in range(blocks):
        ub = u[:, b * bs:(b + 1) * bs]
        r[:, b * bs:(b + 1) * bs] = sigmoid(ub @ w["ra"][b].T + w["ra.b"][b])
        i[:, b * bs:(b + 1) * bs] = sigmoid(ub @ w["ri"][b].T + w["ri.b"][b])
    log_a = -8.0 * r * softplus(w["lam"])
    a = np.exp(log_a)
    drive = np.sqrt(1.0 - a * a) * i * u
    S = np.zeros(C, dtype=h.dtype)
    out = np.empty_like(u)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ w["o"].T


def latent_attention_mixer(h, w, heads, dim, vdim, scale, eps):
    """Attention whose queries and keys/values both pass through normed low-rank latents; no positions; causal softmax."""
    T = h.shape[0]
    cq = rms_unit(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(T, heads, dim)
    c = rms_unit(h @ w["dkv"].T, eps) * w["dkv.norm"]
    k = (c @ w["uk"].T).reshape(T, heads, dim)
    v = (c @ w["uv"].T).reshape(T, heads, vdim)
    out = np.empty((T, heads, vdim), dtype=h.dtype)
    for hd in range(heads):
        s = (q[:, hd] @ k[:, hd].T) * scale
        s = np.where(np.tril(np.ones((T, T), dtype=bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        out[:, hd] = p @ v[:, hd]
    return out.reshape(T, heads * vdim) @ w["o"].T


def expert_ff(h, up, down):
    """down(relu(up h)^2), no biases."""
    a = np.maximum(h @ up.T, 0.0)
    return (a * a) @ down.T


def route(h, router, top):
    """Indices [T, top] of the largest router logits and their weights: softmax over the chosen logits only."""
    z = h @ router.T
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, idx, axis=-1)
    p = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return idx, p / p.sum(axis=-1, keepdims=True)


def moe_ff(h, w, n_experts, top, shared):
    idx, wt = route(h, w["router"], top)
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]), dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wt[t, j] * expert_ff(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if shared:
        out += expert_ff(h, w["shared.up"], w["shared.down"])
    return out


def layer_runs(cfg):
    """Layer indices in the order they run: layers start..stop-1 `times` times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, k = loop["start"], loop["stop"], loop["times"]
    return [(i, 0) for i in range(a)] + [(i, p) for p in range(k) for i in range(a, b)] + [(i, 0) for i in range(b, n)]


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens, dt=np.float64, trace=None):
    """Logits [T, vocab] of one whole sequence.  weights: name -> array.  trace (a list) receives x after every layer run."""
    W = {k: np.asarray(v).astype(dt) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][np.asarray(tokens)]
    x = x0.copy()
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    for (i, p) in layer_runs(cfg):
        if p > 0 and i == loop["start"]:
            x = x + x0
        L = cfg["layers"][i]
        pre = f"l{i}."
        h = token_shift(scalar_norm(x, W[pre + "norm1"], eps), W[pre + "shift"])
        m = L["mixer"]
        mw = sub(W, pre + "mix.")
        if L["type"] == "rglru":
            d = rglru_mixer(h, mw, m["blocks"])
        elif L["type"] == "latent_attention":
            d = latent_attention_mixer(h, mw, m["heads"], m["dim"], m["vdim"], m["scale"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            f = L["mlp"]
            h2 = scalar_norm(x, W[pre + "norm2"], eps)
            d = d + moe_ff(h2, sub(W, pre + "mlp."), f["router"]["experts"], f["router"]["top"], bool(f.get("shared")))
        x = x + d
        if trace is not None:
            trace.append(x.copy())
    return scalar_norm(x, W["final.norm"], eps) @ W["head"].T
