"""A plain, slow float64 NumPy implementation of the Zurerax decoder, one function per mechanism, written from the
design's equations and sharing no code with the engine. It always runs a whole sequence from position 0 with no
cache and no state: what the engine computes in portions, in batches and through its cache must equal it.

Notation: T tokens, H heads, D key (or unrotated query) size, V value size, C latent size, R rotated size.
"""
import numpy as np


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(x):
    return x / (1.0 + np.exp(-x))


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def softplus(x):
    return np.logaddexp(0.0, x)


def causal_conv(x, w):
    """x [T, channels], w [channels, taps] with the current token's weight in the last column; zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = np.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y


def delta_rule(q, k, v, g, beta):
    """q, k [T, H, D] (already unit vectors, q scaled), v [T, H, V], g [T, H, D] decays, beta [T, H]. Returns o [T, H, V]."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = np.zeros((H, D, V))
    o = np.zeros((T, H, V))
    for t in range(T):
        for h in range(H):
            S[h] = g[t, h][:, None] * S[h]
            u = beta[t, h] * (v[t, h] - S[h].T @ k[t, h])
            S[h] = S[h] + np.outer(k[t, h], u)
            o[t, h] = S[h].T @ q[t, h]
    return o


def channel_delta_mixer(h, W, p, m, eps):
    """h [T, width]; W: tensors by name; p: the mixer's name prefix; m: its sizes."""
    T = h.shape[0]
    H, KH, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, KH, D)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, KH, D)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt(np.sum(q * q, -1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt(np.sum(k * k, -1, keepdims=True) + 1e-6)
    group = H // KH
    q, k = np.repeat(q, group, axis=1), np.repeat(k, group, axis=1)          # head h uses q/k head floor(h / group)
    beta = sigmoid(h @ W[p + "b"].T)
    a = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * softplus(a).reshape(T, H, D))
    gate = sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, V)
    o = delta_rule(q, k, v, g, beta)
    o = rms_unit(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * V) @ W[p + "o"].T


def rotate_interleaved(x, positions, base, dims):
    """Rotate the first ``dims`` numbers of the last axis, pair (2i, 2i+1) by the angle position * base^(-2i/dims)."""
    out = np.array(x, dtype=np.float64, copy=True)
    for i in range(dims // 2):
        a = positions * base ** (-2.0 * i / dims)
        a = a.reshape((-1,) + (1,) * (x.ndim - 2))
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * np.cos(a) - v * np.sin(a)
        out[..., 2 * i + 1] = v * np.cos(a) + u * np.sin(a)
    return out


def latent_kv(h, W, p, m, eps):
    """The latent (normed) and the rotated shared key part of every token: what the cache holds."""
    T, C = h.shape[0], m["kv_rank"]
    both = h @ W[p + "dkv"].T
    latent = rms_unit(both[:, :C], eps) * W[p + "dkv.norm"]
    key_rot = rotate_interleaved(both[:, C:], np.arange(T, dtype=np.float64), m["rot"]["base"], m["rot"]["dims"])
    return latent, key_rot


def softmax_with_sink(scores, sink):
    """scores [T, T] with -inf where masked; the denominator also holds exp(sink)."""
    mx = np.maximum(scores.max(-1), sink)
    e = np.exp(scores - mx[:, None])
    return e / (e.sum(-1) + np.exp(sink - mx))[:, None]


def latent_attention_mixer(h, W, p, m, eps, kv=None):
    """kv: (latent, rotated key part) of the layer whose cache this one reads, or None to project its own."""
    T = h.shape[0]
    H, D, R, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    if kv is None:
        kv = latent_kv(h, W, p, m, eps)
    latent, key_rot = kv
    q = (h @ W[p + "q"].T).reshape(T, H, D + R)
    q_rot = rotate_interleaved(q[..., D:], np.arange(T, dtype=np.float64), m["rot"]["base"], m["rot"]["dims"])
    keys = (latent @ W[p + "uk"].T).reshape(T, H, D)
    values = (latent @ W[p + "uv"].T).reshape(T, H, V)
    visible = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, V))
    for head in range(H):
        s = (q[:, head, :D] @ keys[:, head].T + q_rot[:, head] @ key_rot.T) * m["scale"]
        s = np.where(visible, s, -np.inf)
        out[:, head] = softmax_with_sink(s, W[p + "sink"][head]) @ values[:, head]
    return out.reshape(T, H * V) @ W[p + "o"].T, kv


def squared_relu_ffn(h, up, down):
    return np.square(np.maximum(h @ up.T, 0.0)) @ down.T


def forward(cfg, W, tokens, residual_after_layers=None):
    """Logits [T, vocab] of a whole sequence. ``W``: float64 arrays by tensor name."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, W[p + "norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "channel_delta":
            y = channel_delta_mixer(h, W, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            source = m.get("kv_from")
            y, kv = latent_attention_mixer(h, W, p + "mix.", m, eps, kept[source] if source is not None else None)
            kept[i] = kv
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = offset_norm(x, W[p + "norm2"], eps)
            x = x + offset_norm(squared_relu_ffn(h, W[p + "mlp.up"], W[p + "mlp.down"]), W[p + "norm2b"], eps)
        if residual_after_layers is not None:
            residual_after_layers.append(x.copy())
    return offset_norm(x, W["final.norm"], eps) @ W["head"].T * cfg["logit_scale"]
