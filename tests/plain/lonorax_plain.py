"""Lonorax in plain float64 NumPy, one function per mechanism, written from the architecture's equations and sharing no
code with the engine. Slow on purpose: every sum is a visible loop or a single matrix product over a whole sequence.

Notation: T tokens, d model width, a sequence's positions count from 0. ``W`` maps tensor names to float64 arrays
(matrices stored [out, in] and applied as W x).
"""
import numpy as np


def logistic(x):
    return 1.0 / (1.0 + np.exp(-np.asarray(x, dtype=np.float64)))


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis; var = mean of squared deviations."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_unit(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (eps inside the root, plain gain)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def rotate_pairs(x, positions, dims, base):
    """Rotate channels (2i, 2i+1), i < dims/2, of x [T, heads, D] by the angle position * base^(-2i/dims)."""
    out = x.copy()
    for i in range(dims // 2):
        ang = np.asarray(positions, dtype=np.float64) * base ** (-2.0 * i / dims)
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def visible(i, j, window):
    """Whether position i sees position j: itself and the window - 1 tokens before it (no window: all earlier ones)."""
    return j <= i and (window is None or i - j < window)


def sigmoid_attention(h, W, p, m, eps):
    """h [T, d] -> [T, d]. Every visible key weighs sigmoid(score + head bias); nothing is normalised over the keys."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, G, D)
    v = (h @ W[p + "v"].T).reshape(T, G, V)
    q, k = rms_unit(q, W[p + "q.norm"], eps), rms_unit(k, W[p + "k.norm"], eps)
    if m.get("rot") is not None:
        pos = np.arange(T)
        q = rotate_pairs(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_pairs(k, pos, m["rot"]["dims"], m["rot"]["base"])
    window = m["mask"]["size"] if m.get("mask") is not None else None
    out = np.zeros((T, H, V))
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            for j in range(i + 1):
                if visible(i, j, window):
                    weight = logistic(q[i, head] @ k[j, g] * m["scale"] + W[p + "pb"][head])
                    out[i, head] += weight * v[j, g]
    return out.reshape(T, H * V) @ W[p + "o"].T


def mingru(h, W, p, state=None):
    """h [T, d] -> ([T, d], final state). S_t = (1 - z_t) S_(t-1) + z_t c_t, out_t = W_o (S_t * silu(W_g h_t))."""
    z = logistic(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, logistic(u))
    gate = h @ W[p + "g"].T
    S = np.zeros(z.shape[1]) if state is None else np.array(state, dtype=np.float64)
    rows = []
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        rows.append(S * (gate[t] * logistic(gate[t])))
    return np.array(rows).reshape(h.shape[0], -1) @ W[p + "o"].T, S


def route(h_row, W, p, router):
    """One token: (chosen expert indices, their weights). Choice by score + correction among the kept groups; weights are
    the plain scores times the router's scale."""
    E, top = router["experts"], router["top"]
    score = logistic(W[p + "router"] @ h_row)
    pick = score + W[p + "correction"]
    if router.get("groups") is not None:
        count, keep = router["groups"]["count"], router["groups"]["keep"]
        size = E // count
        group_score = [np.sort(pick[g * size:(g + 1) * size])[-2:].sum() for g in range(count)]
        kept = sorted(range(count), key=lambda g: (-group_score[g], g))[:keep]
        pick = np.array([pick[e] if e // size in kept else -np.inf for e in range(E)])
    chosen = sorted(range(E), key=lambda e: (-pick[e], e))[:top]
    return chosen, [score[e] * router.get("scale", 1.0) for e in chosen]


def expert(x, up, down):
    return down @ (np.maximum(up @ x, 0.0) ** 2)


def routed_experts(h, W, p, mlp):
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        chosen, weights = route(h[t], W, p, mlp["router"])
        for e, w in zip(chosen, weights):
            out[t] += w * expert(h[t], W[p + f"e{e}.up"], W[p + f"e{e}.down"])
        if mlp.get("shared") is not None:
            out[t] += logistic(W[p + "shared.sg"][0] @ h[t]) * expert(h[t], W[p + "shared.up"], W[p + "shared.down"])
    return out


def stream_read(xs, read):
    """xs [S, T, d] -> [T, d]: the branch's input, a mix of the streams."""
    return np.tensordot(read, xs, axes=(0, 0))


def stream_write(xs, mix, write, y):
    """All streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + write[t] y."""
    new = np.zeros_like(xs)
    for t in range(xs.shape[0]):
        for s in range(xs.shape[0]):
            new[t] += mix[s, t] * xs[s]
        new[t] += write[t] * y
    return new


def forward(cfg, W, tokens, per_layer=None):
    """Logits [T, vocab] of a whole sequence. ``per_layer`` (a list) receives the residual after every layer (the sum of
    the streams, if there are several)."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    S = cfg.get("streams")
    xs = np.stack([x] * S) if S else None
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        branches = [(1, (lambda h, p=p, L=L: sigmoid_attention(h, W, p + "mix.", L["mixer"], eps)) if L["type"] == "attention"
                     else (lambda h, p=p: mingru(h, W, p + "mix.")[0]))]
        if L.get("mlp") is not None:
            branches.append((2, lambda h, p=p, L=L: routed_experts(h, W, p + "mlp.", L["mlp"])))
        for q, branch in branches:
            w, b = W[p + f"norm{q}"], W[p + f"norm{q}.b"]
            if S:
                y = branch(layer_norm(stream_read(xs, W[p + f"hc{q}.in"]), w, b, eps))
                xs = stream_write(xs, W[p + f"hc{q}.mix"], W[p + f"hc{q}.out"], y)
            else:
                x = x + branch(layer_norm(x, w, b, eps))
        if per_layer is not None:
            per_layer.append(xs.sum(0) if S else x.copy())
    if S:
        x = xs.sum(0)
    return layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
