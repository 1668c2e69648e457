"""Plain numpy statement of the Pidenex design, one function per mechanism, float64 throughout.

It keeps no cache and no state: every function sees the whole sequence.  It shares no code with the product path; the tests
compare the CUDA executor with it.

A model is (cfg, W): cfg the dictionary of config.json, W a dictionary name -> float array (bfloat16 values widened).
"""
from __future__ import annotations

import math

import numpy as np


# ------------------------------------------------------------------------------------------------------------ small pieces
def bf16_round(a):
    """round to the nearest bfloat16 value (ties to even), returned as float32"""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var = mean of squared deviations; no bias"""
    mu = x.mean(-1, keepdims=True)
    d = x - mu
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * w


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def silu(z):
    return z * sigmoid(z)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2"""
    ap, an = softplus(p), 0.5 + softplus(q)
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, an * (np.expm1(zn) - zn) + 0.5 * z)


def rotate_pairs(v, pos, dims, base):
    """v [..., T, n]: the first `dims` entries in neighbouring pairs (2i, 2i + 1), angle pos * base^(-2i / dims)"""
    out = np.array(v, dtype=np.float64, copy=True)
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    a = np.asarray(pos, np.float64)[:, None] * f[None, :]
    c, s = np.cos(a), np.sin(a)
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def window_mask(T, size):
    """[T, T] boolean: query i sees key j when 0 <= i - j < size (size <= 0: every earlier key)"""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    m = j <= i
    if size > 0:
        m &= (i - j) < size
    return m


def pooled_mask(T, size, pool):
    """[T, T // pool] boolean: query i sees block b when its last position b * pool + pool - 1 <= i - size"""
    nb = T // pool
    i, b = np.arange(T)[:, None], np.arange(nb)[None, :]
    return b * pool + pool - 1 <= i - size


def masked_softmax(s, m):
    s = np.where(m, s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    e = np.where(m, np.exp(s), 0.0)
    return e / e.sum(-1, keepdims=True)


def block_means(x, pool):
    """x [G, T, d] -> [G, T // pool, d]: mean over each complete block of `pool` positions"""
    G, T, d = x.shape
    nb = T // pool
    return x[:, :nb * pool].reshape(G, nb, pool, d).mean(2)


# ------------------------------------------------------------------------------------------------------------ mixers
def heads_of(x, n, d):
    """[T, n * d] -> [n, T, d]"""
    return x.reshape(x.shape[0], n, d).transpose(1, 0, 2)


def grouped_attention(q, k, v, scale, mask, bias=None):
    """q [H, T, d], k [G, S, d], v [G, S, dv], mask [T, S], bias [H, T, S] or None -> [T, H * dv]"""
    H, G = q.shape[0], k.shape[0]
    rep = H // G
    out = []
    for h in range(H):
        s = q[h] @ k[h // rep].T * scale
        if bias is not None:
            s = s + bias[h]
        out.append(masked_softmax(s, mask) @ v[h // rep])
    return np.concatenate(out, -1)


def pooled_attention(h, m, W, p):
    """values are the keys; window of mask.size tokens plus one mean key / value per block of mask.pool tokens wholly before it"""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = heads_of(h @ W[p + "q"].T, H, d)
    k = heads_of(h @ W[p + "k"].T, G, d)
    size, pool = int(m["mask"]["size"]), int(m["mask"].get("pool", 0))
    mask = window_mask(T, size)
    keys = k
    if pool > 0 and T // pool > 0:
        keys = np.concatenate([k, block_means(k, pool)], 1)
        mask = np.concatenate([mask, pooled_mask(T, size, pool)], 1)
    return grouped_attention(q, keys, keys, m["scale"], mask) @ W[p + "o"].T


def latent_attention(h, m, W, p, eps):
    T = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    pos = np.arange(T)
    cq = rms_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = heads_of(cq @ W[p + "uq"].T, H, dn + dr)
    t = h @ W[p + "dkv"].T
    c = rms_norm(t[:, :rk], W[p + "dkv.norm"], eps)
    kr = rotate_pairs(t[:, rk:], pos, rot["dims"], rot["base"])
    kn = heads_of(c @ W[p + "uk"].T, H, dn)
    v = heads_of(c @ W[p + "uv"].T, H, dv)
    qr = rotate_pairs(q[..., dn:], pos, rot["dims"], rot["base"])
    mask = window_mask(T, int((m.get("mask") or {}).get("size", 0)))
    out = []
    for hh in range(H):
        s = (q[hh, :, :dn] @ kn[hh].T + qr[hh] @ kr.T) * m["scale"]
        out.append(masked_softmax(s, mask) @ v[hh])
    return np.concatenate(out, -1) @ W[p + "o"].T


def slopes(H):
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])


def gated_biased_attention(h, m, W, p, eps):
    """the left half of a parallel mixer: values are the un-normed keys, q / k normed over the whole projection, a penalty
    slope_h (i - j) on the score, a window, a sigmoid gate on the heads' outputs"""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    qf, kf = h @ W[p + "q"].T, h @ W[p + "k"].T
    v = heads_of(kf, G, d)
    q = heads_of(rms_norm(qf, W[p + "q.norm"], eps), H, d)
    k = heads_of(rms_norm(kf, W[p + "k.norm"], eps), G, d)
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    bias = -slopes(H)[:, None, None] * (i - j)[None]
    o = grouped_attention(q, k, v, m["scale"], window_mask(T, int(m["mask"]["size"])), bias)
    return (o * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def min_gru(h, W, p):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t from zero; z = sigmoid(W_z h + b), c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0)"""
    z = sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    c = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1])
    out = np.empty_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S
    return (out * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def parallel_mixer(h, m, W, p, eps):
    return m["left_scale"] * gated_biased_attention(h, m["left"], W, p + "left.", eps) + m["right_scale"] * min_gru(h, W, p + "right.")


def feed_forward(h, W, p):
    a = W[p + "act"]
    return xielu(h @ W[p + "up"].T, a[0], a[1]) @ W[p + "down"].T


# ------------------------------------------------------------------------------------------------------------ the model
def layer_runs(cfg):
    """[(layer, pass number or None when the run does not open a pass)]"""
    L = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, n = lp["start"], lp["stop"], lp["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(n if b > a else 0):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    runs += [(i, None) for i in range(b, L)]
    return runs


def layer(x, l, W, i, eps):
    p = f"l{i}."
    h = layer_norm(x, W[p + "norm1"], eps)
    kind = l["type"]
    if kind == "attention":
        y = pooled_attention(h, l["mixer"], W, p + "mix.")
    elif kind == "latent_attention":
        y = latent_attention(h, l["mixer"], W, p + "mix.", eps)
    elif kind == "parallel":
        y = parallel_mixer(h, l["mixer"], W, p + "mix.", eps)
    else:
        raise ValueError(kind)
    x = x + layer_norm(y, W[p + "norm1b"], eps)
    if l.get("mlp") is not None:
        x = x + layer_norm(feed_forward(layer_norm(x, W[p + "norm2"], eps), W, p + "mlp."), W[p + "norm2b"], eps)
    return x


def forward(cfg, W, tokens, taps=None):
    """tokens [T] -> logits [T, vocab]; taps (a list) receives the residual stream after every layer run"""
    eps = cfg["norm"]["eps"]
    W = {k: np.asarray(v, np.float64) for k, v in W.items()}
    x0 = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    x = x0
    for i, t in layer_runs(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        x = layer(x, cfg["layers"][i], W, i, eps)
        if taps is not None:
            taps.append(x)
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T
