"""Plain, slow numpy statement of the Dozotar design, one function per mechanism.  Test infrastructure only: it shares no
code with the product path (powerserve_b200/), keeps no cache and no state (every call recomputes the whole sequence, the
recurrences token by token) and works in float64.

Notation: n tokens at positions 0 .. n-1; matrices are stored [out, in] and applied as W @ x; d = i - j >= 0 is the distance
from query i back to key j; U(v) = v / sqrt(mean(v^2) + eps).

  layer            x <- x + U(mixer(x)) * g1;  x <- x + U(ff(x)) * g2        g1, g2 single numbers; the sublayers read x itself
  short conv       y_t[c] = sum_j w[c, j] u_(t - T + 1 + j)[c]  (+ b[c]),  u = 0 before position 0,  T taps
  attention        q, k, v = conv(W_q x), conv(W_k x), conv(W_v x);  q <- U(q) * wq over ALL query rows at once, k likewise
                   s_hij = q_hi . k_g(h)j * c + rel[bucket(d), h],   g(h) = floor(h / (H / G))
                   bucket(d) = d below R/2, else min(R - 1, R/2 + floor(ln(d / (R/2)) / ln(D / (R/2)) * (R - R/2)))   R rows, D last distance
                   visible: j <= i and floor(i / C) = floor(j / C);  soft-max over the visible keys;  out = W_o concat_h(sum_j p_hij v_g(h)j)
  rotation         pair (i, i + R/2), i < R/2, of the first R dims of a head: (u, v) -> (u cos a - v sin a, v cos a + u sin a),
                   a = position * base^(-2i / R)
  retention        q, k rotated; k <- k / sqrt(dim);  S_t = decay_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t
                   out = W_o (concat_h U(o_h) * silu(W_g x))
  mamba2           W_in x = [z | x | B | C | dt];  (x, B, C) <- silu(conv(x, B, C) + b);  dt <- softplus(dt + dt_bias)
                   S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t B_t x_t^T;  y_t = S_t^T C_t + D_h x_t      head h uses group floor(h / (heads / groups))
                   out = W_o (concat over `norm_groups` parts of U(part of (y * silu(z)))) * w_norm
  dense ff         W_down (gelu_tanh(W_gate h) * (W_up h))
  experts          s = softmax(W_r h);  groups of neighbouring experts scored by their best member, the `keep` best groups stay;
                   the `top` best experts of those, weights s / (sum of the chosen s + 1e-20);  expert: W_down (silu(W_gate h) * (W_up h))
                   + sigmoid(w_sg . h) * shared expert (same form)
  output           logits = W_head (U(x) * g_final)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


def bf16_round(a: np.ndarray) -> np.ndarray:
    """round-to-nearest-even of float32 values to bfloat16, returned as float32"""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def unit_rms(v, eps):
    return v / np.sqrt((v * v).mean(-1, keepdims=True) + eps)


def silu(z):
    return z / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return np.logaddexp(0.0, z)


def short_conv(u, w, b=None):
    """u [n, channels], w [channels, taps]: the last tap meets the current token, zeros before the first"""
    n, taps = u.shape[0], w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, u.shape[1])), u], 0)
    y = np.zeros_like(u, dtype=np.float64)
    for j in range(taps):
        y += pad[j:j + n] * w[:, j]
    return y if b is None else y + b


def bucket(d: int, rows: int, last: float) -> int:
    half = rows // 2
    if d < half:
        return d
    return min(rows - 1, half + int(math.floor(math.log(d / half) / math.log(last / half) * (rows - half))))


def chunk_visible(n: int, chunk: Optional[int]):
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    ok = j <= i
    if chunk:
        ok &= (i // chunk) == (j // chunk)
    return ok


def conv_attention(x, w: Dict[str, np.ndarray], m: dict, eps: float):
    n = x.shape[0]
    H, G, dq, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = x @ w["q"].T, x @ w["k"].T, x @ w["v"].T
    if m.get("conv"):
        q, k, v = short_conv(q, w["q.conv"]), short_conv(k, w["k.conv"]), short_conv(v, w["v.conv"])
    q = (unit_rms(q, eps) * w["q.norm"]).reshape(n, H, dq)
    k = (unit_rms(k, eps) * w["k.norm"]).reshape(n, G, dq)
    v = v.reshape(n, G, dv)
    rel = w["rel"]
    rows = rel.shape[0]
    dist = np.maximum(np.arange(n)[:, None] - np.arange(n)[None, :], 0)
    row_of = np.array([bucket(d, rows, m["bias_max"]) for d in range(n)])[dist]
    ok = chunk_visible(n, (m.get("mask") or {}).get("size"))
    out = np.zeros((n, H, dv))
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * m["scale"] + rel[row_of, h]
        s = np.where(ok, s, -np.inf)
        e = np.exp(s - s.max(-1, keepdims=True))
        out[:, h] = (e / e.sum(-1, keepdims=True)) @ v[:, g]
    return out.reshape(n, H * dv) @ w["o"].T


def rotate_half(v, positions, rot: dict):
    """v [n, heads, dim]: the first rot['dims'] dims of every head turn, pairs (i, i + dims / 2)"""
    R = int(rot["dims"])
    if R == 0:
        return v
    f = float(rot["base"]) ** (-2.0 * np.arange(R // 2) / R)
    a = np.asarray(positions, np.float64)[:, None, None] * f
    c, s = np.cos(a), np.sin(a)
    lo, hi = v[..., :R // 2], v[..., R // 2:R]
    return np.concatenate([lo * c - hi * s, hi * c + lo * s, v[..., R:]], -1)


def retention(x, w: Dict[str, np.ndarray], m: dict, eps: float):
    n = x.shape[0]
    H, dq, dv = m["heads"], m["dim"], m["vdim"]
    pos = np.arange(n)
    q = rotate_half((x @ w["q"].T).reshape(n, H, dq), pos, m["rot"])
    k = rotate_half((x @ w["k"].T).reshape(n, H, dq), pos, m["rot"]) / math.sqrt(dq)
    v = (x @ w["v"].T).reshape(n, H, dv)
    o = np.zeros((n, H, dv))
    for h in range(H):
        S = np.zeros((dq, dv))
        for t in range(n):
            S = m["decay"][h] * S + np.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    o = unit_rms(o, eps).reshape(n, H * dv) * silu(x @ w["g"].T)
    return o @ w["o"].T


def mamba2(x, w: Dict[str, np.ndarray], m: dict, eps: float):
    n = x.shape[0]
    H, P, N, G, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    t = x @ w["in"].T
    z, xbc, dt = t[:, :inner], t[:, inner:2 * inner + 2 * G * N], t[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w["conv"], w["conv.b"]))
    u = xbc[:, :inner].reshape(n, H, P)
    Bm = xbc[:, inner:inner + G * N].reshape(n, G, N)
    Cm = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = np.zeros((n, H, P))
    for h in range(H):
        g = h // (H // G)
        S = np.zeros((N, P))
        rate = math.exp(float(w["A_log"][h]))
        for i in range(n):
            S = math.exp(-rate * dt[i, h]) * S + dt[i, h] * np.outer(Bm[i, g], u[i, h])
            y[i, h] = S.T @ Cm[i, g] + w["D"][h] * u[i, h]
    y = y.reshape(n, inner) * silu(z)
    y = unit_rms(y.reshape(n, parts, inner // parts), eps).reshape(n, inner) * w["norm"]
    return y @ w["o"].T


def gated_unit(h, w: Dict[str, np.ndarray], act):
    return (act(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def choose_experts(s: np.ndarray, top: int, count: int, keep: int):
    """s [experts] -> the chosen experts (best first); groups of neighbours, a group is worth its best member"""
    E = s.shape[0]
    per = E // count
    worth = s.reshape(count, per).max(-1)
    kept = np.argsort(-worth, kind="stable")[:keep]
    allowed = np.zeros(E, bool)
    for g in kept:
        allowed[g * per:(g + 1) * per] = True
    order = [e for e in np.argsort(-s, kind="stable") if allowed[e]]
    return order[:top]


def expert_ff(h, w: Dict[str, np.ndarray], mlp: dict, prefix_free: Dict[str, np.ndarray] = None):
    """h [n, width]; w holds 'router', 'e<i>.gate/up/down', and with a shared expert 'shared.gate/up/down/sg'"""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    z = h @ w["router"].T
    s = np.exp(z - z.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    out = np.zeros_like(h, dtype=np.float64)
    for t in range(h.shape[0]):
        chosen = choose_experts(s[t], top, grp["count"], grp["keep"])
        tot = sum(s[t, e] for e in chosen) + 1e-20
        for e in chosen:
            we = {f: w[f"e{e}.{f}"] for f in ("gate", "up", "down")}
            out[t] += s[t, e] / tot * gated_unit(h[t:t + 1], we, silu)[0]
    if mlp.get("shared"):
        ws = {f: w[f"shared.{f}"] for f in ("gate", "up", "down")}
        gate = 1.0 / (1.0 + np.exp(-(h @ w["shared.sg"].T)))
        out += gate * gated_unit(h, ws, silu)
    return out


MIXERS = {"attention": conv_attention, "retention": retention, "mamba2": mamba2}


def sub(tensors: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
    return {k[len(prefix):]: np.asarray(v, np.float64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, np.ndarray], tokens: List[int], taps: Optional[list] = None):
    """logits [n, vocab] of the whole sequence; taps (a list) receives the residual stream after every layer"""
    eps = cfg["norm"]["eps"]
    x = np.asarray(tensors["embed"], np.float64)[np.asarray(tokens)]
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + unit_rms(MIXERS[l["type"]](x, sub(tensors, p + "mix."), l["mixer"], eps), eps) * float(tensors[p + "norm1"])
        mlp = l.get("mlp")
        if mlp is not None:
            w = sub(tensors, p + "mlp.")
            y = gated_unit(x, w, gelu_tanh) if mlp["kind"] == "dense" else expert_ff(x, w, mlp)
            x = x + unit_rms(y, eps) * float(tensors[p + "norm2"])
        if taps is not None:
            taps.append(x.copy())
    return (unit_rms(x, eps) * float(tensors["final.norm"])) @ np.asarray(tensors["head"], np.float64).T
