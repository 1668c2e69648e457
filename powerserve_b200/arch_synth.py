"""Synthetic layer-list model directories (config.json + model.safetensors, random bfloat16 weights) for tests and
bench.py - there are no real checkpoints on the build / GPU boxes.  The result loads through `arch.load_model` like any
other model directory.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np

from . import safetensors


def nufusun_layer(heads: int, kv_heads: int, dim: int, vdim: int, *, scale: Optional[float] = None, bias_max: float = 100.0,
                  experts: int = 0, top: int = 1, ff: int = 0, limit: float = 1.0) -> dict:
    """one entry of a Nufusun config's layer list; experts == 0 means a layer without a feed-forward"""
    layer = {"type": "attention",
             "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5),
                       "bias_max": bias_max},
             "mlp": None}
    if experts:
        layer["mlp"] = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    return layer


def nufusun_config(width: int, vocab: int, layers: List[dict], *, eps: float = 1e-5, embed_scale: float = 1.0) -> dict:
    return {"architecture": "Nufusun", "embedding": {"scale": embed_scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def nufusun_weights(cfg: dict, seed: int = 0, rel_rows: int = 16, fast: bool = False) -> Dict[str, np.ndarray]:
    """float32 arrays holding bfloat16-representable values (what the file will hold), keyed by tensor name.
    fast = True draws the big matrices as random bfloat16 bit patterns of bounded exponent (seconds for gigabytes)."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(out_dim, in_dim, gain=1.0):
        if fast:
            # sign + exponent around 2^-k for the wanted scale + random mantissa; returned as bf16 bit patterns (uint16)
            s = gain / np.sqrt(in_dim)
            e = int(np.floor(np.log2(s))) + 127
            bits = rng.integers(0, 1 << 7, size=(out_dim, in_dim), dtype=np.uint16) | np.uint16(e << 7)
            bits |= (rng.integers(0, 2, size=(out_dim, in_dim), dtype=np.uint16) << 15).astype(np.uint16)
            return bits
        return rnd(rng.standard_normal((out_dim, in_dim), dtype=np.float32) * np.float32(gain / np.sqrt(in_dim)))

    def rnd(a):
        return (safetensors.float32_to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32)

    t: Dict[str, np.ndarray] = {"embed": mat(V, W, np.sqrt(W)), "final.norm": rnd(rng.standard_normal(W).astype(np.float32) * 0.1), "head": mat(V, W)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, G, dq, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        t[p + "norm1"] = rnd(rng.standard_normal(W).astype(np.float32) * 0.1)
        t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * dq, W, 2.0), mat(G * dq, W, 2.0), mat(G * dv, W)
        t[p + "mix.o"] = mat(W, H * dv)
        for n, k in (("q", H * dq), ("k", G * dq), ("v", G * dv), ("o", W)):
            t[p + f"mix.{n}.b"] = rnd(rng.standard_normal(k).astype(np.float32) * 0.1)
        t[p + "mix.rel"] = rnd(rng.standard_normal((rel_rows, H)).astype(np.float32) * 0.7)
        t[p + "mix.talk"] = rnd(np.eye(H, dtype=np.float32) + rng.standard_normal((H, H)).astype(np.float32) * 0.2)
        t[p + "mix.temp"] = rnd(1.0 + rng.standard_normal(H).astype(np.float32) * 0.2)
        if l.get("mlp") is not None:
            E, ff = l["mlp"]["router"]["experts"], l["mlp"]["expert"]["ff"]
            t[p + "mlp.router"] = mat(E, W, 2.0)
            for e in range(E):
                t[p + f"mlp.e{e}.gate"], t[p + f"mlp.e{e}.up"], t[p + f"mlp.e{e}.down"] = mat(ff, W, 1.5), mat(ff, W, 1.5), mat(W, ff)
    return t


def write_model_dir(path: str, cfg: dict, tensors: Dict[str, np.ndarray]) -> str:
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    safetensors.write_file(os.path.join(path, "model.safetensors"), tensors)
    return path


# ------------------------------------------------------------------------------------------------------------ Vanapel
def vanapel_attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, *, window: int, scale: Optional[float] = None, v_mix: bool = False,
                            ff: int = 0, limit: float = 1.0) -> dict:
    """a windowed-attention entry of a Vanapel layer list; ff == 0 means a layer without a feed-forward"""
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": float(scale if scale is not None else dim ** -0.5)}
    if v_mix:
        mixer["v_mix"] = True
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def vanapel_latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, *, scale: Optional[float] = None, rope_base: float = 10000.0,
                         rope_dims: Optional[int] = None, scaling: Optional[dict] = None, ff: int = 0, limit: float = 1.0) -> dict:
    """a latent-attention entry; `scaling` = {"factor", "original", "fast", "slow"} turns YaRN on"""
    rot = {"base": rope_base, "dims": rot_dim if rope_dims is None else rope_dims}
    if scaling:
        rot["scaling"] = dict(scaling)
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "rot": rot,
             "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def vanapel_config(width: int, vocab: int, layers: List[dict], *, eps: float = 1e-6, groups: int = 1) -> dict:
    return {"architecture": "Vanapel", "layers": layers, "norm": {"eps": eps, "groups": groups}, "vocab": vocab, "width": width}


def vanapel_weights(cfg: dict, seed: int = 0, fast: bool = False) -> Dict[str, np.ndarray]:
    """float32 arrays of bfloat16-representable values keyed by tensor name (fast = True: big matrices as random bfloat16 bit patterns)"""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(a):
        return (safetensors.float32_to_bf16_bits(np.asarray(a, np.float32)).astype(np.uint32) << 16).view(np.float32)

    def mat(out_dim, in_dim, gain=1.0):
        if fast:
            e = int(np.floor(np.log2(gain / np.sqrt(in_dim)))) + 127
            bits = rng.integers(0, 1 << 7, size=(out_dim, in_dim), dtype=np.uint16) | np.uint16(e << 7)
            return bits | (rng.integers(0, 2, size=(out_dim, in_dim), dtype=np.uint16) << 15).astype(np.uint16)
        return rnd(rng.standard_normal((out_dim, in_dim), dtype=np.float32) * np.float32(gain / np.sqrt(in_dim)))

    def norm_w(n, mean=1.0):
        return rnd(mean + rng.standard_normal(n).astype(np.float32) * 0.1)

    t: Dict[str, np.ndarray] = {"embed": mat(V, W, np.sqrt(W)), "final.norm": norm_w(W), "head": mat(V, W)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, dv = m["heads"], m["vdim"]
        t[p + "norm1"], t[p + "norm1b"] = norm_w(W), norm_w(W, 0.5)
        if l["type"] == "attention":
            G, dq = m["kv_heads"], m["dim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * dq, W), mat(G * dq, W), mat(G * dv, W)
            t[p + "mix.r1"] = rnd(rng.uniform(0.05, 0.6, H))
            t[p + "mix.r2"] = rnd(rng.uniform(0.05, 1.5, H))
            if m.get("v_mix"):
                t[p + "mix.vmix"] = rnd(np.array(rng.uniform(0.2, 0.8), np.float32))
        else:
            dn, dr, rq, rk = m["dim"], m["rot_dim"], m["q_rank"], m["kv_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = mat(rq, W), norm_w(rq), mat(H * (dn + dr), rq, 2.0)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(rk + dr, W, 2.0), norm_w(rk)
            t[p + "mix.uk"], t[p + "mix.uv"] = mat(H * dn, rk, 2.0), mat(H * dv, rk)
        t[p + "mix.sink"] = rnd(rng.standard_normal(H).astype(np.float32))
        t[p + "mix.o"] = mat(W, H * dv)
        if l.get("mlp") is not None:
            ff = l["mlp"]["ff"]
            t[p + "norm2"], t[p + "norm2b"] = norm_w(W), norm_w(W, 0.5)
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(ff, W, 1.5), mat(ff, W, 1.5), mat(W, ff)
    return t


# ------------------------------------------------------------------------------------------------------------ Dozotar
def _dozotar_mlp(ff: int = 0, experts: int = 0, top: int = 1, route_groups: int = 1, route_keep: int = 1, shared_ff: int = 0) -> Optional[dict]:
    """ff == 0: no feed-forward; experts == 0: dense of ff rows; else routed experts of ff rows (+ a shared expert of shared_ff rows)"""
    if not ff:
        return None
    if not experts:
        return {"kind": "dense", "ff": ff}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": route_groups, "keep": route_keep}}}
    if shared_ff:
        mlp["shared"] = {"ff": shared_ff}
    return mlp


def dozotar_attention_layer(heads: int, kv_heads: int, dim: int, vdim: int, *, chunk: int, conv: int = 3, scale: Optional[float] = None, bias_max: float = 100.0, **mlp) -> dict:
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": chunk}, "bias_max": bias_max,
             "scale": float(scale if scale is not None else dim ** -0.5)}
    return {"type": "attention", "mixer": mixer, "mlp": _dozotar_mlp(**mlp)}


def dozotar_retention_layer(heads: int, dim: int, vdim: int, *, decay: Optional[List[float]] = None, rot_dims: Optional[int] = None, rot_base: float = 10000.0, **mlp) -> dict:
    decay = decay if decay is not None else [1.0 - 2.0 ** (-4 - h) for h in range(heads)]
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [float(x) for x in decay], "rot": {"base": rot_base, "dims": dim if rot_dims is None else rot_dims}}
    return {"type": "retention", "mixer": mixer, "mlp": _dozotar_mlp(**mlp)}


def dozotar_mamba2_layer(heads: int, vdim: int, state: int, *, groups: int = 1, norm_groups: int = 1, conv: int = 4, **mlp) -> dict:
    mixer = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}
    return {"type": "mamba2", "mixer": mixer, "mlp": _dozotar_mlp(**mlp)}


def dozotar_config(width: int, vocab: int, layers: List[dict], *, eps: float = 1e-5) -> dict:
    return {"architecture": "Dozotar", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def dozotar_weights(cfg: dict, seed: int = 0, rel_rows: int = 16, fast: bool = False) -> Dict[str, np.ndarray]:
    """float32 arrays of bfloat16-representable values keyed by tensor name (fast = True: big matrices as random bfloat16 bit patterns)"""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(a):
        return (safetensors.float32_to_bf16_bits(np.asarray(a, np.float32)).astype(np.uint32) << 16).view(np.float32)

    def mat(out_dim, in_dim, gain=1.0):
        if fast:
            e = int(np.floor(np.log2(gain / np.sqrt(in_dim)))) + 127
            bits = rng.integers(0, 1 << 7, size=(out_dim, in_dim), dtype=np.uint16) | np.uint16(e << 7)
            return bits | (rng.integers(0, 2, size=(out_dim, in_dim), dtype=np.uint16) << 15).astype(np.uint16)
        return rnd(rng.standard_normal((out_dim, in_dim), dtype=np.float32) * np.float32(gain / np.sqrt(in_dim)))

    def scalar(mean):
        return rnd(np.array(mean + 0.2 * rng.standard_normal(), np.float32))

    def unit(n):
        return {"gate": mat(n, W, 1.5), "up": mat(n, W, 1.5), "down": mat(W, n)}

    t: Dict[str, np.ndarray] = {"embed": mat(V, W, np.sqrt(W)), "final.norm": scalar(1.0), "head": mat(V, W)}
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        H, dv = m["heads"], m["vdim"]
        t[p + "norm1"] = scalar(0.8)
        if l["type"] == "attention":
            G, dq, taps = m["kv_heads"], m["dim"], m["conv"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * dq, W), mat(G * dq, W), mat(G * dv, W)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = rnd(1.0 + 0.2 * rng.standard_normal(H * dq)), rnd(1.0 + 0.2 * rng.standard_normal(G * dq))
            for n, k in (("q", H * dq), ("k", G * dq), ("v", G * dv)) if taps else ():
                t[p + f"mix.{n}.conv"] = rnd(rng.standard_normal((k, taps)) * 0.5 + np.eye(taps)[taps - 1])
            t[p + "mix.rel"] = rnd(rng.standard_normal((rel_rows, H)) * 0.7)
            t[p + "mix.o"] = mat(W, H * dv)
        elif l["type"] == "retention":
            dq = m["dim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = mat(H * dq, W), mat(H * dq, W), mat(H * dv, W), mat(H * dv, W)
            t[p + "mix.o"] = mat(W, H * dv)
        else:
            N, G, taps = m["state"], m["groups"], m["conv"]
            inner, ch = H * dv, H * dv + 2 * G * N
            t[p + "mix.in"] = mat(2 * inner + 2 * G * N + H, W)
            t[p + "mix.conv"] = rnd(rng.standard_normal((ch, taps)) * 0.4 + np.eye(taps)[taps - 1])
            t[p + "mix.conv.b"] = rnd(rng.standard_normal(ch) * 0.1)
            t[p + "mix.dt_bias"] = rnd(rng.uniform(-3.0, 0.5, H))
            t[p + "mix.A_log"] = rnd(np.log(rng.uniform(0.5, 8.0, H)))
            t[p + "mix.D"] = rnd(1.0 + 0.2 * rng.standard_normal(H))
            t[p + "mix.norm"] = rnd(1.0 + 0.2 * rng.standard_normal(inner))
            t[p + "mix.o"] = mat(W, inner)
        mlp = l.get("mlp")
        if mlp is None:
            continue
        t[p + "norm2"] = scalar(0.8)
        if mlp["kind"] == "dense":
            for f, a in unit(mlp["ff"]).items():
                t[p + "mlp." + f] = a
        else:
            E = mlp["router"]["experts"]
            t[p + "mlp.router"] = mat(E, W, 3.0)
            for e in range(E):
                for f, a in unit(mlp["expert"]["ff"]).items():
                    t[p + f"mlp.e{e}.{f}"] = a
            if mlp.get("shared"):
                for f, a in unit(mlp["shared"]["ff"]).items():
                    t[p + "mlp.shared." + f] = a
                t[p + "mlp.shared.sg"] = mat(1, W, 2.0)
    return t


# ------------------------------------------------------------------------------------------------------------ Pidenex
def _pidenex_mlp(ff: int) -> Optional[dict]:
    return {"kind": "dense", "ff": ff} if ff else None


def pidenex_attention_layer(heads: int, kv_heads: int, dim: int, *, window: int, pool: int = 0, scale: Optional[float] = None, ff: int = 0) -> dict:
    """a windowed attention whose values are its keys (vdim = dim); pool > 0 adds the mean key per block of `pool` tokens before the window"""
    mask = {"size": window}
    if pool:
        mask["pool"] = pool
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": mask, "scale": float(scale if scale is not None else dim ** -0.5)},
            "mlp": _pidenex_mlp(ff)}


def pidenex_parallel_layer(heads: int, kv_heads: int, dim: int, *, window: int, gru_width: int, left_scale: float = 0.8, right_scale: float = 0.9,
                           scale: Optional[float] = None, ff: int = 0) -> dict:
    """a gated attention with a linear distance penalty beside a minGRU of gru_width channels"""
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window}, "scale": float(scale if scale is not None else dim ** -0.5)}
    return {"type": "parallel", "mixer": {"left": left, "left_scale": left_scale, "right": {"width": gru_width}, "right_scale": right_scale}, "mlp": _pidenex_mlp(ff)}


def pidenex_latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, *, window: int = 0, scale: Optional[float] = None,
                         rope_base: float = 10000.0, ff: int = 0) -> dict:
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "rot": {"base": rope_base, "dims": rot_dim},
             "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5)}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": _pidenex_mlp(ff)}


def pidenex_config(width: int, vocab: int, layers: List[dict], *, loop: Optional[tuple] = None, eps: float = 1e-6, embed_scale: float = 1.0) -> dict:
    """loop = (start, stop, times): the layers start .. stop - 1 run `times` times with the same weights"""
    a, b, n = loop if loop else (0, 0, 1)
    return {"architecture": "Pidenex", "embedding": {"scale": embed_scale}, "layers": layers, "loop": {"start": a, "stop": b, "times": n}, "norm": {"eps": eps},
            "vocab": vocab, "width": width}


def pidenex_weights(cfg: dict, seed: int = 0, fast: bool = False) -> Dict[str, np.ndarray]:
    """float32 arrays of bfloat16-representable values keyed by tensor name (fast = True: big matrices as random bfloat16 bit patterns)"""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]

    def rnd(a):
        return (safetensors.float32_to_bf16_bits(np.asarray(a, np.float32)).astype(np.uint32) << 16).view(np.float32)

    def mat(out_dim, in_dim, gain=1.0):
        if fast:
            e = int(np.floor(np.log2(gain / np.sqrt(in_dim)))) + 127
            bits = rng.integers(0, 1 << 7, size=(out_dim, in_dim), dtype=np.uint16) | np.uint16(e << 7)
            return bits | (rng.integers(0, 2, size=(out_dim, in_dim), dtype=np.uint16) << 15).astype(np.uint16)
        return rnd(rng.standard_normal((out_dim, in_dim), dtype=np.float32) * np.float32(gain / np.sqrt(in_dim)))

    def vec(n, mean=0.0, dev=0.1):
        return rnd(mean + rng.standard_normal(n).astype(np.float32) * dev)

    t: Dict[str, np.ndarray] = {"embed": mat(V, W, np.sqrt(W)), "final.norm": vec(W, 1.0), "head": mat(V, W)}
    lp = cfg.get("loop") or {}
    if lp.get("stop", 0) > lp.get("start", 0):
        t["loop.step"] = rnd(rng.standard_normal((lp["times"], W)).astype(np.float32) * 0.5)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        t[p + "norm1"], t[p + "norm1b"] = vec(W, 1.0), vec(W, 0.5)
        if l["type"] == "attention":
            H, G, dq = m["heads"], m["kv_heads"], m["dim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.o"] = mat(H * dq, W, 2.0), mat(G * dq, W, 2.0), mat(W, H * dq)
        elif l["type"] == "parallel":
            a, b, ml, R = p + "mix.left.", p + "mix.right.", m["left"], m["right"]["width"]
            H, G, dq = ml["heads"], ml["kv_heads"], ml["dim"]
            t[a + "q"], t[a + "k"], t[a + "g"], t[a + "o"] = mat(H * dq, W, 2.0), mat(G * dq, W, 2.0), mat(H * dq, W, 2.0), mat(W, H * dq)
            t[a + "q.norm"], t[a + "k.norm"] = vec(H * dq, 1.0, 0.2), vec(G * dq, 1.0, 0.2)
            t[b + "z"], t[b + "x"], t[b + "g"], t[b + "o"] = mat(R, W, 2.0), mat(R, W, 2.0), mat(R, W, 2.0), mat(W, R)
            t[b + "z.b"], t[b + "x.b"] = vec(R, 0.0, 0.5), vec(R, 0.0, 0.5)
        else:
            H, dn, dr, dv, rq, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            t[p + "mix.dq"], t[p + "mix.dq.norm"], t[p + "mix.uq"] = mat(rq, W), vec(rq, 1.0), mat(H * (dn + dr), rq, 2.0)
            t[p + "mix.dkv"], t[p + "mix.dkv.norm"] = mat(rk + dr, W, 2.0), vec(rk, 1.0)
            t[p + "mix.uk"], t[p + "mix.uv"], t[p + "mix.o"] = mat(H * dn, rk, 2.0), mat(H * dv, rk), mat(W, H * dv)
        if l.get("mlp") is not None:
            ff = l["mlp"]["ff"]
            t[p + "norm2"], t[p + "norm2b"] = vec(W, 1.0), vec(W, 0.5)
            t[p + "mlp.up"], t[p + "mlp.down"], t[p + "mlp.act"] = mat(ff, W, 1.5), mat(W, ff), rnd(rng.standard_normal(2).astype(np.float32))
    return t
