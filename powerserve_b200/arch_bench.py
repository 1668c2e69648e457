"""bench.py --arch nufusun | vanapel | dozotar | pidenex: prefill and decode throughput of a layer-list design at layer sizes that resemble real
models (random weights), beside the closest existing model of the framework.

--arch vanapel: the Vanapel design (windowed attention layers and one latent-attention layer, dense gated feed-forward) beside
Nufusun at equal width, head geometry, layer count, vocabulary and as many ACTIVE feed-forward rows per token (top_k x expert
ff = ff) - the same executor, kernels and bfloat16 weights, so the two steps move nearly the same bytes.

--arch dozotar: the Dozotar design (retention, state-space and chunked-attention layers; dense gelu and routed feed-forwards with a
shared expert) beside Nufusun at equal width, attention head geometry, layer count, vocabulary and ACTIVE feed-forward rows per token.

--arch pidenex: the Pidenex design (pooled-window attention whose values are its keys, a gated attention beside a minGRU, latent
attention with rotation in neighbouring pairs, feed-forwards without a gate; the first two layers run twice with the same weights at
sizes s and m) beside Vanapel - the closest existing model: sequential blocks normed on both sides, windowed and latent attention,
dense feed-forward - with as many layer runs, equal width, head geometry, windows, vocabulary and feed-forward bytes (a gated unit of
ff rows against an ungated one of 3 ff / 2).

--arch nufusun: prefill and decode throughput of the Nufusun design at layer sizes that resemble real models
(random weights), beside the closest existing model of the framework - a llama stack (Q4_K) with the same width, head
geometry, layer count, vocabulary and as many ACTIVE feed-forward rows per token (ffn = top_k x expert ff).

Timing: the backend's CUDA events around every forward / decode call (counter last_device_ns), warm-up first; the weights
of every size exceed the 126 MB L2, so consecutive steps do not find them cached.  One JSON line per run.
"""
from __future__ import annotations

import json
import os
import shutil
import tempfile
import time

import numpy as np

from . import arch, arch_synth, capi, gguf, synth

# name: (width, heads, kv_heads, head size, experts, top, expert ff, layers, vocab)
SIZES = {
    "s": (1024, 16, 4, 64, 8, 2, 1024, 4, 32000),
    "m": (2048, 16, 4, 128, 8, 2, 2816, 4, 32000),
    "l": (4096, 32, 8, 128, 8, 2, 7168, 2, 32000),
}


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def _timed_prefill(model, prompt, chunk):
    model.reset()
    ns = 0
    for lo in range(0, len(prompt), chunk):
        model.forward(prompt[lo:lo + chunk], lm_head=False)
        ns += model.be.counter("last_device_ns")
    return ns / 1e9


def _timed_decode(model, tok, steps, warmup):
    model.decode_greedy(tok, warmup)
    model.decode_greedy(tok, steps)
    return model.be.counter("last_device_ns") / 1e9 / steps


def run_size(name, prompt_len, steps, warmup, seed, chunk):
    W, H, G, hs, E, top, ff, nl, V = SIZES[name]
    hbm, tflops, src = _peaks()
    n_ctx = -(-(prompt_len + steps + warmup + 8) // 256) * 256
    prompt = [int(v) for v in np.random.default_rng(1234).integers(0, V, prompt_len)]
    out = {"size": name, "width": W, "heads": [H, G], "head_size": hs, "experts": [E, top, ff], "layers": nl, "vocab": V, "context": prompt_len}

    # ---- Nufusun
    cfg = arch_synth.nufusun_config(W, V, [arch_synth.nufusun_layer(H, G, hs, hs, bias_max=float(prompt_len), experts=E, top=top, ff=ff, limit=7.0) for _ in range(nl)])
    d = tempfile.mkdtemp(prefix="ps_nufusun_")
    try:
        arch_synth.write_model_dir(d, cfg, arch_synth.nufusun_weights(cfg, seed=seed, rel_rows=32, fast=True))
        m = arch.load_model(d, dtype="bfloat16", max_batch=chunk, n_ctx=n_ctx)
    finally:
        shutil.rmtree(d, ignore_errors=True)
    for _ in range(2):
        t_pre = _timed_prefill(m, prompt, chunk)
    l0 = m.be.counter("kernel_launches")
    t_dec = _timed_decode(m, prompt[-1], steps, warmup)
    launches = m.be.counter("kernel_launches") - l0
    t0 = time.perf_counter()
    tok = prompt[-1]
    for _ in range(16):
        tok = int(np.argmax(m.forward([tok])[0]))
    e2e = 16 / (time.perf_counter() - t0)
    m.close()
    qkv = (H + 2 * G) * hs * W
    act_params = nl * (qkv + H * hs * W + E * W + top * 3 * ff * W) + V * W
    kv_bytes = nl * 2 * G * hs * 4 * prompt_len
    attn_flops = nl * 2 * 2 * H * hs * prompt_len / 2                     # per token, averaged over a causal prompt
    out["nufusun"] = {
        "prefill_tok_s": prompt_len / t_pre, "prefill_chunk": chunk,
        "prefill_tflops": (2 * act_params + attn_flops) * prompt_len / t_pre / 1e12,
        "prefill_frac_of_bf16_peak": (2 * act_params + attn_flops) * prompt_len / t_pre / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec, "decode_ms": t_dec * 1e3, "decode_launches_per_step": launches / (steps + warmup),
        "decode_bytes_per_token": 2 * act_params + kv_bytes, "decode_frac_of_hbm_peak": (2 * act_params + kv_bytes) / t_dec / 1e9 / hbm,
        "e2e_decode_tok_s": e2e}

    # ---- the closest existing model: llama, Q4_K, ffn = top x ff
    shape = synth.ModelShape(f"llama-like-{name}", "llama", W, top * ff, nl, H, G, hs, V, False, 0, 5e5, 1e-5, gguf.GGML_Q4_K, n_ctx=n_ctx)
    tensors = synth.generate_tensors(shape, seed)
    tmap = {n: gguf.GGUFTensor(n, t, tuple(s), np.ascontiguousarray(dd).view(np.uint8).reshape(-1)) for n, t, s, dd in tensors}
    lm = capi.CudaModel(desc=capi.desc_from_model_json(synth.model_json(shape), max_batch=128, n_ctx=n_ctx), tensors=tmap)
    for _ in range(2):
        t_pre_l = _timed_prefill(lm, prompt, 128)
    t_dec_l = _timed_decode(lm, prompt[-1], steps, warmup)
    lm.close()
    l_params = nl * (qkv + H * hs * W + 3 * top * ff * W) + V * W
    l_bytes = l_params * 0.5625 + kv_bytes
    out["llama_q4k"] = {
        "prefill_tok_s": prompt_len / t_pre_l, "prefill_chunk": 128,
        "prefill_tflops": (2 * l_params + attn_flops) * prompt_len / t_pre_l / 1e12,
        "prefill_frac_of_bf16_peak": (2 * l_params + attn_flops) * prompt_len / t_pre_l / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec_l, "decode_ms": t_dec_l * 1e3,
        "decode_bytes_per_token": l_bytes, "decode_frac_of_hbm_peak": l_bytes / t_dec_l / 1e9 / hbm}
    out["peaks"] = {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}
    return out


# name: (width, heads, kv_heads, head size, window, ff, latent (heads, plain dims, rotated dims, value dims, q rank, kv rank), layer types, vocab)
VANAPEL_SIZES = {
    "s": (1024, 16, 4, 64, 512, 2048, (16, 64, 32, 64, 384, 256), "aala", 32000),
    "m": (2048, 16, 4, 128, 1024, 5632, (16, 128, 64, 128, 768, 512), "aala", 32000),
    "l": (4096, 32, 8, 128, 1024, 14336, (32, 128, 64, 128, 1536, 512), "al", 32000),
}


def _measure(m, prompt, chunk, steps, warmup):
    for _ in range(2):
        t_pre = _timed_prefill(m, prompt, chunk)
    l0 = m.be.counter("kernel_launches")
    t_dec = _timed_decode(m, prompt[-1], steps, warmup)
    launches = m.be.counter("kernel_launches") - l0
    t0 = time.perf_counter()
    tok = prompt[-1]
    for _ in range(16):
        tok = int(np.argmax(m.forward([tok])[0]))
    return t_pre, t_dec, launches / (steps + warmup), 16 / (time.perf_counter() - t0)


def _load_synth(cfg, tensors, chunk, n_ctx):
    d = tempfile.mkdtemp(prefix="ps_arch_")
    try:
        arch_synth.write_model_dir(d, cfg, tensors)
        return arch.load_model(d, dtype="bfloat16", max_batch=chunk, n_ctx=n_ctx)
    finally:
        shutil.rmtree(d, ignore_errors=True)


def run_size_vanapel(name, prompt_len, steps, warmup, seed, chunk):
    W, H, G, hs, win, ff, (LH, dn, dr, dv, rq, rk), kinds, V = VANAPEL_SIZES[name]
    hbm, tflops, src = _peaks()
    n_ctx = -(-(prompt_len + steps + warmup + 24) // 256) * 256
    prompt = [int(v) for v in np.random.default_rng(1234).integers(0, V, prompt_len)]
    out = {"size": name, "width": W, "heads": [H, G], "head_size": hs, "window": win, "ff": ff, "latent": [LH, dn, dr, dv, rq, rk], "layers": kinds, "vocab": V, "context": prompt_len}
    layers = [arch_synth.vanapel_attention_layer(H, G, hs, hs, window=win, v_mix=True, ff=ff, limit=7.0) if k == "a" else
              arch_synth.vanapel_latent_layer(LH, dn, dr, dv, rq, rk, rope_base=10000.0, scaling={"factor": 8.0, "original": 1024, "fast": 32.0, "slow": 1.0}, ff=ff, limit=7.0)
              for k in kinds]
    cfg = arch_synth.vanapel_config(W, V, layers, groups=2)
    m = _load_synth(cfg, arch_synth.vanapel_weights(cfg, seed=seed, fast=True), chunk, n_ctx)
    t_pre, t_dec, launches, e2e = _measure(m, prompt, chunk, steps, warmup)
    m.close()
    na, nlat = kinds.count("a"), kinds.count("l")
    p_att = (H + 2 * G) * hs * W + H * hs * W
    p_lat = (rq + rk + dr) * W + LH * (dn + dr) * rq + LH * dn * rk + LH * dv * rk + LH * dv * W
    act_params = na * p_att + nlat * p_lat + len(kinds) * 3 * ff * W + V * W
    keys_a = min(win, prompt_len)
    kv_bytes = na * 2 * G * hs * 4 * keys_a + nlat * (2 * rk + dr) * 4 * prompt_len
    # per token, averaged over the prompt: windowed layers see at most `win` keys, the latent layer (queries with W_uk folded in) all before it
    attn_flops = na * 2 * 2 * H * hs * min(win, prompt_len / 2) + nlat * 2 * LH * (2 * rk + dr) * prompt_len / 2
    out["vanapel"] = {
        "prefill_tok_s": prompt_len / t_pre, "prefill_chunk": chunk,
        "prefill_tflops": (2 * act_params + attn_flops) * prompt_len / t_pre / 1e12,
        "prefill_frac_of_bf16_peak": (2 * act_params + attn_flops) * prompt_len / t_pre / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec, "decode_ms": t_dec * 1e3, "decode_launches_per_step": launches,
        "decode_bytes_per_token": 2 * act_params + kv_bytes, "decode_frac_of_hbm_peak": (2 * act_params + kv_bytes) / t_dec / 1e9 / hbm,
        "e2e_decode_tok_s": e2e}

    # ---- the closest existing model: Nufusun, 8 experts of ff / 2 rows, the best 2 active
    nl, E, top, eff = len(kinds), 8, 2, ff // 2
    ncfg = arch_synth.nufusun_config(W, V, [arch_synth.nufusun_layer(H, G, hs, hs, bias_max=float(prompt_len), experts=E, top=top, ff=eff, limit=7.0) for _ in range(nl)])
    m = _load_synth(ncfg, arch_synth.nufusun_weights(ncfg, seed=seed, rel_rows=32, fast=True), chunk, n_ctx)
    t_pre_n, t_dec_n, launches_n, e2e_n = _measure(m, prompt, chunk, steps, warmup)
    m.close()
    n_params = nl * (p_att + E * W + top * 3 * eff * W) + V * W
    n_kv = nl * 2 * G * hs * 4 * prompt_len
    n_flops = nl * 2 * 2 * H * hs * prompt_len / 2
    out["nufusun"] = {
        "prefill_tok_s": prompt_len / t_pre_n, "prefill_chunk": chunk,
        "prefill_tflops": (2 * n_params + n_flops) * prompt_len / t_pre_n / 1e12,
        "prefill_frac_of_bf16_peak": (2 * n_params + n_flops) * prompt_len / t_pre_n / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec_n, "decode_ms": t_dec_n * 1e3, "decode_launches_per_step": launches_n,
        "decode_bytes_per_token": 2 * n_params + n_kv, "decode_frac_of_hbm_peak": (2 * n_params + n_kv) / t_dec_n / 1e9 / hbm,
        "e2e_decode_tok_s": e2e_n}
    out["peaks"] = {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}
    return out

# name: (width, attention (heads, kv heads, head size, chunk), retention (heads, dim, vdim), state space (heads, vdim, state, groups), ff, layer types, vocab)
DOZOTAR_SIZES = {
    "s": (1024, (16, 4, 64, 512), (8, 64, 128), (32, 64, 128, 2), 1024, "rmma", 32000),
    "m": (2048, (16, 4, 128, 1024), (8, 128, 256), (64, 64, 128, 4), 2816, "rmma", 32000),
    "l": (4096, (32, 8, 128, 1024), (16, 128, 256), (128, 64, 128, 8), 7168, "rma", 32000),
}


def run_size_dozotar(name, prompt_len, steps, warmup, seed, chunk):
    W, (H, G, hs, ck), (RH, rd, rv), (MH, mp, N, mg), ff, kinds, V = DOZOTAR_SIZES[name]
    hbm, tflops, src = _peaks()
    n_ctx = -(-(prompt_len + steps + warmup + 24) // 256) * 256
    prompt = [int(v) for v in np.random.default_rng(1234).integers(0, V, prompt_len)]
    E, top = 8, 2
    out = {"size": name, "width": W, "attention": [H, G, hs, ck], "retention": [RH, rd, rv], "state_space": [MH, mp, N, mg], "ff": ff, "experts": [E, top, ff // 2, ff],
           "layers": kinds, "vocab": V, "context": prompt_len}
    # the first layer's feed-forward is dense (2 ff rows), the others route 2 of 8 experts of ff / 2 rows beside a shared expert of ff rows: 2 ff active rows everywhere
    moe = dict(ff=ff // 2, experts=E, top=top, route_groups=4, route_keep=2, shared_ff=ff)
    layers = []
    for i, k in enumerate(kinds):
        mlp = dict(ff=2 * ff) if i == 0 else moe
        if k == "r":
            layers.append(arch_synth.dozotar_retention_layer(RH, rd, rv, rot_base=5e5, **mlp))
        elif k == "m":
            layers.append(arch_synth.dozotar_mamba2_layer(MH, mp, N, groups=mg, norm_groups=mg, conv=4, **mlp))
        else:
            layers.append(arch_synth.dozotar_attention_layer(H, G, hs, hs, chunk=ck, conv=4, bias_max=float(ck), **mlp))
    cfg = arch_synth.dozotar_config(W, V, layers)
    m = _load_synth(cfg, arch_synth.dozotar_weights(cfg, seed=seed, rel_rows=32, fast=True), chunk, n_ctx)
    t_pre, t_dec, launches, e2e = _measure(m, prompt, chunk, steps, warmup)
    m.close()
    na, nr, nm, nl = kinds.count("a"), kinds.count("r"), kinds.count("m"), len(kinds)
    inner = MH * mp
    p_att = (H + 2 * G) * hs * W + H * hs * W
    p_ret = (2 * RH * rd + 2 * RH * rv) * W + RH * rv * W
    p_mam = (2 * inner + 2 * mg * N + MH) * W + inner * W
    p_ff = 3 * 2 * ff * W + (nl - 1) * ((E + 1) * W + top * 3 * (ff // 2) * W + 3 * ff * W)
    act_params = na * p_att + nr * p_ret + nm * p_mam + p_ff + V * W
    keys = min(ck, prompt_len)
    state_bytes = na * 2 * G * hs * 4 * keys + nr * 2 * RH * rd * rv * 4 + nm * 2 * MH * N * mp * 4        # K / V rows read; recurrent state read and written
    mix_flops = na * 2 * 2 * H * hs * keys / 2 + nr * 4 * RH * rd * rv + nm * 4 * MH * N * mp                # per token
    out["dozotar"] = {
        "prefill_tok_s": prompt_len / t_pre, "prefill_chunk": chunk,
        "prefill_tflops": (2 * act_params + mix_flops) * prompt_len / t_pre / 1e12,
        "prefill_frac_of_bf16_peak": (2 * act_params + mix_flops) * prompt_len / t_pre / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec, "decode_ms": t_dec * 1e3, "decode_launches_per_step": launches,
        "decode_bytes_per_token": 2 * act_params + state_bytes, "decode_frac_of_hbm_peak": (2 * act_params + state_bytes) / t_dec / 1e9 / hbm,
        "e2e_decode_tok_s": e2e}

    # ---- the closest existing model: Nufusun, 8 experts of ff rows, the best 2 active
    ncfg = arch_synth.nufusun_config(W, V, [arch_synth.nufusun_layer(H, G, hs, hs, bias_max=float(prompt_len), experts=E, top=top, ff=ff, limit=7.0) for _ in range(nl)])
    m = _load_synth(ncfg, arch_synth.nufusun_weights(ncfg, seed=seed, rel_rows=32, fast=True), chunk, n_ctx)
    t_pre_n, t_dec_n, launches_n, e2e_n = _measure(m, prompt, chunk, steps, warmup)
    m.close()
    n_params = nl * (p_att + E * W + top * 3 * ff * W) + V * W
    n_kv = nl * 2 * G * hs * 4 * prompt_len
    n_flops = nl * 2 * 2 * H * hs * prompt_len / 2
    out["nufusun"] = {
        "prefill_tok_s": prompt_len / t_pre_n, "prefill_chunk": chunk,
        "prefill_tflops": (2 * n_params + n_flops) * prompt_len / t_pre_n / 1e12,
        "prefill_frac_of_bf16_peak": (2 * n_params + n_flops) * prompt_len / t_pre_n / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec_n, "decode_ms": t_dec_n * 1e3, "decode_launches_per_step": launches_n,
        "decode_bytes_per_token": 2 * n_params + n_kv, "decode_frac_of_hbm_peak": (2 * n_params + n_kv) / t_dec_n / 1e9 / hbm,
        "e2e_decode_tok_s": e2e_n}
    out["peaks"] = {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}
    return out


# name: (width, heads, kv heads, head size, window, pool, minGRU channels, gated-equivalent ff, latent geometry, layer types, loop, vocab)
PIDENEX_SIZES = {
    "s": (1024, 16, 4, 64, 512, 16, 512, 2048, (16, 64, 32, 64, 384, 256), "apl", (0, 2, 2), 32000),
    "m": (2048, 16, 4, 128, 1024, 16, 1024, 5632, (16, 128, 64, 128, 768, 512), "apl", (0, 2, 2), 32000),
    "l": (4096, 32, 8, 128, 1024, 16, 2048, 14336, (32, 128, 64, 128, 1536, 512), "apl", None, 32000),
}


def run_size_pidenex(name, prompt_len, steps, warmup, seed, chunk):
    W, H, G, hs, win, pool, R, ff, (LH, dn, dr, dv, rq, rk), kinds, loop, V = PIDENEX_SIZES[name]
    hbm, tflops, src = _peaks()
    n_ctx = -(-(prompt_len + steps + warmup + 24) // 256) * 256
    prompt = [int(v) for v in np.random.default_rng(1234).integers(0, V, prompt_len)]
    ffp = 3 * ff // 2                                                # up and down rows of an ungated unit: the bytes of a gated unit of ff rows
    out = {"size": name, "width": W, "heads": [H, G], "head_size": hs, "window": win, "pool": pool, "gru": R, "ff": ffp, "latent": [LH, dn, dr, dv, rq, rk],
           "layers": kinds, "loop": loop, "vocab": V, "context": prompt_len}
    layers = []
    for k in kinds:
        if k == "a":
            layers.append(arch_synth.pidenex_attention_layer(H, G, hs, window=win, pool=pool, ff=ffp))
        elif k == "p":
            layers.append(arch_synth.pidenex_parallel_layer(H, G, hs, window=win, gru_width=R, ff=ffp))
        else:
            layers.append(arch_synth.pidenex_latent_layer(LH, dn, dr, dv, rq, rk, window=win, rope_base=5e5, ff=ffp))
    cfg = arch_synth.pidenex_config(W, V, layers, loop=loop, embed_scale=2.0)
    m = _load_synth(cfg, arch_synth.pidenex_weights(cfg, seed=seed, fast=True), chunk, n_ctx)
    t_pre, t_dec, launches, e2e = _measure(m, prompt, chunk, steps, warmup)
    m.close()
    runs = "".join(kinds[i] for i, _ in arch._pidenex_runs(cfg))
    na, npar, nlat = runs.count("a"), runs.count("p"), runs.count("l")
    p_att = (H + G) * hs * W + H * hs * W
    p_par = (H + G) * hs * W + 2 * H * hs * W + 4 * R * W
    p_lat = (rq + rk + dr) * W + LH * (dn + dr) * rq + LH * dn * rk + LH * dv * rk + LH * dv * W
    act_params = na * p_att + npar * p_par + nlat * p_lat + len(runs) * 2 * ffp * W + V * W   # every run streams its weights, shared or not
    keys = min(win, prompt_len)
    blocks = max(0, prompt_len - win) // pool
    kv_bytes = (na + npar) * 2 * G * hs * 4 * keys + na * 2 * G * hs * 4 * blocks + npar * 2 * R * 4 + nlat * (2 * rk + dr) * 4 * keys
    mix_flops = (na + npar) * 2 * 2 * H * hs * min(win, prompt_len / 2) + na * 2 * 2 * H * hs * blocks / 2 + nlat * 2 * LH * (2 * rk + dr) * min(win, prompt_len / 2)
    out["pidenex"] = {
        "runs": runs, "prefill_tok_s": prompt_len / t_pre, "prefill_chunk": chunk,
        "prefill_tflops": (2 * act_params + mix_flops) * prompt_len / t_pre / 1e12,
        "prefill_frac_of_bf16_peak": (2 * act_params + mix_flops) * prompt_len / t_pre / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec, "decode_ms": t_dec * 1e3, "decode_launches_per_step": launches,
        "decode_bytes_per_token": 2 * act_params + kv_bytes, "decode_frac_of_hbm_peak": (2 * act_params + kv_bytes) / t_dec / 1e9 / hbm,
        "e2e_decode_tok_s": e2e}

    # ---- the closest existing model: Vanapel with a layer per run (the parallel layer's place taken by a windowed attention layer)
    vkinds = runs.replace("p", "a")
    vlayers = [arch_synth.vanapel_attention_layer(H, G, hs, hs, window=win, ff=ff, limit=7.0) if k == "a" else
               arch_synth.vanapel_latent_layer(LH, dn, dr, dv, rq, rk, rope_base=5e5, ff=ff, limit=7.0) for k in vkinds]
    vcfg = arch_synth.vanapel_config(W, V, vlayers, groups=1)
    m = _load_synth(vcfg, arch_synth.vanapel_weights(vcfg, seed=seed, fast=True), chunk, n_ctx)
    t_pre_v, t_dec_v, launches_v, e2e_v = _measure(m, prompt, chunk, steps, warmup)
    m.close()
    va, vl = vkinds.count("a"), vkinds.count("l")
    v_params = va * ((H + 2 * G) * hs * W + H * hs * W) + vl * p_lat + len(vkinds) * 3 * ff * W + V * W
    v_kv = va * 2 * G * hs * 4 * keys + vl * (2 * rk + dr) * 4 * prompt_len
    v_flops = va * 2 * 2 * H * hs * min(win, prompt_len / 2) + vl * 2 * LH * (2 * rk + dr) * prompt_len / 2
    out["vanapel"] = {
        "layers": vkinds, "prefill_tok_s": prompt_len / t_pre_v, "prefill_chunk": chunk,
        "prefill_tflops": (2 * v_params + v_flops) * prompt_len / t_pre_v / 1e12,
        "prefill_frac_of_bf16_peak": (2 * v_params + v_flops) * prompt_len / t_pre_v / 1e12 / tflops,
        "decode_tok_s": 1 / t_dec_v, "decode_ms": t_dec_v * 1e3, "decode_launches_per_step": launches_v,
        "decode_bytes_per_token": 2 * v_params + v_kv, "decode_frac_of_hbm_peak": (2 * v_params + v_kv) / t_dec_v / 1e9 / hbm,
        "e2e_decode_tok_s": e2e_v}
    out["peaks"] = {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}
    return out


def main(args) -> int:
    if capi.load_library().ps_cuda_device_count() == 0:
        print(json.dumps({"arch": args.arch, "unavailable": "no CUDA device: there is no CPU fallback"}))
        return 1
    sizes = [s for s in args.arch_sizes.split(",") if s]
    if args.arch == "dozotar":
        res = [run_size_dozotar(s, args.arch_prompt, max(args.steps, 8), max(args.warmup, 3), args.seed, args.arch_chunk) for s in sizes]
        print(json.dumps({"arch": "dozotar", "dtype": "bf16", "data": "synthetic", "timing": "CUDA events around every call, warm-up first; weights exceed L2",
                          "sizes": res}))
        return 0
    if args.arch == "pidenex":
        res = [run_size_pidenex(s, args.arch_prompt, max(args.steps, 8), max(args.warmup, 3), args.seed, args.arch_chunk) for s in sizes]
        print(json.dumps({"arch": "pidenex", "dtype": "bf16", "data": "synthetic", "timing": "CUDA events around every call, warm-up first; weights exceed L2",
                          "sizes": res}))
        return 0
    if args.arch == "vanapel":
        res = [run_size_vanapel(s, args.arch_prompt, max(args.steps, 8), max(args.warmup, 3), args.seed, args.arch_chunk) for s in sizes]
        print(json.dumps({"arch": "vanapel", "dtype": "bf16", "data": "synthetic", "timing": "CUDA events around every call, warm-up first; weights exceed L2",
                          "sizes": res}))
        return 0
    res = [run_size(s, args.arch_prompt, max(args.steps, 8), max(args.warmup, 3), args.seed, args.arch_chunk) for s in sizes]
    print(json.dumps({"arch": "nufusun", "dtype": "bf16", "data": "synthetic", "timing": "CUDA events around every call, warm-up first; weights exceed L2",
                      "sizes": res}))
    return 0
