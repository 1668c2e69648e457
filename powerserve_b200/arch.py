"""Layer-list models (config.json + model.safetensors) on the CUDA backend, and the model registry.

`load_model(path)` is how every front end (bin/trace_run, the generation command line, bench.py, tests) gets a model: a
PowerServe model directory (model.json + ggml/weights.gguf) becomes a `capi.CudaModel`, a directory with a config.json
becomes the class its "architecture" names in `ARCHITECTURES`.  Both are the same kind of object - a bound ps_cuda
context with forward / prefill / generate / decode_greedy / sample_topk / sessions.

A design registers a function that turns its config.json into the backend's layer descriptions (include/ps_cuda.h,
"layer-list models") and one that names its tensors; the constants a design fixes live in that function, everything a
config file may vary is read from the file.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from . import capi, safetensors
from .capi import ArchDesc, ArchLayerWeights, ArchWeights, LayerDesc, Tensor


class LayerListModel(capi.CudaModel):
    """A layer-list model bound through ps_cuda_create_arch / ps_cuda_bind_arch.  Everything after construction is
    capi.CudaModel's: the context behaves like a llama context behind the shared entry points."""

    def __init__(self, path: str, *, dtype: str = "bfloat16", max_batch: int = 128, n_ctx: int = 4096, device: int = 0):
        cfg = json.load(open(os.path.join(path, "config.json")))
        name = cfg.get("architecture")
        if name not in ARCHITECTURES:
            raise capi.PsCudaError(f"{path}: unknown architecture {name!r} (known: {sorted(ARCHITECTURES)})")
        describe, tensor_names = ARCHITECTURES[name]
        self.cfg = cfg
        self._keep: List[object] = []
        self._file = safetensors.SafeTensorsFile(os.path.join(path, "model.safetensors"))
        self.tensors = self._file.tensors
        compute = {"bfloat16": capi.COMPUTE_BF16, "float32": capi.COMPUTE_F32}[dtype]
        layers, top = describe(cfg, self.tensors)
        self._layer_descs = (LayerDesc * len(layers))(*layers)
        self.desc = ArchDesc(top["dim"], top["vocab_size"], len(layers), int(n_ctx), int(max_batch), top["norm_eps"], top["embed_scale"],
                             top["norm_unit_offset"], compute, self._layer_descs, int(top.get("norm_groups", 1)), int(top.get("norm_scalar", 0)),
                             int(top.get("norm_kind", 0)), int(top.get("n_pass_steps", 0)))
        self.vocab = self.desc.vocab_size
        self.be = capi.CudaBackend(self.desc, device)

        def T(n) -> Tensor:
            if n is None:
                return Tensor(None, 0, 0)
            if not isinstance(n, str):          # constants of the configuration, handed over as a float32 array
                arr = np.ascontiguousarray(n, np.float32)
                self._keep.append(arr)
                return Tensor(arr.ctypes.data, safetensors.PS_F32, 0)
            if n not in self.tensors:
                raise capi.PsCudaError(f"{path}: tensor {n} is missing")
            t = self.tensors[n]
            return Tensor(t.host_ptr, t.ps_type, 0)

        names = tensor_names(cfg)
        self._lw = (ArchLayerWeights * len(layers))()
        for i, ln in enumerate(names["layers"]):
            lw = ArchLayerWeights()
            for f in ("norm", "q", "q_bias", "k", "k_bias", "v", "v_bias", "o", "o_bias", "rel", "head_mix", "head_temp", "router") + capi.ARCH_LAYER_VECTORS_2:
                setattr(lw, f, T(ln.get(f)))
            for f in ("gate", "up", "down"):
                lst = ln.get(f)
                if lst:
                    arr = (Tensor * len(lst))(*[T(n) for n in lst])
                    self._keep.append(arr)
                    setattr(lw, f, arr)
            self._lw[i] = lw
        self._w = ArchWeights(T(names["embed"]), T(names["final_norm"]), T(names["head"]), self._lw, T(names.get("pass_steps")))
        self.be._ck(self.be.L.ps_cuda_bind_arch(self.be.h, C.byref(self._w)))

    def layer_tap(self, layer: int, bs: int):
        """residual stream after `layer` of the last forward pass (option arch_taps)"""
        import numpy as np
        out = np.empty((bs, self.desc.dim), np.float32)
        self.be._ck(self.be.L.ps_cuda_arch_tap(self.be.h, layer, out.ctypes.data, bs))
        return out


# ------------------------------------------------------------------------------------------------------------ Nufusun
# Decoder-only; every layer is a parallel block (one unit-offset RMS norm feeds the mixer AND the feed-forward).  Mixer:
# grouped-query attention without rotation, projection biases, per-head temperature, a bucketed distance bias, head mixing
# before the soft-max, a value-less sink in the denominator.  Feed-forward: sigmoid-routed experts whose score scales the
# expert's input, scores not renormalised; expert activation g * sigmoid(1.702 g) * (u + 1) on clamped g, u.
def _nufusun_describe(cfg: dict, tensors) -> Tuple[List[LayerDesc], dict]:
    layers = []
    for i, l in enumerate(cfg["layers"]):
        if l["type"] != "attention":
            raise capi.PsCudaError(f"Nufusun layer {i}: unknown mixer type {l['type']!r}")
        m = l["mixer"]
        d = LayerDesc()
        d.mixer_kind = capi.MIXER_ATTENTION
        d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        d.score_scale = m["scale"]
        d.proj_bias, d.head_temp, d.head_mix, d.sink = 1, 1, 1, 1
        d.rel_buckets = int(tensors[f"l{i}.mix.rel"].shape[0])      # the table's own row count
        d.rel_max_dist = m["bias_max"]
        mlp = l.get("mlp")
        if mlp is None:
            d.mlp_kind = capi.MLP_NONE
        elif mlp.get("kind") == "moe":
            d.mlp_kind = capi.MLP_ROUTED
            d.n_experts, d.top_k = mlp["router"]["experts"], mlp["router"]["top"]
            d.expert_ff, d.act_limit = mlp["expert"]["ff"], mlp["expert"]["limit"]
            d.router_act, d.route_on_input, d.route_renorm = 1, 1, 0
            d.act_alpha, d.up_shift = 1.702, 1.0
        else:
            raise capi.PsCudaError(f"Nufusun layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(d)
    top = {"dim": cfg["width"], "vocab_size": cfg["vocab"], "norm_eps": cfg["norm"]["eps"], "embed_scale": cfg["embedding"]["scale"],
           "norm_unit_offset": 1}
    return layers, top


def _nufusun_tensor_names(cfg: dict) -> dict:
    out = {"embed": "embed", "final_norm": "final.norm", "head": "head", "layers": []}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = {"norm": p + "norm1", "q": p + "mix.q", "q_bias": p + "mix.q.b", "k": p + "mix.k", "k_bias": p + "mix.k.b", "v": p + "mix.v",
             "v_bias": p + "mix.v.b", "o": p + "mix.o", "o_bias": p + "mix.o.b", "rel": p + "mix.rel", "head_mix": p + "mix.talk",
             "head_temp": p + "mix.temp"}
        if l.get("mlp") is not None:
            E = l["mlp"]["router"]["experts"]
            n["router"] = p + "mlp.router"
            for f in ("gate", "up", "down"):
                n[f] = [f"{p}mlp.e{e}.{f}" for e in range(E)]
        out["layers"].append(n)
    return out


# ------------------------------------------------------------------------------------------------------------ Vanapel
# Decoder-only; every layer is a sequential block whose sublayers are normed on the way in AND on the way out,
#   x <- x + N1b(mixer(N1(x))),  x <- x + N2b(ff(N2(x))),
# with RMS norms taken over `norm.groups` equal parts of the vector.  Two mixers, chosen per layer by "type":
#   "attention"         grouped-query, no rotation and no biases; q and k of every head scaled to unit RMS; the score loses
#                       r1_h ln(1 + r2_h (i - j)) with distance; a sliding window of mask.size keys; a learned per-head sink
#                       logit in the soft-max denominator; layers marked v_mix blend their values with those of the FIRST marked
#                       layer (weight '.vmix'; the first one's own is unused).
#   "latent_attention"  queries through a normed latent, keys / values up-projected from a shared normed latent plus one
#                       rotated key part common to all heads (rotate-half pairs, YaRN-scaled frequencies); causal; learned sink.
# Feed-forward: one gated unit, y = g sigmoid(1.702 g) (u + 1) on g = min(gate, limit), u = clamp(up, +-limit).
def _vanapel_describe(cfg: dict, tensors) -> Tuple[List[LayerDesc], dict]:
    layers = []
    v_source_seen = False
    for i, l in enumerate(cfg["layers"]):
        m = l["mixer"]
        d = LayerDesc()
        d.block_kind, d.post_norm = capi.BLOCK_SEQUENTIAL, 1
        d.n_heads, d.qk_dim, d.v_dim = m["heads"], m["dim"], m["vdim"]
        d.score_scale = m["scale"]
        d.sink = capi.SINK_LEARNED
        if l["type"] == "attention":
            d.mixer_kind = capi.MIXER_ATTENTION
            d.n_kv_heads = m["kv_heads"]
            d.qk_norm, d.log_bias = 1, 1
            d.window = int((m.get("mask") or {}).get("size", 0))
            if m.get("v_mix"):
                d.v_mix = capi.VMIX_BLEND if v_source_seen else capi.VMIX_SOURCE
                v_source_seen = True
        elif l["type"] == "latent_attention":
            d.mixer_kind = capi.MIXER_LATENT
            d.n_kv_heads = 1
            d.q_rank, d.kv_rank, d.rot_dim = m["q_rank"], m["kv_rank"], m["rot_dim"]
            rot = m.get("rot") or {}
            d.rope_dims, d.rope_base = int(rot.get("dims", d.rot_dim)), float(rot.get("base", 10000.0))
            sc = rot.get("scaling")
            if sc:
                d.rope_factor, d.rope_original, d.rope_fast, d.rope_slow = float(sc["factor"]), int(sc["original"]), float(sc["fast"]), float(sc["slow"])
            d.window = int((m.get("mask") or {}).get("size", 0))
        else:
            raise capi.PsCudaError(f"Vanapel layer {i}: unknown mixer type {l['type']!r}")
        mlp = l.get("mlp")
        if mlp is None:
            d.mlp_kind = capi.MLP_NONE
        elif mlp.get("kind") == "dense":
            d.mlp_kind = capi.MLP_DENSE
            d.expert_ff, d.act_limit = mlp["ff"], mlp["limit"]
            d.act_alpha, d.up_shift = 1.702, 1.0
        else:
            raise capi.PsCudaError(f"Vanapel layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(d)
    top = {"dim": cfg["width"], "vocab_size": cfg["vocab"], "norm_eps": cfg["norm"]["eps"], "embed_scale": 1.0, "norm_unit_offset": 0,
           "norm_groups": int(cfg["norm"].get("groups", 1))}
    return layers, top


def _vanapel_tensor_names(cfg: dict) -> dict:
    out = {"embed": "embed", "final_norm": "final.norm", "head": "head", "layers": []}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = {"norm": p + "norm1", "norm_mix_out": p + "norm1b", "o": p + "mix.o", "sink": p + "mix.sink"}
        if l["type"] == "attention":
            n.update({"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "r1": p + "mix.r1", "r2": p + "mix.r2"})
            if l["mixer"].get("v_mix"):
                n["vmix"] = p + "mix.vmix"
        else:
            n.update({"dq": p + "mix.dq", "dq_norm": p + "mix.dq.norm", "uq": p + "mix.uq", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm",
                      "uk": p + "mix.uk", "uv": p + "mix.uv"})
        if l.get("mlp") is not None:
            n.update({"norm_ff": p + "norm2", "norm_ff_out": p + "norm2b"})
            for f in ("gate", "up", "down"):
                n[f] = [f"{p}mlp.{f}"]
        out["layers"].append(n)
    return out


# ------------------------------------------------------------------------------------------------------------ Dozotar
# Decoder-only; every layer is a sequential block whose sublayers read the residual stream itself and are normed on the way out only,
#   x <- x + N(mixer(x)) g1,  x <- x + N(ff(x)) g2,   N an RMS norm, g1 / g2 single numbers.  Three mixers, chosen per layer by "type":
#   "attention"  grouped-query, no rotation; a short causal convolution on q, k and v after the projections; q and k normed over the
#                whole projection with weights; a bucketed distance bias; attention inside chunks of mask.size positions; plain soft-max.
#   "retention"  linear attention with a fixed decay per head: rotated q / k (rotate-half pairs), k / sqrt(dim), per-head RMS of the
#                output, a silu gate.
#   "mamba2"     state-space recurrence: one input projection [z | x | B | C | dt], convolution + silu on x|B|C, softplus step sizes,
#                gated output normed in norm_groups parts.
# Feed-forward: dense with the tanh form of gelu, or soft-max-routed silu experts chosen inside the best groups of neighbours, weights
# renormalised (+ 1e-20), plus a shared expert behind a sigmoid gate.
def _dozotar_describe(cfg: dict, tensors) -> Tuple[List[LayerDesc], dict]:
    layers = []
    for i, l in enumerate(cfg["layers"]):
        m = l["mixer"]
        d = LayerDesc()
        d.block_kind, d.post_norm, d.raw_input = capi.BLOCK_SEQUENTIAL, 1, 1
        d.n_heads, d.v_dim = m["heads"], m["vdim"]
        if l["type"] == "attention":
            d.mixer_kind = capi.MIXER_ATTENTION
            d.n_kv_heads, d.qk_dim = m["kv_heads"], m["dim"]
            d.score_scale = m["scale"]
            d.qk_norm = capi.QKNORM_WHOLE
            d.conv_taps = int(tensors[f"l{i}.mix.q.conv"].shape[1]) if m.get("conv") else 0    # the taps the stored kernel has
            d.rel_buckets = int(tensors[f"l{i}.mix.rel"].shape[0])      # the table's own row count
            d.rel_max_dist = m["bias_max"]
            d.chunk = int((m.get("mask") or {}).get("size", 0))
        elif l["type"] == "retention":
            d.mixer_kind = capi.MIXER_RETENTION
            d.n_kv_heads, d.qk_dim = m["heads"], m["dim"]
            rot = m.get("rot") or {}
            d.rope_dims, d.rope_base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
            if len(m["decay"]) != m["heads"]:
                raise capi.PsCudaError(f"Dozotar layer {i}: {len(m['decay'])} decays for {m['heads']} heads")
        elif l["type"] == "mamba2":
            d.mixer_kind = capi.MIXER_MAMBA2
            d.n_kv_heads = m["groups"]
            d.ssm_state, d.ssm_groups, d.gate_norm_groups = m["state"], m["groups"], m["norm_groups"]
            d.conv_taps = int(tensors[f"l{i}.mix.conv"].shape[1])      # the taps the stored kernel has
        else:
            raise capi.PsCudaError(f"Dozotar layer {i}: unknown mixer type {l['type']!r}")
        mlp = l.get("mlp")
        d.act_limit, d.act_alpha, d.up_shift = float("inf"), 1.0, 0.0   # silu(gate) * up where the activation is the swish kind
        if mlp is None:
            d.mlp_kind = capi.MLP_NONE
        elif mlp.get("kind") == "dense":
            d.mlp_kind, d.expert_ff, d.act_kind = capi.MLP_DENSE, mlp["ff"], capi.ACT_GELU_TANH
        elif mlp.get("kind") == "moe":
            r = mlp["router"]
            d.mlp_kind, d.act_kind = capi.MLP_ROUTED, capi.ACT_SWISH
            d.n_experts, d.top_k, d.expert_ff = r["experts"], r["top"], mlp["expert"]["ff"]
            d.router_act, d.route_on_input, d.route_renorm, d.route_renorm_eps = capi.ROUTER_SOFTMAX, 0, 1, 1e-20
            g = r.get("groups") or {}
            d.route_groups, d.route_keep = int(g.get("count", 1)), int(g.get("keep", 1))
            if mlp.get("shared"):
                d.shared_ff, d.shared_gate = mlp["shared"]["ff"], 1
        else:
            raise capi.PsCudaError(f"Dozotar layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        layers.append(d)
    top = {"dim": cfg["width"], "vocab_size": cfg["vocab"], "norm_eps": cfg["norm"]["eps"], "embed_scale": 1.0, "norm_unit_offset": 0, "norm_scalar": 1}
    return layers, top


def _dozotar_tensor_names(cfg: dict) -> dict:
    out = {"embed": "embed", "final_norm": "final.norm", "head": "head", "layers": []}
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = {"norm_mix_out": p + "norm1", "o": p + "mix.o"}
        if l["type"] == "attention":
            n.update({"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm", "rel": p + "mix.rel"})
            if l["mixer"].get("conv"):
                n.update({"q_conv": p + "mix.q.conv", "k_conv": p + "mix.k.conv", "v_conv": p + "mix.v.conv"})
        elif l["type"] == "retention":
            n.update({"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "g": p + "mix.g", "decay": np.asarray(l["mixer"]["decay"], np.float32)})
        else:
            n.update({"w_in": p + "mix.in", "conv_w": p + "mix.conv", "conv_b": p + "mix.conv.b", "dt_bias": p + "mix.dt_bias", "a_log": p + "mix.A_log",
                      "d_skip": p + "mix.D", "mix_norm": p + "mix.norm"})
        mlp = l.get("mlp")
        if mlp is not None:
            n["norm_ff_out"] = p + "norm2"
            if mlp.get("kind") == "moe":
                n["router"] = p + "mlp.router"
                for f in ("gate", "up", "down"):
                    n[f] = [f"{p}mlp.e{e}.{f}" for e in range(mlp["router"]["experts"])]
                if mlp.get("shared"):
                    n.update({"shared_gate": p + "mlp.shared.gate", "shared_up": p + "mlp.shared.up", "shared_down": p + "mlp.shared.down", "shared_sg": p + "mlp.shared.sg"})
            else:
                for f in ("gate", "up", "down"):
                    n[f] = [f"{p}mlp.{f}"]
        out["layers"].append(n)
    return out


# ------------------------------------------------------------------------------------------------------------ Pidenex
# Decoder-only; every layer is a sequential block with a layer norm (mean removed, weight, no bias) on the way into AND out of every
# sublayer.  config "loop" runs the layers start .. stop - 1 `times` times with the same weights - every pass with a cache / state of
# its own - then the rest; before every pass but the first the embedding output joins the stream, before every pass row t of "loop.step".
# The descriptor therefore lists layer RUNS; a repeated run names the run whose weights it uses.  Three mixers, chosen by "type":
#   "attention"         grouped-query, no rotation, the values ARE the projected keys; a window of mask.size tokens plus one mean key /
#                       value per block of mask.pool tokens that lies wholly before the window.
#   "parallel"          two mixers on the same input, summed with left_scale / right_scale: "left" an attention whose values are the
#                       un-normed keys, q / k normed over the whole projection with weights, a penalty slope_h (i - j) with
#                       slope_h = 2^(-8 (h + 1) / H), a window, a sigmoid output gate; "right" a minGRU recurrence.
#   "latent_attention"  queries through a normed latent, keys / values from a shared normed latent plus one rotated key part common to
#                       all heads; rotation in neighbouring pairs (2i, 2i + 1); a window.
# Feed-forward: down(xIELU(up h)) with the activation's two numbers per layer.  Embedding scaled; final layer norm; untied head.
def _pidenex_runs(cfg: dict) -> List[Tuple[int, Optional[int]]]:
    """(layer, number of the pass that this run opens or None) in execution order"""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {}
    a, b, times = int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 1))
    if not (0 <= a <= b <= n) or times < 1:
        raise capi.PsCudaError(f"Pidenex: loop {lp!r} does not fit {n} layers")
    runs: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(a)]
    if b > a:
        for t in range(times):
            runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def _pidenex_attention(d: LayerDesc, m: dict) -> None:
    d.mixer_kind = capi.MIXER_ATTENTION
    d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    d.score_scale = m["scale"]
    d.v_is_k = 1
    mask = m.get("mask") or {}
    d.window, d.pool = int(mask.get("size", 0)), int(mask.get("pool", 0))


def _pidenex_describe(cfg: dict, tensors) -> Tuple[List[LayerDesc], dict]:
    layers = []
    first_run: Dict[int, int] = {}
    for r, (i, t) in enumerate(_pidenex_runs(cfg)):
        l = cfg["layers"][i]
        m = l["mixer"]
        d = LayerDesc()
        d.block_kind, d.post_norm = capi.BLOCK_SEQUENTIAL, 1
        if l["type"] == "attention":
            _pidenex_attention(d, m)
        elif l["type"] == "parallel":
            _pidenex_attention(d, m["left"])
            d.qk_norm, d.lin_bias, d.out_gate = capi.QKNORM_WHOLE, 1, 1
            d.side_kind, d.side_width = capi.MIXER_MINGRU, int(m["right"]["width"])
            d.mix_scale, d.side_scale = float(m["left_scale"]), float(m["right_scale"])
        elif l["type"] == "latent_attention":
            d.mixer_kind = capi.MIXER_LATENT
            d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim = m["heads"], 1, m["dim"], m["vdim"]
            d.score_scale = m["scale"]
            d.q_rank, d.kv_rank, d.rot_dim = m["q_rank"], m["kv_rank"], m["rot_dim"]
            rot = m.get("rot") or {}
            d.rope_dims, d.rope_base, d.rope_interleaved = int(rot.get("dims", d.rot_dim)), float(rot.get("base", 10000.0)), 1
            d.window = int((m.get("mask") or {}).get("size", 0))
        else:
            raise capi.PsCudaError(f"Pidenex layer {i}: unknown mixer type {l['type']!r}")
        mlp = l.get("mlp")
        if mlp is None:
            d.mlp_kind = capi.MLP_NONE
        elif mlp.get("kind") == "dense":
            d.mlp_kind, d.expert_ff, d.mlp_ungated, d.act_kind = capi.MLP_DENSE, mlp["ff"], 1, capi.ACT_XIELU
        else:
            raise capi.PsCudaError(f"Pidenex layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        if i in first_run:
            d.share_weights = first_run[i] + 1
        else:
            first_run[i] = r
        if t is not None:
            d.pass_step = t + 1
            d.pass_embed = 1 if t > 0 else 0
        layers.append(d)
    lp = cfg.get("loop") or {}
    looped = int(lp.get("stop", 0)) > int(lp.get("start", 0))
    top = {"dim": cfg["width"], "vocab_size": cfg["vocab"], "norm_eps": cfg["norm"]["eps"], "embed_scale": cfg["embedding"]["scale"], "norm_unit_offset": 0,
           "norm_kind": capi.NORM_LAYER, "n_pass_steps": int(lp.get("times", 1)) if looped else 0}
    return layers, top


def _pidenex_tensor_names(cfg: dict) -> dict:
    out = {"embed": "embed", "final_norm": "final.norm", "head": "head", "layers": []}
    lp = cfg.get("loop") or {}
    if int(lp.get("stop", 0)) > int(lp.get("start", 0)):
        out["pass_steps"] = "loop.step"
    seen = set()
    for i, _ in _pidenex_runs(cfg):
        if i in seen:                 # a repeated run: the weights of its first run
            out["layers"].append({})
            continue
        seen.add(i)
        l = cfg["layers"][i]
        p = f"l{i}."
        n = {"norm": p + "norm1", "norm_mix_out": p + "norm1b"}
        if l["type"] == "attention":
            n.update({"q": p + "mix.q", "k": p + "mix.k", "o": p + "mix.o"})
        elif l["type"] == "parallel":
            a, b = p + "mix.left.", p + "mix.right."
            H = l["mixer"]["left"]["heads"]
            n.update({"q": a + "q", "k": a + "k", "q_norm": a + "q.norm", "k_norm": a + "k.norm", "g": a + "g", "o": a + "o",
                      "lin": np.asarray([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], np.float32),
                      "side_z": b + "z", "side_z_bias": b + "z.b", "side_x": b + "x", "side_x_bias": b + "x.b", "side_g": b + "g", "side_o": b + "o"})
        else:
            n.update({"dq": p + "mix.dq", "dq_norm": p + "mix.dq.norm", "uq": p + "mix.uq", "dkv": p + "mix.dkv", "dkv_norm": p + "mix.dkv.norm",
                      "uk": p + "mix.uk", "uv": p + "mix.uv", "o": p + "mix.o"})
        if l.get("mlp") is not None:
            n.update({"norm_ff": p + "norm2", "norm_ff_out": p + "norm2b", "up": [p + "mlp.up"], "down": [p + "mlp.down"], "act": p + "mlp.act"})
        out["layers"].append(n)
    return out


ARCHITECTURES: Dict[str, Tuple[Callable, Callable]] = {
    "Dozotar": (_dozotar_describe, _dozotar_tensor_names),
    "Pidenex": (_pidenex_describe, _pidenex_tensor_names),
    "Nufusun": (_nufusun_describe, _nufusun_tensor_names),
    "Vanapel": (_vanapel_describe, _vanapel_tensor_names),
}


def load_model(path: str, *, dtype: str = "bfloat16", max_batch: int = 128, n_ctx: Optional[int] = None, device: int = 0):
    """The model class is chosen by what the directory holds."""
    if os.path.exists(os.path.join(path, "model.json")):
        if dtype != "bfloat16" and dtype != "native":
            raise capi.PsCudaError("GGUF models run in their stored quantised formats; --dtype does not apply")
        return capi.CudaModel(path, max_batch=max_batch, device=device)
    if os.path.exists(os.path.join(path, "config.json")):
        return LayerListModel(path, dtype=dtype, max_batch=max_batch, n_ctx=n_ctx or 4096, device=device)
    raise capi.PsCudaError(f"{path}: neither model.json (PowerServe / GGUF) nor config.json (layer list) found")
