"""CPU-only checks around the Dozotar design: the registry's reading of a configuration (every size and constant comes from the
file), the tensor names, and the oracle's own invariants (it is what the GPU tests compare with, so it is checked against
hand-computed cases and second formulations here)."""
import math

import numpy as np
import pytest

from powerserve_b200 import arch, arch_synth, capi
from tests import _dozotar_ref as R

AT, RE, MA = arch_synth.dozotar_attention_layer, arch_synth.dozotar_retention_layer, arch_synth.dozotar_mamba2_layer


class _Shape:
    def __init__(self, *shape):
        self.shape = shape


def test_registry_reads_every_size_from_the_configuration():
    layers = [RE(3, 10, 14, decay=[0.5, 0.75, 0.875], rot_dims=6, rot_base=500.0, ff=44),
              MA(6, 5, 9, groups=3, norm_groups=2, conv=5, ff=12, experts=10, top=3, shared_ff=20),
              AT(6, 3, 12, 20, chunk=9, conv=4, scale=0.21, bias_max=77.0)]
    layers[1]["mlp"]["router"]["groups"] = {"count": 5, "keep": 2}
    cfg = arch_synth.dozotar_config(60, 99, layers, eps=3e-5)
    shapes = {"l1.mix.conv": _Shape(33, 5), "l2.mix.rel": _Shape(22, 6), "l2.mix.q.conv": _Shape(72, 4)}
    descs, top = arch.ARCHITECTURES["Dozotar"][0](cfg, shapes)
    assert top == {"dim": 60, "vocab_size": 99, "norm_eps": 3e-5, "embed_scale": 1.0, "norm_unit_offset": 0, "norm_scalar": 1}
    d = descs[0]
    assert (d.mixer_kind, d.n_heads, d.qk_dim, d.v_dim, d.rope_dims, d.rope_base) == (capi.MIXER_RETENTION, 3, 10, 14, 6, 500.0)
    assert (d.block_kind, d.post_norm, d.raw_input) == (capi.BLOCK_SEQUENTIAL, 1, 1)
    assert (d.mlp_kind, d.expert_ff, d.act_kind) == (capi.MLP_DENSE, 44, capi.ACT_GELU_TANH)
    d = descs[1]
    assert (d.mixer_kind, d.n_heads, d.v_dim, d.ssm_state, d.ssm_groups, d.gate_norm_groups, d.conv_taps) == (capi.MIXER_MAMBA2, 6, 5, 9, 3, 2, 5)
    assert (d.mlp_kind, d.n_experts, d.top_k, d.expert_ff, d.route_groups, d.route_keep, d.shared_ff, d.shared_gate) == (capi.MLP_ROUTED, 10, 3, 12, 5, 2, 20, 1)
    assert (d.router_act, d.route_on_input, d.route_renorm, d.act_kind) == (capi.ROUTER_SOFTMAX, 0, 1, capi.ACT_SWISH)
    assert d.act_alpha == 1.0 and d.up_shift == 0.0 and math.isinf(d.act_limit) and 0 < d.route_renorm_eps < 1e-19
    d = descs[2]
    assert (d.mixer_kind, d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim, d.chunk, d.conv_taps, d.rel_buckets, d.qk_norm) == (capi.MIXER_ATTENTION, 6, 3, 12, 20, 9, 4, 22, capi.QKNORM_WHOLE)
    assert abs(d.score_scale - 0.21) < 1e-7 and d.rel_max_dist == 77.0 and d.sink == capi.SINK_NONE and d.window == 0 and d.mlp_kind == capi.MLP_NONE


def test_tensor_names_follow_the_layer_types():
    cfg = arch_synth.dozotar_config(16, 8, [RE(2, 4, 4, ff=8), MA(2, 4, 3, ff=8, experts=3, top=1, shared_ff=4), AT(2, 1, 4, 4, chunk=3)])
    n = arch.ARCHITECTURES["Dozotar"][1](cfg)
    assert (n["embed"], n["final_norm"], n["head"]) == ("embed", "final.norm", "head")
    l0, l1, l2 = n["layers"]
    assert "norm" not in l0 and l0["norm_mix_out"] == "l0.norm1" and l0["norm_ff_out"] == "l0.norm2" and l0["g"] == "l0.mix.g" and l0["gate"] == ["l0.mlp.gate"]
    assert list(l0["decay"]) == [np.float32(x) for x in cfg["layers"][0]["mixer"]["decay"]]
    assert l1["w_in"] == "l1.mix.in" and l1["conv_b"] == "l1.mix.conv.b" and l1["a_log"] == "l1.mix.A_log" and l1["d_skip"] == "l1.mix.D"
    assert l1["up"] == ["l1.mlp.e0.up", "l1.mlp.e1.up", "l1.mlp.e2.up"] and l1["shared_sg"] == "l1.mlp.shared.sg" and l1["router"] == "l1.mlp.router"
    assert l2["q_conv"] == "l2.mix.q.conv" and l2["k_norm"] == "l2.mix.k.norm" and l2["rel"] == "l2.mix.rel" and "norm_ff_out" not in l2
    t = arch_synth.dozotar_weights(cfg, seed=1)
    for ln in n["layers"]:
        for v in ln.values():
            for name in (v if isinstance(v, list) else [v]):
                assert not isinstance(name, str) or name in t, name
    assert t["l0.norm1"].shape == () and t["final.norm"].shape == ()


def test_unknown_parts_are_refused():
    cfg = arch_synth.dozotar_config(16, 8, [RE(2, 4, 4)])
    cfg["layers"][0]["type"] = "convolution"
    with pytest.raises(capi.PsCudaError):
        arch.ARCHITECTURES["Dozotar"][0](cfg, {})
    cfg = arch_synth.dozotar_config(16, 8, [RE(2, 4, 4, ff=8)])
    cfg["layers"][0]["mlp"]["kind"] = "sparse"
    with pytest.raises(capi.PsCudaError):
        arch.ARCHITECTURES["Dozotar"][0](cfg, {})
    cfg = arch_synth.dozotar_config(16, 8, [RE(2, 4, 4, decay=[0.5])])
    with pytest.raises(capi.PsCudaError):
        arch.ARCHITECTURES["Dozotar"][0](cfg, {})


# ------------------------------------------------------------------------------------------------- the oracle itself
def test_short_conv_by_hand():
    u = np.array([[1.0], [2.0], [4.0], [8.0]])
    w = np.array([[100.0, 10.0, 1.0]])                                  # oldest tap first, the last one meets the current token
    np.testing.assert_allclose(R.short_conv(u, w)[:, 0], [1.0, 12.0, 124.0, 248.0])
    np.testing.assert_allclose(R.short_conv(u, w, np.array([0.5]))[:, 0], [1.5, 12.5, 124.5, 248.5])


def test_bucket_map_by_hand():
    assert [R.bucket(d, 8, 16.0) for d in (0, 1, 3, 4, 5, 7, 8, 15, 16, 1000)] == [0, 1, 3, 4, 4, 5, 6, 7, 7, 7]
    assert all(R.bucket(d, 24, 100.0) <= R.bucket(d + 1, 24, 100.0) for d in range(600))


def test_chunks_are_counted_from_position_zero():
    ok = R.chunk_visible(7, 3)
    assert [int(r.sum()) for r in ok] == [1, 2, 3, 1, 2, 3, 1]
    assert ok[5, 3] and not ok[5, 2] and not ok[3, 2]
    assert R.chunk_visible(4, None).sum() == 10


def test_retention_recurrence_equals_the_sum_over_the_past():
    rng = np.random.default_rng(0)
    n, W = 9, 12
    m = RE(2, 4, 3, decay=[0.5, 0.9], rot_dims=2, rot_base=50.0)["mixer"]
    w = {k: rng.standard_normal(s) for k, s in (("q", (8, W)), ("k", (8, W)), ("v", (6, W)), ("g", (6, W)), ("o", (W, 6)))}
    x = rng.standard_normal((n, W))
    got = R.retention(x, w, m, 1e-6)
    pos = np.arange(n)
    q = R.rotate_half((x @ w["q"].T).reshape(n, 2, 4), pos, m["rot"])
    k = R.rotate_half((x @ w["k"].T).reshape(n, 2, 4), pos, m["rot"]) / 2.0
    v = (x @ w["v"].T).reshape(n, 2, 3)
    o = np.zeros((n, 2, 3))
    for h in range(2):
        for i in range(n):
            for j in range(i + 1):
                o[i, h] += m["decay"][h] ** (i - j) * (q[i, h] @ k[j, h]) * v[j, h]
    want = (R.unit_rms(o, 1e-6).reshape(n, 6) * R.silu(x @ w["g"].T)) @ w["o"].T
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-12)
    # a rotation leaves lengths alone and turns position 0 by nothing
    z = rng.standard_normal((3, 2, 4))
    np.testing.assert_allclose(np.linalg.norm(R.rotate_half(z, [5, 6, 7], m["rot"]), axis=-1), np.linalg.norm(z, axis=-1))
    np.testing.assert_allclose(R.rotate_half(z, [0, 0, 0], m["rot"]), z)


def test_state_space_recurrence_by_hand():
    """one head, one state, one channel, one tap: S_t = exp(-a dt) S + dt B x, y = S C + D x"""
    m = MA(1, 1, 1, conv=1)["mixer"]
    w = {"in": np.array([[0.3], [1.0], [0.5], [2.0], [0.7]]), "conv": np.ones((3, 1)), "conv.b": np.zeros(3), "dt_bias": np.array([0.1]),
         "A_log": np.array([math.log(2.0)]), "D": np.array([0.25]), "norm": np.array([1.0]), "o": np.array([[1.0]])}
    xs = np.array([[1.0], [-2.0], [0.5]])
    S, want = 0.0, []
    for x in xs[:, 0]:
        z, u, B, Cc, dt = 0.3 * x, R.silu(x), R.silu(0.5 * x), R.silu(2.0 * x), math.log1p(math.exp(0.7 * x + 0.1))
        S = math.exp(-2.0 * dt) * S + dt * B * u
        y = (S * Cc + 0.25 * u) * R.silu(z)
        want.append(y / math.sqrt(y * y + 1e-6))
    np.testing.assert_allclose(R.mamba2(xs, w, m, 1e-6)[:, 0], want, rtol=1e-12)


def test_expert_choice_by_hand():
    s = np.array([0.05, 0.30, 0.04, 0.06, 0.20, 0.10, 0.12, 0.13])
    assert R.choose_experts(s, 3, 1, 1) == [1, 4, 7]
    # four pairs worth 0.30, 0.06, 0.20, 0.13: with two kept only experts 0, 1, 4, 5 can be chosen
    assert R.choose_experts(s, 3, 4, 2) == [1, 4, 5]
    assert R.choose_experts(s, 2, 4, 3) == [1, 4]
    assert R.choose_experts(s, 4, 4, 3) == [1, 4, 7, 6]


def test_expert_weights_sum_to_one_and_the_shared_gate_scales():
    rng = np.random.default_rng(1)
    W, E, ff = 10, 6, 5
    w = {"router": rng.standard_normal((E, W))}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rng.standard_normal((ff, W)), rng.standard_normal((ff, W)), rng.standard_normal((W, ff))
    mlp = {"expert": {"ff": ff}, "router": {"experts": E, "top": E, "groups": {"count": 1, "keep": 1}}}
    h = rng.standard_normal((4, W))
    got = R.expert_ff(h, w, mlp)
    z = h @ w["router"].T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)                    # every expert chosen: the weights are the soft-max itself
    want = sum(s[:, e:e + 1] * R.gated_unit(h, {f: w[f"e{e}.{f}"] for f in ("gate", "up", "down")}, R.silu) for e in range(E))
    np.testing.assert_allclose(got, want, rtol=1e-9)
    w.update({"shared.gate": rng.standard_normal((3, W)), "shared.up": rng.standard_normal((3, W)), "shared.down": rng.standard_normal((W, 3)), "shared.sg": np.zeros((1, W))})
    mlp["shared"] = {"ff": 3}
    extra = R.expert_ff(h, w, mlp) - got
    np.testing.assert_allclose(extra, 0.5 * R.gated_unit(h, {f: w[f"shared.{f}"] for f in ("gate", "up", "down")}, R.silu), rtol=1e-9)


def test_gelu_and_softplus():
    z = np.linspace(-6, 6, 25)
    np.testing.assert_allclose(R.gelu_tanh(z), z / (1.0 + np.exp(-2.0 * math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3))), atol=1e-12)
    np.testing.assert_allclose(R.softplus(np.array([-50.0, 0.0, 50.0])), [math.exp(-50.0), math.log(2.0), 50.0], rtol=1e-12)


def test_forward_uses_single_number_norms_on_the_outputs_only():
    cfg = arch_synth.dozotar_config(12, 20, [RE(1, 4, 4, ff=8)])
    t = arch_synth.dozotar_weights(cfg, seed=2)
    toks = [3, 7, 7, 1, 19]
    taps = []
    R.forward(cfg, t, toks, taps=taps)
    x0 = np.asarray(t["embed"], np.float64)[toks]
    eps = cfg["norm"]["eps"]
    a = R.retention(x0, R.sub(t, "l0.mix."), cfg["layers"][0]["mixer"], eps)
    x1 = x0 + a / np.sqrt((a * a).mean(-1, keepdims=True) + eps) * float(t["l0.norm1"])
    f = R.gated_unit(x1, R.sub(t, "l0.mlp."), R.gelu_tanh)
    x2 = x1 + f / np.sqrt((f * f).mean(-1, keepdims=True) + eps) * float(t["l0.norm2"])
    np.testing.assert_allclose(taps[0], x2, rtol=1e-10)
