"""CPU-only checks around the Pidenex design: the registry's reading of a configuration (every size and constant comes from the
file, a looped group of layers becomes runs that share weights), the tensor names, and the oracle's own invariants (it is what
the GPU tests compare with, so it is checked against hand-computed cases and second formulations here)."""
import math

import numpy as np
import pytest

from powerserve_b200 import arch, arch_synth, capi
from tests import _pidenex_ref as R

AT, PA, LA = arch_synth.pidenex_attention_layer, arch_synth.pidenex_parallel_layer, arch_synth.pidenex_latent_layer


def test_registry_reads_every_size_from_the_configuration():
    layers = [LA(5, 12, 6, 9, 33, 21, window=77, scale=0.19, rope_base=1234.0, ff=44), AT(6, 3, 10, window=31, pool=7, scale=0.21),
              PA(8, 2, 14, window=19, gru_width=55, left_scale=0.3, right_scale=1.9, scale=0.11, ff=12)]
    cfg = arch_synth.pidenex_config(60, 99, layers, loop=(1, 3, 2), eps=3e-5, embed_scale=2.5)
    descs, top = arch.ARCHITECTURES["Pidenex"][0](cfg, {})
    assert top == {"dim": 60, "vocab_size": 99, "norm_eps": 3e-5, "embed_scale": 2.5, "norm_unit_offset": 0, "norm_kind": capi.NORM_LAYER, "n_pass_steps": 2}
    assert len(descs) == 5                                           # latent, then (attention, parallel) twice
    d = descs[0]
    assert (d.mixer_kind, d.n_heads, d.n_kv_heads, d.qk_dim, d.rot_dim, d.v_dim, d.q_rank, d.kv_rank, d.window) == (capi.MIXER_LATENT, 5, 1, 12, 6, 9, 33, 21, 77)
    assert (d.rope_dims, d.rope_base, d.rope_interleaved, d.rope_factor) == (6, 1234.0, 1, 0.0) and abs(d.score_scale - 0.19) < 1e-7
    assert (d.block_kind, d.post_norm, d.raw_input, d.sink) == (capi.BLOCK_SEQUENTIAL, 1, 0, capi.SINK_NONE)
    assert (d.mlp_kind, d.expert_ff, d.mlp_ungated, d.act_kind) == (capi.MLP_DENSE, 44, 1, capi.ACT_XIELU)
    assert (d.share_weights, d.pass_embed, d.pass_step) == (0, 0, 0)
    d = descs[1]
    assert (d.mixer_kind, d.n_heads, d.n_kv_heads, d.qk_dim, d.v_dim, d.window, d.pool, d.v_is_k) == (capi.MIXER_ATTENTION, 6, 3, 10, 10, 31, 7, 1)
    assert (d.qk_norm, d.lin_bias, d.out_gate, d.side_kind, d.mlp_kind) == (capi.QKNORM_NONE, 0, 0, 0, capi.MLP_NONE) and abs(d.score_scale - 0.21) < 1e-7
    assert (d.share_weights, d.pass_embed, d.pass_step) == (0, 0, 1)  # opens pass 0: the step row, not the embedding
    d = descs[2]
    assert (d.n_heads, d.n_kv_heads, d.qk_dim, d.window, d.pool, d.v_is_k, d.qk_norm, d.lin_bias, d.out_gate) == (8, 2, 14, 19, 0, 1, capi.QKNORM_WHOLE, 1, 1)
    assert (d.side_kind, d.side_width) == (capi.MIXER_MINGRU, 55) and abs(d.mix_scale - 0.3) < 1e-7 and abs(d.side_scale - 1.9) < 1e-7
    assert (d.share_weights, d.pass_embed, d.pass_step, d.expert_ff) == (0, 0, 0, 12)
    assert (descs[3].share_weights, descs[3].pass_embed, descs[3].pass_step, descs[3].pool) == (2, 1, 2, 7)   # pass 1 of run 1's weights
    assert (descs[4].share_weights, descs[4].pass_embed, descs[4].pass_step, descs[4].side_width) == (3, 0, 0, 55)


@pytest.mark.parametrize("loop,want", [((0, 2, 3), [0, 1, 0, 1, 0, 1, 2]), ((1, 3, 2), [0, 1, 2, 1, 2]), ((0, 1, 1), [0, 1, 2]), ((2, 3, 4), [0, 1, 2, 2, 2, 2]),
                                       (None, [0, 1, 2]), ((1, 1, 5), [0, 1, 2])])
def test_runs_follow_the_loop(loop, want):
    cfg = arch_synth.pidenex_config(16, 8, [AT(1, 1, 4, window=3), AT(1, 1, 4, window=3), AT(1, 1, 4, window=3)], loop=loop)
    runs = arch._pidenex_runs(cfg)
    assert [i for i, _ in runs] == want == [i for i, _ in R.layer_runs(cfg)]
    assert runs == R.layer_runs(cfg)
    if loop and loop[1] > loop[0]:
        assert [t for i, t in runs if t is not None] == list(range(loop[2]))
        assert all(i == loop[0] for i, t in runs if t is not None)
    descs, top = arch.ARCHITECTURES["Pidenex"][0](cfg, {})
    firsts = {}
    for r, ((i, t), d) in enumerate(zip(runs, descs)):
        assert d.share_weights == (firsts[i] + 1 if i in firsts else 0)
        firsts.setdefault(i, r)
        assert (d.pass_step, d.pass_embed) == ((t + 1, int(t > 0)) if t is not None else (0, 0))


def test_bad_loops_and_types_are_refused():
    for loop in ((2, 1, 2), (0, 4, 2), (0, 1, 0), (-1, 1, 1)):
        with pytest.raises(capi.PsCudaError):
            arch._pidenex_runs(arch_synth.pidenex_config(16, 8, [AT(1, 1, 4, window=3)] * 3, loop=loop))
    cfg = arch_synth.pidenex_config(16, 8, [AT(1, 1, 4, window=3)])
    cfg["layers"][0]["type"] = "retention"
    with pytest.raises(capi.PsCudaError):
        arch.ARCHITECTURES["Pidenex"][0](cfg, {})
    cfg = arch_synth.pidenex_config(16, 8, [AT(1, 1, 4, window=3, ff=8)])
    cfg["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(capi.PsCudaError):
        arch.ARCHITECTURES["Pidenex"][0](cfg, {})


def test_tensor_names_follow_the_layer_types():
    cfg = arch_synth.pidenex_config(16, 8, [AT(2, 1, 4, window=3, pool=2, ff=8), PA(4, 2, 4, window=3, gru_width=6), LA(2, 4, 2, 4, 6, 5, ff=8)], loop=(0, 2, 2))
    n = arch.ARCHITECTURES["Pidenex"][1](cfg)
    assert (n["embed"], n["final_norm"], n["head"], n["pass_steps"]) == ("embed", "final.norm", "head", "loop.step")
    l0, l1, r0, r1, l2 = n["layers"]
    assert r0 == {} and r1 == {}                                     # repeated runs name no tensors of their own
    assert l0["norm"] == "l0.norm1" and l0["norm_mix_out"] == "l0.norm1b" and l0["norm_ff"] == "l0.norm2" and l0["norm_ff_out"] == "l0.norm2b"
    assert l0["q"] == "l0.mix.q" and l0["k"] == "l0.mix.k" and "v" not in l0 and l0["up"] == ["l0.mlp.up"] and "gate" not in l0 and l0["act"] == "l0.mlp.act"
    assert l1["q"] == "l1.mix.left.q" and l1["k_norm"] == "l1.mix.left.k.norm" and l1["g"] == "l1.mix.left.g" and l1["side_x_bias"] == "l1.mix.right.x.b"
    assert l1["side_o"] == "l1.mix.right.o" and "norm_ff" not in l1
    np.testing.assert_allclose(l1["lin"], [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8])
    assert l2["dq_norm"] == "l2.mix.dq.norm" and l2["uv"] == "l2.mix.uv" and l2["dkv"] == "l2.mix.dkv"
    t = arch_synth.pidenex_weights(cfg, seed=1)
    assert t["loop.step"].shape == (2, 16) and t["l1.mix.right.z.b"].shape == (6,) and t["l0.mlp.act"].shape == (2,)
    for ln in n["layers"]:
        for v in ln.values():
            for name in (v if isinstance(v, list) else [v]):
                assert not isinstance(name, str) or name in t, name
    plain = arch.ARCHITECTURES["Pidenex"][1](arch_synth.pidenex_config(16, 8, [AT(2, 1, 4, window=3)]))
    assert "pass_steps" not in plain


# ------------------------------------------------------------------------------------------------- the oracle by hand
def test_layer_norm_by_hand():
    x = np.array([[1.0, 2.0, 3.0, 6.0]])
    w = np.array([1.0, 2.0, 0.5, -1.0])
    mu, var = 3.0, (4 + 1 + 0 + 9) / 4
    np.testing.assert_allclose(R.layer_norm(x, w, 0.25), (x - mu) / math.sqrt(var + 0.25) * w)
    np.testing.assert_allclose(R.layer_norm(x + 100.0, w, 0.25), R.layer_norm(x, w, 0.25))      # the mean is taken off
    assert abs(R.layer_norm(x, np.ones(4), 0.0).mean()) < 1e-12
    np.testing.assert_allclose(R.rms_norm(x, w, 0.5), x / math.sqrt(50 / 4 + 0.5) * w)


def test_activation_by_hand():
    p, q = 0.3, -0.7
    sp = lambda v: math.log(1 + math.exp(v))
    for z in (-5.0, -0.5, 0.0, 1e-9, 0.5, 4.0):
        want = sp(p) * z * z + z / 2 if z > 0 else (0.5 + sp(q)) * (math.exp(z) - 1 - z) + z / 2
        assert abs(float(R.xielu(np.array(z), p, q)) - want) < 1e-12
    # value and slope meet at zero
    e = 1e-6
    assert abs(float(R.xielu(np.array(e), p, q)) - float(R.xielu(np.array(-e), p, q)) - e) < 1e-10
    assert R.softplus(np.array(800.0)) == 800.0 and abs(R.softplus(np.array(-800.0))) < 1e-300


def test_rotation_in_neighbouring_pairs():
    v = np.arange(1.0, 9.0)[None, :]                                 # one position, 8 entries, 6 of them rotate
    out = R.rotate_pairs(v, [3], 6, 100.0)
    for i in range(3):
        a = 3 * 100.0 ** (-2.0 * i / 6)
        u, w = v[0, 2 * i], v[0, 2 * i + 1]
        np.testing.assert_allclose(out[0, 2 * i:2 * i + 2], [u * math.cos(a) - w * math.sin(a), w * math.cos(a) + u * math.sin(a)])
    np.testing.assert_array_equal(out[0, 6:], v[0, 6:])
    np.testing.assert_allclose(R.rotate_pairs(v, [0], 6, 100.0), v)
    # a rotated query against a rotated key depends on the distance only
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((1, 8)), rng.standard_normal((1, 8))
    s1 = R.rotate_pairs(a, [17], 8, 50.0) @ R.rotate_pairs(b, [5], 8, 50.0).T
    s2 = R.rotate_pairs(a, [112], 8, 50.0) @ R.rotate_pairs(b, [100], 8, 50.0).T
    np.testing.assert_allclose(s1, s2, atol=1e-12)


def test_window_and_blocks_by_hand():
    m = R.window_mask(6, 3)
    assert [list(np.nonzero(r)[0]) for r in m] == [[0], [0, 1], [0, 1, 2], [1, 2, 3], [2, 3, 4], [3, 4, 5]]
    # window 3, blocks of 2: block b (positions 2b, 2b + 1) is seen when 2b + 1 <= i - 3
    pm = R.pooled_mask(9, 3, 2)
    assert [list(np.nonzero(r)[0]) for r in pm] == [[], [], [], [], [0], [0], [0, 1], [0, 1], [0, 1, 2]]
    # position 3 has lost token 0 from its window and does not see block 0 yet: token 0 is not seen at all
    assert not m[3, 0] and not pm[3, 0]
    x = np.arange(14.0).reshape(1, 7, 2)
    np.testing.assert_allclose(R.block_means(x, 3), [[[2.0, 3.0], [8.0, 9.0]]])


def test_pooled_attention_against_an_explicit_loop():
    rng = np.random.default_rng(1)
    T, W, H, G, d, size, pool = 23, 10, 4, 2, 3, 5, 4
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": 0.7, "mask": {"size": size, "pool": pool}}
    Wt = {"q": rng.standard_normal((H * d, W)), "k": rng.standard_normal((G * d, W)), "o": rng.standard_normal((W, H * d))}
    h = rng.standard_normal((T, W))
    got = R.pooled_attention(h, m, Wt, "")
    q, k = h @ Wt["q"].T, h @ Wt["k"].T
    want = np.zeros((T, H * d))
    for i in range(T):
        for hh in range(H):
            g = hh // (H // G)
            keys = [k[j, g * d:(g + 1) * d] for j in range(max(0, i - size + 1), i + 1)]
            b = 0
            while b * pool + pool - 1 <= i - size:
                keys.append(np.mean([k[j, g * d:(g + 1) * d] for j in range(b * pool, (b + 1) * pool)], 0))
                b += 1
            keys = np.array(keys)
            s = keys @ q[i, hh * d:(hh + 1) * d] * 0.7
            p = np.exp(s - s.max())
            want[i, hh * d:(hh + 1) * d] = (p / p.sum()) @ keys
    np.testing.assert_allclose(got, want @ Wt["o"].T, atol=1e-10)


def test_min_gru_by_hand():
    W = {"z": np.array([[1.0]]), "z.b": np.array([0.0]), "x": np.array([[2.0]]), "x.b": np.array([-1.0]), "g": np.array([[1.0]]), "o": np.array([[1.0]])}
    h = np.array([[1.0], [0.0], [-2.0]])
    sg = lambda v: 1 / (1 + math.exp(-v))
    S, want = 0.0, []
    for x in (1.0, 0.0, -2.0):
        z, u = sg(x), 2 * x - 1
        c = u + 0.5 if u >= 0 else sg(u)
        S = (1 - z) * S + z * c
        want.append(S * x * sg(x))
    np.testing.assert_allclose(R.min_gru(h, W, "")[:, 0], want)
    assert R.slopes(4).tolist() == [0.25, 0.0625, 0.015625, 0.00390625]


def test_forward_adds_the_embedding_and_the_steps_once_a_pass():
    cfg = arch_synth.pidenex_config(16, 12, [AT(2, 1, 4, window=3, ff=8), LA(2, 4, 2, 4, 6, 5)], loop=(0, 1, 3), embed_scale=2.0)
    t = {k: v.astype(np.float64) for k, v in arch_synth.pidenex_weights(cfg, seed=2).items()}
    toks = [3, 1, 4, 1, 5]
    taps = []
    R.forward(cfg, t, toks, taps=taps)
    assert len(taps) == 4
    x0 = t["embed"][toks] * 2.0
    x = R.layer(x0 + t["loop.step"][0], cfg["layers"][0], t, 0, cfg["norm"]["eps"])
    np.testing.assert_allclose(taps[0], x)
    x = R.layer(x + x0 + t["loop.step"][1], cfg["layers"][0], t, 0, cfg["norm"]["eps"])
    np.testing.assert_allclose(taps[1], x)
    # a later position never changes an earlier one
    a = R.forward(cfg, t, toks)
    b = R.forward(cfg, t, toks[:3])
    np.testing.assert_allclose(a[:3], b, atol=1e-10)
