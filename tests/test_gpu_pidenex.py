"""GPU tests of the Pidenex design on the layer-list path: the CUDA backend (forward / sessions / decode_greedy behind
arch.load_model) against the plain numpy oracle in tests/_pidenex_ref.py, on small random models made here.

float32 mode is compared tightly with the oracle; bfloat16 mode loosely with the oracle."""
import json
import os
import subprocess

import numpy as np
import pytest

from powerserve_b200 import arch, arch_synth, capi
from tests import _pidenex_ref as R

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
AT, PA, LA = arch_synth.pidenex_attention_layer, arch_synth.pidenex_parallel_layer, arch_synth.pidenex_latent_layer
# every mixer, a looped pair in the middle, unequal head counts and windows
MIXED = [LA(3, 8, 6, 10, 20, 14, window=21, ff=40), AT(4, 2, 10, window=19, pool=4, ff=56), PA(6, 3, 8, window=13, gru_width=50, ff=24),
         AT(2, 1, 12, window=40, pool=7)]
MIXED_LOOP = (1, 3, 3)


def make(tmp_path, layers, width=48, vocab=96, seed=0, eps=1e-5, edit=None, name="m", loop=None, embed_scale=1.7):
    cfg = arch_synth.pidenex_config(width, vocab, layers, loop=loop, eps=eps, embed_scale=embed_scale)
    t = arch_synth.pidenex_weights(cfg, seed=seed)
    if edit:
        edit(t)
        t = {k: R.bf16_round(v) for k, v in t.items()}
    d = str(tmp_path / name)
    arch_synth.write_model_dir(d, cfg, t)
    return d, cfg, t


def tokens(vocab, n, seed=0):
    return [int(v) for v in np.random.default_rng(seed).integers(0, vocab, n)]


def run(model, toks, cuts=None):
    """logits of every position, the sequence fed in portions of the given sizes (cycled); None = one portion per batch cap"""
    model.reset()
    cap, out, lo, k = model.desc.max_batch, [], 0, 0
    while lo < len(toks):
        s = min(cap if cuts is None else min(cuts[k % len(cuts)], cap), len(toks) - lo)
        out.append(model.forward(toks[lo:lo + s]))
        lo, k = lo + s, k + 1
    return np.concatenate(out)


def rel_err(got, ref):
    """per position: rms of the difference over rms of the reference"""
    return np.sqrt(((got - ref) ** 2).mean(-1)) / np.maximum(np.sqrt((ref ** 2).mean(-1)), 1e-6)


TOL = {"float32": 4e-5, "bfloat16": 6e-2}


def check(got, ref, dtype, what=""):
    e = rel_err(got, ref)
    assert e.max() < TOL[dtype], f"{what}: worst relative error {e.max():.3g} at position {int(e.argmax())} ({dtype})"
    if dtype == "bfloat16":
        assert np.median(e) < 2e-2, f"{what}: median relative error {np.median(e):.3g}"


def both_paths(d, toks, ref, what, n_ctx, cap=64, cuts=([7, 2, 33, 1],), decode_from=None):
    """float32: portions of the batch cap, ragged portions, and the tail decoded token by token, all against the oracle"""
    m = arch.load_model(d, dtype="float32", max_batch=cap, n_ctx=n_ctx)
    check(run(m, toks), ref, "float32", what + ", portions of the batch cap")
    for c in cuts:
        check(run(m, toks, list(c)), ref, "float32", what + f", portions {list(c)}")
    k = decode_from if decode_from is not None else len(toks) // 2
    m.reset()
    for lo in range(0, k, cap):
        m.forward(toks[lo:min(k, lo + cap)], lm_head=False)
    dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(k, len(toks))])
    check(dec, ref[k:], "float32", what + ", decoded alone")
    m.close()


def alone(tmp_path, layer, what, seed, n=45, width=48, n_ctx=64, **kw):
    d, cfg, t = make(tmp_path, [layer], seed=seed, width=width, **kw)
    toks = tokens(96, n, seed)
    taps = []
    ref = R.forward(cfg, t, toks, taps=taps)
    m = arch.load_model(d, dtype="float32", max_batch=64, n_ctx=n_ctx)
    m.be.set_option("arch_taps", 1)
    check(run(m, toks), ref, "float32", what)
    check(m.layer_tap(0, len(toks)), taps[0], "float32", "residual after the layer")
    m.close()
    both_paths(d, toks, ref, what, n_ctx, cuts=([7, 2, 33, 1], [2]))


# ------------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("heads,kv_heads,dim,window,pool", [(4, 2, 10, 9, 4), (3, 3, 8, 16, 5), (4, 1, 12, 5, 1), (2, 2, 6, 1, 3), (2, 1, 8, 12, 0), (5, 5, 7, 100, 6)])
def test_pooled_attention_layer_alone(tmp_path, heads, kv_heads, dim, window, pool):
    alone(tmp_path, AT(heads, kv_heads, dim, window=window, pool=pool), "attention-only layer", 1)


@pytest.mark.parametrize("heads,kv_heads,dim,window,width", [(4, 2, 12, 11, 40), (2, 1, 8, 64, 7), (3, 3, 6, 3, 100), (8, 2, 4, 17, 33)])
def test_parallel_layer_alone(tmp_path, heads, kv_heads, dim, window, width):
    alone(tmp_path, PA(heads, kv_heads, dim, window=window, gru_width=width, left_scale=0.6, right_scale=1.3), "gated attention beside a minGRU", 2)


@pytest.mark.parametrize("geometry,window", [((3, 8, 6, 10, 20, 14), 9), ((2, 4, 8, 4, 9, 12), 0), ((1, 6, 2, 5, 7, 5), 4), ((4, 16, 16, 12, 24, 32), 33)])
def test_latent_layer_alone(tmp_path, geometry, window):
    alone(tmp_path, LA(*geometry, window=window, rope_base=500.0), "latent attention, rotation in neighbouring pairs", 3)


@pytest.mark.parametrize("p,q", [(0.5, -0.25), (-3.0, 2.0), (4.0, -6.0)])
def test_feed_forward_alone(tmp_path, p, q):
    """large up rows: both branches of the activation over a wide range, for several pairs of its numbers"""
    def edit(t):
        t["l0.mlp.up"] = t["l0.mlp.up"] * 3.0
        t["l0.mlp.act"] = np.array([p, q], np.float32)
    alone(tmp_path, AT(1, 1, 8, window=4, ff=72), "feed-forward without a gate", 4, edit=edit)


def test_each_half_of_the_parallel_mixer_shows(tmp_path):
    """the oracle itself: without the gate, the distance penalty, the whole-projection norms or the recurrence the logits move,
    so the comparisons above see every one of them"""
    d, cfg, t = make(tmp_path, [PA(4, 2, 8, window=30, gru_width=24)], seed=5)
    toks = tokens(96, 50, 5)
    ref = R.forward(cfg, t, toks)
    for name, new in (("l0.mix.left.g", 0.0), ("l0.mix.left.q.norm", 1.0), ("l0.mix.right.z.b", 3.0), ("l0.mix.right.o", 0.0)):
        t2 = dict(t)
        t2[name] = np.full_like(t[name], new)
        assert rel_err(R.forward(cfg, t2, toks), ref).max() > 1e-2, name
    slopes = R.slopes
    try:
        R.slopes = lambda H: slopes(H)[::-1]                        # the heads' penalties the other way round
        assert rel_err(R.forward(cfg, t, toks), ref).max() > 1e-2
    finally:
        R.slopes = slopes


# ------------------------------------------------------------------------------------------------- windows, blocks, far keys
def peaky(t, gain=4.0):
    """larger queries and keys: a few keys carry the soft-max, so one key or block too many or too few moves the output by O(1)"""
    for k in list(t):
        if k.endswith("mix.q") or k.endswith("mix.k") or k.endswith("left.q") or k.endswith("left.k"):
            t[k] = t[k] * gain


@pytest.mark.parametrize("window,pool", [(15, 3), (16, 16), (17, 1), (63, 17), (64, 5), (65, 16), (33, 64), (2, 2)])
def test_window_and_block_edges(tmp_path, window, pool):
    """windows and blocks around the 16-key blocks and 64-key tiles of the kernels, in prompts of several cuts and decoded alone; the
    oracle with a window or a block size that is one off differs by far more than the tolerance (blocks of one token make every
    token visible whatever the window: there only the block size shows)"""
    d, cfg, t = make(tmp_path, [AT(3, 1, 8, window=window, pool=pool)], seed=6, width=32)
    toks = tokens(96, 200, 6)
    ref = R.forward(cfg, t, toks)
    for dw, dp, least in ((1, 0, 5e-2), (-1, 0, 5e-2), (0, 1, 2e-4)):
        if window + dw < 1 or (pool == 1 and dp == 0):
            continue
        c2 = json.loads(json.dumps(cfg))
        c2["layers"][0]["mixer"]["mask"] = {"size": window + dw, "pool": pool + dp}
        assert rel_err(R.forward(c2, t, toks), ref).max() > least, (dw, dp)
    both_paths(d, toks, ref, f"window {window}, blocks of {pool}", 208, cap=80, cuts=([64, 16, 1], [5, 2, 70]), decode_from=90)


@pytest.mark.parametrize("window", [1, 15, 16, 17, 64, 65])
def test_window_edges_of_the_biased_and_latent_layers(tmp_path, window):
    layers = [PA(2, 2, 8, window=window, gru_width=16), LA(2, 8, 4, 6, 12, 10, window=window)]
    d, cfg, t = make(tmp_path, layers, seed=7, edit=peaky, width=32)
    toks = tokens(96, 150, 7)
    ref = R.forward(cfg, t, toks)
    c2 = json.loads(json.dumps(cfg))
    c2["layers"][0]["mixer"]["left"]["mask"]["size"] = window + 1
    assert rel_err(R.forward(c2, t, toks), ref).max() > 1e-3
    both_paths(d, toks, ref, f"window {window}", 160, cap=70, cuts=([64, 16, 1], [3, 2, 61]), decode_from=60)


def test_a_far_token_reaches_through_its_block(tmp_path):
    """a token that occurs once, 300 positions back, and is seen only through the mean of its block: the queries at the end carry the
    same embedding and q = k / 2, so that block's score stands out among hundreds"""
    def edit(t):
        t["l0.mix.q"] = 0.5 * t["l0.mix.k"]
        t["embed"][39] = t["embed"][0]
    d, cfg, t = make(tmp_path, [AT(1, 1, 8, window=20, pool=2)], seed=8, width=32, vocab=40, edit=edit)
    toks = [1 + int(v) for v in np.random.default_rng(8).integers(0, 38, 340)]
    toks[27] = 0
    for p in (333, 336, 339):
        toks[p] = 39
    ref = R.forward(cfg, t, toks)
    other = list(toks)
    other[27] = 5
    assert rel_err(R.forward(cfg, t, other)[[333, 336, 339]], ref[[333, 336, 339]]).min() > 1e-3      # the far token matters at the end
    both_paths(d, toks, ref, "far token", 352, cap=128, cuts=([100, 3, 128],), decode_from=300)


# ------------------------------------------------------------------------------------------------- passes
@pytest.mark.parametrize("loop", [(0, 2, 3), (1, 3, 2), (0, 1, 1), (2, 3, 4), (0, 3, 2), None])
def test_looped_runs(tmp_path, loop):
    """every run's residual stream against the oracle's: shared weights, a cache and state per run, the pass additions"""
    layers = [AT(2, 2, 8, window=9, pool=3, ff=24), PA(2, 1, 8, window=7, gru_width=20), LA(2, 6, 4, 6, 10, 8, window=11, ff=16)]
    d, cfg, t = make(tmp_path, layers, seed=9, loop=loop, width=40)
    toks = tokens(96, 37, 9)
    taps = []
    ref = R.forward(cfg, t, toks, taps=taps)
    assert len(taps) == (3 if not loop else 3 + (loop[1] - loop[0]) * (loop[2] - 1))
    m = arch.load_model(d, dtype="float32", max_batch=64, n_ctx=48)
    m.be.set_option("arch_taps", 1)
    check(run(m, toks), ref, "float32", f"loop {loop}")
    for i, tap in enumerate(taps):
        check(m.layer_tap(i, len(toks)), tap, "float32", f"residual after run {i}")
    m.close()
    both_paths(d, toks, ref, f"loop {loop}", 48, cap=16, cuts=([5, 2, 16], [2]))


# ------------------------------------------------------------------------------------------------- schedules
def test_whole_prompt_portions_and_decoding_agree_in_both_precisions(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=10, loop=MIXED_LOOP)
    toks = tokens(130, 150, 10)
    ref = R.forward(cfg, t, toks)
    both_paths(d, toks, ref, "mixed model", 160, cap=64, cuts=([7, 2, 33, 1], [2], [64, 3]))
    m = arch.load_model(d, dtype="bfloat16", max_batch=64, n_ctx=160)
    whole = run(m, toks)
    check(whole, ref, "bfloat16", "whole prompt")
    for cuts in ([1], [2], [5, 40, 3]):
        got = run(m, toks, cuts)
        check(got, ref, "bfloat16", f"portions {cuts}")
        assert np.median(rel_err(got, whole)) < 2e-2
    m.close()


def test_single_token_kernels_match_the_batch_kernels(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=11, loop=MIXED_LOOP)
    toks = tokens(130, 100, 11)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=32, n_ctx=112)
        a = run(m, toks, [1])
        m.be.set_option("arch_simple", 1)
        b = run(m, toks, [1])
        assert np.median(rel_err(a, b)) < (1e-5 if dtype == "float32" else 2e-2) and rel_err(a, b).max() < (8e-5 if dtype == "float32" else 1e-1), dtype
        m.close()


def test_replayed_step_matches_the_plain_launches(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=12, loop=MIXED_LOOP)
    toks = tokens(130, 90, 12)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=40, n_ctx=96)
        g0 = m.be.counter("graph_replays")
        a = run(m, toks, [1])
        assert m.be.counter("graph_replays") - g0 == len(toks)
        m.reset()
        m.forward(toks[:40], lm_head=False)
        ids_a = list(m.decode_greedy(toks[40], 20))
        m.be.set_option("graph", 0)
        b = run(m, toks, [1])
        m.reset()
        m.forward(toks[:40], lm_head=False)
        ids_b = list(m.decode_greedy(toks[40], 20))
        np.testing.assert_array_equal(a, b)                         # the same kernels on the same data
        assert ids_a == ids_b
        m.be.set_option("graph", 1)
        m.be.set_option("arch_pdl", 0)
        np.testing.assert_array_equal(run(m, toks, [1]), a)
        m.close()


def test_tensor_core_gemm_matches_the_tile_kernels(tmp_path):
    """bfloat16 batches: the tcgen05 GEMM (projections, up rows with the activation in the epilogue, down) against the fp32-FMA tiles"""
    layers = [AT(6, 3, 24, window=50, pool=9, ff=200), PA(5, 5, 24, window=70, gru_width=150, ff=136), LA(4, 24, 16, 20, 72, 40, window=90, ff=72)]
    d, cfg, t = make(tmp_path, layers, width=136, vocab=300, seed=13, loop=(0, 2, 2))
    toks = tokens(300, 300, 13)
    m = arch.load_model(d, dtype="bfloat16", max_batch=160, n_ctx=304)
    n0 = m.be.counter("kernel_launches")
    a = run(m, toks)
    n1 = m.be.counter("kernel_launches")
    m.be.set_option("arch_tc", 0)
    b = run(m, toks)
    n2 = m.be.counter("kernel_launches")
    assert n1 - n0 > n2 - n1                                        # the tensor-core path adds its operand-tiling launches: it did run
    e = rel_err(a, b)
    assert np.median(e) < 1e-2 and e.max() < 4e-2, (np.median(e), e.max())
    check(a, R.forward(cfg, t, toks), "bfloat16", "tensor-core path against the oracle")
    m.close()


def test_sessions_interleaved_and_sets_reused(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=14, loop=MIXED_LOOP)
    reqs = [tokens(130, n, 20 + i) for i, n in enumerate((50, 9, 33, 64))]
    refs = [R.forward(cfg, t, r) for r in reqs]
    m = arch.load_model(d, dtype="float32", max_batch=16, n_ctx=64)
    sid = [m.session_create() for _ in range(3)]
    got = [[] for _ in reqs]
    at = [0, 0, 0, 0]
    sizes = [5, 2, 16, 1, 7]
    live, k = [0, 1, 2], 0
    while live:
        for r in list(live):
            s = min(sizes[k % len(sizes)], len(reqs[r]) - at[r])
            k += 1
            m.session_select(sid[r])
            assert m.position == at[r]
            got[r].append(m.forward(reqs[r][at[r]:at[r] + s]))
            at[r] += s
            if at[r] == len(reqs[r]):
                live.remove(r)
                if r == 1:              # the short request ends first: its set is freed and a new request takes a new one
                    m.session_select(0)
                    m.session_destroy(sid[1])
                    sid.append(m.session_create())
                    live.append(3)
    for r in range(4):
        check(np.concatenate(got[r]), refs[r], "float32", f"request {r} among others")
    # the same set used again from position 0: the recurrent state and the block means of the longer request must not leak
    m.session_select(sid[0])
    m.reset()
    check(run(m, reqs[2], [16]), refs[2], "float32", "set reused after reset")
    check(run(m, reqs[1], [1]), refs[1], "float32", "set reused once more, token by token")
    m.reset()
    m.forward(reqs[2][:16])
    with pytest.raises(capi.PsCudaError):                           # recurrent state cannot be cut back, only to the start
        m.be.kv_rollback(13)
    m.be.kv_rollback(16)
    assert m.position == 0
    check(m.forward(reqs[2][:16]), refs[2][:16], "float32", "from the start after a rollback to 0")
    m.close()


def test_long_decoding_past_every_window(tmp_path):
    layers = [AT(4, 1, 8, window=37, pool=5, ff=16), PA(2, 1, 8, window=50, gru_width=12), LA(2, 8, 4, 6, 12, 10, window=130), AT(2, 2, 8, window=16, pool=16)]
    d, cfg, t = make(tmp_path, layers, width=32, vocab=50, seed=15, loop=(0, 2, 2))
    toks = tokens(50, 400, 15)
    ref = R.forward(cfg, t, toks)
    for dtype in ("float32", "bfloat16"):
        m = arch.load_model(d, dtype=dtype, max_batch=8, n_ctx=400)
        m.reset()
        m.forward(toks[:6], lm_head=False)
        dec = np.concatenate([m.forward(toks[i:i + 1]) for i in range(6, 400)])
        check(dec, ref[6:], dtype, "394 tokens decoded alone")
        m.close()


@pytest.mark.parametrize("layers,width,vocab,loop", [
    ([AT(1, 1, 4, window=3, pool=2)], 8, 11, None),                                                 # the smallest of everything
    ([PA(1, 1, 4, window=2, gru_width=1)], 8, 11, (0, 1, 2)),
    ([LA(1, 4, 2, 4, 4, 4, window=2)], 8, 11, None),
    ([AT(8, 8, 8, window=1000, pool=3, ff=8)], 40, 64, None),                                       # no key sharing; a window nothing leaves
    ([AT(8, 1, 12, window=7, pool=70, ff=20)], 56, 77, (0, 1, 3)),                                  # one shared key head; blocks longer than the prompt part they cover
    ([PA(5, 5, 6, window=5, gru_width=37, ff=37), LA(3, 5, 6, 7, 11, 9, window=6, ff=13)], 50, 101, (1, 2, 2)),   # nothing a multiple of four
    ([LA(4, 32, 16, 24, 48, 64, ff=96), AT(16, 4, 32, window=48, pool=12, ff=96), PA(16, 16, 16, window=30, gru_width=256)], 128, 300, (0, 3, 2)),
    ([PA(2, 2, 8, window=9, gru_width=8), PA(4, 1, 8, window=4, gru_width=24, ff=16)], 32, 60, (0, 2, 2)),
])
def test_other_sizes(tmp_path, layers, width, vocab, loop):
    d, cfg, t = make(tmp_path, layers, width=width, vocab=vocab, seed=16, eps=3e-6, loop=loop, embed_scale=0.5)
    toks = tokens(vocab, 75, 16)
    ref = R.forward(cfg, t, toks)
    m = arch.load_model(d, dtype="float32", max_batch=32, n_ctx=80)
    check(run(m, toks), ref, "float32", "portions of 32")
    check(run(m, toks, [2, 31, 1]), ref, "float32", "ragged portions")
    check(run(m, toks[:40], [1]), ref[:40], "float32", "token by token")
    m.close()
    m = arch.load_model(d, dtype="bfloat16", max_batch=80, n_ctx=80)
    check(run(m, toks), ref, "bfloat16", "whole prompt")
    m.close()


# ------------------------------------------------------------------------------------------------- entry points
def test_greedy_generation_through_the_entry_points(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=17, loop=MIXED_LOOP)
    prompt = tokens(130, 21, 17)
    m = arch.load_model(d, dtype="float32", max_batch=8, n_ctx=64)
    ids, lg = m.generate(prompt, 12, batch_size=8)                  # prefill in portions + one forward per token
    m.reset()
    m.prefill(prompt, 8)
    ids2 = [int(v) for v in m.decode_greedy(prompt[-1], 12)]        # the device-side greedy loop
    assert ids == ids2
    assert m.position == len(prompt) - 1 + 12
    seq = list(prompt)
    for step, tok in enumerate(ids):
        ref = R.forward(cfg, t, seq)[-1]
        assert rel_err(lg[step][None], ref[None]).max() < 4e-5
        assert ref[tok] >= ref.max() - 1e-4 * np.abs(ref).max()
        seq.append(tok)
    m.forward_lazy([seq[-1]])
    vals, idx = m.sample_topk(5)
    full = R.forward(cfg, t, seq)[-1]
    assert list(idx) == [int(v) for v in np.argsort(-full, kind="stable")[:5]]
    m.close()


def test_bad_configurations_are_refused(tmp_path):
    bad = AT(2, 2, 8, window=9, pool=3)
    bad["mixer"]["vdim"] = 6                                         # the values are the keys: they cannot have another size
    for i, (layers, loop) in enumerate([([bad], None), ([AT(3, 2, 8, window=4)], None), ([AT(2, 2, 8, window=4)], (1, 0, 2))]):
        with pytest.raises((capi.PsCudaError, KeyError)):
            d, cfg, t = make(tmp_path, layers, seed=18, name=f"bad{i}", loop=loop)
            arch.load_model(d, dtype="float32", max_batch=8, n_ctx=16)


def test_trace_runner_and_generation_command_lines(tmp_path):
    d, cfg, t = make(tmp_path, MIXED, width=72, vocab=130, seed=19, loop=MIXED_LOOP)
    a, b = tokens(130, 40, 30), tokens(130, 17, 31)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[32:], "want": [7, 3]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [16]}], "end": ["b"]}]
    out = tmp_path / "out"
    ra, rb = R.forward(cfg, t, a), R.forward(cfg, t, b)
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "40", "--max-batch", "16"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        check(np.fromfile(out / "0.f32", "<f4").reshape(2, 130), ra[[0, 29]], dtype, "step 0")
        assert not (out / "1.f32").exists()
        check(np.fromfile(out / "2.f32", "<f4").reshape(2, 130), ra[[39, 35]], dtype, "step 2 (order of `want`)")
        check(np.fromfile(out / "3.f32", "<f4").reshape(1, 130), rb[[16]], dtype, "step 3")
        for f in out.iterdir():
            f.unlink()
    prompt = tokens(130, 19, 19)
    exe = os.path.join(ROOT, "bin", "ps_generate")
    p = subprocess.run([exe, "--model", d, "--dtype", "float32", "--ids", " ".join(map(str, prompt)), "--n", "10", "--prefill-batch", "8"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    ids = json.loads(p.stdout.strip().splitlines()[-1])["ids"]
    m = arch.load_model(d, dtype="float32", max_batch=32, n_ctx=32)
    want, _ = m.generate(prompt, 10, batch_size=8)
    assert ids == want
    m.close()
