"""Pins oracle/attn_oracle.py against outputs of the reference's own CPU code
(tests/golden/ref_vectors.npz, made by tests/golden/make_golden.py) and against the algebraic
identities the reference's tests assert (ref/test_prefill.py)."""
import os

import numpy as np
import pytest

from oracle import attn_oracle as ao

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz"))


@pytest.mark.parametrize("rows", [1, 3, 64, 65, 130])
def test_gdn_small_heads_match_reference(rows):
    a = {n: G[f"gdn8_{rows}_{n}"] for n in ("q", "k", "v", "g", "beta", "init", "ys", "ss", "yc", "sc")}
    ys, ss = ao.gdn_serial(a["q"], a["k"], a["v"], a["g"], a["beta"], a["init"])
    yc, sc = ao.gdn_chunked(a["q"], a["k"], a["v"], a["g"], a["beta"], a["init"])
    np.testing.assert_allclose(ys, a["ys"], rtol=2e-13, atol=2e-14)
    np.testing.assert_allclose(ss, a["ss"], rtol=2e-13, atol=2e-14)
    np.testing.assert_allclose(yc, a["yc"], rtol=2e-12, atol=2e-13)
    np.testing.assert_allclose(sc, a["sc"], rtol=2e-12, atol=2e-13)
    # ref/test_prefill.py:18-19: chunk == serial
    np.testing.assert_allclose(yc, ys, rtol=2e-13, atol=2e-14)
    np.testing.assert_allclose(sc, ss, rtol=2e-13, atol=2e-14)


def test_gdn_full_head_matches_reference():
    a = {n: G[f"gdn128_{n}"] for n in ("q", "k", "v", "g", "beta", "init", "ys", "ss", "yc", "sc")}
    ys, ss = ao.gdn_serial(a["q"], a["k"], a["v"], a["g"], a["beta"], a["init"])
    yc, sc = ao.gdn_chunked(a["q"], a["k"], a["v"], a["g"], a["beta"], a["init"])
    np.testing.assert_allclose(ys, a["ys"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(ss, a["ss"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(yc, a["yc"], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(sc, a["sc"], rtol=1e-10, atol=1e-12)


def test_decay_underflow_stays_finite():
    q = k = v = np.ones((64, 2)) / np.sqrt(2)
    g, b, s0 = np.full(64, -100.0), np.ones(64), np.ones((2, 2))
    yc, sc = ao.gdn_chunked(q, k, v, g, b, s0)
    ys, ss = ao.gdn_serial(q, k, v, g, b, s0)
    assert np.isfinite(yc).all()
    np.testing.assert_allclose(yc, ys)
    np.testing.assert_allclose(sc, ss)
    np.testing.assert_allclose(yc, G["underflow_y"])
    np.testing.assert_allclose(sc, G["underflow_s"])


def _tokens(scores, n):
    nb = n // 4
    sel = ao.qsa_select(scores, nb)
    return ao.qsa_positions(n - 1, sel)


@pytest.mark.parametrize("n", [2047, 2048, 2049, 2051, 2052, 2055, 2060])
def test_visibility_matches_reference(n):
    scores = np.zeros(n // 4)
    if n // 4 > 512:
        scores[512] = 1
    tokens = _tokens(scores, n)
    np.testing.assert_array_equal(tokens, G[f"vis_{n}"])
    assert len(tokens) == min(n // 4, 512) * 4 + n % 4


@pytest.mark.parametrize("n", [2100, 4099, 9001])
def test_selection_with_ties_matches_reference(n):
    np.testing.assert_array_equal(_tokens(G[f"sel_scores_{n}"], n), G[f"sel_tokens_{n}"])


def test_helpers_match_reference():
    assert int(G["helpers"]) == 1, "golden file was generated without ref/oracle.py helpers"
    x = G["rope_x"]
    np.testing.assert_allclose(ao.rope64(x, G["rope_pos"]), G["rope_y"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(ao.cn_rmsnorm(x, G["rms_w1"]), G["rms_y"], rtol=1e-13)
    np.testing.assert_allclose(ao.sigmoid(x), G["sigmoid_y"], rtol=1e-13)
    np.testing.assert_allclose(ao.silu(x), G["silu_y"], rtol=1e-12, atol=1e-15)
    np.testing.assert_allclose(ao.wht128(x), G["had_y"], rtol=1e-12, atol=1e-12)


def test_all_tied_scores_select_first_blocks():
    # bench/prefill_qsa.hip:213-223: all-tied scores => blocks 0..511 and a 3-token tail
    n = 4 * 700 + 3
    tokens = _tokens(np.zeros(700, np.float32), n)
    np.testing.assert_array_equal(tokens[:2048], np.arange(2048))
    np.testing.assert_array_equal(tokens[2048:], np.arange(2800, 2803))


def test_dense_equals_sparse_when_everything_is_selected():
    g = ao.Geometry(q_heads=4, kv_heads=2)
    rng = np.random.default_rng(0)
    n = 64
    cache = ao.QsaCache(g, 128)
    norms = [1 + 0.1 * rng.normal(size=s) for s in (256, 256, 128, 128)]
    q = rng.normal(size=(n, 4, 512)); k = rng.normal(size=(n, 512)); v = rng.normal(size=(n, 512))
    idx = rng.normal(size=(n, 640))
    out = ao.qsa_rows(q, k, v, idx, norms, cache, 0, g)
    # the same rows one at a time (decode) give the same result: row invariance (bench/qsa_long.hip:213-222)
    cache2 = ao.QsaCache(g, 128)
    rows = [ao.qsa_rows(q[i:i + 1], k[i:i + 1], v[i:i + 1], idx[i:i + 1], norms, cache2, i, g) for i in range(n)]
    np.testing.assert_allclose(np.concatenate(rows), out, rtol=1e-12, atol=1e-12)
    np.testing.assert_array_equal(cache.ik_pool, cache2.ik_pool)


def test_gdn_step_replay_commit_equals_serial_decode():
    """Lazy commit (engine/layers/ops.h:272-293, :361-368): verify span with commit=1 then a pass that
    replays `a` accepted rows must leave the state serial decoding of those tokens would."""
    g = ao.Geometry(hidden=64, gdn_vheads=4, gdn_kheads=2)
    rng = np.random.default_rng(1)
    W = g.gdn_qkv_width
    conv = rng.normal(size=(W, 4)) * 0.5
    ab = (rng.normal(size=(2 * g.gdn_vheads, g.hidden)) * 0.1).astype(np.float16)
    A_log, dtb, gamma = rng.normal(size=4), rng.normal(size=4) * 0.5, 1 + 0.1 * rng.normal(size=128)
    T = 14
    qkv, z, x = rng.normal(size=(T, W)), rng.normal(size=(T, 4 * 128)), rng.normal(size=(T, g.hidden))
    # serial decode, one row per call
    a = ao.GdnDecodeState(g)
    ser = [ao.gdn_step(a, qkv[t:t + 1], z[t:t + 1], x[t:t + 1], ab, conv, A_log, dtb, gamma, t, 0, 1) for t in range(T)]
    ser = np.concatenate(ser)
    # speculative: rows 0..4 as a span (commit 1), 3 drafts accepted -> next span starts at 4 with replay 3
    b = ao.GdnDecodeState(g)
    o1 = ao.gdn_step(b, qkv[0:5], z[0:5], x[0:5], ab, conv, A_log, dtb, gamma, 0, 0, 1)
    o2 = ao.gdn_step(b, qkv[4:10], z[4:10], x[4:10], ab, conv, A_log, dtb, gamma, 4, 3, 1)
    o3 = ao.gdn_step(b, qkv[10:14], z[10:14], x[10:14], ab, conv, A_log, dtb, gamma, 10, 5, 4)
    np.testing.assert_allclose(o1, ser[0:5], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(o2, ser[4:10], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(o3, ser[10:14], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(b.state, a.state, rtol=1e-10, atol=1e-12)


def test_gdn_layer_chunk_equals_serial():
    g = ao.Geometry(gdn_vheads=4, gdn_kheads=2)
    rng = np.random.default_rng(2)
    n = 150
    qkv = rng.normal(size=(n, g.gdn_qkv_width)); z = rng.normal(size=(n, 512))
    a, b = rng.normal(size=(n, 4)), rng.normal(size=(n, 4))
    conv = rng.normal(size=(g.gdn_qkv_width, 4)) * 0.5
    s0 = rng.normal(size=(4, 128, 128)) * 0.05
    args = (qkv, z, a, b, conv, rng.normal(size=4), rng.normal(size=4) * .5, np.ones(128), s0, g)
    o1, s1, _ = ao.gdn_layer(*args)
    o2, s2, _ = ao.gdn_layer(*args, chunk=64)
    np.testing.assert_allclose(o2, o1, rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(s2, s1, rtol=1e-9, atol=1e-11)


def test_gdn_layer_matches_the_references_own_layer_function():
    """ref/oracle.py::gdn (:101-130) run on a duck-typed checkpoint at the reference geometry (48 value / 16 key
    heads): conv + SiLU, L2 norms, head repetition, gates, serial recurrence from a zero state, gated RMSNorm."""
    assert int(G["layers"]) == 1, "golden file was generated without ref/oracle.py's layer functions"
    f = lambda name: G["layer_gdn_" + name].astype(np.float64)
    g = ao.Geometry(hidden=128, q_heads=24, kv_heads=2, gdn_vheads=48, gdn_kheads=16)
    x = f("x")
    a, b = x @ f("wa").T, x @ f("wb").T                 # ref/oracle.py:105-106
    out, state, _ = ao.gdn_layer(f("qkv"), f("z"), a, b, f("conv"), f("A_log"), f("dt_bias"), f("gamma"), np.zeros((48, 128, 128)), g)
    np.testing.assert_allclose(out, G["layer_gdn_out"], rtol=1e-9, atol=1e-11)
    # the chunked form of the same layer agrees as well
    out_c, _, _ = ao.gdn_layer(f("qkv"), f("z"), a, b, f("conv"), f("A_log"), f("dt_bias"), f("gamma"), np.zeros((48, 128, 128)), g, chunk=64)
    np.testing.assert_allclose(out_c, G["layer_gdn_out"], rtol=1e-8, atol=1e-10)


def test_qsa_dense_rows_match_the_references_own_layer_function():
    """ref/oracle.py::qsa (:147-165) on a duck-typed checkpoint at the reference geometry (24 query / 2 KV heads):
    CN-RMSNorm with (1 + w), partial RoPE, scale 1/16, causal softmax, KV head h // 12, sigmoid gate.  The oracle's
    cache holds K and V in fp16 (as the engine does), the reference function keeps them in fp64: the tolerance is the
    fp16 rounding of K (2^-11 relative on a logit of a few units) and V."""
    assert int(G["layers"]) == 1
    f = lambda name: G["layer_qsa_" + name].astype(np.float64)
    g = ao.Geometry(hidden=128, q_heads=24, kv_heads=2, gdn_vheads=48, gdn_kheads=16)
    n = len(f("q"))
    cache = ao.QsaCache(g, 64)
    norms = [1 + f("q_norm"), 1 + f("k_norm"), np.ones(128), np.ones(128)]
    out, sels, _, qn, _ = ao.qsa_rows(f("q").reshape(n, 24, 512), f("k"), f("v"), np.zeros((n, 640)), norms, cache, 0, g, return_detail=True)
    assert all(s is None for s in sels)                  # dense below 512 blocks
    ref = G["layer_qsa_out"]
    assert np.abs(out - ref).max() < 4e-3 and np.linalg.norm(out - ref) / np.linalg.norm(ref) < 1e-3
    # with K and V kept in fp64 (no cache rounding) the two agree to rounding: the algebra is the same
    D = 256
    q64 = f("q").reshape(n, 24, 512)
    pos = np.arange(n, dtype=np.float64)
    kn = ao.rope64(ao.cn_rmsnorm(f("k").reshape(n, 2, D), norms[1]), pos, g)
    v64 = f("v").reshape(n, 2, D)
    exact = np.empty((n, 24, D))
    for r in range(n):
        for h in range(24):
            lg = kn[:r + 1, h // 12] @ qn[r, h] / 16.0
            pr = np.exp(lg - lg.max())
            exact[r, h] = (pr / pr.sum()) @ v64[:r + 1, h // 12]
    exact = (exact * ao.sigmoid(q64[..., D:])).reshape(n, -1)
    np.testing.assert_allclose(exact, ref, rtol=1e-9, atol=1e-11)


@pytest.mark.parametrize("factor", [2, 4])
def test_yarn_tables_match_the_references_rows(factor):
    """The YaRN rows of engine/layers/rope_tables.h (32 inverse frequencies + the cos/sin multiplier), recomputed: equal to
    one or two units in the last place of float32 (the rows were generated with torch's float32 power function)."""
    ref = G["yarn_table_%d" % factor]
    inv, mult = ao.yarn_table(factor)
    np.testing.assert_allclose(inv, ref[:32], rtol=4e-7, atol=0)
    np.testing.assert_allclose(mult, ref[32], rtol=1e-7)
    plain, one = ao.yarn_table(1)
    np.testing.assert_array_equal(inv[:8], plain[:8])                  # fast frequencies are kept
    np.testing.assert_allclose(inv[24:], plain[24:] / factor, rtol=2e-7)   # slow ones are divided by the factor


def test_multimodal_rope_with_equal_axes_is_the_text_rotation():
    """Rope64Axes with t = h = w equals Rope64 (engine/layers/ops.h:515-536); distinct axes rotate frequency j by the h
    position when j % 3 == 1, by w when j % 3 == 2 and j < 30."""
    rng = np.random.default_rng(4)
    x = rng.normal(size=(5, 3, 256))
    pos = np.array([0., 7., 300., 4096., 99999.])
    axes = np.stack([pos, pos, pos], -1)
    np.testing.assert_allclose(ao.rope64(x, pos, axes=axes), ao.rope64(x, pos), rtol=0, atol=1e-15)
    axes = np.stack([pos, pos + 3, pos + 11], -1)
    got = ao.rope64(x, pos, axes=axes)
    inv = ao.rope_inv_freq(ao.GEOM_BENCH)
    for j, which in ((0, 0), (1, 1), (2, 2), (29, 2), (30, 0), (31, 1)):
        ang = axes[:, which] * inv[j]
        want = x[:, :, j] * np.cos(ang)[:, None] - x[:, :, j + 32] * np.sin(ang)[:, None]
        np.testing.assert_allclose(got[:, :, j], want, rtol=1e-12, atol=1e-12)
