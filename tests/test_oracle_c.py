"""The C port of the oracle (timed CPU baseline) agrees with the numpy oracle."""
import ctypes as C

import numpy as np
import pytest

from oracle import attn_oracle as ao


@pytest.fixture(scope="module")
def clib():
    from oracle import build
    lib = C.CDLL(build.build_oracle())
    lib.oracle_threads.restype = C.c_int
    return lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def test_gdn_layer_matches_numpy(clib):
    g = ao.Geometry(gdn_vheads=4, gdn_kheads=2)
    rng = np.random.default_rng(0)
    n, Cw = 90, g.gdn_qkv_width
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    qkv, z, ab = f32(rng.normal(size=(n, Cw))), f32(rng.normal(size=(n, 512))), f32(rng.normal(size=(n, 8)))
    conv, A_log, dtb, gamma = f32(rng.normal(size=(Cw, 4)) * .5), f32(rng.normal(size=4)), f32(rng.normal(size=4) * .5), f32(1 + .1 * rng.normal(size=128))
    hist = f32(rng.normal(size=(3, Cw)))
    s0 = f32(rng.normal(size=(4, 128, 128)) * 0.05)
    state, out = s0.copy(), np.zeros((n, 512), np.float32)
    clib.oracle_gdn_layer(_p(qkv), _p(z), _p(ab), _p(conv), _p(A_log), _p(dtb), _p(gamma), _p(hist), _p(state), _p(out), n, 4, 2)
    d = lambda a: a.astype(np.float64)
    ref, st, _ = ao.gdn_layer(d(qkv), d(z), d(ab[:, :4]), d(ab[:, 4:]), d(conv), d(A_log), d(dtb), d(gamma), d(s0), g, history=d(hist))
    assert np.abs(out - ref).max() < 2e-4
    assert np.linalg.norm(state - st) / np.linalg.norm(st) < 1e-5
    assert clib.oracle_threads() >= 1


def test_qsa_decode_row_matches_numpy(clib):
    g = ao.Geometry(q_heads=16, kv_heads=2)
    rng = np.random.default_rng(1)
    ctx = 2400
    cache = ao.QsaCache(g, ctx)
    norms = [1 + 0.1 * rng.normal(size=s) for s in (256, 256, 128, 128)]
    n = ctx - 1
    ao.qsa_prep(rng.normal(size=(n, 16, 512)), rng.normal(size=(n, 512)), rng.normal(size=(n, 512)), rng.normal(size=(n, 640)), *norms, cache, 0, g)
    q, k, v, idx = rng.normal(size=(1, 16, 512)), rng.normal(size=(1, 512)), rng.normal(size=(1, 512)), rng.normal(size=(1, 640))
    ref, sels, scs, qn, iq = ao.qsa_rows(q, k, v, idx, norms, cache, n, g, return_detail=True)
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    out, sel, nsel = np.zeros((16, 256), np.float32), np.zeros(512, np.int32), np.zeros(1, np.int32)
    qn32, gate32, iq32 = f32(qn[0]), f32(q[0, :, 256:]), f32(iq[0])
    kc, vc = np.ascontiguousarray(cache.k), np.ascontiguousarray(cache.v)
    clib.oracle_qsa_decode_row(_p(qn32), _p(gate32), _p(iq32), n, _p(kc), _p(vc), _p(cache.ik_pool), _p(out), _p(sel), _p(nsel), 16, 2)
    assert nsel[0] == 512
    assert ao.selection_agrees(scs[0], sel, sels[0])
    if np.array_equal(sel, sels[0]):
        assert np.abs(out.reshape(1, -1) - ref).max() < 1e-4
