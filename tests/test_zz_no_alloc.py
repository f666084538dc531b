"""cr_qsa_attn_static: the attention entry point for hosts that cannot allocate or pass scratch (a server whose
HBM is all committed to caches, a plugin without its host's allocator, a caller inside a capture-sensitive
section).  It must give what cr_qsa_attn gives with caller scratch, call after call, since every call reuses the
same built-in array.  Collected last on purpose: a failure here cannot hide the other tests under `-x`."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _spans(capi, layers, w, g, rng, ctxs, rows):
    sess, args, keep = [], [], []
    for ctx, R in zip(ctxs, rows):
        s = layers.QsaSession(g, ctx + 16, max_rows=13)
        s.k.copy_(torch.randn(ctx + 16, 2, 256, device="cuda").half())
        s.v.copy_(torch.randn(ctx + 16, 2, 256, device="cuda").half())
        s.ik_pool.normal_()
        s.ik_raw.normal_()
        t = [torch.randn(R, 16, 512, device="cuda"), torch.randn(R, 512, device="cuda"), torch.randn(R, 512, device="cuda"),
             torch.randn(R, 640, device="cuda")]
        out = torch.zeros(R, 16 * 256, device="cuda")
        keep.append((s, t, out))
        args.append(layers.qsa_args(w, s, *t, out, ctx))
    arr = (capi.QsaArgs * len(args))(*args)
    return arr, keep


def test_static_scratch_attention_equals_caller_scratch_twice():
    from crucible_strix_halo_b200 import capi, layers
    torch.manual_seed(0)
    g = capi.GEOM_BENCH
    rng = np.random.default_rng(0)
    w = layers.QsaWeights(g, *[1 + 0.1 * rng.normal(size=n) for n in (256, 256, 128, 128)])
    arr, keep = _spans(capi, layers, w, g, rng, ctxs=[2500, 1000], rows=[3, 2])   # one sparse span, one dense span
    n = len(keep)
    capi.check(capi.lib.cr_qsa_prep(C.byref(g), arr, n, None))
    capi.check(capi.lib.cr_qsa_select(C.byref(g), arr, n, None, 0, None))
    scratch = torch.zeros(capi.lib.cr_qsa_scratch_bytes(C.byref(g), 5), dtype=torch.uint8, device="cuda")
    capi.check(capi.lib.cr_qsa_attn(C.byref(g), arr, n, scratch.data_ptr(), scratch.numel(), capi.OUT_RAW_F32, None))
    torch.cuda.synchronize()
    want = [k[2].clone() for k in keep]
    assert all(torch.isfinite(x).all() and x.abs().max() > 0 for x in want)
    for call in range(2):                      # the array keeps the previous call's contents: results must not change
        for k in keep:
            k[2].zero_()
        capi.check(capi.lib.cr_qsa_attn_static(C.byref(g), arr, n, capi.OUT_RAW_F32, None))
        torch.cuda.synchronize()
        for got, ref in zip((k[2] for k in keep), want):
            assert torch.allclose(got, ref, rtol=0, atol=1e-6), "call %d: max diff %g" % (call, (got - ref).abs().max().item())


def test_static_scratch_rejects_oversized_calls():
    from crucible_strix_halo_b200 import capi, layers
    g = capi.GEOM_BENCH
    rng = np.random.default_rng(1)
    w = layers.QsaWeights(g, *[1 + 0.1 * rng.normal(size=n) for n in (256, 256, 128, 128)])
    arr, keep = _spans(capi, layers, w, g, rng, ctxs=[600, 600], rows=[9, 8])     # 17 rows x 16 heads = 272 > 256
    assert capi.lib.cr_qsa_attn_static(C.byref(g), arr, 2, capi.OUT_RAW_F32, None) == capi.ERR_INVALID
    assert b"exceed the built-in scratch" in capi.lib.cr_last_error()
