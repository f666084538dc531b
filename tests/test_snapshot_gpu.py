"""State snapshot / restore through the C ABI (cr_state_save / cr_state_restore): an in-slot checkpoint holds exactly
the spans that change after its position (engine/runtime/slot_checkpoint_io.h:5-26), so a stream restored from it
replays the following steps bit for bit."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.gpu_util import dev

pytestmark = pytest.mark.gpu


def _stream_setup(seed, ctx0, compact):
    from crucible_strix_halo_b200 import capi, layers
    g = capi.Geometry(256, 16, 2, 4, 2)
    rng = np.random.default_rng(seed)
    qw = layers.QsaWeights(g, *[1 + 0.1 * rng.normal(size=n) for n in (256, 256, 128, 128)])
    gw = [layers.GdnWeights(g, 0.5 * rng.normal(size=(g.gdn_channels, 4)), rng.normal(size=4) - 1, 0.5 * rng.normal(size=4),
                            1 + 0.1 * rng.normal(size=128), ab=0.1 * rng.normal(size=(8, 256))) for _ in range(2)]
    qs = layers.QsaSession(g, ctx0 + 64, max_rows=1024, raw_slots=16 if compact else 0)
    gs = [layers.GdnSession(g) for _ in range(2)]
    # bring the stream to ctx0 positions: QSA cache rows through the prefill cache entry, GDN states through a prefill
    plan = layers.QsaPrefillPlan(qw, 1024)
    for p0 in range(0, ctx0, 1024):
        n = min(1024, ctx0 - p0)
        a = (capi.QsaArgs * 1)(layers.qsa_args(qw, qs, dev(rng.normal(size=(n, 16, 512))), dev(rng.normal(size=(n, 512))),
                                               dev(rng.normal(size=(n, 512))), dev(rng.normal(size=(n, 640))), plan.out, p0))
        capi.check(capi.lib.cr_qsa_prefill_cache(C.byref(g), a, None))
    for i in range(2):
        layers.GdnPrefillPlan(gw[i], 200).run(gs[i], dev(rng.normal(size=(200, g.gdn_channels))), dev(rng.normal(size=(200, 512))),
                                              dev(rng.normal(size=(200, 8))), ctx0 - 200)
    torch.cuda.synchronize()
    return capi, layers, g, rng, qw, gw, qs, gs


def _decode(layers, g, qw, gw, qs, gs, rows, pos0):
    """One-row steps of the two GDN layers and the QSA layer; returns every output."""
    outs = []
    plan = layers.QsaStepPlan(qw, 1)
    for t, (q, k, v, idx, qkv, z, x) in enumerate(rows):
        for i in range(2):
            outs.append(layers.gdn_step(gw[i], [dict(session=gs[i], qkv=dev(qkv[i]), z=dev(z[i]), x=dev(x[i]), pos0=pos0 + t)])[0].clone())
        outs.append(plan.run([dict(session=qs, q=dev(q), k=dev(k), v=dev(v), idx=dev(idx), pos0=pos0 + t)])[0].clone())
    torch.cuda.synchronize()
    return outs


@pytest.mark.parametrize("ctx0", [2300, 2304])          # inside a pool tile / on a tile boundary (no pool span)
def test_slot_checkpoint_restores_a_stream(ctx0):
    capi, layers, g, rng, qw, gw, qs, gs = _stream_setup(11, ctx0, compact=True)
    rows = [(rng.normal(size=(1, 16, 512)), rng.normal(size=(1, 512)), rng.normal(size=(1, 512)), rng.normal(size=(1, 640)),
             [rng.normal(size=(1, g.gdn_channels)) for _ in range(2)], [rng.normal(size=(1, 512)) for _ in range(2)],
             [rng.normal(size=(1, 256)) for _ in range(2)]) for _ in range(9)]
    tensors = layers.checkpoint_spans(gs, [qs], ctx0)
    assert len(tensors) == 6 + 1 + (1 if ctx0 % 128 else 0)
    cp = layers.SlotCheckpoint(tensors)
    assert cp.bytes == sum(t.numel() * t.element_size() for t in tensors)
    cp.save()
    torch.cuda.synchronize()
    flat = torch.cat([t.contiguous().view(torch.uint8).reshape(-1) for t in tensors])
    assert torch.equal(cp.buffer, flat), "the buffer holds the spans in order, back to back"
    first = _decode(layers, g, qw, gw, qs, gs, rows, ctx0)
    after = [t.clone() for t in tensors]
    assert not torch.equal(after[0], flat[:after[0].numel() * 4].view(torch.float32)), "the steps changed the state"
    cp.restore()
    torch.cuda.synchronize()
    assert torch.equal(torch.cat([t.contiguous().view(torch.uint8).reshape(-1) for t in tensors]), flat)
    again = _decode(layers, g, qw, gw, qs, gs, rows, ctx0)
    for a, b in zip(first, again):
        assert torch.equal(a, b), "a restored stream replays its steps bit for bit"
    for a, t in zip(after, tensors):
        assert torch.equal(a, t)
    # the compact ring changes nothing in the outputs: the same stream with full raw rows gives the same bits
    capi, layers, g, rng2, qw2, gw2, qs2, gs2 = _stream_setup(11, ctx0, compact=False)
    full = _decode(layers, g, qw2, gw2, qs2, gs2, rows, ctx0)
    for a, b in zip(first, full):
        assert torch.equal(a, b)


def test_snapshot_copy_many_spans_and_argument_checks():
    from crucible_strix_halo_b200 import capi, layers
    gen = torch.Generator(device="cuda").manual_seed(3)
    sizes = [16, 2048, 16384, 16400, 3 * 16384 + 32, 2 * 1024 * 1024 + 256] * 40            # 240 spans: three launches
    src = [torch.randint(0, 255, (n,), device="cuda", dtype=torch.uint8, generator=gen) for n in sizes]
    cp = layers.SlotCheckpoint(src)
    cp.buffer.fill_(0xEE)
    cp.save()
    torch.cuda.synchronize()
    assert torch.equal(cp.buffer, torch.cat(src))
    keep = [t.clone() for t in src]
    for t in src:
        t.zero_()
    cp.restore()
    torch.cuda.synchronize()
    for a, b in zip(keep, src):
        assert torch.equal(a, b)
    # a pinned host buffer takes a conversation snapshot without a staging copy
    host = torch.empty(cp.bytes, dtype=torch.uint8).pin_memory()
    capi.check(capi.lib.cr_state_save(cp.spans, len(src), host.data_ptr(), cp.bytes, None))
    torch.cuda.synchronize()
    assert torch.equal(host, torch.cat(keep).cpu())
    # refusals: a buffer smaller than the spans, a span that is not 16-byte sized, a span off a 16-byte boundary
    assert capi.lib.cr_state_save(cp.spans, len(src), cp.buffer.data_ptr(), cp.bytes - 16, None) == capi.ERR_INVALID
    odd = (capi.Span * 1)(capi.Span(src[1].data_ptr(), 24))
    assert capi.lib.cr_state_restore(odd, 1, cp.buffer.data_ptr(), cp.bytes, None) == capi.ERR_INVALID
    off = (capi.Span * 1)(capi.Span(src[1].data_ptr() + 8, 32))
    assert capi.lib.cr_state_save(off, 1, cp.buffer.data_ptr(), cp.bytes, None) == capi.ERR_INVALID
    assert capi.lib.cr_state_save(None, 0, None, 0, None) == capi.OK
