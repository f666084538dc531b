"""CPU checks of the C-ABI library: it loads, exports every function include/crucible_attn.h declares, and
rejects contract violations before touching a device (no compute calls here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def capi():
    import __graft_entry__ as ge
    ge.build()
    from crucible_strix_halo_b200 import capi
    return capi


def test_exports_every_declared_symbol(capi):
    header = open(os.path.join(ROOT, "include", "crucible_attn.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(cr_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 20
    for name in sorted(declared):
        assert hasattr(capi.lib, name), name
    assert declared == set(capi.EXPORTS)
    assert capi.lib.cr_version() >= 1


def test_struct_sizes_match_header(capi):
    # 13 pointers + 6 ints; 4 pointers + int (padded); see include/crucible_attn.h
    assert C.sizeof(capi.GdnArgs) == 13 * 8 + 6 * 4
    assert C.sizeof(capi.QsaCache) == 4 * 8 + 8
    assert C.sizeof(capi.Geometry) == 5 * 4


def test_contract_violations_are_reported_without_a_device(capi):
    g = capi.GEOM_BENCH
    a = (capi.GdnArgs * 1)()
    a[0].R, a[0].commit = 0, 0
    assert capi.lib.cr_gdn_step(C.byref(g), a, 1, 8, capi.OUT_RAW_F32, None) == capi.ERR_INVALID
    assert b"R=0" in capi.lib.cr_last_error()
    a[0].R, a[0].commit = 4, 0          # zero-prefix rollback is unsupported (retained_prefix.h:14-15)
    assert capi.lib.cr_gdn_step(C.byref(g), a, 1, 8, capi.OUT_RAW_F32, None) == capi.ERR_INVALID
    a[0].R, a[0].commit = 14, 1         # ring headroom: at most 13 rows per span
    assert capi.lib.cr_gdn_step(C.byref(g), a, 1, 16, capi.OUT_RAW_F32, None) == capi.ERR_INVALID
    bad = capi.Geometry(2048, 15, 2, 32, 16)
    assert capi.lib.cr_gdn_step(C.byref(bad), a, 1, 8, capi.OUT_RAW_F32, None) == capi.ERR_INVALID
    q = (capi.QsaArgs * 1)()
    q[0].R, q[0].pos0 = 2049, 0
    assert capi.lib.cr_qsa_select(C.byref(g), q, 1, None, 0, None) == capi.ERR_INVALID
    p = capi.QsaPrefillArgs()
    p.input.R, p.input.pos0, p.input.sstride = 64, 0, 1   # stride too small
    assert capi.lib.cr_qsa_prefill(C.byref(g), C.byref(p), 0, capi.OUT_RAW_F32, None) == capi.ERR_INVALID


def test_sizing_helpers(capi):
    g = capi.GEOM_BENCH
    assert capi.lib.cr_qsa_pool_floats(262144) == 2048 * 4096          # QsaPoolFloats, ops.h:420
    out = (C.c_size_t * 4)()
    assert capi.lib.cr_qsa_cache_bytes(C.byref(g), 262144, 0, out) == capi.OK
    assert list(out) == [262144 * 1024, 262144 * 1024, 262144 * 512, 2048 * 4096 * 4]   # cache_storage.h:40-46
    assert capi.lib.cr_qsa_cache_bytes(C.byref(g), 262144, 1, out) == capi.OK and out[2] == 16 * 512
    assert capi.lib.cr_qsa_cache_bytes(C.byref(g), 0, 0, out) == capi.ERR_INVALID
    assert capi.lib.cr_qsa_scratch_bytes(C.byref(g), 1) == 16 * 32 * 258 * 4          # QsaScratchFloats, qsa_long.h:396
    assert capi.lib.cr_gdn_prefill_workspace_bytes(C.byref(g), 2048) > 0


def test_gdn_prefill_part_schedule_covers_every_row():
    """cr_gdn_prefill_parts is host-only: the parts of a long call tile the rows exactly, every part but the last is a
    whole number of 64-row chunks, none exceeds the part the workspace is sized for, the first is short and the
    last ones shrink."""
    import ctypes as C
    from crucible_strix_halo_b200 import capi
    part = 111 * 64
    for rows in (1, 63, 64, 7104, 7105, 8004, 14541, 32768, 100000, 262144):
        first, n = (C.c_int * 64)(), (C.c_int * 64)()
        k = capi.lib.cr_gdn_prefill_parts(rows, first, n, 64)
        assert 1 <= k <= 64
        assert first[0] == 0 and sum(n[:k]) == rows
        for i in range(k):
            assert 1 <= n[i] <= part
            if i + 1 < k:
                assert n[i] % 64 == 0 and first[i + 1] == first[i] + n[i]
        if rows <= part:
            assert k == 1
        if rows >= 32768:
            assert n[0] == 32 * 64 and n[k - 1] <= n[k - 2] <= n[k - 3]
    assert capi.lib.cr_gdn_prefill_parts(0, None, None, 0) == 0


def test_options_are_validated_and_bound_the_part_schedule():
    """cr_get_options / cr_set_options are host-only: bad values are refused and leave the options unchanged; with a
    part option below the default every part of a long call, the short first one included, stays within the part the
    workspace is sized for."""
    import ctypes as C
    from crucible_strix_halo_b200 import capi
    old = capi.get_options()
    assert (old.gdn_part_chunks, old.pdl, old.qsa_score_simt) == (111, 1, 0)
    for bad in (dict(gdn_part_chunks=8), dict(gdn_part_chunks=5000), dict(pdl=2), dict(qsa_score_simt=-1), dict(qsa_union_rows=5)):
        with pytest.raises(capi.CrError):
            capi.set_options(**bad)
        assert capi.get_options().gdn_part_chunks == 111
    try:
        for chunks in (32, 33, 50, 111, 400):
            capi.set_options(gdn_part_chunks=chunks)
            for rows in (chunks * 64, chunks * 64 + 1, 3 * chunks * 64 + 5, 32768, 262144):
                first, n = (C.c_int * 256)(), (C.c_int * 256)()
                k = capi.lib.cr_gdn_prefill_parts(rows, first, n, 256)
                assert 1 <= k <= 256 and sum(n[:k]) == rows
                assert max(n[:k]) <= chunks * 64, (chunks, rows, list(n[:k]))
    finally:
        capi.check(capi.lib.cr_set_options(C.byref(old)))
