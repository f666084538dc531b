"""Projection GEMM either side of the attention core (cr_proj_gemm): bf16 operands, fp32 accumulation on tcgen05,
columns scattered into the buffers the core reads.  Compared with a torch fp32 product of the same bf16 operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(R, K, widths, f32, seed):
    from crucible_strix_halo_b200 import capi, layers
    gen = torch.Generator(device="cuda").manual_seed(seed)
    N = sum(widths)
    x = torch.randn(R, K, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=gen) / K ** 0.5).bfloat16()
    outs = [torch.full((R, c), float("nan"), device="cuda", dtype=torch.float32 if f else torch.bfloat16) for c, f in zip(widths, f32)]
    layers.proj_gemm(x, w, outs)
    torch.cuda.synchronize()
    assert capi.lib.cr_device_status() == 0
    ref = x.float() @ w.float().t()
    col = 0
    for o, c, f in zip(outs, widths, f32):
        want = ref[:, col:col + c]
        err = (o.float() - want).abs().max().item()
        assert err < (2e-4 if f else 2e-2), "columns %d..%d: max error %g" % (col, col + c, err)      # fp32 out: accumulation order only; bf16 out: one rounding
        col += c


@pytest.mark.parametrize("R,K,widths,f32", [
    (128, 64, [256], [True]),                                   # one tile, one K step
    (300, 256, [512, 256, 64], [False, False, False]),          # ragged rows, a narrow last output, partial last tile
    (1000, 2048, [1024, 512, 32], [True, False, True]),         # mixed output types, more K steps than stages
    (77, 128, [32], [False]),                                   # narrower than a tile in both directions
])
def test_projection_matches_torch(R, K, widths, f32):
    _check(R, K, widths, f32, R + K)


def test_gdn_input_projection_feeds_the_prefill_entry():
    """hidden rows -> qkv | z | gate logits in bf16 -> cr_gdn_prefill (CR_IN_BF16): the same layer output as with rows
    projected by torch and rounded to bf16."""
    from crucible_strix_halo_b200 import capi, layers
    g = capi.Geometry(256, 16, 2, 4, 2)
    gen = torch.Generator(device="cuda").manual_seed(9)
    rn = lambda *s, std=1.0: torch.randn(*s, device="cuda", generator=gen) * std
    R, C, Z = 517, g.gdn_channels, 4 * 128
    x = rn(R, 256).bfloat16()
    w = rn(C + Z + 32, 256, std=1 / 16).bfloat16()             # a,b logits padded to 32 columns (8 used)
    gw = layers.GdnWeights(g, rn(C, 4, std=0.5), rn(4) - 1, rn(4, std=0.5), 1 + rn(128, std=0.1))
    qkv, z, ab = (torch.empty(R, c, device="cuda", dtype=torch.bfloat16) for c in (C, Z, 32))
    layers.proj_gemm(x, w, [qkv, z, ab])
    ref = (x.float() @ w.float().t()).bfloat16()
    assert (qkv.float() - ref[:, :C].float()).abs().max().item() < 3e-2
    outs = []
    for rows in ((qkv, z, ab[:, :8].contiguous()), (ref[:, :C].contiguous(), ref[:, C:C + Z].contiguous(), ref[:, C + Z:C + Z + 8].contiguous())):
        ses = layers.GdnSession(g)
        plan = layers.GdnPrefillPlan(gw, R, in_dtype=capi.IN_BF16)
        outs.append(plan.run(ses, *rows, 0, capi.GDN_CHUNK_TC).clone())
    torch.cuda.synchronize()
    # the two inputs differ by bf16 roundings of single elements; the layer outputs stay within the path's tolerance
    assert (outs[0] - outs[1]).abs().max().item() < 2e-2


def test_projection_argument_checks():
    from crucible_strix_halo_b200 import capi
    x = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    o = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    one = lambda col0, cols: (capi.ProjOut * 1)(capi.ProjOut(o.data_ptr(), col0, cols, 64, 0))
    assert capi.lib.cr_proj_gemm(x.data_ptr(), x.data_ptr(), 64, 48, 64, one(0, 64), 1, None) == capi.ERR_INVALID      # K not a multiple of 64
    assert capi.lib.cr_proj_gemm(x.data_ptr(), x.data_ptr(), 64, 64, 64, one(0, 32), 1, None) == capi.ERR_INVALID      # outputs do not cover N
    assert capi.lib.cr_proj_gemm(x.data_ptr(), x.data_ptr(), 64, 64, 64, one(32, 32), 1, None) == capi.ERR_INVALID     # gap before the first output
    assert capi.lib.cr_proj_gemm(x.data_ptr(), x.data_ptr(), 64, 64, 64, one(0, 64), 1, None) == capi.OK
