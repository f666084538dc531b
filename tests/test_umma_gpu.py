"""tcgen05 building blocks: a 128 x N x K tf32 product on tensor memory equals torch.  This pins the
shared-memory / instruction descriptor conventions the production kernels use."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K,N", [(8, 32), (64, 64), (128, 128), (128, 32), (64, 96)])
def test_umma_gemm(K, N):
    from crucible_strix_halo_b200 import capi
    g = torch.Generator(device="cuda").manual_seed(K * 1000 + N)
    A = torch.randn(128, K, device="cuda", generator=g)
    B = torch.randn(N, K, device="cuda", generator=g)
    D = torch.zeros(128, N, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.check(capi.lib.cr_debug_umma_gemm(A.data_ptr(), B.data_ptr(), D.data_ptr(), K, N, status.data_ptr(), None))
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "the bounded wait on the MMA gave up"
    ref = A.double() @ B.double().t()
    err = (D.double() - ref).abs().max().item()
    assert err < 3e-2 * (K ** 0.5) / 8 + 1e-3, "max error %g" % err     # tf32 operands: about 1e-3 relative per term


@pytest.mark.parametrize("K,N", [(16, 32), (64, 256), (32, 64), (128, 128)])
def test_umma_f16_gemm_with_mn_major_b(K, N):
    """kind::f16 with the B operand as a V tile lies in memory (keys x channels, channels contiguous): the descriptor
    whose leading offset is the step along keys and whose stride offset is the step along channels gives A B; the
    other assignment does not.  Pins the convention the tiled prefill attention relies on."""
    from crucible_strix_halo_b200 import capi
    g = torch.Generator(device="cuda").manual_seed(K * 7 + N)
    A = torch.randn(128, K, device="cuda", generator=g).half()
    B = torch.randn(K, N, device="cuda", generator=g).half()
    ref = A.double() @ B.double()
    errs = []
    for variant in (1, 0):
        D = torch.zeros(128, N, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        capi.check(capi.lib.cr_debug_umma_f16_gemm(A.data_ptr(), B.data_ptr(), D.data_ptr(), K, N, variant, status.data_ptr(), None))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        errs.append((D.double() - ref).abs().max().item())
    assert errs[0] < 1e-4, errs
    assert errs[1] > 1.0, errs


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """A wait on an mbarrier that nothing completes gives up after its time limit: the kernel returns, the status word
    and cr_device_check() report it (CR_ERR_TIMEOUT), clearing works, and the next ordinary launch is correct."""
    from crucible_strix_halo_b200 import capi
    import time
    capi.check(capi.lib.cr_device_status_clear())
    assert capi.lib.cr_device_status() == 0 and capi.lib.cr_device_check() == capi.OK
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    capi.check(capi.lib.cr_debug_wait_timeout(status.data_ptr(), 200, None))      # 200 microseconds
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0                       # it returned on its own
    assert int(status.item()) == 1
    assert capi.lib.cr_device_status() == 8
    assert capi.lib.cr_device_check() == capi.ERR_TIMEOUT
    assert b"debug_wait_kernel" in capi.lib.cr_last_error()
    capi.check(capi.lib.cr_device_status_clear())
    assert capi.lib.cr_device_status() == 0 and capi.lib.cr_device_check() == capi.OK
    test_umma_gemm(64, 64)                                      # the context is intact


@pytest.mark.parametrize("kv_heads,head,rows", [(2, 1, 4096), (2, 0, 130), (1, 0, 64)])
def test_tensor_map_tiles_feed_both_products_of_an_attention_step(kv_heads, head, rows):
    """Sixteen 4-token blocks of a K and a V cache copied by tensor-map boxes into 128-byte-swizzled tiles: the K tile
    read K-major gives S = Q K^T, the same kind of tile read MN-major gives O = P V; positions past the cache read as
    zeros.  Pins the copy layout and both descriptors of the tiled prefill attention."""
    from crucible_strix_halo_b200 import capi
    g = torch.Generator(device="cuda").manual_seed(rows)
    kc = torch.randn(rows, kv_heads, 256, device="cuda", generator=g).half()
    vc = torch.randn(rows, kv_heads, 256, device="cuda", generator=g).half()
    nb = (rows + 3) // 4
    blocks = torch.randperm(nb, device="cuda", generator=g)[:16].sort().values.int() if nb >= 16 else torch.arange(16, device="cuda").int()
    blocks[-1] = nb - 1                                           # the last block may hang over the end of the cache
    if rows == 64:
        blocks[-1] = nb + 3                                       # and one wholly past it
    Q = torch.randn(128, 256, device="cuda", generator=g).half()
    Pm = torch.rand(128, 64, device="cuda", generator=g).half()
    S = torch.zeros(128, 64, device="cuda"); O = torch.zeros(128, 256, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    capi.check(capi.lib.cr_debug_umma_kv_step(kc.data_ptr(), vc.data_ptr(), kv_heads, rows, head, blocks.data_ptr(), Q.data_ptr(), Pm.data_ptr(),
                                              S.data_ptr(), O.data_ptr(), status.data_ptr(), None))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    pos = (blocks.long()[:, None] * 4 + torch.arange(4, device="cuda")[None]).reshape(-1)
    live = pos < rows
    kt = torch.zeros(64, 256, device="cuda", dtype=torch.float64); vt = torch.zeros(64, 256, device="cuda", dtype=torch.float64)
    kt[live] = kc[pos[live], head].double(); vt[live] = vc[pos[live], head].double()
    assert (S.double() - Q.double() @ kt.t()).abs().max().item() < 1e-3
    assert (O.double() - Pm.double() @ vt).abs().max().item() < 1e-3
