"""Split-KV over real ranks: two processes, one GPU each, NCCL for the exchange (all-to-all of candidates and partials,
all-gathers of selections and output rows); the result equals the single-device path.  Skipped on a single-GPU box;
the same exchange runs there with emulated ranks (tests/test_qsa_gpu.py) and on CPU ranks over gloo
(tests/test_parallel_cpu.py)."""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, pos0, R, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from crucible_strix_halo_b200 import capi, layers, parallel as par
    g = capi.Geometry(256, 16, 2, 4, 2)
    gen = torch.Generator(device="cuda").manual_seed(5)                  # the same sequence on every rank
    rn = lambda *s: torch.randn(*s, device="cuda", generator=gen)
    w = layers.QsaWeights(g, *[1 + 0.1 * rn(n).cpu().numpy() for n in (256, 256, 128, 128)])
    ses = layers.QsaSession(g, pos0 + R, max_rows=max(R, 1024))
    plan = layers.QsaPrefillPlan(w, max(R, 1024))
    for p0 in range(0, pos0, 1024):                                       # cache rows through the prefill cache entry
        n = min(1024, pos0 - p0)
        a = (capi.QsaArgs * 1)(layers.qsa_args(w, ses, rn(n, 16, 512), rn(n, 512), rn(n, 512), rn(n, 640), plan.out, p0))
        capi.check(capi.lib.cr_qsa_prefill_cache(C.byref(g), a, None))
    rows = [rn(R, 16, 512), rn(R, 512), rn(R, 512), rn(R, 640)]
    capi.set_options(qsa_union_rows=-1)                                   # the fp32-level row-wise kernels on both sides
    single = plan.run(ses, rows[0].clone(), rows[1], rows[2], rows[3].clone(), pos0).float().clone()
    sel_single, nsel_single = ses.sel[:R].clone(), ses.nsel[:R].clone()
    # the sharded path on the prepared part: queries normalised in place, cache rows of the part already written
    qd, idxd = rows[0].clone(), rows[3].clone()
    out = torch.zeros(R, 16 * 256, device="cuda")
    args = layers.qsa_args(w, ses, qd, rows[1], rows[2], idxd, out, pos0)
    capi.check(capi.lib.cr_qsa_prep_queries(C.byref(g), (capi.QsaArgs * 1)(args), 1, None))
    ses.scores.fill_(-1.0)
    backend = par.CudaQsaBackend(g, args, R, capi.OUT_RAW_F32, out)
    got = par.SplitKvQsa(backend).run(pos0 + R)
    torch.cuda.synchronize()
    ok = torch.equal(backend.nsel, nsel_single)
    sparse = nsel_single > 0
    ok = ok and torch.equal(backend.sel[sparse], sel_single[sparse])
    err = (got - single).abs().max().item()
    q.put((rank, bool(ok), err, capi.lib.cr_device_status()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("pos0,R", [(3000, 300), (2300, 13)])          # rows the ranks divide, and rows they do not
def test_split_kv_over_nccl_equals_the_single_device_path(pos0, R):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, pos0, R, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, ok, err, status in res:
        assert ok, "rank %d: the merged selection differs from the single-device selection" % rank
        assert err < 2e-4 and status == 0, (rank, err, status)
