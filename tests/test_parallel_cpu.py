"""Host logic of the multi-GPU partitioning on CPU: shard ranges, and the split-KV exchange (candidate all-gather,
global merge, partial all-gather, LSE merge) run as two gloo ranks with the numpy oracle as the compute backend;
the result must equal the single-rank oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from crucible_strix_halo_b200 import parallel as par
from oracle import attn_oracle as ao


def test_shard_ranges_cover_and_balance():
    for n, w in [(32, 8), (7, 4), (1, 2), (65536, 3)]:
        spans = [par.shard_range(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    (b0, b1), (p0, p1) = par.kv_block_range(2603, 2, 1)
    assert (b0, b1) == (325, 650) and p0 == 1300 and p1 > 2603      # the tail 2600..2602 belongs to the last rank
    assert par.kv_block_range(2603, 2, 0) == ((0, 325), (0, 1300))


class OracleBackend:
    """Numpy stand-in for the CUDA kernels, same record formats."""

    def __init__(self, g, cache, qn, gate, iq, pos0):
        self.g, self.cache, self.qn, self.gate, self.iq, self.pos0 = g, cache, qn, gate, iq, pos0
        self.R = len(qn)
        self.sel = [None] * self.R

    def shard_candidates(self, b0, b1):
        cs = np.full((self.R, 512), -1.0, np.float32); ci = np.full((self.R, 512), -1, np.int32)
        for r in range(self.R):
            nb = (self.pos0 + r + 1) // 4
            hi = min(nb, b1)
            if nb <= 512 or hi <= b0:
                continue
            sc = ao.qsa_scores(self.iq[r], self.cache.pool_rows(nb)).astype(np.float32)[b0:hi]
            order = np.lexsort((np.arange(len(sc)), -sc))[:512]
            order.sort()
            cs[r, :len(order)] = sc[order]; ci[r, :len(order)] = order + b0
        return torch.from_numpy(cs), torch.from_numpy(ci)

    rows = property(lambda self: self.R)

    def merge_candidates(self, scores, ids, r0, r1):
        s, i = scores.numpy(), ids.numpy()
        sel = np.zeros((r1 - r0, 512), np.int32); nsel = np.full(r1 - r0, -1, np.int32)
        for r in range(r0, r1):
            if (self.pos0 + r + 1) // 4 <= 512:
                continue
            sc, idv = s[:, r - r0].ravel(), i[:, r - r0].ravel()
            keep = idv >= 0
            sc, idv = sc[keep], idv[keep]
            order = np.lexsort((idv, -sc.astype(np.float64)))[:512]
            sel[r - r0], nsel[r - r0] = np.sort(idv[order]), 512
        return torch.from_numpy(sel), torch.from_numpy(nsel)

    def set_selection(self, sel, nsel):
        self.sel = [sel[r].numpy().astype(np.int32) if int(nsel[r]) > 0 else None for r in range(self.R)]

    def shard_attn(self, p0, p1):
        g = self.g
        out = np.zeros((self.R, g.q_heads, 258), np.float32)
        for r in range(self.R):
            pos = ao.qsa_positions(self.pos0 + r, self.sel[r], g)
            pos = pos[(pos >= p0) & (pos < p1)]
            out[r, :, 0] = -np.inf
            if len(pos) == 0:
                continue
            K, V = self.cache.k[pos].astype(np.float64), self.cache.v[pos].astype(np.float64)
            for h in range(g.q_heads):
                lg = K[:, h // g.gqa] @ self.qn[r, h] / 16.0
                m = lg.max(); e = np.exp(lg - m)
                out[r, h, 0], out[r, h, 1], out[r, h, 2:] = m, e.sum(), e @ V[:, h // g.gqa]
        return torch.from_numpy(out)

    def merge_partials(self, parts, r0, r1):
        p = parts.numpy().astype(np.float64)
        out = np.zeros((r1 - r0, self.g.q_heads, 256))
        for r in range(r1 - r0):
            for h in range(self.g.q_heads):
                out[r, h] = ao.lse_merge([(p[w, r, h, 0], p[w, r, h, 1], p[w, r, h, 2:]) for w in range(p.shape[0])])
        return torch.from_numpy(out * ao.sigmoid(self.gate[r0:r1]))


def _problem(R=6):
    g = ao.Geometry(q_heads=16, kv_heads=2)
    rng = np.random.default_rng(0)
    ctx0 = 2110
    cache = ao.QsaCache(g, ctx0 + R)
    norms = [1 + 0.1 * rng.normal(size=s) for s in (256, 256, 128, 128)]
    ao.qsa_prep(rng.normal(size=(ctx0, 16, 512)), rng.normal(size=(ctx0, 512)), rng.normal(size=(ctx0, 512)), rng.normal(size=(ctx0, 640)),
                *norms, cache, 0, g)
    rows = (rng.normal(size=(R, 16, 512)), rng.normal(size=(R, 512)), rng.normal(size=(R, 512)), rng.normal(size=(R, 640)))
    return g, cache, norms, rows, ctx0, R


def _worker(rank, world, port, q, R):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g, cache, norms, rows, ctx0, R = _problem(R)
    qn, gate, iq = ao.qsa_prep(*rows, *norms, cache, ctx0, g)
    out = par.SplitKvQsa(OracleBackend(g, cache, qn, gate, iq, ctx0)).run(ctx0 + R)
    if rank == 0:
        q.put(out.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("R", [6, 5])         # rows the ranks divide (every rank merges its own rows) and rows they do not
def test_split_kv_two_ranks_equals_single_rank(R):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, R)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    g, cache, norms, rows, ctx0, R = _problem(R)
    ref = ao.qsa_rows(*rows, norms, cache, ctx0, g)
    np.testing.assert_allclose(out.reshape(R, -1), ref, rtol=1e-6, atol=1e-7)


def _gdn_problem():
    g = ao.Geometry(hidden=64, gdn_vheads=8, gdn_kheads=4)
    rng = np.random.default_rng(11)
    n, C = 70, g.gdn_qkv_width
    return (g, rng.normal(size=(n, C)), rng.normal(size=(n, g.gdn_value_width)), rng.normal(size=(n, 8)), rng.normal(size=(n, 8)),
            rng.normal(size=(C, 4)) * 0.5, np.clip(rng.normal(-1, 1.5, 8), -5, 1.5), rng.normal(size=8) * 0.5,
            1 + 0.1 * rng.normal(size=128), rng.normal(size=(8, 128, 128)) * 0.05)


def _gdn_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g, qkv, z, al, bl, conv, A_log, dtb, gamma, state = _gdn_problem()
    sh = par.GdnHeadShard(g.gdn_vheads, g.gdn_kheads, world, rank)
    sg = ao.Geometry(hidden=64, gdn_vheads=sh.vheads, gdn_kheads=sh.kheads)
    cols, hs = sh.qkv_columns, sh.head_slice
    out, st, _ = ao.gdn_layer(qkv[:, cols], z[:, sh.value_columns], al[:, hs], bl[:, hs], conv[cols], A_log[hs], dtb[hs], gamma,
                              state[hs], sg)
    outs = [torch.empty(len(out), sh.vheads * 128, dtype=torch.float64) for _ in range(world)]     # equal shards here
    dist.all_gather(outs, torch.from_numpy(np.ascontiguousarray(out)))
    sts = [torch.empty(sh.vheads, 128, 128, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(sts, torch.from_numpy(np.ascontiguousarray(st)))
    if rank == 0:
        q.put((torch.cat(outs, 1).numpy(), torch.cat(sts, 0).numpy()))
    dist.barrier()
    dist.destroy_process_group()


def test_gdn_head_shards_two_ranks_equal_the_full_layer():
    """GDN value heads shard with no exchange: every rank runs the layer on its own heads (channels picked by
    GdnHeadShard), outputs and states are concatenated in rank order."""
    sh = [par.GdnHeadShard(32, 16, 8, r) for r in range(8)]
    assert [s.vheads for s in sh] == [4] * 8 and sh[3].v0 == 12 and sh[3].k0 == 6
    cols = sorted(c for s in sh for c in s.qkv_columns)
    assert cols == list(range(2 * 16 * 128 + 32 * 128))                       # every channel owned exactly once
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gdn_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out, st = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    g, qkv, z, al, bl, conv, A_log, dtb, gamma, state = _gdn_problem()
    ref, ref_st, _ = ao.gdn_layer(qkv, z, al, bl, conv, A_log, dtb, gamma, state, g)
    np.testing.assert_allclose(out, ref, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(st, ref_st, rtol=1e-12, atol=1e-12)
