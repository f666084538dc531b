"""Multi-GPU partitioning of the attention path: one process per GPU, torch.distributed for the exchange.

Natural shards need no exchange: sessions (decode / verify) and sequences (prefill) are independent, GDN value
heads are independent recurrences (GdnHeadShard).  One long sequence of the QSA layer is split over the KV positions:

    rank g owns positions [lo_g, hi_g)  (whole 4-token blocks; the newest rows belong to the last rank)
    and the merges of the rows [g R / W, (g + 1) R / W) of the part
    1. local scores + top-512 candidates over the owned blocks, all rows    cr_qsa_shard_select
    2. candidates of rows r go to the owner of r (all-to-all)               -> owner: cr_qsa_merge_candidates
    3. all-gather of the selections [rows][512]
    4. attention over the owned part of the attended positions, all rows    cr_qsa_shard_attn -> (m, l, acc[256])
    5. partials of rows r go to the owner of r (all-to-all)                 -> owner: cr_qsa_merge_partials (LSE merge + gate)
    6. all-gather of the output rows
Per rank and part (2,048 rows, 16 heads) that is (W - 1) / W x (8 + 4 + 34 + 17) MB on the wire instead of
(W - 1) x 42 MB when every rank gathers and merges everything (the form kept for row counts W does not divide).

The record formats are the reference's own split-KV formats (engine/layers/qsa_long.h:228-234, :442-474), which is
what makes the single-device merge kernels reusable across devices.  The compute steps go through a backend
object so the host logic (ranges, gather layouts, ordering) is testable on CPU ranks with gloo.
"""
import ctypes as C


def shard_range(n, world, rank):
    """Contiguous, balanced [lo, hi) of n items for `rank` of `world`."""
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def kv_block_range(total_positions, world, rank, block=4):
    """Block range [b0, b1) and position range [p0, p1) owned by `rank` when `total_positions` cache positions are
    split over `world` ranks.  Complete blocks are dealt out contiguously; the incomplete tail block and everything
    after it belongs to the last rank (its positions are the newest rows)."""
    nb = total_positions // block
    b0, b1 = shard_range(nb, world, rank)
    p0, p1 = b0 * block, b1 * block
    if rank == world - 1:
        p1 = 1 << 30
    return (b0, b1), (p0, p1)


class GdnHeadShard:
    """Value heads of a GDN layer dealt to ranks with no exchange: each value head is an independent recurrence, and
    the rep = Hv / Hk value heads that share a key head stay together (engine/layers/ops.h:258).  The shard is
    itself a GDN layer of vheads x kheads heads: `qkv_columns` picks its channels out of a projection row
    [q heads | k heads | v heads], `value_columns` its slice of z / output rows, `head_slice` its entries of the
    per-head vectors (A_log, dt_bias, a/b logits) and of the state; conv weights follow `qkv_columns`."""

    def __init__(self, vheads, kheads, world, rank, dim=128):
        assert vheads % kheads == 0 and kheads >= world, "need at least one key head per rank"
        rep = vheads // kheads
        k0, k1 = shard_range(kheads, world, rank)
        self.k0, self.k1, self.v0, self.v1 = k0, k1, k0 * rep, k1 * rep
        self.kheads, self.vheads, self.dim = k1 - k0, (k1 - k0) * rep, dim
        self._full = (vheads, kheads)

    @property
    def head_slice(self):
        return slice(self.v0, self.v1)

    @property
    def value_columns(self):
        return slice(self.v0 * self.dim, self.v1 * self.dim)

    @property
    def qkv_columns(self):
        """Channel indices (ascending) of this shard in a full [q | k | v] row."""
        vheads, kheads = self._full
        d = self.dim
        q = range(self.k0 * d, self.k1 * d)
        k = range(kheads * d + self.k0 * d, kheads * d + self.k1 * d)
        v = range(2 * kheads * d + self.v0 * d, 2 * kheads * d + self.v1 * d)
        return list(q) + list(k) + list(v)


class SplitKvQsa:
    """Runs the selection and attention of one QSA part (rows already prepared, caches holding the part) across the
    ranks of `group`.  backend: object with `rows` and
        shard_candidates(b0, b1)                  -> (scores [R,512] f32, ids [R,512] i32) over the rank's own blocks
        merge_candidates(scores [W,n,512], ids, r0, r1) -> (sel [n,512] i32, nsel [n] i32) of the rows [r0, r1)
        set_selection(sel [R,512], nsel [R])      the global selection every rank attends with
        shard_attn(p0, p1)                        -> partials [R,Hq,258] over the rank's own positions
        merge_partials(parts [W,n,Hq,258], r0, r1) -> output rows [n, ...] of the rows [r0, r1)
    tensors are torch tensors on the backend's device."""

    def __init__(self, backend, group=None):
        import torch.distributed as dist
        self.backend, self.group, self.dist = backend, group, dist
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def _all_gather(self, t):
        import torch
        if self.world == 1:
            return t.unsqueeze(0)
        out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        self.dist.all_gather(list(out.unbind(0)), t.contiguous(), group=self.group)   # rank-major [W, ...]
        return out

    def _rows_to_owners(self, t, r0, r1):
        """t [R, ...] on every rank -> [W, r1 - r0, ...]: what every rank holds for this rank's rows.  An all-to-all
        where the backend has one (NCCL); elsewhere an all-gather of which the own rows are kept."""
        import torch
        if self.world == 1:
            return t.unsqueeze(0)
        if t.is_cuda:
            out = torch.empty((self.world, r1 - r0) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
            self.dist.all_to_all_single(out.view((-1,) + tuple(t.shape[1:])), t.contiguous(), group=self.group)
            return out
        return self._all_gather(t)[:, r0:r1].contiguous()

    def run(self, total_positions):
        """total_positions = pos0 + R (positions in the cache after this part).  Returns the gated output rows [R, ...]."""
        b, W = self.backend, self.world
        (b0, b1), (p0, p1) = kv_block_range(total_positions, W, self.rank)
        cs, ci = b.shard_candidates(b0, b1)
        R = b.rows
        if R % W == 0:                                        # every rank merges its own rows
            r0, r1 = shard_range(R, W, self.rank)
            sel, nsel = b.merge_candidates(self._rows_to_owners(cs, r0, r1), self._rows_to_owners(ci, r0, r1), r0, r1)
            b.set_selection(self._all_gather(sel).reshape(R, -1), self._all_gather(nsel).reshape(R))
            out = b.merge_partials(self._rows_to_owners(b.shard_attn(p0, p1), r0, r1), r0, r1)
            return self._all_gather(out).reshape((R,) + tuple(out.shape[1:]))
        sel, nsel = b.merge_candidates(self._all_gather(cs), self._all_gather(ci), 0, R)      # every rank merges every row
        b.set_selection(sel, nsel)
        return b.merge_partials(self._all_gather(b.shard_attn(p0, p1)), 0, R)


def run_emulated_ranks(backend, world, total_positions):
    """The exchange of SplitKvQsa.run with the ranks played one after the other by ONE process on one device (tests and
    single-GPU checks): every rank's candidates, the merges of every rank's rows, every rank's partials, the merges of
    every rank's rows."""
    import torch
    R = backend.rows
    ranges = [kv_block_range(total_positions, world, r) for r in range(world)]
    rows = [shard_range(R, world, r) for r in range(world)]
    cands = [backend.shard_candidates(b0, b1) for (b0, b1), _ in ranges]
    cs, ci = torch.stack([c[0] for c in cands]), torch.stack([c[1] for c in cands])
    merged = [backend.merge_candidates(cs[:, r0:r1].contiguous(), ci[:, r0:r1].contiguous(), r0, r1) for r0, r1 in rows if r1 > r0]
    backend.set_selection(torch.cat([m[0] for m in merged]), torch.cat([m[1] for m in merged]))
    parts = torch.stack([backend.shard_attn(p0, p1).clone() for _, (p0, p1) in ranges])
    return torch.cat([backend.merge_partials(parts[:, r0:r1].contiguous(), r0, r1).clone() for r0, r1 in rows if r1 > r0])


class CudaQsaBackend:
    """The C-ABI calls behind SplitKvQsa for one prepared part: `args` is the cr_qsa_args of the part (queries
    normalised, caches holding the part); `out` [rows, Hq * 256] receives the output rows."""

    def __init__(self, geometry, args, rows, fmt, out):
        import torch
        from . import capi
        self.capi, self.torch, self.g, self.rows, self.fmt, self.out = capi, torch, geometry, rows, fmt, out
        self.args = args
        self.arr = (capi.QsaArgs * 1)(args)
        self.scratch = torch.empty(rows * geometry.q_heads * 32 * 258 * 4, dtype=torch.uint8, device="cuda")
        self.sel = torch.zeros(rows, 512, device="cuda", dtype=torch.int32)        # the part's selection, wherever it was merged
        self.nsel = torch.zeros(rows, device="cuda", dtype=torch.int32)

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _rows_args(self, r0, r1):
        """The argument block of the rows [r0, r1): the same buffers, row pointers moved to row r0."""
        capi, g = self.capi, self.g
        a = capi.QsaArgs.from_buffer_copy(self.args)
        esz = self.out.element_size()
        a.q += r0 * g.q_heads * 512 * 4; a.idx += r0 * 640 * 4
        a.k += r0 * g.kv_heads * 256 * 4; a.v += r0 * g.kv_heads * 256 * 4
        if a.scores:
            a.scores += r0 * a.sstride * 4
        a.sel, a.nsel = self.sel.data_ptr() + r0 * 512 * 4, self.nsel.data_ptr() + r0 * 4
        a.out = self.out.data_ptr() + r0 * g.q_heads * 256 * esz
        a.pos0 += r0; a.R = r1 - r0
        return (capi.QsaArgs * 1)(a)

    def shard_candidates(self, b0, b1):
        """Scores of the rank's own blocks [b0, b1), then its best 512 per row."""
        t = self.torch
        cs = t.empty(self.rows, 512, device="cuda"); ci = t.empty(self.rows, 512, device="cuda", dtype=t.int32)
        self.capi.check(self.capi.lib.cr_qsa_shard_select(C.byref(self.g), self.arr, b0, b1, cs.data_ptr(), ci.data_ptr(), self._stream()))
        return cs, ci

    def merge_candidates(self, scores, ids, r0, r1):
        self.capi.check(self.capi.lib.cr_qsa_merge_candidates(C.byref(self.g), self._rows_args(r0, r1), scores.shape[0], scores.data_ptr(),
                                                                ids.data_ptr(), self._stream()))
        return self.sel[r0:r1], self.nsel[r0:r1]

    def set_selection(self, sel, nsel):
        """The global selection into the buffers the part's argument block names."""
        capi, t = self.capi, self.torch
        if sel.data_ptr() != self.sel.data_ptr():
            self.sel.copy_(sel); self.nsel.copy_(nsel)
        a = capi.QsaArgs.from_buffer_copy(self.args)
        a.sel, a.nsel = self.sel.data_ptr(), self.nsel.data_ptr()
        self.args = a
        self.arr = (capi.QsaArgs * 1)(a)

    def shard_attn(self, p0, p1):
        parts = self.torch.empty(self.rows, self.g.q_heads, 258, device="cuda")
        self.capi.check(self.capi.lib.cr_qsa_shard_attn(C.byref(self.g), self.arr, p0, min(p1, 2 ** 31 - 1), parts.data_ptr(),
                                                          self.scratch.data_ptr(), self.scratch.numel(), self._stream()))
        return parts

    def merge_partials(self, parts, r0, r1):
        self.capi.check(self.capi.lib.cr_qsa_merge_partials(C.byref(self.g), self._rows_args(r0, r1), parts.shape[0], parts.data_ptr(), self.fmt,
                                                              self._stream()))
        return self.out[r0:r1]
