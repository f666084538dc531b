"""Multi-GPU partitioning of the attention path: one process per GPU, torch.distributed for the exchange.

Natural shards need no exchange: sessions (decode / verify) and sequences (prefill) are independent, GDN value
heads are independent recurrences (GdnHeadShard).  One long sequence of the QSA layer is split over the KV positions:

    rank g owns positions [lo_g, hi_g)  (whole 4-token blocks; the newest rows belong to the last rank)
    1. local scores + top-512 candidates over the owned blocks          cr_qsa_shard_select
    2. all-gather candidates [ranks][rows][512] (score, id)             -> every rank: cr_qsa_merge_candidates
    3. attention over the owned part of the attended positions          cr_qsa_shard_attn -> (m, l, acc[256])
    4. all-gather partials [ranks][rows][heads][258]                    -> cr_qsa_merge_partials (LSE merge + gate)

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
    ranks of `group`.  backend: object with shard_candidates(b0, b1) -> (scores [R,512] f32, ids [R,512] i32),
    merge_candidates(all_scores [W,R,512], all_ids), shard_attn(p0, p1) -> partials [R,Hq,258],
    merge_partials(all_partials [W,R,Hq,258]) -> output; tensors are torch tensors on the backend's device."""

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

    def run(self, total_positions):
        """total_positions = pos0 + R (positions in the cache after this part).  Returns the gated output rows."""
        (b0, b1), (p0, p1) = kv_block_range(total_positions, self.world, self.rank)
        cs, ci = self.backend.shard_candidates(b0, b1)
        self.backend.merge_candidates(self._all_gather(cs), self._all_gather(ci))
        parts = self.backend.shard_attn(p0, p1)
        return self.backend.merge_partials(self._all_gather(parts))


def run_emulated_ranks(backend, world, total_positions):
    """The exchange of SplitKvQsa.run with the ranks played one after the other by ONE process on one device (tests and
    single-GPU checks): every rank's candidates, one merge, every rank's partials, one merge."""
    import torch
    ranges = [kv_block_range(total_positions, world, r) for r in range(world)]
    cands = [backend.shard_candidates(b0, b1) for (b0, b1), _ in ranges]
    backend.merge_candidates(torch.stack([c[0] for c in cands]), torch.stack([c[1] for c in cands]))
    parts = [backend.shard_attn(p0, p1).clone() for _, (p0, p1) in ranges]
    return backend.merge_partials(torch.stack(parts))


class CudaQsaBackend:
    """The C-ABI calls behind SplitKvQsa for one prepared part: `args` is the cr_qsa_args of the part (scores
    already computed for the owned blocks by cr_qsa_select or cr_qsa_prefill's score stage)."""

    def __init__(self, geometry, args, rows, fmt, out):
        import torch
        from . import capi
        self.capi, self.torch, self.g, self.rows, self.fmt, self.out = capi, torch, geometry, rows, fmt, out
        self.arr = (capi.QsaArgs * 1)(args)
        self.scratch = torch.empty(rows * geometry.q_heads * 32 * 258 * 4, dtype=torch.uint8, device="cuda")

    def _stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def shard_candidates(self, b0, b1):
        """Scores of the rank's own blocks [b0, b1), then its best 512 per row."""
        t = self.torch
        cs = t.empty(self.rows, 512, device="cuda"); ci = t.empty(self.rows, 512, device="cuda", dtype=t.int32)
        self.capi.check(self.capi.lib.cr_qsa_shard_select(C.byref(self.g), self.arr, b0, b1, cs.data_ptr(), ci.data_ptr(), self._stream()))
        return cs, ci

    def merge_candidates(self, all_scores, all_ids):
        self.capi.check(self.capi.lib.cr_qsa_merge_candidates(C.byref(self.g), self.arr, all_scores.shape[0], all_scores.data_ptr(),
                                                                all_ids.data_ptr(), self._stream()))

    def shard_attn(self, p0, p1):
        parts = self.torch.empty(self.rows, self.g.q_heads, 258, device="cuda")
        self.capi.check(self.capi.lib.cr_qsa_shard_attn(C.byref(self.g), self.arr, p0, min(p1, 2 ** 31 - 1), parts.data_ptr(),
                                                          self.scratch.data_ptr(), self.scratch.numel(), self._stream()))
        return parts

    def merge_partials(self, all_parts):
        self.capi.check(self.capi.lib.cr_qsa_merge_partials(C.byref(self.g), self.arr, all_parts.shape[0], all_parts.data_ptr(), self.fmt,
                                                              self._stream()))
        return self.out
