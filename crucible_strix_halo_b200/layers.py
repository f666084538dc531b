"""Torch-tensor wrappers over the C ABI: they own device buffers the way the engine's SequenceState does
(engine/runtime/sequence_state.h:84-112) and fill the argument structs of include/crucible_attn.h.
Plumbing only: every computation happens in libcrucible_attn.so."""
import ctypes as C

import torch

from . import capi
from .capi import (GdnArgs, GdnPrefillArgs, QsaArgs, QsaCache, QsaPrefillArgs, Geometry, check, dptr, lib)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _out_dtype(fmt):
    return {capi.OUT_RAW_F32: torch.float32, capi.OUT_RAW_BF16: torch.bfloat16, capi.OUT_EXL3_WHT: torch.float16}[fmt]


class GdnWeights:
    """Per-layer constants of a GDN layer (struct Gdn, engine/model/flashnext/model.h:60-70)."""

    def __init__(self, g: Geometry, conv, A_log, dt_bias, gamma, ab=None, suh=None, device="cuda"):
        f = dict(device=device, dtype=torch.float32)
        self.g = g
        self.conv = torch.as_tensor(conv).to(**f).contiguous()          # [channels][4]
        self.A_log = torch.as_tensor(A_log).to(**f).contiguous()
        self.dt_bias = torch.as_tensor(dt_bias).to(**f).contiguous()
        self.gamma = torch.as_tensor(gamma).to(**f).contiguous()
        self.ab = None if ab is None else torch.as_tensor(ab).to(device=device, dtype=torch.float16).contiguous()
        self.suh = None if suh is None else torch.as_tensor(suh).to(device=device, dtype=torch.float16).contiguous()


class GdnSession:
    """Per-sequence GDN buffers: state (+64 scale floats), 16-row raw ring, pending rows."""

    def __init__(self, g: Geometry, pend_rows=8, device="cuda"):
        self.g, self.pend_rows = g, pend_rows
        self.state = torch.zeros(g.gdn_vheads * 128 * 128 + 64, device=device, dtype=torch.float32)
        self.hist = torch.zeros(16, g.gdn_channels, device=device, dtype=torch.float32)
        self.pend = torch.zeros(g.gdn_vheads, pend_rows, capi.PEND_FLOATS, device=device, dtype=torch.float32)

    def state_view(self):
        return self.state[:self.g.gdn_vheads * 16384].view(self.g.gdn_vheads, 128, 128)


def _gdn_args(w: GdnWeights, s: GdnSession, qkv, z, x, out, pos0, R, replay, commit, pack_rows=0, pack_off=0):
    return GdnArgs(dptr(qkv), dptr(z), dptr(x), dptr(w.ab), dptr(w.conv), dptr(w.A_log), dptr(w.dt_bias),
                   dptr(w.gamma), dptr(s.hist), dptr(s.state), dptr(w.suh), dptr(out), dptr(s.pend),
                   pos0, R, replay, commit, pack_rows, pack_off)


def gdn_step(w: GdnWeights, spans, fmt=capi.OUT_RAW_F32, outs=None):
    """spans: list of dicts(session, qkv [R,C] f32, z [R,Hv*128] f32, x [R,hidden] f32, pos0, replay, commit).
    One launch for all spans (LaunchGdnCore / packed verify).  Returns the list of outputs [R, Hv*128]."""
    g = w.g
    given, outs, arr = outs, [], (GdnArgs * len(spans))()
    pend_rows = spans[0]["session"].pend_rows
    for i, sp in enumerate(spans):
        R = sp["qkv"].shape[0]
        out = given[i] if given is not None else torch.empty(R, g.gdn_vheads * 128, device=sp["qkv"].device, dtype=_out_dtype(fmt))
        outs.append(out)
        arr[i] = _gdn_args(w, sp["session"], sp["qkv"], sp["z"], sp["x"], out, sp["pos0"], R,
                           sp.get("replay", 0), sp.get("commit", R))
    check(lib.cr_gdn_step(C.byref(g), arr, len(spans), pend_rows, fmt, _stream()))
    return outs


class GdnPrefillPlan:
    """Workspace + argument block for repeated prefill calls of a fixed row count."""

    def __init__(self, w: GdnWeights, rows, in_dtype=capi.IN_F32, fmt=capi.OUT_RAW_F32, raw_y=False, device="cuda"):
        self.w, self.rows, self.in_dtype, self.fmt = w, rows, in_dtype, fmt
        nbytes = lib.cr_gdn_prefill_workspace_bytes(C.byref(w.g), rows)
        self.workspace = torch.empty(nbytes, device=device, dtype=torch.uint8)
        self.out = torch.empty(rows, w.g.gdn_vheads * 128, device=device, dtype=_out_dtype(fmt))
        self.raw_y = torch.empty(rows, w.g.gdn_vheads * 128, device=device, dtype=torch.float32) if raw_y else None

    def run(self, s: GdnSession, qkv, z, ab_logits, pos0, algo=capi.GDN_SERIAL_F32):
        R = qkv.shape[0]
        assert R == self.rows
        a = GdnPrefillArgs(_gdn_args(self.w, s, qkv, z, None, self.out, pos0, R, 0, R), dptr(ab_logits), self.in_dtype,
                           dptr(self.workspace), self.workspace.numel(), dptr(self.raw_y))
        check(lib.cr_gdn_prefill(C.byref(self.w.g), C.byref(a), algo, self.fmt, _stream()))
        return self.out


class QsaWeights:
    """Per-layer constants of a QSA layer: (1 + w) norm vectors, RoPE table, optional suh."""

    def __init__(self, g: Geometry, q_norm1, k_norm1, iq_norm1, ik_norm1, suh=None, device="cuda", rope_factor=1):
        f = dict(device=device, dtype=torch.float32)
        self.g = g
        self.q_norm1 = torch.as_tensor(q_norm1).to(**f).contiguous()
        self.k_norm1 = torch.as_tensor(k_norm1).to(**f).contiguous()
        self.iq_norm1 = torch.as_tensor(iq_norm1).to(**f).contiguous()
        self.ik_norm1 = torch.as_tensor(ik_norm1).to(**f).contiguous()
        self.suh = None if suh is None else torch.as_tensor(suh).to(device=device, dtype=torch.float16).contiguous()
        self.rope = torch.empty(64, **f)
        check(lib.cr_rope_table_fill_yarn(dptr(self.rope), rope_factor, _stream()))   # factor 1: the plain table
        torch.cuda.current_stream().synchronize()


class QsaSession:
    """Per-sequence, per-layer QSA cache (struct QsaCache, engine/layers/ops.h:407-413) and selection buffers."""

    def __init__(self, g: Geometry, ctx, max_rows=13, device="cuda", raw_slots=0):
        self.g, self.ctx, self.raw_slots = g, ctx, raw_slots
        self.k = torch.zeros(ctx, g.kv_heads, 256, device=device, dtype=torch.float16)
        self.v = torch.zeros(ctx, g.kv_heads, 256, device=device, dtype=torch.float16)
        self.ik_raw = torch.zeros(raw_slots if raw_slots else ctx, 128, device=device, dtype=torch.float32)
        self.ik_pool = torch.zeros(lib.cr_qsa_pool_floats(ctx), device=device, dtype=torch.float32)
        self.sstride = (ctx + 3) // 4
        self.scores = torch.zeros(max_rows, self.sstride, device=device, dtype=torch.float32)
        self.sel = torch.zeros(max_rows, capi.SEL_BLOCKS, device=device, dtype=torch.int32)
        self.nsel = torch.zeros(max_rows, device=device, dtype=torch.int32)

    def cache_struct(self):
        return QsaCache(dptr(self.k), dptr(self.v), dptr(self.ik_raw), dptr(self.ik_pool), self.raw_slots)

    def pool_rows(self, nb):
        """Pooled keys of blocks [0, nb) as [nb, 128] (un-tiled view, for tests)."""
        return self.ik_pool.view(-1, 128, 32).transpose(1, 2).reshape(-1, 128)[:nb]


def qsa_args(w: QsaWeights, s: QsaSession, q, k, v, idx, out, pos0, context=None, pack_rows=0, pack_off=0, mrope=None):
    R = q.shape[0]
    return QsaArgs(dptr(q), dptr(k), dptr(v), dptr(idx), dptr(w.q_norm1), dptr(w.k_norm1), dptr(w.iq_norm1),
                   dptr(w.ik_norm1), s.cache_struct(), dptr(s.scores), s.sstride, dptr(s.sel), dptr(s.nsel),
                   dptr(w.suh), dptr(out), pos0, R, dptr(context), pack_rows, pack_off, dptr(mrope), dptr(w.rope))


class QsaStepPlan:
    """Scratch + outputs for batched decode / verify steps (cr_qsa_step over spans)."""

    def __init__(self, w: QsaWeights, total_rows, fmt=capi.OUT_RAW_F32, device="cuda"):
        self.w, self.fmt = w, fmt
        n = lib.cr_qsa_scratch_bytes(C.byref(w.g), total_rows)
        self.scratch = torch.zeros(n, device=device, dtype=torch.uint8)

    def run(self, spans, want_context=False, outs=None):
        """spans: list of dicts(session, q [R,Hq,512] f32 (modified in place), k, v [R,Hkv*256], idx [R,640], pos0)."""
        g = self.w.g
        arr = (QsaArgs * len(spans))()
        given, outs, ctxs = outs, [], []
        for i, sp in enumerate(spans):
            R = sp["q"].shape[0]
            out = given[i] if given is not None else torch.empty(R, g.q_heads * 256, device=sp["q"].device, dtype=_out_dtype(self.fmt))
            ctx = torch.empty(R, g.q_heads, 256, device=sp["q"].device, dtype=torch.float32) if want_context else None
            outs.append(out)
            ctxs.append(ctx)
            arr[i] = qsa_args(self.w, sp["session"], sp["q"], sp["k"], sp["v"], sp["idx"], out, sp["pos0"], ctx)
        check(lib.cr_qsa_step(C.byref(g), arr, len(spans), dptr(self.scratch), self.scratch.numel(), self.fmt, _stream()))
        return (outs, ctxs) if want_context else outs


class QsaPrefillPlan:
    """Scratch + outputs for prefill parts of up to `rows` rows (cr_qsa_prefill)."""

    def __init__(self, w: QsaWeights, rows, fmt=capi.OUT_RAW_F32, device="cuda"):
        self.w, self.rows, self.fmt = w, rows, fmt
        g = w.g
        self.scratch = torch.empty(lib.cr_qsa_prefill_scratch_bytes(C.byref(g), rows), device=device, dtype=torch.uint8)
        self.q_hi = torch.empty(rows, g.q_heads, 256, device=device, dtype=torch.float16)
        self.out = torch.empty(rows, g.q_heads * 256, device=device, dtype=_out_dtype(fmt))

    def run(self, s: QsaSession, q, k, v, idx, pos0, skip=0, context=None):
        R = q.shape[0]
        assert R <= self.rows and s.scores.shape[0] >= R
        a = QsaPrefillArgs(qsa_args(self.w, s, q, k, v, idx, self.out, pos0, context), dptr(self.q_hi),
                           dptr(self.scratch), self.scratch.numel())
        check(lib.cr_qsa_prefill(C.byref(self.w.g), C.byref(a), skip, self.fmt, _stream()))
        return self.out[:R]


def checkpoint_spans(gdn_sessions, qsa_sessions, position):
    """The spans an in-slot checkpoint at `position` holds, in the reference's order (SlotCheckpointIO::Spans,
    engine/runtime/slot_checkpoint_io.h:14-26 over VisitFixedState, engine/model/flashnext/fixed_state.h:17-23):
    every GDN state, then every conv ring, then every pending-row buffer, then per QSA cache its compact raw ring and
    the 128-position pool tile that holds `position` when the position lies inside one."""
    tensors = [s.state for s in gdn_sessions] + [s.hist for s in gdn_sessions] + [s.pend for s in gdn_sessions]
    for s in qsa_sessions:
        if s.raw_slots:
            tensors.append(s.ik_raw)
        if position % 128:
            tensors.append(s.ik_pool[position // 128 * 4096:(position // 128 + 1) * 4096])
    return tensors


class SlotCheckpoint:
    """One device buffer that holds a list of spans (SlotCheckpointIO::Buffer, slot_checkpoint_io.h:33-48), filled and
    read back by cr_state_save / cr_state_restore."""

    def __init__(self, tensors, device="cuda"):
        self.tensors = tensors                                # keeps the views alive
        self.spans = (capi.Span * len(tensors))(*[capi.Span(t.data_ptr(), t.numel() * t.element_size()) for t in tensors])
        self.bytes = lib.cr_spans_bytes(self.spans, len(tensors))
        self.buffer = torch.empty(self.bytes, device=device, dtype=torch.uint8)

    def save(self):
        check(lib.cr_state_save(self.spans, len(self.tensors), dptr(self.buffer), self.bytes, _stream()))

    def restore(self):
        check(lib.cr_state_restore(self.spans, len(self.tensors), dptr(self.buffer), self.bytes, _stream()))


def proj_gemm(x, w, outs):
    """x [R, K] bf16, w [N, K] bf16 (out x in); outs: list of (tensor [R, cols] bf16 or fp32, contiguous rows) whose
    widths add up to N.  One cr_proj_gemm launch (the input or output GEMM group of a prefill layer)."""
    R, K = x.shape
    N = w.shape[0]
    arr = (capi.ProjOut * len(outs))()
    col = 0
    for i, o in enumerate(outs):
        cols = o.shape[-1] if o.dim() == 2 else o[0].numel()
        arr[i] = capi.ProjOut(o.data_ptr(), col, cols, cols, 1 if o.dtype == torch.float32 else 0)
        col += cols
    check(lib.cr_proj_gemm(dptr(x), dptr(w), R, K, N, arr, len(outs), _stream()))
    return outs
