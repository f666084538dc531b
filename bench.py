#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input.  Workloads:
  gdn_prefill_32k     one Gated DeltaNet layer, chunked prefill, batch 1, seq 32768, 16 QK x 128 / 32 V x 128 heads,
                      bf16 inputs, fp32 state (the headline: the config the metric is quoted on)
  decode_262k         QSA sparse attention decode + GDN recurrent update, 4 sessions x 262,144-token fp16 KV cache
  decode_262k_x16     the same step with 16 sessions per GPU (the dependent kernels' latency amortised)
  qsa_prefill_262k    one QSA layer, the last 2,048-row part of a 262,144-token prefill (scores, top-512, attention),
                      selections from the random indexer (nearly independent per row)
  qsa_attend_262k_drift  the attention stage of the same part with injected selections that drift from row to row
                      (a 512-block set, every member replaced with probability 0.25 per row), as real selections overlap
  verify_131k         speculative verify: 8 sessions x 131,072 context, 9-row spans (1 certain row + 8 drafts), QSA +
                      GDN with lazy commit, replay counts uniform 0..8
  prefill_262k_stack  long cold prefill of 262,144 tokens through a 3:1 stack of GDN:QSA layers (16,384-row launches, QSA in
                      2,048-row parts against the growing cache)
  gdn_in_proj_32k     the input projection of a GDN layer over 32,768 tokens (hidden 2048 -> qkv | z | a,b), one GEMM launch
With no --workload the line's headline is gdn_prefill_32k and a `workloads` object carries the figures of all of them
(shorter runs).  Under torchrun (N > 1) every rank runs the headline on its own sequence (weak scaling, no data-path
collective) and the `workloads` object carries qsa_prefill_262k_split_kv: ONE sequence whose KV positions are split
over the ranks, with all-to-alls of candidates and partials and all-gathers of selections and outputs over NCCL (strong scaling).  Time is the max over ranks.
Prints ONE JSON line (rank 0).  --impl reference times the CPU restatement of the reference's algorithm
(oracle/_build/liboracle.so) on the host cores, on a bounded sample of the same workload.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GDN_BYTES_PER_TOKEN = (8192 + 4096) * 2 + 4096 * 2 + 2 * 32 * 4      # bf16 qkv + z in, bf16 out, fp32 a/b logits
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch from the ncu captures summarised under
# profiles/, per unit of work (GDN: per token of a 7,104-token part; decode: per step of 4 sessions), scaled to
# the launch by the units it processes (traffic grows in proportion to them).
NCU_TRAFFIC = {
    "gdn_prefill_32k": {"gdn_chunk_scan_tc_kernel": ("token", (526.36e6 + 102.34e6) / 7104),
                        "gdn_chunk_local_kernel": ("token", (121.44e6 + 464.28e6) / 7104),
                        "gdn_gate_kernel": ("token", (174.63e6 + 37.16e6) / 7104)},
    "decode_262k": {"qsa_score_kernel": ("step", 134.25e6 + 3.57e6), "qsa_attn_split_kernel": ("step", 16.87e6),
                    "qsa_topk_cluster_kernel": ("step", 1.11e6), "qsa_merge_kernel": ("step", 2.21e6), "qsa_prep_kernel": ("step", 0.13e6),
                    "gdn_step_kernel": ("step", 9.47e6)},
    "qsa_prefill_262k": {"qsa_attn_split_kernel": ("step", 6737.66e6 + 135.26e6), "qsa_score_tc_kernel": ("step", 475.9e6),
                         "qsa_topk_kernel": ("step", 537.4e6 + 7.0e6)},
    "qsa_attend_262k_drift": {"qsa_flash_tc_kernel": ("step", 704.4e6 + 13.6e6)},
    "verify_131k": {"qsa_attn_split_kernel": ("step", 281.55e6 + 29.26e6), "gdn_step_kernel": ("step", 23.2e6)},
}
DECODE_BYTES_PER_SESSION = 65536 * 512 + 2051 * 2048 + 2 * 2097152   # pool scan + K/V gather + GDN state in/out


def load_peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.lines, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------------------

class GdnPrefill32k:
    """configs[1]: seeded qkv ~ N(0,1) bf16 [T,8192], z ~ N(0,1) [T,4096], conv ~ N(0,0.25), a/b logits ~ N(0,1),
    A_log ~ clamp(N(-1,1.5),-5,1.5), dt_bias ~ N(0,0.5), gamma = 1 + N(0,0.1); initial state 0."""
    name = "gdn_prefill_32k"
    T = 32768
    unit, metric, dtype = "tokens/s", "gdn_layer_prefill_tokens_per_s", "bf16 in / fp32 state"

    def __init__(self, rank, algo):
        import torch
        from crucible_strix_halo_b200 import capi, layers
        self.torch, self.capi, self.layers = torch, capi, layers
        g = capi.GEOM_BENCH
        gen = torch.Generator(device="cuda").manual_seed(1000 + rank)
        T, Cw = self.T, g.gdn_channels
        rn = lambda *s, std=1.0, mean=0.0: torch.randn(*s, device="cuda", generator=gen) * std + mean
        self.w = layers.GdnWeights(g, rn(Cw, 4, std=0.5), rn(32, std=1.5, mean=-1).clamp(-5, 1.5), rn(32, std=0.5), 1 + rn(128, std=0.1))
        self.qkv = rn(T, Cw).bfloat16()
        self.z = rn(T, 4096).bfloat16()
        self.ab = rn(T, 64)                                   # fp32 logits from the a/b GEMM
        self.ses = layers.GdnSession(g)
        self.plan = layers.GdnPrefillPlan(self.w, T, in_dtype=capi.IN_BF16, fmt=capi.OUT_RAW_BF16)
        self.algo = algo
        # the a/b logits are read as bf16-or-fp32 by in_dtype: keep them in the input dtype
        self.ab_in = self.ab.bfloat16()
        self.units_per_step = T
        self.alg_bytes = GDN_BYTES_PER_TOKEN * T
        # host copies for the end-to-end leg
        self.h_qkv = self.qkv.cpu().pin_memory(); self.h_z = self.z.cpu().pin_memory(); self.h_ab = self.ab_in.cpu().pin_memory()
        self.h_out = torch.empty(T, 4096, dtype=torch.bfloat16).pin_memory()
        self.h2d = self.h_qkv.numel() * 2 + self.h_z.numel() * 2 + self.h_ab.numel() * 2
        self.d2h = self.h_out.numel() * 2
        # the layer's algorithmic bytes are charged to its longest kernel (the scan or the local kernel)
        self.kernel_bytes = {}
        self.launches_per_step = 4 if algo == capi.GDN_SERIAL_F32 else 5

    def step(self):
        self.ses.state.zero_()
        return self.plan.run(self.ses, self.qkv, self.z, self.ab_in, 0, self.algo)

    step_eager = step

    PIECE = 4736                                            # rows per host piece (each piece is a single-part call)

    def _e2e_setup(self):
        torch = self.torch
        self.s_in = [torch.cuda.Stream()]                    # one copy stream saturates PCIe (two or three measured 3-5 % slower)
        self.s_out = torch.cuda.Stream()
        self.piece_plans = [self.layers.GdnPrefillPlan(self.w, self.PIECE, in_dtype=self.capi.IN_BF16, fmt=self.capi.OUT_RAW_BF16)
                            for _ in range(2)]
        n = (self.T + self.PIECE - 1) // self.PIECE
        self.ev_in = [torch.cuda.Event() for _ in range(n)]
        self.ev_c = [torch.cuda.Event() for _ in range(n)]
        self.ev_out = [torch.cuda.Event() for _ in range(n)]

    def step_e2e(self):
        """Host buffers in, host buffer out, as a caller with a long prompt would drive the C ABI: the rows go to
        the device in pieces on a copy stream, each piece is one cr_gdn_prefill call (the state carries), and its
        output returns on a third stream, so the PCIe transfers in both directions overlap the kernels."""
        torch = self.torch
        if not hasattr(self, "s_in"):
            self._e2e_setup()
        cur = torch.cuda.current_stream()
        self.ses.state.zero_()
        for st in self.s_in:
            st.wait_stream(cur)
        self.s_out.wait_stream(cur)
        for i, p0 in enumerate(range(0, self.T, self.PIECE)):
            n = min(self.PIECE, self.T - p0)
            sl = slice(p0, p0 + n)
            with torch.cuda.stream(self.s_in[i % len(self.s_in)]):
                self.qkv[sl].copy_(self.h_qkv[sl], non_blocking=True)
                self.z[sl].copy_(self.h_z[sl], non_blocking=True)
                self.ab_in[sl].copy_(self.h_ab[sl], non_blocking=True)
                self.ev_in[i].record()
            cur.wait_event(self.ev_in[i])
            if i >= 2:
                cur.wait_event(self.ev_out[i - 2])             # the output buffer of this plan has been read back
            plan = self.piece_plans[i & 1]
            if n == self.PIECE:
                out = plan.run(self.ses, self.qkv[sl], self.z[sl], self.ab_in[sl], p0, self.algo)
            else:
                if not hasattr(self, "tail_plan"):
                    self.tail_plan = self.layers.GdnPrefillPlan(self.w, n, in_dtype=self.capi.IN_BF16, fmt=self.capi.OUT_RAW_BF16)
                out = self.tail_plan.run(self.ses, self.qkv[sl], self.z[sl], self.ab_in[sl], p0, self.algo)
            self.ev_c[i].record()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_c[i])
                self.h_out[sl].copy_(out, non_blocking=True)
                self.ev_out[i].record()
        cur.wait_stream(self.s_out)

    def config(self):
        return {"workload": self.name, "seq_len": self.T, "gdn_heads": "16qk/32v x128", "chunk": 64, "sessions_per_gpu": 1,
                "algo": {0: "serial_f32", 1: "chunk64_tcgen05"}[self.algo],
                "l2": "inputs (0.8 GB per step) exceed the 126 MB L2"}


class Decode262k:
    """configs[2]: 4 sessions, each a 262,144-token fp16 KV cache (K,V ~ N(0,1)), pooled keys from raw keys ~ N(0,1),
    one new token per step (q,k,v,idx ~ N(0,1)), 16/2 GQA, plus the GDN update of a 32x128x128 fp32 state."""
    name = "decode_262k"
    CTX, SESSIONS = 262144, 4
    unit, metric, dtype = "tokens/s", "qsa_gdn_decode_tokens_per_s", "fp16 kv / fp32"

    def __init__(self, rank, algo):
        import torch
        from crucible_strix_halo_b200 import capi, layers
        self.torch, self.capi, self.layers = torch, capi, layers
        g = capi.GEOM_BENCH
        gen = torch.Generator(device="cuda").manual_seed(2000 + rank)
        rn = lambda *s, std=1.0, mean=0.0: torch.randn(*s, device="cuda", generator=gen) * std + mean
        self.qw = layers.QsaWeights(g, 1 + rn(256, std=0.1), 1 + rn(256, std=0.1), 1 + rn(128, std=0.1), 1 + rn(128, std=0.1))
        self.gw = layers.GdnWeights(g, rn(g.gdn_channels, 4, std=0.5), rn(32, std=1.5, mean=-1).clamp(-5, 1.5), rn(32, std=0.5),
                                    1 + rn(128, std=0.1), ab=rn(64, 2048, std=0.05))
        self.pos = self.CTX - 1                                 # the new token completes the cache
        S = self.SESSIONS
        # one contiguous block of projection rows per step (what the engine's GEMMs would write), with views per session
        sizes = dict(q=16 * 512, idx=640, k=512, v=512, qkv=g.gdn_channels, z=4096, x=2048)   # q and idx adjacent: one work copy
        width = sum(sizes.values())
        self.inp_all = rn(S, width)
        self.qs, self.gs, self.inp = [], [], []
        for s in range(S):
            q = layers.QsaSession(g, self.CTX, max_rows=1)
            q.k.copy_(rn(self.CTX, 2, 256).half()); q.v.copy_(rn(self.CTX, 2, 256).half())
            q.ik_pool.copy_(rn(q.ik_pool.numel()))              # pooled keys: unit-RMS rows, tiled layout
            q.ik_raw.copy_(rn(self.CTX, 128))
            gs = layers.GdnSession(g)
            gs.state[:32 * 16384].copy_(rn(32 * 16384, std=0.05))
            self.qs.append(q); self.gs.append(gs)
            views, off = {}, 0
            for name, n in sizes.items():
                views[name] = self.inp_all[s, off:off + n].view(1, 16, 512) if name == "q" else self.inp_all[s, off:off + n].view(1, n)
                off += n
            self.inp.append(views)
        # q and idx are normalised in place by the step: they are copied to work buffers first
        self.qi_work = torch.empty(S, 8192 + 640, device="cuda")
        self.q_work = [self.qi_work[s, :8192].view(1, 16, 512) for s in range(S)]
        self.idx_work = [self.qi_work[s, 8192:].view(1, 640) for s in range(S)]
        self.plan = layers.QsaStepPlan(self.qw, S)
        self.units_per_step = S
        self.alg_bytes = DECODE_BYTES_PER_SESSION * S
        self.h_in = self.inp_all.cpu().pin_memory()
        self.out_all = torch.empty(S, 2, 4096, device="cuda")
        self.h_out = torch.empty(S, 2, 4096).pin_memory()
        self.h2d = self.h_in.numel() * 4
        self.d2h = self.h_out.numel() * 4
        # per-kernel algorithmic bytes: pool scan; K/V gather; GDN state in + out; scores read by the select
        self.kernel_bytes = {"qsa_score_kernel": 65536 * 512 * S, "qsa_attn_split_kernel": 2051 * 2048 * S,
                             "gdn_step_kernel": 2 * 2097152 * S, "qsa_topk_cluster_kernel": 65536 * 4 * S}
        self.side = torch.cuda.Stream()
        self.graph = None
        self.graph_e2e = None

    def _work_copies(self):
        self.qi_work.copy_(self.inp_all[:, :8192 + 640])

    def _qsa(self, in_place=False):
        # in_place: q and idx are normalised where they arrived (fresh every step on the host-buffer leg)
        spans = [dict(session=self.qs[s], q=self.inp[s]["q"] if in_place else self.q_work[s], k=self.inp[s]["k"], v=self.inp[s]["v"],
                      idx=self.inp[s]["idx"] if in_place else self.idx_work[s], pos0=self.pos) for s in range(self.SESSIONS)]
        return self.plan.run(spans, outs=[self.out_all[s, 0:1] for s in range(self.SESSIONS)])

    def _gdn(self):
        return self.layers.gdn_step(self.gw, [dict(session=self.gs[s], qkv=self.inp[s]["qkv"], z=self.inp[s]["z"], x=self.inp[s]["x"],
                                                   pos0=self.pos) for s in range(self.SESSIONS)],
                                    outs=[self.out_all[s, 1:2] for s in range(self.SESSIONS)])

    def step_eager(self, parallel=True, in_place=False):
        torch = self.torch
        if not in_place:
            self._work_copies()
        cur = torch.cuda.current_stream()
        if parallel:                              # the GDN layer does not depend on the QSA layer: a parallel branch
            self.side.wait_stream(cur)
            with torch.cuda.stream(self.side):
                go = self._gdn()
            qo = self._qsa(in_place)
            cur.wait_stream(self.side)
        else:
            qo = self._qsa(in_place)
            go = self._gdn()
        return self.out_all

    def step_profile(self):
        return self.step_eager(parallel=False)    # one stream, so consecutive events bracket single kernels

    def step(self):
        """One decode step of all sessions, replayed from a CUDA graph."""
        torch = self.torch
        if self.graph is None:
            for _ in range(2):
                self.step_eager()
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.step_eager()
        self.graph.replay()
        return self.out_all

    def step_e2e(self):
        """Host buffers in, host buffer out: the step's rows are copied from pinned memory, the kernels run from a
        graph that normalises q and idx where they landed (they are fresh every step), the outputs are copied back.
        (Copy nodes inside the graph measured slower than the two plain asynchronous copies: 107 us against 99.)"""
        torch = self.torch
        if self.graph_e2e is None:
            for _ in range(2):
                self.step_eager(in_place=True)
            torch.cuda.synchronize()
            self.graph_e2e = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph_e2e):
                self.step_eager(in_place=True)
        self.inp_all.copy_(self.h_in, non_blocking=True)
        self.graph_e2e.replay()
        self.h_out.copy_(self.out_all, non_blocking=True)

    def config(self):
        return {"workload": self.name, "sessions_per_gpu": self.SESSIONS, "context": self.CTX, "qsa_heads": "16q/2kv x256",
                "block": 4, "top_k_blocks": 512, "gdn_state": "32x128x128 fp32",
                "l2": "per-step traffic (%d MB) exceeds the 126 MB L2" % (self.alg_bytes // 1000000)}


class Decode262kX16(Decode262k):
    """The same step with 16 sessions per GPU: the latency of the dependent kernels behind the pool scan is shared by
    four times the bytes, which shows the HBM fraction the kernels reach once it is amortised."""
    name = "decode_262k_x16"
    SESSIONS = 16


class QsaPrefill262k:
    """The last 2,048-row part of a 262,144-token prefill of one QSA layer (configs[3], attention stage with i.i.d.
    selections): cache K,V fp16 ~ N(0,1) and pooled keys ~ N(0,1) for positions < 260,096; the part's rows
    q [R,16,512], k,v [R,512], idx [R,640] ~ N(0,1) fp32.  Per row: scores over up to 65,536 blocks, exact top-512,
    attention over 2,051 positions for 16 heads; all rows are causal within the part."""
    name = "qsa_prefill_262k"
    POS0, R = 262144 - 2048, 2048
    unit, metric, dtype = "tokens/s", "qsa_layer_prefill_tokens_per_s_at_262k", "fp16 kv / fp32 q / fp16x2 tensor-core products"

    def __init__(self, rank, algo):
        import torch
        from crucible_strix_halo_b200 import capi, layers
        self.torch, self.capi, self.layers = torch, capi, layers
        g = capi.GEOM_BENCH
        gen = torch.Generator(device="cuda").manual_seed(3000 + rank)
        rn = lambda *s, std=1.0: torch.randn(*s, device="cuda", generator=gen) * std
        R, ctx = self.R, self.POS0 + self.R
        self.w = layers.QsaWeights(g, 1 + rn(256, std=0.1), 1 + rn(256, std=0.1), 1 + rn(128, std=0.1), 1 + rn(128, std=0.1))
        self.ses = layers.QsaSession(g, ctx, max_rows=R)
        self.ses.k.copy_(rn(ctx, 2, 256).half()); self.ses.v.copy_(rn(ctx, 2, 256).half())
        self.ses.ik_pool.copy_(rn(self.ses.ik_pool.numel())); self.ses.ik_raw.copy_(rn(ctx, 128))
        self.plan = layers.QsaPrefillPlan(self.w, R, fmt=capi.OUT_RAW_BF16)
        self.inp = {"q": rn(R, 16, 512), "k": rn(R, 512), "v": rn(R, 512), "idx": rn(R, 640)}     # the part's projection rows
        self.work = {n: torch.empty_like(t) for n, t in self.inp.items() if n in ("q", "idx")}    # normalised in place: a fresh copy per step
        self.h_in = {n: t.cpu().pin_memory() for n, t in self.inp.items()}
        self.h_out = torch.empty(R, 4096, dtype=torch.bfloat16).pin_memory()
        self.h2d, self.d2h = sum(t.numel() * 4 for t in self.h_in.values()), self.h_out.numel() * 2
        self.units_per_step = R
        # gathered K/V rows of every query row + one pass over the pooled keys + the rows in and out
        self.alg_bytes = R * 2051 * 2048 + 65536 * 512 + self.h2d + self.d2h
        self.kernel_bytes = {"qsa_attn_split_kernel": R * 2051 * 2048, "qsa_flash_tc_kernel": R * 2051 * 2048}
        # useful flops: attention 4 * Hq * D * n per row + scoring 2 * 4 * 128 * nb per row
        self.alg_flops = R * (4 * 16 * 256 * 2051) + sum(1024 * ((self.POS0 + r + 1) // 4) for r in range(R))

    def _run(self):
        return self.plan.run(self.ses, self.work["q"], self.inp["k"], self.inp["v"], self.work["idx"], self.POS0)

    def step(self):
        for n, t in self.work.items():
            t.copy_(self.inp[n])
        return self._run()

    step_eager = step

    def step_e2e(self):
        for n, t in self.inp.items():
            (self.work[n] if n in self.work else t).copy_(self.h_in[n], non_blocking=True)
        self.h_out.copy_(self._run(), non_blocking=True)

    def config(self):
        return {"workload": self.name, "context": self.POS0 + self.R, "part_rows": self.R, "qsa_heads": "16q/2kv x256", "block": 4,
                "top_k_blocks": 512, "selections": "i.i.d. (random indexer)", "l2": "the K/V cache (0.5 GB) exceeds the 126 MB L2"}




def drift_selections(R, nb0, seed, drift=0.25):
    """Selections that drift from row to row: a 512-block set of which every member is replaced with probability
    `drift` per row by a block drawn uniformly from the nb0 complete blocks; ascending ids per row, [R, 512] int32."""
    rng = np.random.default_rng(seed)
    cur = np.sort(rng.choice(nb0, 512, replace=False))
    rows = np.empty((R, 512), np.int32)
    for r in range(R):
        keep = cur[rng.random(512) >= drift]
        while True:                                           # refill with fresh blocks until 512 distinct ones
            cur = np.union1d(keep, rng.integers(0, nb0, 512 - len(keep)))
            if len(cur) == 512:
                break
            keep = cur
        rows[r] = cur
    return rows


class QsaAttendDrift(QsaPrefill262k):
    """The attention stage of the same 2,048-row part (union lists + tiled attention + gate) with injected selections
    that overlap from row to row the way real selections do: the drift model of the reference's attention probe
    (512-block set, each member replaced with probability 0.25 per row; bench/qsa_attn.hip:46-90), generated here."""
    name = "qsa_attend_262k_drift"
    metric = "qsa_prefill_attention_stage_tokens_per_s_at_262k"

    def __init__(self, rank, algo):
        super().__init__(rank, algo)
        torch, capi, layers = self.torch, self.capi, self.layers
        R = self.R
        self.ses.sel.copy_(torch.from_numpy(drift_selections(R, (self.POS0 + 1) // 4, 3500 + rank)))
        self.ses.nsel.fill_(512)
        self.plan.q_hi.copy_(self.inp["q"][:, :, :256].half())
        self.args = capi.QsaPrefillArgs(layers.qsa_args(self.w, self.ses, self.inp["q"], self.inp["k"], self.inp["v"], self.inp["idx"], self.plan.out, self.POS0),
                                        capi.dptr(self.plan.q_hi), capi.dptr(self.plan.scratch), self.plan.scratch.numel())
        union = torch.unique(self.ses.sel[:16]).numel()
        self.union_16 = int(union)
        self.h_q = self.plan.q_hi.cpu().pin_memory()
        self.h2d, self.d2h = self.h_q.numel() * 2, self.h_out.numel() * 2
        # bytes: every block of a 16-row tile's union once per KV head pair (4 KB of K + V per block), rows in and out
        self.alg_bytes = (R // 16) * union * 2 * 4096 + self.h2d + self.d2h
        self.kernel_bytes = {"qsa_flash_tc_kernel": (R // 16) * union * 2 * 4096}
        self.alg_flops = R * (4 * 16 * 256 * 2051)

    def step(self):
        g = self.capi.GEOM_BENCH
        self.capi.check(self.capi.lib.cr_qsa_prefill_attend(C.byref(g), C.byref(self.args), 0, self.capi.OUT_RAW_BF16,
                                                            C.c_void_p(self.torch.cuda.current_stream().cuda_stream)))
        return self.plan.out

    step_eager = step

    def step_e2e(self):
        self.plan.q_hi.copy_(self.h_q, non_blocking=True)
        self.h_out.copy_(self.step(), non_blocking=True)

    def config(self):
        c = super().config()
        c.update(workload=self.name, selections="drift 0.25 per row (injected); a 16-row tile attends %d distinct blocks" % self.union_16)
        return c


class Verify131k:
    """configs[4]: 8 sessions at 131,072 context, each verifying 8 draft tokens: a span is 1 certain row + 8 drafts
    (commit = 1, 9 rows, pending-row stride 16), the pass before it accepted a ~ U{0..8} drafts, which this pass replays
    into the GDN state first.  QSA: one packed launch chain over the 8 spans (72 rows); GDN: one launch over 8 spans."""
    name = "verify_131k"
    CTX, SESSIONS, ROWS = 131072, 8, 9
    unit, metric, dtype = "rows/s", "qsa_gdn_verify_rows_per_s_at_131k", "fp16 kv / fp32"

    def __init__(self, rank, algo):
        import torch
        from crucible_strix_halo_b200 import capi, layers
        self.torch, self.capi, self.layers = torch, capi, layers
        g = capi.GEOM_BENCH
        gen = torch.Generator(device="cuda").manual_seed(5000 + rank)
        rn = lambda *s, std=1.0, mean=0.0: torch.randn(*s, device="cuda", generator=gen) * std + mean
        S, R = self.SESSIONS, self.ROWS
        self.qw = layers.QsaWeights(g, 1 + rn(256, std=0.1), 1 + rn(256, std=0.1), 1 + rn(128, std=0.1), 1 + rn(128, std=0.1))
        self.gw = layers.GdnWeights(g, rn(g.gdn_channels, 4, std=0.5), rn(32, std=1.5, mean=-1).clamp(-5, 1.5), rn(32, std=0.5),
                                    1 + rn(128, std=0.1), ab=rn(64, 2048, std=0.05))
        self.pos = self.CTX - R
        sizes = dict(q=16 * 512, idx=640, k=512, v=512, qkv=g.gdn_channels, z=4096, x=2048)
        self.inp = {n: rn(S, R, w_) for n, w_ in sizes.items()}                 # projection rows of the pass, one tensor per input
        self.work = {n: torch.empty_like(self.inp[n]) for n in ("q", "idx")}     # normalised in place: a fresh copy per step
        self.qs, self.gs = [], []
        for s in range(S):
            q = layers.QsaSession(g, self.CTX, max_rows=R)
            q.k.copy_(rn(self.CTX, 2, 256).half()); q.v.copy_(rn(self.CTX, 2, 256).half())
            q.ik_pool.copy_(rn(q.ik_pool.numel())); q.ik_raw.copy_(rn(self.CTX, 128))
            gs = layers.GdnSession(g, pend_rows=16)
            gs.state[:32 * 16384].copy_(rn(32 * 16384, std=0.05))
            gs.pend.copy_(rn(*gs.pend.shape, std=0.1))
            gs.pend[:, :, 256] = 0.5 + 0.5 * torch.rand(32, 16, device="cuda", generator=gen)      # decay
            gs.pend[:, :, 257] = torch.rand(32, 16, device="cuda", generator=gen)                  # beta
            self.qs.append(q); self.gs.append(gs)
        # accepted drafts of the previous pass per (step, session), uniform 0..8, seeded
        self.replays = torch.randint(0, 9, (16, S), generator=torch.Generator().manual_seed(5100 + rank)).tolist()
        self.t = 0
        self.graphs = {}
        self.plan = layers.QsaStepPlan(self.qw, S * R)
        self.out_all = torch.empty(S, 2, R, 4096, device="cuda")
        self.h_in = {n: t.cpu().pin_memory() for n, t in self.inp.items()}
        self.h_out = torch.empty(S, 2, R, 4096).pin_memory()
        self.h2d, self.d2h = sum(t.numel() * 4 for t in self.h_in.values()), self.h_out.numel() * 4
        self.units_per_step = S * R
        # per session-pass: one pool scan for all rows, the K/V rows of the union of the 9 rows' positions (upper bound:
        # 9 x 2051 rows; the rows of one span select nearly the same blocks, so about one row's worth is fetched from
        # DRAM), the GDN state in and out, pending rows in and out
        self.alg_bytes = S * (32768 * 512 + 2051 * 2048 + 2 * 2097152 + 2 * 32 * 8 * 258 * 4)
        self.kernel_bytes = {"qsa_score_kernel": 32768 * 512 * S, "gdn_step_kernel": 2 * 2097152 * S}
        self.side = torch.cuda.Stream()

    def _step(self, in_place=False, pattern=None):
        torch = self.torch
        S = self.SESSIONS
        if pattern is None:
            pattern = self.t % len(self.replays)
            self.t += 1
        replay = self.replays[pattern]
        if not in_place:
            for n, t in self.work.items():
                t.copy_(self.inp[n])
        cur = torch.cuda.current_stream()
        self.side.wait_stream(cur)
        with torch.cuda.stream(self.side):
            self.layers.gdn_step(self.gw, [dict(session=self.gs[s], qkv=self.inp["qkv"][s], z=self.inp["z"][s], x=self.inp["x"][s], pos0=self.pos,
                                                 replay=replay[s], commit=1) for s in range(S)], outs=[self.out_all[s, 1] for s in range(S)])
        src = self.inp if in_place else self.work
        spans = [dict(session=self.qs[s], q=src["q"][s].view(self.ROWS, 16, 512), k=self.inp["k"][s], v=self.inp["v"][s], idx=src["idx"][s], pos0=self.pos)
                 for s in range(S)]
        self.plan.run(spans, outs=[self.out_all[s, 0] for s in range(S)])
        cur.wait_stream(self.side)
        return self.out_all

    def _replay_graph(self, in_place):
        """The pass of the next replay pattern as a CUDA graph (one graph per pattern and leg: the replay counts are
        kernel arguments), captured on first use."""
        torch = self.torch
        if (0, in_place) not in self.graphs:                 # first use of the leg: every pattern is captured, outside any timed region
            for pattern in range(len(self.replays)):
                self._step(in_place, pattern)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._step(in_place, pattern)
                self.graphs[(pattern, in_place)] = g
        pattern = self.t % len(self.replays)
        self.t += 1
        return self.graphs[(pattern, in_place)]

    def step(self):
        self._replay_graph(False).replay()
        return self.out_all

    def step_eager(self):
        return self._step()

    def step_profile(self):
        return self._step()

    def step_e2e(self):
        g = self._replay_graph(True)
        for n, t in self.inp.items():
            t.copy_(self.h_in[n], non_blocking=True)
        g.replay()
        self.h_out.copy_(self.out_all, non_blocking=True)

    def config(self):
        return {"workload": self.name, "sessions_per_gpu": self.SESSIONS, "context": self.CTX, "span_rows": self.ROWS, "commit": 1,
                "replay": "uniform 0..8 per session and pass (seeded, 16 patterns in turn, each pass replayed from a CUDA graph)", "pend_rows": 16, "qsa_heads": "16q/2kv x256",
                "gdn_state": "32x128x128 fp32", "l2": "per-pass traffic (202 MB) exceeds the 126 MB L2"}


class PrefillStack262k:
    """configs[3]: cold prefill of 262,144 tokens through a 3:1 stack of GDN:QSA layers (4 layers).  The host walks the
    sequence in launches of 16,384 rows, layer by layer, as the reference's prefill does (launches of up to 16,384 rows,
    engine/model/flashnext/prefill_launch.h:14-34): a GDN layer takes a launch in one cr_gdn_prefill call (its internal
    parts pipeline the chunk-local and the scan kernels), the QSA layer runs in 2,048-row parts against the growing cache
    (cr_qsa_prefill).  A step is the whole sequence.  Every launch reuses one seeded block of projection rows per layer
    (positions, caches and states differ from launch to launch); the indexer rows get a launch-dependent mixture so that
    the pooled keys do not repeat along the sequence."""
    name = "prefill_262k_stack"
    T, PART, LAUNCH = 262144, 2048, 16384
    unit, metric, dtype = "tokens/s", "gdn3_qsa1_stack_prefill_tokens_per_s_at_262k", "bf16 in (GDN) / fp32 in (QSA) / fp16 kv / fp32 state"

    def __init__(self, rank, algo, launches=None):
        import torch
        from crucible_strix_halo_b200 import capi, layers
        self.torch, self.capi, self.layers = torch, capi, layers
        g = capi.GEOM_BENCH
        gen = torch.Generator(device="cuda").manual_seed(6000 + rank)
        rn = lambda *s, std=1.0, mean=0.0: torch.randn(*s, device="cuda", generator=gen) * std + mean
        R, L = self.PART, self.LAUNCH
        self.launches = launches if launches is not None else list(range(self.T // L))
        self.algo = algo
        self.gw = [layers.GdnWeights(g, rn(g.gdn_channels, 4, std=0.5), rn(32, std=1.5, mean=-1).clamp(-5, 1.5), rn(32, std=0.5),
                                     1 + rn(128, std=0.1)) for _ in range(3)]
        self.gses = [layers.GdnSession(g) for _ in range(3)]
        self.gplan = layers.GdnPrefillPlan(self.gw[0], L, in_dtype=capi.IN_BF16, fmt=capi.OUT_RAW_BF16)     # one workspace for the three layers
        self.g_in = [(rn(L, g.gdn_channels).bfloat16(), rn(L, 4096).bfloat16(), rn(L, 64).bfloat16()) for _ in range(3)]
        self.qw = layers.QsaWeights(g, 1 + rn(256, std=0.1), 1 + rn(256, std=0.1), 1 + rn(128, std=0.1), 1 + rn(128, std=0.1))
        self.qses = layers.QsaSession(g, self.T, max_rows=R)
        self.qplan = layers.QsaPrefillPlan(self.qw, R, fmt=capi.OUT_RAW_BF16)
        self.q_in = {"q": rn(L, 16, 512), "k": rn(L, 512), "v": rn(L, 512), "idx": rn(L, 640)}
        self.idx_mix = [rn(L, 640) for _ in range(3)]                       # launch l uses idx + mixtures chosen by l % 2, l % 3, l % 5
        self.q_work = {n: torch.empty_like(self.q_in[n]) for n in ("q", "idx")}
        self.q_out = torch.empty(L, 4096, device="cuda", dtype=torch.bfloat16)
        if len(self.launches) < self.T // L:                                # a subset of launches: the rows below them are never
            for t in (self.qses.k, self.qses.v, self.qses.ik_pool):          # written, so the caches get seeded values instead
                t.copy_(torch.randn(t.shape, device="cuda", generator=gen).to(t.dtype))
        self.units_per_step = len(self.launches) * L
        rows = [l * L + r for l in self.launches for r in range(0, L, 64)]                           # sampled rows (every 64th)
        att = sum(min(p + 1, 2051) for p in rows) * 64
        self.alg_bytes = 3 * GDN_BYTES_PER_TOKEN * self.units_per_step + att * 2048 + sum(((p + 1) // 4) * 512 for p in rows if (p + 1) // 4 > 512) * 64 // 2048
        self.alg_flops = 3 * 5.4e6 * self.units_per_step + att * 4 * 16 * 256 + sum(1024 * ((p + 1) // 4) for p in rows if (p + 1) // 4 > 512) * 64
        self.kernel_bytes = {}
        self.h_g = [tuple(t.cpu().pin_memory() for t in tpl) for tpl in self.g_in]
        self.h_q = {n: t.cpu().pin_memory() for n, t in self.q_in.items()}
        self.h_out = torch.empty(4, L, 4096, dtype=torch.bfloat16).pin_memory()
        self.h2d = (sum(t.numel() * 2 for tpl in self.h_g for t in tpl) + sum(t.numel() * 4 for t in self.h_q.values())) * len(self.launches)
        self.d2h = self.h_out.numel() * 2 * len(self.launches)

    def _reset(self):
        for s in self.gses:
            s.state.zero_(); s.hist.zero_()

    def _launch(self, l, e2e=False):
        R, L, torch = self.PART, self.LAUNCH, self.torch
        for i in range(3):                                                   # layers 0-2: Gated DeltaNet, one call per launch
            if e2e:
                for d, h in zip(self.g_in[i], self.h_g[i]):
                    d.copy_(h, non_blocking=True)
            qkv, z, ab = self.g_in[i]
            self.gplan.w = self.gw[i]
            out = self.gplan.run(self.gses[i], qkv, z, ab, l * L, self.algo)
            if e2e:
                self.h_out[i].copy_(out, non_blocking=True)
        for n, t in self.q_in.items():                                       # layer 3: QSA in parts of 2,048 rows
            dst = self.q_work[n] if n in self.q_work else t
            if e2e:
                dst.copy_(self.h_q[n], non_blocking=True)
            elif n in self.q_work:
                dst.copy_(t)
        self.q_work["idx"].add_(self.idx_mix[0], alpha=0.7 * (l % 2)).add_(self.idx_mix[1], alpha=0.5 * (l % 3)).add_(self.idx_mix[2], alpha=0.4 * (l % 5))
        for p in range(L // R):
            sl = slice(p * R, (p + 1) * R)
            out = self.qplan.run(self.qses, self.q_work["q"][sl], self.q_in["k"][sl], self.q_in["v"][sl], self.q_work["idx"][sl], l * L + p * R)
            self.q_out[sl].copy_(out)
        if e2e:
            self.h_out[3].copy_(self.q_out, non_blocking=True)

    def step(self):
        self._reset()
        for l in self.launches:
            self._launch(l)

    step_eager = step

    def step_e2e(self):
        self._reset()
        for l in self.launches:
            self._launch(l, e2e=True)

    def config(self):
        return {"workload": self.name, "seq_len": self.T, "launch_rows": self.LAUNCH, "qsa_part_rows": self.PART, "launches_run": len(self.launches),
                "layers": "GDN, GDN, GDN, QSA", "gdn_heads": "16qk/32v x128", "qsa_heads": "16q/2kv x256", "block": 4, "top_k_blocks": 512,
                "selections": "i.i.d. (random indexer)", "l2": "the K/V cache (0.5 GB) and the GDN inputs exceed the 126 MB L2"}


class GdnInProj32k:
    """The input projection of a GDN layer over 32,768 tokens (the caller's side of configs[1]): hidden rows
    x [T, 2048] bf16 ~ N(0,1) times W [12,352, 2048] bf16 ~ N(0, 1/2048) -> qkv [T, 8192] | z [T, 4096] | a,b logits
    [T, 64] as bf16 rows, the inputs cr_gdn_prefill takes.  One cr_proj_gemm launch per step."""
    name = "gdn_in_proj_32k"
    bound = "tensor"
    T, K, WIDTHS = 32768, 2048, (8192, 4096, 64)
    unit, metric, dtype = "tokens/s", "gdn_input_projection_tokens_per_s_at_32k", "bf16 operands / fp32 accumulate (tcgen05) / bf16 out"

    def __init__(self, rank, algo):
        import torch
        from crucible_strix_halo_b200 import layers
        self.torch, self.layers = torch, layers
        gen = torch.Generator(device="cuda").manual_seed(7000 + rank)
        T, K, N = self.T, self.K, sum(self.WIDTHS)
        self.x = torch.randn(T, K, device="cuda", generator=gen).bfloat16()
        self.w = (torch.randn(N, K, device="cuda", generator=gen) / K ** 0.5).bfloat16()
        self.outs = [torch.empty(T, c, device="cuda", dtype=torch.bfloat16) for c in self.WIDTHS]
        self.h_x = self.x.cpu().pin_memory()
        self.h_out = [torch.empty(T, c, dtype=torch.bfloat16).pin_memory() for c in self.WIDTHS]
        self.h2d, self.d2h = self.x.numel() * 2, T * N * 2
        self.units_per_step = T
        self.alg_flops = 2.0 * T * K * N
        self.alg_bytes = (T * K + N * K + T * N) * 2
        self.kernel_bytes = {}
        # the library GEMM on the same operands, for context (not part of the step)
        y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            torch.matmul(self.x, self.w.t(), out=y)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            torch.matmul(self.x, self.w.t(), out=y)
        e1.record()
        torch.cuda.synchronize()
        self.cublas_ms = e0.elapsed_time(e1) / 5
        del y

    def step(self):
        return self.layers.proj_gemm(self.x, self.w, self.outs)

    step_eager = step

    def step_e2e(self):
        self.x.copy_(self.h_x, non_blocking=True)
        self.step()
        for h, o in zip(self.h_out, self.outs):
            h.copy_(o, non_blocking=True)

    def config(self):
        return {"workload": self.name, "tokens": self.T, "hidden": self.K, "columns": "qkv 8192 | z 4096 | a,b 64",
                "library_gemm_ms_same_operands": self.cublas_ms, "l2": "x (134 MB) and the outputs (810 MB) exceed the 126 MB L2"}


class SplitKvPrefill262k:
    """The QSA part of qsa_prefill_262k with the KV sequence split over the ranks (strong scaling: ONE sequence): rank g
    owns the cache positions of blocks [b0_g, b1_g) (its cache pointers are biased, so it stores only its share) and the
    merges of the rows [g R / N, (g + 1) R / N).  It scores its own blocks for every row, sends each rank the 512
    candidates of that rank's rows (all-to-all), merges the candidates of its rows into the global selection, all-gathers
    the selections, attends its own positions for every row, sends each rank the (m, l, acc) partials of that rank's rows
    (all-to-all), merges its rows and all-gathers the output rows (NCCL over NVLink)."""
    name = "qsa_prefill_262k_split_kv"
    POS0, R = 262144 - 2048, 2048
    unit, metric, dtype = "tokens/s", "qsa_layer_prefill_tokens_per_s_at_262k_split_kv", "fp16 kv / fp32 q"

    def __init__(self, rank, world):
        import torch
        import torch.distributed as dist
        from crucible_strix_halo_b200 import capi, layers, parallel
        self.torch, self.capi, self.layers, self.dist = torch, capi, layers, dist
        g = capi.GEOM_BENCH
        R, ctx = self.R, self.POS0 + self.R
        self.rank, self.world = rank, world
        (b0, b1), (p0, p1) = parallel.kv_block_range(ctx, world, rank)
        self.b0, self.b1, self.p0, self.p1 = b0, b1, p0, min(p1, ctx)
        own = self.p1 - self.p0
        gen = torch.Generator(device="cuda").manual_seed(7000)          # the same sequence on every rank
        rn = lambda *s, std=1.0: torch.randn(*s, device="cuda", generator=gen) * std
        self.w = layers.QsaWeights(g, 1 + rn(256, std=0.1), 1 + rn(256, std=0.1), 1 + rn(128, std=0.1), 1 + rn(128, std=0.1))
        self.inp = {"q": rn(R, 16, 512), "k": rn(R, 512), "v": rn(R, 512), "idx": rn(R, 640)}
        lgen = torch.Generator(device="cuda").manual_seed(7100 + rank)   # the rank's own share of the cache
        lrn = lambda *s: torch.randn(*s, device="cuda", generator=lgen)
        # own share only: K, V [own][2][256]; pool tiles covering the own blocks; bases biased to absolute positions
        self.k = lrn(own + 8, 2, 256).half(); self.v = lrn(own + 8, 2, 256).half()
        t0 = b0 // 32
        self.pool = lrn(((b1 + 31) // 32 - t0 + 1) * 4096)
        self.raw = torch.zeros(16, 128, device="cuda")
        self.scores = torch.empty(R, b1 - b0 + 64, device="cuda")        # the rank's own columns; biased base
        self.sel = torch.zeros(R, 512, device="cuda", dtype=torch.int32)
        self.nsel = torch.zeros(R, device="cuda", dtype=torch.int32)
        self.out = torch.empty(R, 4096, device="cuda", dtype=torch.bfloat16)
        self.work = {n: torch.empty_like(self.inp[n]) for n in ("q", "idx")}
        cache = capi.QsaCache(self.k.data_ptr() - self.p0 * 1024, self.v.data_ptr() - self.p0 * 1024, self.raw.data_ptr(),
                              self.pool.data_ptr() - t0 * 4096 * 4, 16)
        score_stride = self.scores.shape[1]
        self.args = capi.QsaArgs(capi.dptr(self.work["q"]), capi.dptr(self.inp["k"]), capi.dptr(self.inp["v"]), capi.dptr(self.work["idx"]),
                                 capi.dptr(self.w.q_norm1), capi.dptr(self.w.k_norm1), capi.dptr(self.w.iq_norm1), capi.dptr(self.w.ik_norm1),
                                 cache, self.scores.data_ptr() - b0 * 4, score_stride, capi.dptr(self.sel), capi.dptr(self.nsel), None,
                                 capi.dptr(self.out), self.POS0, R, None, 0, 0, None, capi.dptr(self.w.rope))
        assert R % world == 0, "the part's rows are dealt evenly to the ranks"
        Rr = self.Rr = R // world
        r0 = self.r0 = rank * Rr
        self.cs = torch.empty(R, 512, device="cuda"); self.ci = torch.empty(R, 512, device="cuda", dtype=torch.int32)
        self.my_cs = torch.empty(world, Rr, 512, device="cuda"); self.my_ci = torch.empty(world, Rr, 512, device="cuda", dtype=torch.int32)
        self.sel_mine = torch.zeros(Rr, 512, device="cuda", dtype=torch.int32); self.nsel_mine = torch.zeros(Rr, device="cuda", dtype=torch.int32)
        self.part = torch.empty(R, 16, 258, device="cuda"); self.my_part = torch.empty(world, Rr, 16, 258, device="cuda")
        self.out_mine = torch.empty(Rr, 4096, device="cuda", dtype=torch.bfloat16)
        self.scratch = torch.empty(R * 16 * 4 * 258 * 4, dtype=torch.uint8, device="cuda")
        # the argument block of this rank's rows: same buffers, row pointers moved to row r0, selections and outputs of its own
        mine = capi.QsaArgs.from_buffer_copy(self.args)
        mine.q += r0 * 16 * 512 * 4; mine.idx += r0 * 640 * 4; mine.k += r0 * 512 * 4; mine.v += r0 * 512 * 4
        mine.scores += r0 * score_stride * 4
        mine.sel, mine.nsel, mine.out = self.sel_mine.data_ptr(), self.nsel_mine.data_ptr(), self.out_mine.data_ptr()
        mine.pos0 += r0; mine.R = Rr
        self.args_mine = mine
        self.units_per_step = R
        f = (world - 1) / world                                              # share of a buffer that crosses the wire
        self.wire_bytes = int(f * (self.cs.numel() * 8 + self.sel.numel() * 4 + self.nsel.numel() * 4 + self.part.numel() * 4 + self.out.numel() * 2))
        self.ev = [torch.cuda.Event(enable_timing=True) for _ in range(9)]
        self.stage_ms = [0.0, 0.0, 0.0, 0.0]
        self.coll_ms = [0.0, 0.0, 0.0, 0.0]
        self.h_in = {n: t.cpu().pin_memory() for n, t in self.inp.items()}
        self.h_out = torch.empty(R, 4096, dtype=torch.bfloat16).pin_memory()
        self.h2d, self.d2h = sum(t.numel() * 4 for t in self.h_in.values()), self.h_out.numel() * 2

    def _prep(self):
        """q and the indexer queries normalised + roped in place (every rank does this cheap step for all rows)."""
        capi, g = self.capi, self.capi.GEOM_BENCH
        capi.check(capi.lib.cr_qsa_prep_queries(C.byref(g), (capi.QsaArgs * 1)(self.args), 1, C.c_void_p(self.torch.cuda.current_stream().cuda_stream)))

    def _run(self, timed=False):
        capi, dist, g = self.capi, self.dist, self.capi.GEOM_BENCH
        st = C.c_void_p(self.torch.cuda.current_stream().cuda_stream)
        arr = (capi.QsaArgs * 1)(self.args)
        # the cache rows of the part belong to the last rank's positions and are part of the synthetic cache here
        if timed: self.ev[8].record()
        self._prep()
        mine = (capi.QsaArgs * 1)(self.args_mine)
        capi.check(capi.lib.cr_qsa_shard_select(C.byref(g), arr, self.b0, self.b1, self.cs.data_ptr(), self.ci.data_ptr(), st))
        if timed: self.ev[0].record()
        if self.world > 1:
            dist.all_to_all_single(self.my_cs.view(-1, 512), self.cs); dist.all_to_all_single(self.my_ci.view(-1, 512), self.ci)
        else:
            self.my_cs.copy_(self.cs.unsqueeze(0)); self.my_ci.copy_(self.ci.unsqueeze(0))
        if timed: self.ev[1].record()
        capi.check(capi.lib.cr_qsa_merge_candidates(C.byref(g), mine, self.world, self.my_cs.data_ptr(), self.my_ci.data_ptr(), st))
        if timed: self.ev[2].record()
        if self.world > 1:
            dist.all_gather_into_tensor(self.sel, self.sel_mine); dist.all_gather_into_tensor(self.nsel, self.nsel_mine)
        else:
            self.sel.copy_(self.sel_mine); self.nsel.copy_(self.nsel_mine)
        if timed: self.ev[3].record()
        capi.check(capi.lib.cr_qsa_shard_attn(C.byref(g), arr, self.p0, self.p1 if self.rank < self.world - 1 else 2 ** 31 - 1,
                                              self.part.data_ptr(), self.scratch.data_ptr(), self.scratch.numel(), st))
        if timed: self.ev[4].record()
        if self.world > 1:
            dist.all_to_all_single(self.my_part.view(-1, 16, 258), self.part)
        else:
            self.my_part.copy_(self.part.unsqueeze(0))
        if timed: self.ev[5].record()
        capi.check(capi.lib.cr_qsa_merge_partials(C.byref(g), mine, self.world, self.my_part.data_ptr(), capi.OUT_RAW_BF16, st))
        if timed: self.ev[6].record()
        if self.world > 1:
            dist.all_gather_into_tensor(self.out, self.out_mine)
        else:
            self.out.copy_(self.out_mine)
        if timed: self.ev[7].record()
        return self.out

    def _fresh(self):
        for n, t in self.work.items():
            t.copy_(self.inp[n])

    def step(self):
        self._fresh()
        return self._run()

    def step_timed(self):
        self._fresh()
        out = self._run(timed=True)
        self.torch.cuda.synchronize()
        for i in range(4):
            self.coll_ms[i] += self.ev[2 * i].elapsed_time(self.ev[2 * i + 1])
            self.stage_ms[i] += (self.ev[8] if i == 0 else self.ev[2 * i - 1]).elapsed_time(self.ev[2 * i])
        return out

    def step_e2e(self):
        for n, t in self.inp.items():
            (self.work[n] if n in self.work else t).copy_(self.h_in[n], non_blocking=True)
        self.h_out.copy_(self._run(), non_blocking=True)

    def config(self):
        return {"workload": self.name, "context": self.POS0 + self.R, "part_rows": self.R, "ranks": self.world,
                "split": "KV positions by whole blocks, the newest rows on the last rank", "collectives": "all-to-all of candidates, all-gather of selections, all-to-all of partials, all-gather of output rows (NCCL)",
                "wire_bytes_received_per_rank_per_part": self.wire_bytes}


WORKLOADS = {"gdn_prefill_32k": GdnPrefill32k, "decode_262k": Decode262k, "qsa_prefill_262k": QsaPrefill262k,
             "qsa_attend_262k_drift": QsaAttendDrift, "verify_131k": Verify131k, "prefill_262k_stack": PrefillStack262k,
             "gdn_in_proj_32k": GdnInProj32k, "decode_262k_x16": Decode262kX16}
SUB_WORKLOADS = ["decode_262k", "decode_262k_x16", "qsa_prefill_262k", "qsa_attend_262k_drift", "verify_131k", "prefill_262k_stack", "gdn_in_proj_32k"]
SUB_STEPS = {"decode_262k": (20, 5), "decode_262k_x16": (20, 5), "qsa_prefill_262k": (5, 3), "qsa_attend_262k_drift": (5, 3), "verify_131k": (20, 5), "prefill_262k_stack": (2, 1),
             "gdn_in_proj_32k": (5, 3)}
BF16_PEAK_FALLBACK = 1590.0


# ------------------------------------------------------------------------------------------------------------
# CPU baseline (the oracle's C port on the host cores)
# ------------------------------------------------------------------------------------------------------------

def cpu_baseline(workload, seconds=6.0):
    """Times the C port of the oracle on every host core this process may use, for at least `seconds` seconds, on a
    bounded sample of the workload."""
    from oracle import build as oracle_build
    lib = C.CDLL(oracle_build.build_oracle())
    lib.oracle_threads.restype = C.c_int
    lib.oracle_set_threads(C.c_int(len(os.sched_getaffinity(0))))
    cores = lib.oracle_threads()
    rng = np.random.default_rng(0)
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    Hv, Hk, Hq, Hkv = 32, 16, 16, 2
    Cw = 2 * Hk * 128 + Hv * 128
    conv, A_log = f32(rng.normal(size=(Cw, 4)) * 0.5), f32(np.clip(rng.normal(-1, 1.5, Hv), -5, 1.5))
    dtb, gamma = f32(rng.normal(size=Hv) * 0.5), f32(1 + 0.1 * rng.normal(size=128))

    def gdn_rows(n):
        qkv, z, ab = f32(rng.normal(size=(n, Cw))), f32(rng.normal(size=(n, Hv * 128))), f32(rng.normal(size=(n, 2 * Hv)))
        state, out = f32(rng.normal(size=(Hv, 128, 128)) * 0.05), np.zeros((n, Hv * 128), np.float32)
        return lambda: lib.oracle_gdn_layer(ptr(qkv), ptr(z), ptr(ab), ptr(conv), ptr(A_log), ptr(dtb), ptr(gamma), None, ptr(state), ptr(out), n, Hv, Hk)

    def qsa_row(ctx):
        kc = rng.normal(size=(ctx, Hkv, 256)).astype(np.float16); vc = rng.normal(size=(ctx, Hkv, 256)).astype(np.float16)
        pool = f32(rng.normal(size=((ctx + 127) // 128) * 4096))
        qn, gate, iq = f32(rng.normal(size=(Hq, 256))), f32(rng.normal(size=(Hq, 256))), f32(rng.normal(size=(4, 128)))
        out, sel, nsel = np.zeros((Hq, 256), np.float32), np.zeros(512, np.int32), np.zeros(1, np.int32)
        return lambda p=ctx - 1: lib.oracle_qsa_decode_row(ptr(qn), ptr(gate), ptr(iq), int(p), ptr(kc), ptr(vc), ptr(pool), ptr(out), ptr(sel), ptr(nsel), Hq, Hkv)

    def run(fn, units, what):
        fn()                                              # warm the caches and the thread pool
        t0, reps = time.perf_counter(), 0
        while True:
            fn()
            reps += 1
            dt = time.perf_counter() - t0
            if dt >= seconds:
                break
        return {"value": units * reps / dt, "unit": WORKLOADS[workload].unit if workload in WORKLOADS else "tokens/s", "cores": cores, "kind": "port",
                "sample": "%d x %s, %.1f s" % (reps, what, dt)}

    if workload == "gdn_prefill_32k":
        return run(gdn_rows(2048), 2048, "2048 tokens of the 32768-token layer (serial fp32 recurrence, all 32 heads)")
    if workload in ("qsa_prefill_262k", "qsa_attend_262k_drift", "qsa_prefill_262k_split_kv"):
        row = qsa_row(262144)
        what = "8 rows of the 2,048-row part at 262,144 context (score, top-512, attention)"
        return run(lambda: [row(262143 - i) for i in range(8)], 8, what)
    if workload in ("decode_262k", "decode_262k_x16"):
        row, upd = qsa_row(262144), gdn_rows(1)
        return run(lambda: (row(), upd()), 1, "1 session-step at 262,144 context (QSA row + GDN update)")
    if workload == "verify_131k":
        row, upd = qsa_row(131072), gdn_rows(9)
        return run(lambda: ([row(131071 - i) for i in range(9)], upd()), 9, "one 9-row span at 131,072 context (9 QSA rows + 9 GDN rows)")
    if workload == "prefill_262k_stack":
        # per token of the stack: 3 GDN tokens + 1 QSA row at a context drawn evenly from the sequence
        row, upd = qsa_row(262144), gdn_rows(64)
        ctxs = [int(c) for c in np.linspace(2048, 262143, 8)]
        def fn():
            for _ in range(3):
                upd()
            for c in ctxs * 8:
                row(c)
        return run(fn, 64, "64 tokens of the stack (3 x 64 GDN tokens + 64 QSA rows at contexts spread over the sequence)")
    if workload == "gdn_in_proj_32k":
        x, w = f32(rng.normal(size=(1024, 2048))), f32(rng.normal(size=(12352, 2048)))
        res = run(lambda: x @ w.T, 1024, "1024 of the 32768 rows (numpy fp32 product, the host's BLAS threads)")
        res["cores"] = len(os.sched_getaffinity(0))
        return res
    raise ValueError(workload)


def run_reference(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals, cb = [], None
    for _ in range(max(1, min(args.steps, 3))):
        cb = cpu_baseline(workload, seconds=6.0)
        vals.append(cb["value"])
    v = float(np.mean(vals))
    cb["value"] = v
    W = WORKLOADS[workload]
    line = {"impl": "reference", "metric": W.metric, "value": v, "unit": W.unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": workload}, "cpu_baseline": cb,
            "e2e": {"value": v, "unit": W.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


def load_tensor_peak():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["bf16_tflops"]), "measured"
    except Exception:
        return BF16_PEAK_FALLBACK, "fallback"


def measure(wl, steps, warmup, world, dist, sampler=None):
    """Runs one workload: device-timed steps, the host-buffer leg, per-kernel times.  Returns the figures of the line."""
    import torch
    from crucible_strix_halo_b200 import capi

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(warmup, 3) if steps > 2 else max(warmup, 1)):
        wl.step()
    if sampler:
        sampler.start()
    ms = timed(wl.step, steps)
    clocks = sampler.stop() if sampler else None
    for _ in range(2 if steps > 2 else 1):
        wl.step_e2e()
    ms_e2e = timed(wl.step_e2e, steps)
    capi.lib.cr_profile_enable(1)
    barrier()
    psteps = min(steps, 5)
    for _ in range(psteps):
        capi.lib.cr_profile_begin(C.c_void_p(torch.cuda.current_stream().cuda_stream))
        (wl.step_profile if hasattr(wl, "step_profile") else wl.step_eager)()
    prof = capi.profile_collect()
    capi.lib.cr_profile_enable(0)
    status = capi.lib.cr_device_status()
    peak, peak_kind = load_peaks()
    tpeak, tpeak_kind = load_tensor_peak()
    dominant = max(prof, key=lambda k: prof[k][0]) if prof else None
    dom_ms, dom_calls = prof.get(dominant, (0.0, 0))
    per_launch_ms = dom_ms / dom_calls if dom_calls else None
    launches_per_step = dom_calls / psteps if dom_calls else 1
    dominant_bytes = wl.kernel_bytes.get(dominant, wl.alg_bytes)
    achieved = (dominant_bytes / launches_per_step) / (per_launch_ms * 1e-3) / 1e9 if per_launch_ms else None
    traffic = None
    if dominant in NCU_TRAFFIC.get(wl.name, {}):
        per, val = NCU_TRAFFIC[wl.name][dominant]
        traffic = val * (wl.units_per_step if per == "token" else 1.0) / launches_per_step
    step_ms = ms / steps
    step_frac = (wl.alg_bytes / peak / 1e9) / (step_ms * 1e-3)
    roof = {"bound": "hbm", "achieved": wl.alg_bytes / (step_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s", "frac": step_frac,
            "frac_is": "step: algorithmic bytes of the step / ms_per_step / peak",
            "peak_source": (peak_kind + " (of measured copy bandwidth)") if peak_kind == "measured" else "fallback",
            "traffic": traffic, "step_algorithmic_bytes": wl.alg_bytes,
            "dominant_kernel": {"name": dominant, "ms_per_launch": per_launch_ms, "algorithmic_bytes_per_launch": dominant_bytes / launches_per_step,
                                "achieved_gbs": achieved, "frac": (achieved / peak) if achieved else None},
            "kernels": {k: {"ms_per_step": v[0] / psteps, "launches_per_step": v[1] / psteps} for k, v in prof.items()}}
    if getattr(wl, "alg_flops", None):
        tf = wl.alg_flops / (step_ms * 1e-3) / 1e12
        roof["tensor"] = {"useful_tflops": tf, "peak": tpeak, "frac": tf / tpeak, "peak_source": tpeak_kind + " (cuBLAS bf16, burst)",
                          "step_useful_flops": wl.alg_flops}
        if getattr(wl, "bound", "hbm") == "tensor":          # a contraction: the tensor figure leads, the byte figure stays beside it
            roof = {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak,
                    "frac_is": "step: flops of the step / ms_per_step / peak", "peak_source": tpeak_kind + " (of measured cuBLAS bf16, burst)",
                    "traffic": None, "step_flops": wl.alg_flops, "hbm": {k: roof[k] for k in ("achieved", "peak", "frac", "step_algorithmic_bytes")},
                    "dominant_kernel": roof["dominant_kernel"], "kernels": roof["kernels"]}
    total_units = wl.units_per_step * world * steps
    return {"metric": wl.metric, "value": total_units / (ms * 1e-3), "unit": wl.unit, "steps": steps, "ms_per_step": step_ms,
            "dtype": wl.dtype, "config": wl.config(),
            "e2e": {"value": total_units / (ms_e2e * 1e-3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                    "ms_per_step": ms_e2e / steps},
            "gpu_launches": int(sum(v[1] for v in prof.values()) * steps / psteps), "roofline": roof, "device_status": status}, clocks


def measure_split_kv(rank, world, dist, steps=5, warmup=3):
    import torch
    wl = SplitKvPrefill262k(rank, world)
    for _ in range(warmup):
        wl.step()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    res = {}
    for name, fn in (("device", wl.step), ("e2e", wl.step_e2e)):
        fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        res[name] = float(ms.item()) / steps
    for _ in range(steps):
        wl.step_timed()
    coll = torch.tensor(wl.coll_ms + wl.stage_ms, device="cuda") / steps
    if world > 1:
        dist.all_reduce(coll, op=dist.ReduceOp.MAX)
    out = {"metric": wl.metric, "value": wl.R / (res["device"] * 1e-3), "unit": wl.unit, "ms_per_step": res["device"], "scaling": "strong",
           "steps": steps, "config": wl.config(),
           "e2e": {"value": wl.R / (res["e2e"] * 1e-3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "ms_per_step": res["e2e"]},
           "collectives_ms_per_step": {"all_to_all_candidates": float(coll[0]), "all_gather_selections": float(coll[1]),
                                       "all_to_all_partials": float(coll[2]), "all_gather_outputs": float(coll[3])},
           "stages_ms_per_step": {"prep_and_shard_select": float(coll[4]), "merge_candidates": float(coll[5]), "shard_attn": float(coll[6]),
                                  "merge_partials": float(coll[7])},
           "wire_bytes_received_per_rank_per_step": wl.wire_bytes}
    del wl
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + ["qsa_prefill_262k_split_kv"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--algo", default="auto", choices=["auto", "serial", "chunk"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub-workloads", action="store_true", help="headline only (no `workloads` object)")
    ap.add_argument("--seq", type=int, default=0, help="gdn_prefill_32k only: a shorter sequence, for profiler captures")
    ap.add_argument("--parts", type=int, default=0, help="prefill_262k_stack only: run every n-th 16,384-row launch, for profiler captures")
    args = ap.parse_args()
    headline = args.workload or "gdn_prefill_32k"
    if args.impl == "reference":
        return run_reference(args, headline)

    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if rank == 0:
        ge.build()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist.barrier()
    from crucible_strix_halo_b200 import capi
    algo = {"serial": capi.GDN_SERIAL_F32, "chunk": capi.GDN_CHUNK_TC}.get(args.algo)
    if algo is None:
        algo = capi.GDN_CHUNK_TC if capi.lib.cr_gdn_algo_available(capi.GDN_CHUNK_TC) else capi.GDN_SERIAL_F32
    if args.seq and headline == "gdn_prefill_32k":
        GdnPrefill32k.T = args.seq

    if headline == "qsa_prefill_262k_split_kv":            # the strong-scaling workload alone (any number of ranks)
        res = measure_split_kv(rank, world, dist, steps=args.steps, warmup=max(args.warmup, 3))
        res.update(n_gpus=world, warmup=max(args.warmup, 3), higher_is_better=True, vs_baseline=None, dtype=SplitKvPrefill262k.dtype, data="synthetic")
        if rank == 0:
            print(json.dumps(res))
        if world > 1:
            dist.destroy_process_group()
        return

    def make(name):
        if name == "prefill_262k_stack" and args.parts:
            return PrefillStack262k(rank, algo, launches=list(range(args.parts - 1, 16, args.parts)))
        return WORKLOADS[name](rank, algo)

    wl = make(headline)
    sampler = ClockSampler(local) if rank == 0 else None
    res, clocks = measure(wl, args.steps, args.warmup, world, dist, sampler)
    del wl
    torch.cuda.empty_cache()
    line = {"metric": res["metric"], "value": res["value"], "unit": res["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": res["dtype"], "data": "synthetic", "config": res["config"], "e2e": res["e2e"],
            "gpu_launches": res["gpu_launches"], "clocks": clocks, "roofline": res["roofline"], "device_status": res["device_status"]}
    if not args.no_cpu_baseline and rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_baseline(headline)
    if args.workload is None and not args.no_sub_workloads:
        subs = {}
        if world == 1:
            subs[headline] = {k: line[k] for k in ("metric", "value", "unit", "ms_per_step", "e2e", "roofline") if k in line}
            if "cpu_baseline" in line:
                subs[headline]["cpu_baseline"] = line["cpu_baseline"]
            for name in SUB_WORKLOADS:
                steps, warm = SUB_STEPS[name]
                try:
                    w2 = make(name)
                    r2, _ = measure(w2, steps, warm, world, dist)
                    del w2
                    torch.cuda.empty_cache()
                    if not args.no_cpu_baseline:
                        r2["cpu_baseline"] = cpu_baseline(name)
                    subs[name] = r2
                except Exception as e:                      # a failing sub-workload must not cost the headline line
                    subs[name] = {"error": "%s: %s" % (type(e).__name__, e)}
        else:
            try:
                subs["qsa_prefill_262k_split_kv"] = measure_split_kv(rank, world, dist)
            except Exception as e:
                subs["qsa_prefill_262k_split_kv"] = {"error": "%s: %s" % (type(e).__name__, e)}
        line["workloads"] = subs
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
