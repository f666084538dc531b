#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input.  Workloads:
  gdn_prefill_32k  one Gated DeltaNet layer, chunked prefill, batch 1, seq 32768, 16 QK x 128 / 32 V x 128 heads,
                   bf16 inputs, fp32 state (the default: the config the headline metric is quoted on)
  decode_262k      QSA sparse attention decode + GDN recurrent update, 4 sessions x 262,144-token fp16 KV cache
  qsa_prefill_262k one QSA layer, the last 2,048-row part of a 262,144-token prefill (scores, top-512, attention)
Under torchrun (N > 1) every rank runs the same workload on its own sequences / sessions (weak scaling, no
data-path collective); time is the max over ranks, value the whole-job throughput.
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
    "gdn_prefill_32k": {"gdn_chunk_scan_tc_kernel": ("token", (526.546e6 + 102.534e6) / 7104),
                        "gdn_chunk_local_kernel": ("token", (120.665e6 + 465.678e6) / 7104),
                        "gdn_gate_kernel": ("token", (174.630e6 + 38.259e6) / 7104)},
    "decode_262k": {"qsa_score_kernel": ("step", 134.26e6 + 4.22e6), "qsa_attn_split_kernel": ("step", 16.88e6),
                    "qsa_topk_cluster_kernel": ("step", 1.07e6), "qsa_merge_kernel": ("step", 2.20e6), "qsa_prep_kernel": ("step", 0.13e6),
                    "gdn_step_kernel": ("step", 9.47e6)},
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
                "l2": "per-step traffic (168 MB) exceeds the 126 MB L2"}


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
        self.inp = rn(R, 8192 + 512 + 512 + 640)
        self.work = torch.empty_like(self.inp)               # q and idx are normalised in place: a fresh copy per step
        self.h_in = self.inp.cpu().pin_memory()
        self.h_out = torch.empty(R, 4096, dtype=torch.bfloat16).pin_memory()
        self.h2d, self.d2h = self.h_in.numel() * 4, self.h_out.numel() * 2
        self.units_per_step = R
        # gathered K/V rows of every query row + one pass over the pooled keys + the rows in and out
        self.alg_bytes = R * 2051 * 2048 + 65536 * 512 + self.h2d + self.d2h
        self.kernel_bytes = {"qsa_attn_split_kernel": R * 2051 * 2048}

    def _run(self, src):
        R = self.R
        q, k = src[:, :8192].view(R, 16, 512), src[:, 8192:8704]
        v, idx = src[:, 8704:9216], src[:, 9216:]
        return self.plan.run(self.ses, q, k, v, idx, self.POS0)

    def step(self):
        self.work.copy_(self.inp)
        return self._run(self.work)

    step_eager = step

    def step_e2e(self):
        self.work.copy_(self.h_in, non_blocking=True)
        self.h_out.copy_(self._run(self.work), non_blocking=True)

    def config(self):
        return {"workload": self.name, "context": self.POS0 + self.R, "part_rows": self.R, "qsa_heads": "16q/2kv x256", "block": 4,
                "top_k_blocks": 512, "selections": "i.i.d. (random indexer)", "l2": "the K/V cache (0.5 GB) exceeds the 126 MB L2"}


WORKLOADS = {"gdn_prefill_32k": GdnPrefill32k, "decode_262k": Decode262k, "qsa_prefill_262k": QsaPrefill262k}


# ------------------------------------------------------------------------------------------------------------
# CPU baseline (the oracle's C port on the host cores)
# ------------------------------------------------------------------------------------------------------------

def cpu_baseline(workload, seconds_hint=10.0):
    from oracle import build as oracle_build
    lib_path = oracle_build.build_oracle()
    lib = C.CDLL(lib_path)
    lib.oracle_threads.restype = C.c_int
    lib.oracle_set_threads(C.c_int(len(os.sched_getaffinity(0))))   # every core this process may run on
    cores = lib.oracle_threads()
    rng = np.random.default_rng(0)
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    if workload == "gdn_prefill_32k":
        Hv, Hk, n = 32, 16, 2048
        Cw = 2 * Hk * 128 + Hv * 128
        qkv, z, ab = f32(rng.normal(size=(n, Cw))), f32(rng.normal(size=(n, Hv * 128))), f32(rng.normal(size=(n, 2 * Hv)))
        conv, A_log = f32(rng.normal(size=(Cw, 4)) * 0.5), f32(np.clip(rng.normal(-1, 1.5, Hv), -5, 1.5))
        dtb, gamma = f32(rng.normal(size=Hv) * 0.5), f32(1 + 0.1 * rng.normal(size=128))
        state, out = np.zeros((Hv, 128, 128), np.float32), np.zeros((n, Hv * 128), np.float32)
        t0 = time.perf_counter()
        reps = 0
        while True:
            lib.oracle_gdn_layer(ptr(qkv), ptr(z), ptr(ab), ptr(conv), ptr(A_log), ptr(dtb), ptr(gamma), None, ptr(state), ptr(out),
                                 n, Hv, Hk)
            reps += 1
            if time.perf_counter() - t0 > seconds_hint or reps >= 64:
                break
        dt = time.perf_counter() - t0
        return {"value": n * reps / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": "%d x %d tokens of the 32768-token layer (serial fp32 recurrence, all 32 heads), %.1f s" % (reps, n, dt)}
    # decode: one session at a reduced number of steps, full 262,144-token context
    Hq, Hkv, ctx = 16, 2, 262144
    kc = rng.normal(size=(ctx, Hkv, 256)).astype(np.float16)
    vc = rng.normal(size=(ctx, Hkv, 256)).astype(np.float16)
    pool = f32(rng.normal(size=(ctx // 128) * 4096))
    qn, gate, iq = f32(rng.normal(size=(Hq, 256))), f32(rng.normal(size=(Hq, 256))), f32(rng.normal(size=(4, 128)))
    out, sel, nsel = np.zeros((Hq, 256), np.float32), np.zeros(512, np.int32), np.zeros(1, np.int32)
    Hv, Hk = 32, 16
    Cw = 2 * Hk * 128 + Hv * 128
    g_in = [f32(rng.normal(size=(1, Cw))), f32(rng.normal(size=(1, Hv * 128))), f32(rng.normal(size=(1, 2 * Hv)))]
    conv, A_log = f32(rng.normal(size=(Cw, 4)) * 0.5), f32(np.clip(rng.normal(-1, 1.5, Hv), -5, 1.5))
    dtb, gamma = f32(rng.normal(size=Hv) * 0.5), f32(1 + 0.1 * rng.normal(size=128))
    state, gout = f32(rng.normal(size=(Hv, 128, 128)) * 0.05), np.zeros((1, Hv * 128), np.float32)
    if workload == "qsa_prefill_262k":      # a prefill row costs what a decode row costs: score, select, attend
        t0 = time.perf_counter()
        reps = 0
        while True:
            lib.oracle_qsa_decode_row(ptr(qn), ptr(gate), ptr(iq), ctx - 1 - reps % 2048, ptr(kc), ptr(vc), ptr(pool), ptr(out), ptr(sel),
                                      ptr(nsel), Hq, Hkv)
            reps += 1
            if time.perf_counter() - t0 > seconds_hint or reps >= 2048:
                break
        dt = time.perf_counter() - t0
        return {"value": reps / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": "%d rows of the 2,048-row part at 262,144 context (score, top-512, attention), %.1f s" % (reps, dt)}
    t0 = time.perf_counter()
    reps = 0
    while True:
        lib.oracle_qsa_decode_row(ptr(qn), ptr(gate), ptr(iq), ctx - 1, ptr(kc), ptr(vc), ptr(pool), ptr(out), ptr(sel), ptr(nsel), Hq, Hkv)
        lib.oracle_gdn_layer(ptr(g_in[0]), ptr(g_in[1]), ptr(g_in[2]), ptr(conv), ptr(A_log), ptr(dtb), ptr(gamma), None, ptr(state),
                             ptr(gout), 1, Hv, Hk)
        reps += 1
        if time.perf_counter() - t0 > seconds_hint or reps >= 2000:
            break
    dt = time.perf_counter() - t0
    return {"value": reps / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": "%d session-steps of one session at 262,144 context (QSA row + GDN update), %.1f s" % (reps, dt)}


def run_reference(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    cb = None
    for _ in range(max(1, min(args.steps, 3))):
        cb = cpu_baseline(workload, seconds_hint=8.0)
        vals.append(cb["value"])
    v = float(np.mean(vals))
    cb["value"] = v
    W = WORKLOADS[workload]
    line = {"impl": "reference", "metric": W.metric, "value": v, "unit": W.unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": workload}, "cpu_baseline": cb,
            "e2e": {"value": v, "unit": W.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="gdn_prefill_32k", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--algo", default="auto", choices=["auto", "serial", "chunk"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--seq", type=int, default=0, help="gdn_prefill_32k only: a shorter sequence, for profiler captures")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args, args.workload)

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
    if args.seq and args.workload == "gdn_prefill_32k":
        GdnPrefill32k.T = args.seq
    wl = WORKLOADS[args.workload](rank, algo)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
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
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        wl.step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(wl.step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    # end to end: pinned host inputs -> device, step, result -> host, inside the timed region
    for _ in range(2):
        wl.step_e2e()
    ms_e2e = timed(wl.step_e2e, args.steps)
    # dominant kernel, timed live with events on the launching stream
    capi.lib.cr_profile_enable(1)
    barrier()
    for _ in range(args.steps):
        capi.lib.cr_profile_begin(C.c_void_p(torch.cuda.current_stream().cuda_stream))
        (wl.step_profile if hasattr(wl, "step_profile") else wl.step_eager)()
    prof = capi.profile_collect()
    capi.lib.cr_profile_enable(0)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, peak_kind = load_peaks()
    # the dominant kernel is the one with the largest share of the measured kernel time
    dominant = max(prof, key=lambda k: prof[k][0]) if prof else None
    dom_ms, dom_calls = prof.get(dominant, (0.0, 0))
    per_launch_ms = dom_ms / dom_calls if dom_calls else None
    launches_per_step = dom_calls / args.steps if dom_calls else 1
    dominant_bytes = wl.kernel_bytes.get(dominant, wl.alg_bytes)
    achieved = (dominant_bytes / launches_per_step) / (per_launch_ms * 1e-3) / 1e9 if per_launch_ms else None
    traffic = None
    if dominant in NCU_TRAFFIC.get(args.workload, {}):
        per, val = NCU_TRAFFIC[args.workload][dominant]
        traffic = val * (wl.units_per_step if per == "token" else 1.0) / launches_per_step
    launches = sum(v[1] for v in prof.values())   # library kernels per timed region (graph replays launch the same kernels)
    total_units = wl.units_per_step * world * args.steps
    line = {
        "metric": wl.metric, "value": total_units / (ms * 1e-3), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(),
        "e2e": {"value": total_units / (ms_e2e * 1e-3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": (achieved / peak) if achieved else None, "peak_source": peak_kind + " (of measured copy bandwidth)"
                     if peak_kind == "measured" else "fallback", "traffic": traffic,
                     "algorithmic_bytes_per_launch": dominant_bytes / launches_per_step, "step_algorithmic_bytes": wl.alg_bytes,
                     "step_frac_of_hbm_roofline": (wl.alg_bytes / peak / 1e9) / (ms / args.steps * 1e-3), "kernel_ms_per_launch": per_launch_ms,
                     "kernels": {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps} for k, v in prof.items()}},
    }
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.workload)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
