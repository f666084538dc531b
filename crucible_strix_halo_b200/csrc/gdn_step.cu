// Gated DeltaNet decode / speculative-verify step for sm_100a.
//
// One thread-block CLUSTER of 4 CTAs per (value head, span): CTA c of the cluster owns value columns
// [32c, 32c+32) of the head's 128x128 fp32 state (16 KB, 16 registers per thread), because the delta rule
// never mixes value columns.  The only cross-column quantity, the RMS of the 128-wide readout, is
// exchanged through distributed shared memory once per call.  The state slice is streamed with 128-bit loads
// (each warp load covers 4 key rows x 128 B) while the row prologue (conv + SiLU, L2 norms, a/b GEMV) runs.
//
// Semantics follow GdnKernel (engine/layers/ops.h:252-401): replay of pending rows, per-row update with the
// readout from the updated state, state stored after row commit-1, rows >= commit recorded as
// (khat, v, decay, beta), gated RMSNorm readout, raw-row ring update.
#include <cooperative_groups.h>
#include "common.cuh"

namespace cg = cooperative_groups;

namespace cr {

constexpr int kStepRows = CR_MAX_STEP_ROWS;

struct GdnStepParams {
  cr_gdn_args span[kMaxSpans];
  int Hv, Hk, hidden, pend_rows, fmt;
};

__global__ void __cluster_dims__(4, 1, 1) __launch_bounds__(256)
gdn_step_kernel(const __grid_constant__ GdnStepParams P) {
  const cr_gdn_args& a = P.span[blockIdx.y];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int h = blockIdx.x >> 2;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int rep = P.Hv / P.Hk, kh = h / rep;
  const int KW = P.Hk * 128, VW = P.Hv * 128, C = 2 * KW + VW;
  const int colbase = rank * 32, c4 = (l & 7) * 4;
  const int R = a.R;

  __shared__ __align__(16) float qs[kStepRows][128];
  __shared__ __align__(16) float ks[kStepRows][128];
  __shared__ __align__(16) float vs[kStepRows][32];
  __shared__ __align__(16) float ys[kStepRows][32];
  __shared__ __align__(16) float kbuf[128];
  __shared__ __align__(16) float part[8][32];
  __shared__ __align__(16) float party[8][32];
  __shared__ float red_qk[kStepRows][8], red_a[kStepRows][8], red_b[kStepRows][8];
  __shared__ float dec[kStepRows], bet[kStepRows];
  __shared__ float ssq[kStepRows];                       // read by the other CTAs of the cluster
  __shared__ __align__(16) float ob[kStepRows][128];     // rank 0's copy is written by the whole cluster

  // ---- state slice -> registers: lane holds key rows 16w + 4i + l/8 (i < 4), columns colbase + c4 .. +3
  float S[4][4];
  int krow[4];
  float* st = a.state + (size_t)h * 16384 + colbase + c4;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    krow[i] = 16 * w + 4 * i + (l >> 3);
    const float4 v = *reinterpret_cast<const float4*>(st + (size_t)krow[i] * 128);
    S[i][0] = v.x; S[i][1] = v.y; S[i][2] = v.z; S[i][3] = v.w;
  }

  // One delta-rule update of the register slice.  kv: the 128 normalised key values; qv: the query values or
  // nullptr (replay has no readout).  Two block barriers per call.
  auto update = [&](const float* kv, const float* qv, float decay, float beta, const float vcol[4], float* yrow) {
    float kk[4], m[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      kk[i] = kv[krow[i]];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        S[i][c] *= decay;
        m[c] = fmaf(S[i][c], kk[i], m[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      m[c] += __shfl_xor_sync(0xffffffffu, m[c], 8);
      m[c] += __shfl_xor_sync(0xffffffffu, m[c], 16);
    }
    if (l < 8) *reinterpret_cast<float4*>(&part[w][c4]) = make_float4(m[0], m[1], m[2], m[3]);
    __syncthreads();
    float mem[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ww = 0; ww < 8; ++ww) {
      const float4 p = *reinterpret_cast<const float4*>(&part[ww][c4]);
      mem[0] += p.x; mem[1] += p.y; mem[2] += p.z; mem[3] += p.w;
    }
    float delta[4], y[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < 4; ++c) delta[c] = beta * (vcol[c] - mem[c]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float qq = qv ? qv[krow[i]] : 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        S[i][c] = fmaf(kk[i], delta[c], S[i][c]);
        y[c] = fmaf(S[i][c], qq, y[c]);
      }
    }
    if (qv) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        y[c] += __shfl_xor_sync(0xffffffffu, y[c], 8);
        y[c] += __shfl_xor_sync(0xffffffffu, y[c], 16);
      }
      if (l < 8) *reinterpret_cast<float4*>(&party[w][c4]) = make_float4(y[0], y[1], y[2], y[3]);
    }
    __syncthreads();
    if (qv && t < 32) {
      float s = 0.f;
#pragma unroll
      for (int ww = 0; ww < 8; ++ww) s += party[ww][t];
      yrow[t] = s;
    }
  };

  // ---- lazy commit: fold the accepted rows of the previous pass into the state (no readout)
  for (int i = 0; i < a.replay; ++i) {
    const float* pe = a.pend + ((size_t)h * P.pend_rows + i) * CR_PEND_FLOATS;
    __syncthreads();
    if (t < 128) kbuf[t] = pe[t];
    __syncthreads();
    float vcol[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) vcol[c] = pe[128 + colbase + c4 + c];
    update(kbuf, nullptr, pe[256], pe[257], vcol, nullptr);
  }
  // Every CTA of the cluster has read the old pending rows before any of them records new ones.
  if (a.replay > 0 && R > a.commit) cluster.sync();

  // ---- row prologue for all rows: conv + SiLU, squared norms, a/b dot products
  const float A = -__expf(a.A_log[h]), dtb = a.dt_bias[h];
  const float* qkv = reinterpret_cast<const float*>(a.qkv);
  const float* zrow = reinterpret_cast<const float*>(a.z);
  for (int r = 0; r < R; ++r) {
    const int p = a.pos0 + r;
    auto tap = [&](int ch, int back) -> float {
      const int rr = r - back;
      if (rr >= 0) return qkv[(size_t)rr * C + ch];
      if (p - back < 0) return 0.f;
      return a.hist[(size_t)((p - back) & 15) * C + ch];
    };
    auto conv = [&](int ch) -> float {
      const float4 wv = *reinterpret_cast<const float4*>(a.conv + (size_t)ch * 4);
      float c = wv.x * tap(ch, 3);
      c = fmaf(wv.y, tap(ch, 2), c);
      c = fmaf(wv.z, tap(ch, 1), c);
      c = fmaf(wv.w, tap(ch, 0), c);
      return siluf_(c);
    };
    const float cqk = conv(t < 128 ? kh * 128 + t : KW + kh * 128 + (t - 128));
    if (t < 128) qs[r][t] = cqk; else ks[r][t - 128] = cqk;
    if (t < 32) vs[r][t] = conv(2 * KW + h * 128 + colbase + t);
    float pa = 0.f, pb = 0.f;
    const float* xr = a.x + (size_t)r * P.hidden;
    const __half* wa = reinterpret_cast<const __half*>(a.ab) + (size_t)h * P.hidden;
    const __half* wb = reinterpret_cast<const __half*>(a.ab) + (size_t)(P.Hv + h) * P.hidden;
    for (int i8 = t; i8 < P.hidden / 8; i8 += 256) {
      const float4 x0 = *reinterpret_cast<const float4*>(xr + i8 * 8);
      const float4 x1 = *reinterpret_cast<const float4*>(xr + i8 * 8 + 4);
      const uint4 ua = *reinterpret_cast<const uint4*>(wa + i8 * 8);
      const uint4 ub = *reinterpret_cast<const uint4*>(wb + i8 * 8);
      const __half2* ha = reinterpret_cast<const __half2*>(&ua);
      const __half2* hb = reinterpret_cast<const __half2*>(&ub);
      const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __half22float2(ha[j]), fb = __half22float2(hb[j]);
        pa = fmaf(fa.x, xs[2 * j], pa); pa = fmaf(fa.y, xs[2 * j + 1], pa);
        pb = fmaf(fb.x, xs[2 * j], pb); pb = fmaf(fb.y, xs[2 * j + 1], pb);
      }
    }
    const float s2 = warp_sum(cqk * cqk);
    pa = warp_sum(pa);
    pb = warp_sum(pb);
    if (l == 0) { red_qk[r][w] = s2; red_a[r][w] = pa; red_b[r][w] = pb; }
  }
  __syncthreads();
  for (int r = 0; r < R; ++r) {
    if (t < 128) {
      const float sq = red_qk[r][0] + red_qk[r][1] + red_qk[r][2] + red_qk[r][3];
      qs[r][t] *= rsqrtf(sq + kEps) * kInvSqrt128;
    } else {
      const float sk = red_qk[r][4] + red_qk[r][5] + red_qk[r][6] + red_qk[r][7];
      ks[r][t - 128] *= rsqrtf(sk + kEps);
    }
  }
  if (t < R) {
    float pa = 0.f, pb = 0.f;
#pragma unroll
    for (int ww = 0; ww < 8; ++ww) { pa += red_a[t][ww]; pb += red_b[t][ww]; }
    const float sp = pa + dtb;
    const float softplus = sp > 20.f ? sp : log1pf(expf(sp));
    dec[t] = expf(A * softplus);
    bet[t] = sigmoidf_(pb);
  }
  __syncthreads();

  // ---- speculative rows: record (khat, v, decay, beta) for the next pass's replay
  for (int r = a.commit; r < R; ++r) {
    float* pe = a.pend + ((size_t)h * P.pend_rows + (r - a.commit)) * CR_PEND_FLOATS;
    if (rank == 0) {
      if (t < 128) pe[t] = ks[r][t];
      if (t == 128) pe[256] = dec[r];
      if (t == 129) pe[257] = bet[r];
    }
    if (t < 32) pe[128 + colbase + t] = vs[r][t];
  }

  // ---- the recurrence
  for (int r = 0; r < R; ++r) {
    float vcol[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) vcol[c] = vs[r][c4 + c];
    update(ks[r], qs[r], dec[r], bet[r], vcol, ys[r]);
    if (r == a.commit - 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<float4*>(st + (size_t)krow[i] * 128) = make_float4(S[i][0], S[i][1], S[i][2], S[i][3]);
    }
  }
  __syncthreads();

  // ---- gated RMSNorm over the head's 128 columns: partial sums of squares exchanged through DSMEM
  for (int r = w; r < R; r += 8) {
    const float v = ys[r][l];
    const float s = warp_sum(v * v);
    if (l == 0) ssq[r] = s;
  }
  cluster.sync();
  float* ob0 = cluster.map_shared_rank(&ob[0][0], 0);
  for (int r = w; r < R; r += 8) {
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) tot += cluster.map_shared_rank(ssq, k)[r];
    const int col = h * 128 + colbase + l;
    const float o = ys[r][l] * rsqrtf(tot * (1.f / 128.f) + kEps) * a.gamma[colbase + l] *
                    sigmoidf_(zrow[(size_t)r * VW + col]);
    if (P.fmt == CR_OUT_RAW_F32) reinterpret_cast<float*>(a.out)[(size_t)r * VW + col] = o;
    else if (P.fmt == CR_OUT_RAW_BF16) reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)r * VW + col] = __float2bfloat16(o);
    else ob0[r * 128 + colbase + l] = round_h(round_h(o) * __half2float(reinterpret_cast<const __half*>(a.suh_out)[col]));
  }
  cluster.sync();   // remote reads of ssq and remote writes of ob are complete
  if (P.fmt == CR_OUT_EXL3_WHT && rank == 0) {
    for (int r = w; r < R; r += 8) {
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = ob[r][l * 4 + i];
      wht128(v);
      __half* dst = reinterpret_cast<__half*>(a.out);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        dst[out_index(r, h * 128 + l * 4 + i, VW, a.pack_rows, a.pack_off)] = __float2half(v[i] * kHadNorm);
    }
  }

  // ---- raw-row ring: slots of this call never alias the three slots any CTA reads (R + 3 <= 16)
  for (int r = 0; r < R; ++r) {
    float* hs = a.hist + (size_t)((a.pos0 + r) & 15) * C;
    const float* q = qkv + (size_t)r * C;
    if (t < 32) {
      const int ch = 2 * KW + h * 128 + colbase + t;
      hs[ch] = q[ch];
    } else if (t < 96 && h % rep == 0) {
      const int ch = (t < 64 ? 0 : KW) + kh * 128 + colbase + ((t - 32) & 31);
      hs[ch] = q[ch];
    }
  }
}

}  // namespace cr

extern "C" cr_status cr_gdn_step(const cr_geometry* g, const cr_gdn_args* spans, int n_spans, int pend_rows,
                                 cr_out_format fmt, void* stream) {
  using namespace cr;
  if (cr_status s = check_geometry(g)) return s;
  CR_REQUIRE(spans && n_spans >= 1, "cr_gdn_step: no spans");
  use_stream((cudaStream_t)stream);
  CR_REQUIRE(pend_rows >= 1 && pend_rows <= 64, "cr_gdn_step: pend_rows %d out of range", pend_rows);
  CR_REQUIRE(fmt == CR_OUT_RAW_F32 || fmt == CR_OUT_RAW_BF16 || fmt == CR_OUT_EXL3_WHT, "cr_gdn_step: bad output format");
  for (int s = 0; s < n_spans; ++s) {
    const cr_gdn_args& a = spans[s];
    CR_REQUIRE(a.R >= 1 && a.R <= CR_MAX_STEP_ROWS, "cr_gdn_step: span %d has R=%d, need 1..%d", s, a.R, CR_MAX_STEP_ROWS);
    CR_REQUIRE(a.pos0 >= 0, "cr_gdn_step: span %d has negative pos0", s);
    CR_REQUIRE(a.commit >= 1 && a.commit <= a.R, "cr_gdn_step: span %d commit=%d must be in 1..R (a verify pass keeps at least one row)", s, a.commit);
    CR_REQUIRE(a.replay >= 0 && a.replay <= pend_rows, "cr_gdn_step: span %d replay=%d exceeds the pending rows", s, a.replay);
    CR_REQUIRE(a.R - a.commit <= pend_rows, "cr_gdn_step: span %d records %d pending rows, stride is %d", s, a.R - a.commit, pend_rows);
    CR_REQUIRE(a.qkv && a.z && a.x && a.ab && a.conv && a.A_log && a.dt_bias && a.gamma && a.hist && a.state && a.out,
               "cr_gdn_step: span %d has a null buffer", s);
    CR_REQUIRE(a.pend || (a.replay == 0 && a.commit == a.R), "cr_gdn_step: span %d needs a pending-row buffer", s);
    CR_REQUIRE(fmt != CR_OUT_EXL3_WHT || a.suh_out, "cr_gdn_step: span %d needs suh_out for the EXL3 output", s);
    CR_REQUIRE(fmt == CR_OUT_EXL3_WHT || a.pack_rows == 0, "cr_gdn_step: packed layout only with the EXL3 output");
  }
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    GdnStepParams P;
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    for (int s = 0; s < n; ++s) P.span[s] = spans[s0 + s];
    P.Hv = g->gdn_vheads; P.Hk = g->gdn_kheads; P.hidden = g->hidden; P.pend_rows = pend_rows; P.fmt = (int)fmt;
    gdn_step_kernel<<<dim3(4 * g->gdn_vheads, n), 256, 0, (cudaStream_t)stream>>>(P);
    CR_LAUNCH_CHECK("gdn_step_kernel");
  }
  return CR_OK;
}
