// QSA attention over the attended positions for sm_100a (decode, verify, and the row-wise prefill path).
//
// Split-KV gather (QsaGqaSplitKernel, engine/layers/qsa_long.h:399-456): one CTA per (split, row, KV head);
// its warps are the query heads of the KV group and share every K/V row.  Positions are staged 32 at a time
// as fp16 in shared memory with 128-bit loads (the next tile is prefetched into registers while the current
// one is consumed).  QK^T runs position-parallel (lane = position, fp32 query broadcast from shared memory),
// PV runs channel-parallel (lane = 8 channels), so the only shuffles are one max and one sum per tile.
// Each CTA writes the partial (m, l, acc[256]) of its heads; the merge kernel (QsaMergeKernel,
// qsa_long.h:458-499) combines them by log-sum-exp, applies the sigmoid gate and the output transform.
// No CTA waits on another CTA.
#include <climits>
#include "qsa.cuh"

namespace cr {

constexpr int kTile = 32;            // positions per shared-memory tile
constexpr int kKRow = 264;           // padded K row (halves): 528 B keeps 128-bit column reads conflict-free
constexpr int kMaxGqa = 12;

__device__ __forceinline__ int qsa_position(const int* sel, int t, int ns, int nb) {
  return ns < 0 ? t : (t < ns * 4 ? sel[t >> 2] * 4 + (t & 3) : nb * 4 + t - ns * 4);
}

// grid (splits, Rmax * Hkv, spans); blockDim = 32 * gqa.
__global__ void __launch_bounds__(384) qsa_attn_split_kernel(const __grid_constant__ QsaParams P, float* partials,
                                                             int splits, int p0, int p1) {
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int r = blockIdx.y / P.Hkv, g = blockIdx.y % P.Hkv;
  if (r >= a.R) return;
  const int gqa = P.Hq / P.Hkv, nthr = 32 * gqa;
  const int t = threadIdx.x, w = t >> 5, l = t & 31, h = g * gqa + w;
  const int split = blockIdx.x;
  const int p = a.pos0 + r, ns = a.nsel[r], nb = (p + 1) / 4;
  const int n = ns < 0 ? p + 1 : ns * 4 + (p + 1) % 4;
  const int per = max(kTile, (n / splits) / kTile * kTile);   // decode: 64 per split, the last takes the rest
  const int begin = split * per, end = split == splits - 1 ? n : min(begin + per, n);
  const int* sel = a.sel + (size_t)r * CR_SEL_BLOCKS;

  __shared__ __align__(16) __half ksm[kTile][kKRow];
  __shared__ __align__(16) __half vsm[kTile][256];
  __shared__ __align__(16) float qsm[kMaxGqa][256];
  __shared__ int psm[kTile];

  for (int i = t; i < gqa * 256; i += nthr) qsm[i >> 8][i & 255] = a.q[((size_t)r * P.Hq + g * gqa + (i >> 8)) * 512 + (i & 255)];

  // Stage one tile: 32 positions x (32 K + 32 V) 16-byte pieces, spread over the CTA's threads.
  const int pieces = kTile * 64;
  const int ppt = (pieces + nthr - 1) / nthr;             // <= 8: the geometry check keeps gqa >= 8
  constexpr int kMaxPieces = 8;    // 2048 pieces over >= 256 threads
  uint4 stage[kMaxPieces];
  const __half* kc = reinterpret_cast<const __half*>(a.c.k);
  const __half* vc = reinterpret_cast<const __half*>(a.c.v);
  auto fetch = [&](int tile0) {
#pragma unroll
    for (int i = 0; i < kMaxPieces; ++i) {
      if (i >= ppt) break;
      const int piece = t + i * nthr;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (piece < pieces) {
        const int j = piece >> 6, c = piece & 63;
        const int ti = tile0 + j;
        if (ti < end) {
          const int pos = qsa_position(sel, ti, ns, nb);
          if (pos >= p0 && pos < p1) {
            const size_t off = ((size_t)pos * P.Hkv + g) * 256 + (c & 31) * 8;
            v = *reinterpret_cast<const uint4*>((c < 32 ? kc : vc) + off);
          }
        }
      }
      stage[i] = v;
    }
  };
  auto commit = [&](int tile0) {
#pragma unroll
    for (int i = 0; i < kMaxPieces; ++i) {
      if (i >= ppt) break;
      const int piece = t + i * nthr;
      if (piece < pieces) {
        const int j = piece >> 6, c = piece & 63;
        if (c < 32) *reinterpret_cast<uint4*>(&ksm[j][c * 8]) = stage[i];
        else *reinterpret_cast<uint4*>(&vsm[j][(c - 32) * 8]) = stage[i];
      }
    }
    if (t < kTile) {
      const int ti = tile0 + t;
      int pos = -1;
      if (ti < end) {
        pos = qsa_position(sel, ti, ns, nb);
        if (pos < p0 || pos >= p1) pos = -1;
      }
      psm[t] = pos;
    }
  };

  float m = -INFINITY, lsum = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (begin < end) fetch(begin);
  for (int tile0 = begin; tile0 < end; tile0 += kTile) {
    __syncthreads();                 // previous tile fully consumed (and qsm visible on the first pass)
    commit(tile0);
    __syncthreads();
    if (tile0 + kTile < end) fetch(tile0 + kTile);
    // QK^T: lane = position of the tile
    float s = -INFINITY;
    if (psm[l] >= 0) {
      const __half* krow = &ksm[l][0];
      const float* q = &qsm[w][0];
      float d0 = 0.f, d1 = 0.f;
#pragma unroll 4
      for (int c = 0; c < 256; c += 8) {
        const uint4 kv = *reinterpret_cast<const uint4*>(krow + c);
        const float4 qa = *reinterpret_cast<const float4*>(q + c);
        const float4 qb = *reinterpret_cast<const float4*>(q + c + 4);
        const __half2* kh = reinterpret_cast<const __half2*>(&kv);
        const float2 k0 = __half22float2(kh[0]), k1 = __half22float2(kh[1]);
        const float2 k2 = __half22float2(kh[2]), k3 = __half22float2(kh[3]);
        d0 = fmaf(qa.x, k0.x, d0); d1 = fmaf(qa.y, k0.y, d1);
        d0 = fmaf(qa.z, k1.x, d0); d1 = fmaf(qa.w, k1.y, d1);
        d0 = fmaf(qb.x, k2.x, d0); d1 = fmaf(qb.y, k2.y, d1);
        d0 = fmaf(qb.z, k3.x, d0); d1 = fmaf(qb.w, k3.y, d1);
      }
      s = (d0 + d1) * 0.0625f;
    }
    const float tmax = warp_max(s);
    if (tmax > -INFINITY) {            // warp uniform
      const float mn = fmaxf(m, tmax);
      const float corr = __expf(m - mn);      // m = -inf on the first tile: exp(-inf) = 0
      const float e = s > -INFINITY ? __expf(s - mn) : 0.f;
      lsum = lsum * corr + warp_sum(e);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= corr;
      m = mn;
      // PV: lane = channels 8l..8l+7
#pragma unroll 4
      for (int j = 0; j < kTile; ++j) {
        const float pj = __shfl_sync(0xffffffffu, e, j);
        const uint4 vv = *reinterpret_cast<const uint4*>(&vsm[j][l * 8]);
        const __half2* vh = reinterpret_cast<const __half2*>(&vv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(vh[i]);
          acc[2 * i] = fmaf(pj, f.x, acc[2 * i]);
          acc[2 * i + 1] = fmaf(pj, f.y, acc[2 * i + 1]);
        }
      }
    }
  }
  float* dst = partials + (((size_t)(P.base[blockIdx.z] + r) * P.Hq + h) * splits + split) * CR_QSA_PART;
  if (l == 0) { dst[0] = m; dst[1] = lsum; }
  // records are 8-byte aligned (258 floats): store pairs
#pragma unroll
  for (int i = 0; i < 8; i += 2) *reinterpret_cast<float2*>(dst + 2 + l * 8 + i) = make_float2(acc[i], acc[i + 1]);
}

// grid (Hq, Rmax, spans), 256 threads: thread d = output channel.
// Partial p of (row, head) is at partials[(part_major ? (p * rows_total + row) * Hq + h : (row * Hq + h) * nparts + p) * 258].
__global__ void __launch_bounds__(256) qsa_merge_kernel(const __grid_constant__ QsaParams P, const float* partials, int nparts,
                                                        int part_major, int rows_total, float* partial_out, int fmt) {
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int h = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
  if (r >= a.R) return;
  const int row = P.base[blockIdx.z] + r;
  __shared__ float ob[256];
  auto rec = [&](int p) -> const float* {
    const size_t i = part_major ? ((size_t)p * rows_total + row) * P.Hq + h : ((size_t)row * P.Hq + h) * nparts + p;
    return partials + i * CR_QSA_PART;
  };
  // (m, l) of the parts are combined by the first warp; every thread then sums its channel with the factors
  // from shared memory, so the loads of the second pass are independent of each other.
  __shared__ float fs[32];
  __shared__ float ml[2];
  if (d < 32) {
    float pm = -INFINITY, pl = 0.f;
    if (d < nparts) {
      const float2 v = *reinterpret_cast<const float2*>(rec(d));
      pl = v.y;
      pm = pl != 0.f ? v.x : -INFINITY;
    }
    const float mx = warp_max(pm);
    const float f = pl != 0.f ? __expf(pm - mx) : 0.f;
    const float lt = warp_sum(pl * f);
    fs[d] = f;
    if (d == 0) { ml[0] = mx; ml[1] = lt; }
  }
  __syncthreads();
  const float m = ml[0], lsum = ml[1];
  float o = 0.f;
#pragma unroll 8
  for (int p = 0; p < nparts; ++p) o = fmaf(rec(p)[2 + d], fs[p], o);
  if (partial_out) {      // shard mode: one merged partial per (row, head)
    float* dst = partial_out + ((size_t)row * P.Hq + h) * CR_QSA_PART;
    if (d == 0) { dst[0] = m; dst[1] = lsum; }
    dst[2 + d] = o;
    return;
  }
  o /= lsum;
  const size_t W = (size_t)P.Hq * 256;
  if (a.context) a.context[((size_t)r * P.Hq + h) * 256 + d] = o;
  o *= sigmoidf_(a.q[((size_t)r * P.Hq + h) * 512 + 256 + d]);
  if (fmt == CR_OUT_RAW_F32) { reinterpret_cast<float*>(a.out)[(size_t)r * W + h * 256 + d] = o; return; }
  if (fmt == CR_OUT_RAW_BF16) { reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)r * W + h * 256 + d] = __float2bfloat16(o); return; }
  ob[d] = round_h(round_h(o) * __half2float(reinterpret_cast<const __half*>(a.suh_o)[h * 256 + d]));
  __syncthreads();
  if (d < 64) {
    const int half = d >> 5, lane = d & 31;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = ob[half * 128 + lane * 4 + i];
    wht128(v);
    __half* dst = reinterpret_cast<__half*>(a.out);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      dst[out_index(r, h * 256 + half * 128 + lane * 4 + i, (int)W, a.pack_rows, a.pack_off)] = __float2half(v[i] * kHadNorm);
  }
}

cr_status qsa_attn_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, float* partials, int splits,
                          int p0, int p1, cudaStream_t stream) {
  use_stream(stream);
  int row_base = 0;
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    for (int s = 0; s < n; ++s) P.base[s] += row_base;
    const int Rmax = qsa_max_rows(spans + s0, n);
    qsa_attn_split_kernel<<<dim3(splits, Rmax * g->kv_heads, n), 32 * (g->q_heads / g->kv_heads), 0, stream>>>(P, partials, splits, p0, p1);
    CR_LAUNCH_CHECK("qsa_attn_split_kernel");
    for (int s = 0; s < n; ++s) row_base += spans[s0 + s].R;
  }
  return CR_OK;
}

cr_status qsa_merge_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, const float* partials, int nparts,
                           bool part_major, float* partial_out, cr_out_format fmt, cudaStream_t stream) {
  use_stream(stream);
  int rows_total = 0, row_base = 0;
  for (int s = 0; s < n_spans; ++s) rows_total += spans[s].R;
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    for (int s = 0; s < n; ++s) P.base[s] += row_base;
    const int Rmax = qsa_max_rows(spans + s0, n);
    qsa_merge_kernel<<<dim3(g->q_heads, Rmax, n), 256, 0, stream>>>(P, partials, nparts, part_major ? 1 : 0, rows_total, partial_out, (int)fmt);
    CR_LAUNCH_CHECK("qsa_merge_kernel");
    for (int s = 0; s < n; ++s) row_base += spans[s0 + s].R;
  }
  return CR_OK;
}

static cr_status check_out(const cr_qsa_args* spans, int n, cr_out_format fmt, const char* who) {
  CR_REQUIRE(fmt == CR_OUT_RAW_F32 || fmt == CR_OUT_RAW_BF16 || fmt == CR_OUT_EXL3_WHT, "%s: bad output format", who);
  for (int s = 0; s < n; ++s) {
    CR_REQUIRE(spans[s].out, "%s: span %d has no output buffer", who, s);
    CR_REQUIRE(fmt != CR_OUT_EXL3_WHT || spans[s].suh_o, "%s: span %d needs suh_o for the EXL3 output", who, s);
    CR_REQUIRE(fmt == CR_OUT_EXL3_WHT || spans[s].pack_rows == 0, "%s: packed layout only with the EXL3 output", who);
  }
  return CR_OK;
}

static size_t total_rows(const cr_qsa_args* spans, int n) {
  size_t r = 0;
  for (int s = 0; s < n; ++s) r += (size_t)spans[s].R;
  return r;
}

}  // namespace cr

extern "C" size_t cr_qsa_scratch_bytes(const cr_geometry* g, int rows) {
  if (!g || rows < 1) return 0;
  return (size_t)rows * g->q_heads * CR_QSA_SPLITS * CR_QSA_PART * sizeof(float);
}

extern "C" cr_status cr_qsa_attn(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* scratch, size_t scratch_bytes,
                                 cr_out_format fmt, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, spans, n_spans, CR_MAX_STEP_ROWS, "cr_qsa_attn")) return s;
  if (cr_status s = check_out(spans, n_spans, fmt, "cr_qsa_attn")) return s;
  const size_t need = cr_qsa_scratch_bytes(g, (int)total_rows(spans, n_spans));
  CR_REQUIRE(scratch && scratch_bytes >= need, "cr_qsa_attn: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  if (cr_status s = qsa_attn_launch(g, spans, n_spans, (float*)scratch, CR_QSA_SPLITS, 0, INT_MAX, (cudaStream_t)stream)) return s;
  return qsa_merge_launch(g, spans, n_spans, (const float*)scratch, CR_QSA_SPLITS, false, nullptr, fmt, (cudaStream_t)stream);
}

extern "C" cr_status cr_qsa_step(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* scratch, size_t scratch_bytes,
                                 cr_out_format fmt, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, spans, n_spans, CR_MAX_STEP_ROWS, "cr_qsa_step")) return s;
  if (cr_status s = check_out(spans, n_spans, fmt, "cr_qsa_step")) return s;
  const size_t need = cr_qsa_scratch_bytes(g, (int)total_rows(spans, n_spans));
  CR_REQUIRE(scratch && scratch_bytes >= need, "cr_qsa_step: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  if (cr_status s = qsa_prep_launch(g, spans, n_spans, 0, nullptr, 0, st)) return s;
  if (cr_status s = qsa_select_launch(g, spans, n_spans, st)) return s;
  if (cr_status s = qsa_attn_launch(g, spans, n_spans, (float*)scratch, CR_QSA_SPLITS, 0, INT_MAX, st)) return s;
  return qsa_merge_launch(g, spans, n_spans, (const float*)scratch, CR_QSA_SPLITS, false, nullptr, fmt, st);
}

extern "C" cr_status cr_qsa_shard_attn(const cr_geometry* g, const cr_qsa_args* a, int p0, int p1, float* partials, void* scratch,
                                       size_t scratch_bytes, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_shard_attn")) return s;
  CR_REQUIRE(partials && p0 >= 0 && p1 >= p0, "cr_qsa_shard_attn: bad position window or null output");
  const int splits = a->R <= CR_MAX_STEP_ROWS ? CR_QSA_SPLITS : 4;
  const size_t need = (size_t)a->R * g->q_heads * splits * CR_QSA_PART * sizeof(float);
  CR_REQUIRE(scratch && scratch_bytes >= need, "cr_qsa_shard_attn: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  if (cr_status s = qsa_attn_launch(g, a, 1, (float*)scratch, splits, p0, p1, (cudaStream_t)stream)) return s;
  return qsa_merge_launch(g, a, 1, (const float*)scratch, splits, false, partials, CR_OUT_RAW_F32, (cudaStream_t)stream);
}

extern "C" cr_status cr_qsa_merge_partials(const cr_geometry* g, const cr_qsa_args* a, int ranks, const float* partials,
                                           cr_out_format fmt, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_merge_partials")) return s;
  if (cr_status s = check_out(a, 1, fmt, "cr_qsa_merge_partials")) return s;
  CR_REQUIRE(partials && ranks >= 1 && ranks <= 32, "cr_qsa_merge_partials: need gathered partials of 1..32 ranks");
  return qsa_merge_launch(g, a, 1, partials, ranks, true, nullptr, fmt, (cudaStream_t)stream);
}
