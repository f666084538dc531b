// QSA block selection for sm_100a: indexer scores over the pooled keys and the exact top-512.
//
// Scores (QsaScoreKernel / QsaScoreRowsKernel, engine/layers/qsa_long.h:9-108): HBM-bound scan of the tiled
// fp32 pool [b/32][128][32].  One warp owns one 16 KB tile: lane = block, every load of the warp is one full
// 128-byte line, and a group of up to RT rows is scored from one read of the tile.
//
// Top-512 (LaunchQsaTop, engine/layers/qsa_long.h:111-380): total order (score desc, block id asc), emitted
// in ascending id.  Scores are >= +0, so their fp32 bit patterns order like unsigned integers: four byte-radix
// histogram passes find the bit pattern of the 512th score and how many of its ties are taken; ordered ballots
// emit.  The same body serves a rank's local candidates and the merge of gathered candidates (split-KV).
#include <climits>
#include "qsa.cuh"

namespace cr {

// ---- scores --------------------------------------------------------------------------------------------
// grid (ceil(tiles/8), row groups, spans), 256 threads; blockIdx.y = group of RT consecutive rows.
template <int RT>
__global__ void __launch_bounds__(256) qsa_score_kernel(const __grid_constant__ QsaParams P) {
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int rg0 = blockIdx.y * RT;
  if (rg0 >= a.R) return;
  const int nr = min(RT, a.R - rg0);
  const int nb_hi = (a.pos0 + rg0 + nr) / 4;        // blocks complete for the last row of the group
  if (nb_hi <= CR_SEL_BLOCKS) return;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  __shared__ float4 iqs[128][RT];                    // [dim][row] = the 4 indexer heads
  for (int i = t; i < 128 * RT; i += 256) {
    const int d = i / RT, r = i % RT;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < nr) {
      const float* iq = a.idx + (size_t)(rg0 + r) * 640;
      v = make_float4(iq[d], iq[128 + d], iq[256 + d], iq[384 + d]);
    }
    iqs[d][r] = v;
  }
  __syncthreads();
  const int tile = blockIdx.x * 8 + w;
  if (tile * 32 >= nb_hi) return;
  const int b = tile * 32 + l;
  const float* pt = a.c.ik_pool + (size_t)tile * 4096 + l;
  float acc[RT][4];
#pragma unroll
  for (int r = 0; r < RT; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
#pragma unroll 4
  for (int d0 = 0; d0 < 128; d0 += 16) {
    float key[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) key[j] = __ldg(pt + (d0 + j) * 32);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        const float4 q = iqs[d0 + j][r];
        acc[r][0] = fmaf(q.x, key[j], acc[r][0]);
        acc[r][1] = fmaf(q.y, key[j], acc[r][1]);
        acc[r][2] = fmaf(q.z, key[j], acc[r][2]);
        acc[r][3] = fmaf(q.w, key[j], acc[r][3]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RT; ++r) {
    if (r >= nr) break;
    const int nb = (a.pos0 + rg0 + r + 1) / 4;
    if (nb <= CR_SEL_BLOCKS || b >= nb) continue;
    float s = fmaxf(acc[r][0], 0.f);
    s += fmaxf(acc[r][1], 0.f);
    s += fmaxf(acc[r][2], 0.f);
    s += fmaxf(acc[r][3], 0.f);
    a.scores[(size_t)(rg0 + r) * a.sstride + b] = s * kInvSqrt128;
  }
}

// Same scores for one or two rows with 128-bit loads: lane l reads blocks 4(l%8)..+3 of dims l/8, l/8+4, ...,
// so a warp load covers four 128-byte lines and the tile costs 32 load instructions per lane instead of 128.
// The four lanes that share a block group add their partial dots with two shuffles.
template <int RT>
__global__ void __launch_bounds__(256) qsa_score4_kernel(const __grid_constant__ QsaParams P) {
  pdl_release();
  pdl_wait();
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int rg0 = blockIdx.y * RT;
  if (rg0 >= a.R) return;
  const int nr = min(RT, a.R - rg0);
  const int nb_hi = (a.pos0 + rg0 + nr) / 4;
  if (nb_hi <= CR_SEL_BLOCKS) return;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  __shared__ float4 iqs[128][RT];
  for (int i = t; i < 128 * RT; i += 256) {
    const int d = i / RT, r = i % RT;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < nr) {
      const float* iq = a.idx + (size_t)(rg0 + r) * 640;
      v = make_float4(iq[d], iq[128 + d], iq[256 + d], iq[384 + d]);
    }
    iqs[d][r] = v;
  }
  __syncthreads();
  const int tile = blockIdx.x * 8 + w;
  if (tile * 32 >= nb_hi) return;
  const int bq = (l & 7) * 4, dl = l >> 3;
  const float4* pt = reinterpret_cast<const float4*>(a.c.ik_pool + (size_t)tile * 4096 + dl * 32 + bq);
  float acc[RT][4][4];                        // [row][block][head]
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[r][b][0] = acc[r][b][1] = acc[r][b][2] = acc[r][b][3] = 0.f;
#pragma unroll
  for (int it0 = 0; it0 < 32; it0 += 8) {
    float4 key[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) key[j] = __ldg(pt + (it0 + j) * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float kb[4] = {key[j].x, key[j].y, key[j].z, key[j].w};
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        const float4 q = iqs[(it0 + j) * 4 + dl][r];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          acc[r][b][0] = fmaf(q.x, kb[b], acc[r][b][0]);
          acc[r][b][1] = fmaf(q.y, kb[b], acc[r][b][1]);
          acc[r][b][2] = fmaf(q.z, kb[b], acc[r][b][2]);
          acc[r][b][3] = fmaf(q.w, kb[b], acc[r][b][3]);
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RT; ++r)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        acc[r][b][h] += __shfl_xor_sync(0xffffffffu, acc[r][b][h], 8);
        acc[r][b][h] += __shfl_xor_sync(0xffffffffu, acc[r][b][h], 16);
      }
  if (dl != 0) return;
#pragma unroll
  for (int r = 0; r < RT; ++r) {
    if (r >= nr) break;
    const int nb = (a.pos0 + rg0 + r + 1) / 4;
    if (nb <= CR_SEL_BLOCKS) continue;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int blk = tile * 32 + bq + b;
      if (blk >= nb) continue;
      float s = fmaxf(acc[r][b][0], 0.f);
      s += fmaxf(acc[r][b][1], 0.f);
      s += fmaxf(acc[r][b][2], 0.f);
      s += fmaxf(acc[r][b][3], 0.f);
      a.scores[(size_t)(rg0 + r) * a.sstride + blk] = s * kInvSqrt128;
    }
  }
}

// ---- exact top-512 ------------------------------------------------------------------------------------
// Source element idx lives at keys[(idx / 512) * group_stride + idx % 512] (group_stride = 512: contiguous);
// ids (optional) uses the same addressing and marks padding with id < 0.  1024 threads.
// REG: the row's bit patterns stay in PT registers per thread; otherwise every pass re-reads them.
template <int PT, bool REG>
__device__ __forceinline__ void topk_body(const float* keys, const int* ids, size_t group_stride, int count, int id_base,
                                          int* out_ids, float* out_scores) {
  __shared__ unsigned hist[8][256];
  __shared__ unsigned wtot[32], gt_pre[33], eq_pre[33];
  __shared__ unsigned s_prefix, s_remaining;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int per = (count + 1023) / 1024;
  const int span = per * 32, begin = w * span, end = min(begin + span, count);
  auto addr = [&](int idx) -> size_t { return (size_t)(idx >> 9) * group_stride + (idx & 511); };
  auto fetch = [&](int i, bool& valid) -> unsigned {
    const int idx = begin + 32 * i + l;
    valid = idx < end;
    if (!valid) return 0u;
    const size_t ad = addr(idx);
    if (ids && ids[ad] < 0) { valid = false; return 0u; }
    return __float_as_uint(keys[ad]);
  };
  unsigned u[REG ? PT : 1];
  unsigned long long vmask = 0ull;
  if constexpr (REG) {
#pragma unroll
    for (int i = 0; i < PT; ++i) {
      bool valid = false;
      u[i] = i < per ? fetch(i, valid) : 0u;
      if (valid) vmask |= 1ull << i;
    }
  }
  auto get = [&](int i, bool& valid) -> unsigned {
    if constexpr (REG) { valid = (vmask >> i) & 1ull; return u[i]; }
    else return fetch(i, valid);
  };
  if (t == 0) { s_prefix = 0u; s_remaining = CR_SEL_BLOCKS; }
  unsigned mask = 0u;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = t; i < 8 * 256; i += 1024) (&hist[0][0])[i] = 0u;
    __syncthreads();
    const unsigned prefix = s_prefix, remaining = s_remaining;
    unsigned last = 0u, run = 0u;
    auto body = [&](int i) {
      bool valid;
      const unsigned v = get(i, valid);
      if (!valid || (v & mask) != prefix) return;
      const unsigned bin = (v >> shift) & 255u;
      if (run && bin != last) { atomicAdd(&hist[w & 7][last], run); run = 0u; }
      last = bin; ++run;
    };
    if constexpr (REG) {
#pragma unroll
      for (int i = 0; i < PT; ++i) body(i);
    } else {
      for (int i = 0; i < per; ++i) body(i);
    }
    if (run) atomicAdd(&hist[w & 7][last], run);
    __syncthreads();
    unsigned c = 0u, inc = 0u;
    if (t < 256) {                       // thread j looks at bin 255 - j: descending key order
#pragma unroll
      for (int rep = 0; rep < 8; ++rep) c += hist[rep][255 - t];
      inc = c;
#pragma unroll
      for (int step = 1; step < 32; step <<= 1) {
        const unsigned v = __shfl_up_sync(0xffffffffu, inc, step);
        if (l >= step) inc += v;
      }
      if (l == 31) wtot[w] = inc;
    }
    __syncthreads();
    if (t < 256) {
      for (int ww = 0; ww < w; ++ww) inc += wtot[ww];
      const unsigned exc = inc - c;
      if (exc < remaining && inc >= remaining) {
        s_prefix = prefix | ((unsigned)(255 - t) << shift);
        s_remaining = remaining - exc;
      }
    }
    __syncthreads();
    mask |= 255u << shift;
  }
  const unsigned thr = s_prefix, need = s_remaining;
  unsigned gt = 0u, eq = 0u;
  auto tally = [&](int i) {
    bool valid;
    const unsigned v = get(i, valid);
    if (valid) { gt += v > thr; eq += v == thr; }
  };
  if constexpr (REG) {
#pragma unroll
    for (int i = 0; i < PT; ++i) tally(i);
  } else {
    for (int i = 0; i < per; ++i) tally(i);
  }
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) {
    gt += __shfl_xor_sync(0xffffffffu, gt, step);
    eq += __shfl_xor_sync(0xffffffffu, eq, step);
  }
  if (l == 0) { gt_pre[w + 1] = gt; eq_pre[w + 1] = eq; }
  __syncthreads();
  if (t == 0) {
    gt_pre[0] = eq_pre[0] = 0u;
    for (int ww = 1; ww <= 32; ++ww) { gt_pre[ww] += gt_pre[ww - 1]; eq_pre[ww] += eq_pre[ww - 1]; }
  }
  __syncthreads();
  unsigned tie = eq_pre[w];
  unsigned out = gt_pre[w] + min(tie, need);
  const unsigned lower = (1u << l) - 1u;
  auto emit = [&](int i) {
    bool valid;
    const unsigned v = get(i, valid);
    const unsigned eqmask = __ballot_sync(0xffffffffu, valid && v == thr);
    const bool keep = valid && (v > thr || (v == thr && tie + __popc(eqmask & lower) < need));
    const unsigned chosen = __ballot_sync(0xffffffffu, keep);
    if (keep) {
      const int idx = begin + 32 * i + l;
      const unsigned pos = out + __popc(chosen & lower);
      out_ids[pos] = ids ? ids[addr(idx)] : id_base + idx;
      if (out_scores) out_scores[pos] = __uint_as_float(v);
    }
    tie += __popc(eqmask);
    out += __popc(chosen);
  };
  if constexpr (REG) {
#pragma unroll
    for (int i = 0; i < PT; ++i) {
      if (begin + 32 * i >= end) break;    // warp uniform
      emit(i);
    }
  } else {
    for (int i = 0; i < per && begin + 32 * i < end; ++i) emit(i);
  }
}

template <int PT, bool REG>
__global__ void __launch_bounds__(1024) qsa_topk_kernel(const __grid_constant__ QsaParams P) {
  const cr_qsa_args& a = P.span[blockIdx.y];
  const int r = blockIdx.x;
  if (r >= a.R) return;
  const int nb = (a.pos0 + r + 1) / 4;
  if (nb <= CR_SEL_BLOCKS) { if (threadIdx.x == 0) a.nsel[r] = -1; return; }
  topk_body<PT, REG>(a.scores + (size_t)r * a.sstride, nullptr, 512, nb, 0, a.sel + (size_t)r * CR_SEL_BLOCKS, nullptr);
  if (threadIdx.x == 0) a.nsel[r] = CR_SEL_BLOCKS;
}

// A rank's candidates among blocks [b0, b1): its top-512 (score, id), ascending id, padded with -1.
template <int PT, bool REG>
__global__ void __launch_bounds__(1024) qsa_candidates_kernel(const __grid_constant__ QsaParams P, int b0, int b1,
                                                              float* cand_scores, int* cand_ids) {
  const cr_qsa_args& a = P.span[0];
  const int r = blockIdx.x, t = threadIdx.x;
  const int nb = (a.pos0 + r + 1) / 4;
  float* cs = cand_scores + (size_t)r * CR_SEL_BLOCKS;
  int* ci = cand_ids + (size_t)r * CR_SEL_BLOCKS;
  const int hi = min(nb, b1), count = hi - b0;
  if (nb <= CR_SEL_BLOCKS || count <= CR_SEL_BLOCKS) {
    if (t < CR_SEL_BLOCKS) {
      const bool have = nb > CR_SEL_BLOCKS && t < count;
      cs[t] = have ? a.scores[(size_t)r * a.sstride + b0 + t] : -1.f;
      ci[t] = have ? b0 + t : -1;
    }
    return;
  }
  topk_body<PT, REG>(a.scores + (size_t)r * a.sstride + b0, nullptr, 512, count, b0, ci, cs);
}

// Global selection from the gathered candidates [ranks][rows][512] of all ranks.
__global__ void __launch_bounds__(1024) qsa_merge_candidates_kernel(const __grid_constant__ QsaParams P, int ranks,
                                                                    const float* cand_scores, const int* cand_ids) {
  const cr_qsa_args& a = P.span[0];
  const int r = blockIdx.x;
  const int nb = (a.pos0 + r + 1) / 4;
  if (nb <= CR_SEL_BLOCKS) { if (threadIdx.x == 0) a.nsel[r] = -1; return; }
  const size_t off = (size_t)r * CR_SEL_BLOCKS;
  topk_body<8, true>(cand_scores + off, cand_ids + off, (size_t)a.R * CR_SEL_BLOCKS, ranks * CR_SEL_BLOCKS, 0,
                     a.sel + off, nullptr);
  if (threadIdx.x == 0) a.nsel[r] = CR_SEL_BLOCKS;
}

template <int RT>
static cr_status score_launch_t(const QsaParams& P, int tiles, int Rmax, int n, cudaStream_t stream) {
  qsa_score_kernel<RT><<<dim3((tiles + 7) / 8, (Rmax + RT - 1) / RT, n), 256, 0, stream>>>(P);
  CR_LAUNCH_CHECK("qsa_score_kernel");
  return CR_OK;
}

cr_status qsa_score_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream) {
  use_stream(stream);
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    const int Rmax = qsa_max_rows(spans + s0, n);
    int nb_max = 0;
    for (int s = 0; s < n; ++s) nb_max = max(nb_max, (spans[s0 + s].pos0 + spans[s0 + s].R) / 4);
    if (nb_max <= CR_SEL_BLOCKS) continue;
    const int tiles = (nb_max + 31) / 32;
    cr_status st;
    if (Rmax <= 2) {
      const dim3 grid((tiles + 7) / 8, 1, n);
      if (Rmax == 1) CR_CUDA(launch_pdl(qsa_score4_kernel<1>, grid, dim3(256), 0, stream, P));
      else CR_CUDA(launch_pdl(qsa_score4_kernel<2>, grid, dim3(256), 0, stream, P));
      CR_LAUNCH_CHECK("qsa_score_kernel");
      st = CR_OK;
    }
    else if (Rmax >= 32 && !options().qsa_score_simt) st = qsa_score_tc_launch(P, Rmax, n, stream);
    else if (Rmax <= 4) st = score_launch_t<4>(P, tiles, Rmax, n, stream);
    else st = score_launch_t<8>(P, tiles, Rmax, n, stream);
    if (st) return st;
  }
  return CR_OK;
}

// Picks the values held per thread from the largest block count of the launch.
template <typename F>
static cr_status topk_dispatch(int nb_max, F&& launch) {
  if (nb_max <= 8192) return launch(std::integral_constant<int, 8>{}, std::true_type{});
  if (nb_max <= 32768) return launch(std::integral_constant<int, 32>{}, std::true_type{});
  return launch(std::integral_constant<int, 1>{}, std::false_type{});
}

cr_status qsa_topk_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream) {
  use_stream(stream);
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    const int Rmax = qsa_max_rows(spans + s0, n);
    int nb_max = 0;
    for (int s = 0; s < n; ++s) nb_max = max(nb_max, (spans[s0 + s].pos0 + spans[s0 + s].R) / 4);
    if (nb_max > 8192 && nb_max <= 262144) {   // long rows: 8 SMs per row
      if (cr_status st = qsa_topk_cluster_launch(P, Rmax, n, nb_max, stream)) return st;
      continue;
    }
    cr_status st = topk_dispatch(nb_max, [&](auto pt, auto reg) -> cr_status {
      qsa_topk_kernel<decltype(pt)::value, decltype(reg)::value><<<dim3(Rmax, n), 1024, 0, stream>>>(P);
      CR_LAUNCH_CHECK("qsa_topk_kernel");
      return CR_OK;
    });
    if (st) return st;
  }
  return CR_OK;
}

cr_status qsa_select_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream) {
  if (cr_status s = qsa_score_launch(g, spans, n_spans, stream)) return s;
  return qsa_topk_launch(g, spans, n_spans, stream);
}

}  // namespace cr

extern "C" size_t cr_qsa_select_scratch_bytes(const cr_geometry*, int) { return 0; }

extern "C" cr_status cr_qsa_select(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void*, size_t, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, spans, n_spans, CR_MAX_PREFILL_ROWS, "cr_qsa_select")) return s;
  return qsa_select_launch(g, spans, n_spans, (cudaStream_t)stream);
}

extern "C" cr_status cr_qsa_shard_candidates(const cr_geometry* g, const cr_qsa_args* a, int b0, int b1, float* cand_scores,
                                             int* cand_ids, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_shard_candidates")) return s;
  CR_REQUIRE(cand_scores && cand_ids && b0 >= 0 && b1 >= b0, "cr_qsa_shard_candidates: bad block range or null output");
  QsaParams P;
  qsa_fill_params(P, g, a, 1);
  use_stream((cudaStream_t)stream);
  return topk_dispatch(b1 - b0, [&](auto pt, auto reg) -> cr_status {
    qsa_candidates_kernel<decltype(pt)::value, decltype(reg)::value><<<a->R, 1024, 0, (cudaStream_t)stream>>>(P, b0, b1, cand_scores, cand_ids);
    CR_LAUNCH_CHECK("qsa_candidates_kernel");
    return CR_OK;
  });
}

extern "C" cr_status cr_qsa_merge_candidates(const cr_geometry* g, const cr_qsa_args* a, int ranks, const float* cand_scores,
                                             const int* cand_ids, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_merge_candidates")) return s;
  CR_REQUIRE(cand_scores && cand_ids && ranks >= 1 && ranks <= 16, "cr_qsa_merge_candidates: need 1..16 ranks and candidate buffers");
  QsaParams P;
  qsa_fill_params(P, g, a, 1);
  use_stream((cudaStream_t)stream);
  qsa_merge_candidates_kernel<<<a->R, 1024, 0, (cudaStream_t)stream>>>(P, ranks, cand_scores, cand_ids);
  CR_LAUNCH_CHECK("qsa_merge_candidates_kernel");
  return CR_OK;
}
