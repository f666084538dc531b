// QSA block selection for sm_100a: indexer scores over the pooled keys.
//
// Scores (QsaScoreKernel / QsaScoreRowsKernel, engine/layers/qsa_long.h:9-108): HBM-bound scan of the tiled
// fp32 pool [b/32][128][32].  One warp owns one 16 KB tile: lane = block, every load of the warp is one full
// 128-byte line, and a group of up to RT rows is scored from one read of the tile.
//
// The exact top-512 over these scores is in qsa_topk.cu.
#include <climits>
#include "qsa.cuh"

namespace cr {

// ---- scores --------------------------------------------------------------------------------------------
// grid (ceil(tiles/8), row groups, spans), 256 threads; blockIdx.y = group of RT consecutive rows.
template <int RT, bool RANGED>
__global__ void __launch_bounds__(256) qsa_score_kernel(const __grid_constant__ QsaParams P) {
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int rg0 = blockIdx.y * RT;
  if (rg0 >= a.R) return;
  const int nr = min(RT, a.R - rg0);
  const int nb_all = (a.pos0 + rg0 + nr) / 4;       // blocks complete for the last row of the group
  if (nb_all <= CR_SEL_BLOCKS) return;
  const int nb_hi = RANGED ? min(nb_all, P.b_hi) : nb_all;   // the scored range ends here
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
  const int tile = (RANGED ? P.b_lo / 32 : 0) + blockIdx.x * 8 + w;
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
    if constexpr (RANGED) { if (b < P.b_lo || b >= P.b_hi) continue; }
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
// RANGED: only the blocks [P.b_lo, P.b_hi) are scored (a rank's own blocks).  A separate instantiation: with the range
// tests in it the whole-row kernel measured 40 us instead of 29 for four 262,144-token rows.
template <int RT, bool RANGED>
__global__ void __launch_bounds__(256) qsa_score4_kernel(const __grid_constant__ QsaParams P) {
  pdl_release();
  pdl_wait();
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int rg0 = blockIdx.y * RT;
  if (rg0 >= a.R) return;
  const int nr = min(RT, a.R - rg0);
  const int nb_all = (a.pos0 + rg0 + nr) / 4;
  if (nb_all <= CR_SEL_BLOCKS) return;
  const int nb_hi = RANGED ? min(nb_all, P.b_hi) : nb_all;
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
  const int tile = (RANGED ? P.b_lo / 32 : 0) + blockIdx.x * 8 + w;
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
      if constexpr (RANGED) { if (blk < P.b_lo || blk >= P.b_hi) continue; }
      float s = fmaxf(acc[r][b][0], 0.f);
      s += fmaxf(acc[r][b][1], 0.f);
      s += fmaxf(acc[r][b][2], 0.f);
      s += fmaxf(acc[r][b][3], 0.f);
      a.scores[(size_t)(rg0 + r) * a.sstride + blk] = s * kInvSqrt128;
    }
  }
}

template <int RT>
static cr_status score_launch_t(const QsaParams& P, int tiles, int Rmax, int n, bool ranged, cudaStream_t stream) {
  const dim3 grid((tiles + 7) / 8, (Rmax + RT - 1) / RT, n);
  if (ranged) qsa_score_kernel<RT, true><<<grid, 256, 0, stream>>>(P);
  else qsa_score_kernel<RT, false><<<grid, 256, 0, stream>>>(P);
  CR_LAUNCH_CHECK("qsa_score_kernel");
  return CR_OK;
}

cr_status qsa_score_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream, int b_lo, int b_hi) {
  use_stream(stream);
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    P.b_lo = b_lo; P.b_hi = b_hi;
    const bool ranged = b_lo > 0 || b_hi < INT_MAX;
    const int Rmax = qsa_max_rows(spans + s0, n);
    int nb_max = 0;
    for (int s = 0; s < n; ++s) nb_max = max(nb_max, (spans[s0 + s].pos0 + spans[s0 + s].R) / 4);
    if (nb_max <= CR_SEL_BLOCKS) continue;
    const int hi = nb_max < b_hi ? nb_max : b_hi;
    if (hi <= b_lo) continue;                       // the range holds no complete block of these rows
    const int tiles = (hi + 31) / 32 - b_lo / 32;   // 32-block pool tiles that overlap the scored range
    cr_status st;
    if (Rmax <= 2) {
      const dim3 grid((tiles + 7) / 8, 1, n);
      if (ranged) {
        if (Rmax == 1) CR_CUDA(launch_pdl(qsa_score4_kernel<1, true>, grid, dim3(256), 0, stream, P));
        else CR_CUDA(launch_pdl(qsa_score4_kernel<2, true>, grid, dim3(256), 0, stream, P));
      } else {
        if (Rmax == 1) CR_CUDA(launch_pdl(qsa_score4_kernel<1, false>, grid, dim3(256), 0, stream, P));
        else CR_CUDA(launch_pdl(qsa_score4_kernel<2, false>, grid, dim3(256), 0, stream, P));
      }
      CR_LAUNCH_CHECK("qsa_score_kernel");
      st = CR_OK;
    }
    else if (Rmax <= 16 && !ranged && !options().qsa_score_simt) st = qsa_score_mma_launch(P, tiles, Rmax, n, stream);   // verify spans
    else if (Rmax >= 8 && !options().qsa_score_simt) st = qsa_score_tc_launch(P, Rmax, n, stream);   // prefill parts (and a rank's range of a span)
    else if (Rmax <= 4) st = score_launch_t<4>(P, tiles, Rmax, n, ranged, stream);
    else st = score_launch_t<8>(P, tiles, Rmax, n, ranged, stream);
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
