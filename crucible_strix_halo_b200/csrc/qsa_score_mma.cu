// Indexer scores of short spans (3..16 rows: verify passes, short decode batches) as an HBM stream through
// mma.sync: the job of QsaScoreRowsKernel (engine/layers/qsa_long.h:44-108) for spans too long for the one-row stream
// (qsa_score4_kernel) and too short to fill the 128-row tiles of the tcgen05 kernel (qsa_score_tc.cu).
//
// The pool tile [128 dims][32 blocks] fp32 is, as it lies in HBM, the "column" operand of m16n8k16: a thread's B
// fragment is pool[d][b] for four dims and one block, so every load instruction of a warp is four full 32-byte sectors
// and nothing is transposed or staged.  Rows of the product are (row, indexer head) pairs, m = 4 r + h, so the four
// heads of a row sit in four neighbouring lanes and relu + sum is two shuffles.  Queries and pool values are split
// into fp16 head + remainder (hi hi + lo hi + hi lo, fp32 accumulation): scores agree with fp32 dot products to 1e-5.
// One warp owns whole tiles and walks them in steps of 16 dims x 16 blocks; the loads of three steps are in flight
// ahead of the one that multiplies.
#include "qsa.cuh"

namespace cr {

constexpr int kSmLd = 136;                   // halves per query row in shared memory (272 bytes: conflict-free ldmatrix)
constexpr int kSmTilesPerWarp = 4;

__device__ __forceinline__ void sm_ldsm_x4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sm_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// (x, y) as fp16 pair and the fp16 pair of what the rounding lost
__device__ __forceinline__ void split_pair(float x, float y, unsigned& hi, unsigned& lo) {
  const __half2 h = __floats2half2_rn(x, y);
  const float2 b = __half22float2(h);
  const __half2 r = __floats2half2_rn(x - b.x, y - b.y);
  hi = *reinterpret_cast<const unsigned*>(&h);
  lo = *reinterpret_cast<const unsigned*>(&r);
}

// grid (tile groups, 1, spans), 128 threads; MT = ceil(rows / 4) m-tiles of 16 (row, head) pairs.
template <int MT>
__global__ void __launch_bounds__(128, 4) qsa_score_mma_kernel(const __grid_constant__ QsaParams P) {
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int nb_all = (a.pos0 + a.R) / 4;              // blocks complete for the last row
  if (nb_all <= CR_SEL_BLOCKS || a.R > 4 * MT) return;
  __shared__ __align__(16) __half qh[16 * MT][kSmLd], ql[16 * MT][kSmLd];
  const int t = threadIdx.x, w = t >> 5, l = t & 31, g = l >> 2, tq = l & 3;
  for (int i = t; i < 16 * MT * 64; i += 128) {        // pairs of dims: row m = 4 r + h of the span's normalised indexer queries
    const int m = i >> 6, d = (i & 63) * 2, r = m >> 2, h = m & 3;
    float2 v = make_float2(0.f, 0.f);
    if (r < a.R) v = *reinterpret_cast<const float2*>(a.idx + (size_t)r * 640 + h * 128 + d);
    unsigned hi, lo;
    split_pair(v.x, v.y, hi, lo);
    *reinterpret_cast<unsigned*>(&qh[m][d]) = hi;
    *reinterpret_cast<unsigned*>(&ql[m][d]) = lo;
  }
  __syncthreads();
  const int tiles = (nb_all + 31) / 32;
  const int first = (blockIdx.x * 4 + w) * kSmTilesPerWarp;
  if (first >= tiles) return;
  const int last = min(first + kSmTilesPerWarp, tiles);
  // A step is one k-step (16 dims) of one half tile (16 blocks): this thread's 8 values are the dims
  // 16 ks + 2 tq + {0, 1, 8, 9} of the blocks 16 half + 8 nt + g.  Three steps are in flight ahead of the one in use.
  const int total = (last - first) * 16;
  auto fetch = [&](float (&v)[8], int step) {
    const int tile = first + (step >> 4), half = (step >> 3) & 1, ks = step & 7;
    const float* pt = a.c.ik_pool + (size_t)tile * 4096 + (16 * ks + 2 * tq) * 32 + 16 * half + g;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      v[4 * nt] = __ldg(pt + 8 * nt); v[4 * nt + 1] = __ldg(pt + 32 + 8 * nt);
      v[4 * nt + 2] = __ldg(pt + 256 + 8 * nt); v[4 * nt + 3] = __ldg(pt + 288 + 8 * nt);
    }
  };
  float ring[4][8];
  fetch(ring[0], 0); fetch(ring[1], 1); fetch(ring[2], 2);          // total >= 16
  float acc[MT][2][4];
  for (int s0 = 0; s0 < total; s0 += 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int step = s0 + j, ks = step & 7;
      if (step + 3 < total) fetch(ring[(j + 3) & 3], step + 3);
      if (ks == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) acc[m][nt][0] = acc[m][nt][1] = acc[m][nt][2] = acc[m][nt][3] = 0.f;
      }
      unsigned bh[2][2], bl[2][2];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        split_pair(ring[j][4 * nt], ring[j][4 * nt + 1], bh[nt][0], bl[nt][0]);
        split_pair(ring[j][4 * nt + 2], ring[j][4 * nt + 3], bh[nt][1], bl[nt][1]);
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        unsigned ah[4], al[4];
        sm_ldsm_x4(ah, &qh[16 * m + (l & 15)][16 * ks + (l >> 4) * 8]);
        sm_ldsm_x4(al, &ql[16 * m + (l & 15)][16 * ks + (l >> 4) * 8]);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          sm_mma(acc[m][nt], ah, bh[nt][0], bh[nt][1]);
          sm_mma(acc[m][nt], al, bh[nt][0], bh[nt][1]);
          sm_mma(acc[m][nt], ah, bl[nt][0], bl[nt][1]);
        }
      }
      if (ks != 7) continue;
      // relu per head, sum over the four heads of a row (lanes g, g ^ 1, g ^ 2, g ^ 3 of the same row quartet), scale, store
      const int blk0 = (first + (step >> 4)) * 32 + 16 * ((step >> 3) & 1);
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float sc[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            sc[i] = fmaxf(acc[m][nt][i], 0.f);
            sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], 4);
            sc[i] += __shfl_xor_sync(0xffffffffu, sc[i], 8);
          }
          if ((g & 3) == 0) {
            const int blk = blk0 + 8 * nt + 2 * tq;
#pragma unroll
            for (int half = 0; half < 2; ++half) {                   // accumulator rows g and g + 8: span rows 4 m + g / 4 and + 2
              const int r = 4 * m + 2 * half + (g >> 2);
              if (r >= a.R) continue;
              const int nb = (a.pos0 + r + 1) / 4;
              if (nb <= CR_SEL_BLOCKS) continue;
              float* dst = a.scores + (size_t)r * a.sstride + blk;
              if (blk < nb) dst[0] = sc[2 * half] * kInvSqrt128;
              if (blk + 1 < nb) dst[1] = sc[2 * half + 1] * kInvSqrt128;
            }
          }
        }
    }
  }
}

// Spans of 3..16 rows, every block of every row.
cr_status qsa_score_mma_launch(const QsaParams& P, int tiles, int Rmax, int n, cudaStream_t stream) {
  const dim3 grid((tiles + 4 * kSmTilesPerWarp - 1) / (4 * kSmTilesPerWarp), 1, n);
  const int mt = (Rmax + 3) / 4;
  if (mt <= 1) qsa_score_mma_kernel<1><<<grid, 128, 0, stream>>>(P);
  else if (mt == 2) qsa_score_mma_kernel<2><<<grid, 128, 0, stream>>>(P);
  else if (mt == 3) qsa_score_mma_kernel<3><<<grid, 128, 0, stream>>>(P);
  else qsa_score_mma_kernel<4><<<grid, 128, 0, stream>>>(P);
  CR_LAUNCH_CHECK("qsa_score_mma_kernel");
  return CR_OK;
}

}  // namespace cr
