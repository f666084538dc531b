// qsa_score_tc_kernel: indexer scores of a prefill part on tcgen05 tensor cores (kind::f16) (QsaPrefillSgprScoreKernel,
// engine/layers/kernels/prefill_qsa_score_sgpr.h:19-81, computes the same scores with fp32 FMAs).
//
//   score[r][b] = (sum_{h<4} max(iq[r][h] . pool[b], 0)) / sqrt(128)        for b < (pos0 + r + 1) / 4
//
// is four GEMMs of shape [blocks x 128] x [128 x rows] with a ReLU between them and their sum.  One CTA owns 64
// rows and a range of 128-block pool tiles.  M = 128 blocks (the pool tile is the A operand), N = 64 rows (the
// query panel of all four heads stays in shared memory as the B operand: N = 4 heads x 64 rows = 256 columns of one
// MMA), K = 128; the heads are the four 64-column quarters of a TMEM accumulator, two accumulators used in turn, so the epilogue of a tile (ReLU, sum over heads, scale, store)
// runs while the next tile is multiplied.  Precision: both operands are split into an fp16 head and an fp16
// remainder (22 mantissa bits together; the values are normalised rows, well inside the fp16 range) and three
// products are accumulated in fp32 (head x head, head x remainder, remainder x head); the error of a score
// stays below 1e-5 (measured 9e-6 against fp64 scores of the same operands; 4e-6 for the fp32 FMA kernel), far
// inside the 1e-3 gap within which selections may differ.  The pool is stored [dim][32 blocks] per 32-block tile, i.e. transposed for a K-major
// operand: eight staging warps read it with coalesced loads (prefetched into registers while the previous tile
// is multiplied), split it and write 16-byte K-major units.  Every wait is bounded and raises a status word.
#include "qsa.cuh"
#include "umma.cuh"

namespace cr {

CR_DEFINE_STATUS_WORD(qsa_score)

constexpr int kScRows = 64;                 // query rows per CTA (N)
constexpr int kScBlocks = 128;              // pool blocks per tile (M)
constexpr int kScThreads = 32 * 13;         // 4 epilogue warps, 8 staging warps, 1 issuer warp
constexpr int kQopBytes = 2 * 16 * 4 * kScRows * 16;      // [hi/lo][dim / 8][head][row][8 fp16]: N = (head, row) = 256 columns
constexpr int kPopBytes = 2 * 16 * kScBlocks * 16;        // [hi/lo][dim / 8][block][8 fp16]
constexpr size_t kScoreSmem = kQopBytes + kPopBytes + 128;

using umma::mma_f16_ss;
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N) { return umma::idesc_f16(M, N, false, false); }
// eight fp32 values -> fp16 heads and fp16 remainders, each packed into 16 bytes
__device__ __forceinline__ void split8(const float (&x)[8], uint4& hi, uint4& lo) {
  unsigned h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 a = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
    const float2 b = __half22float2(a);
    const __half2 c = __floats2half2_rn(x[2 * i] - b.x, x[2 * i + 1] - b.y);
    h[i] = *reinterpret_cast<const unsigned*>(&a);
    l[i] = *reinterpret_cast<const unsigned*>(&c);
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// grid (row tiles, splits, spans).
template <bool RANGED>
__global__ void __launch_bounds__(kScThreads, 1) qsa_score_tc_kernel(const __grid_constant__ QsaParams P) {
  extern __shared__ __align__(128) unsigned char sm[];
  unsigned char* Qop = sm;
  unsigned char* Pop = sm + kQopBytes;
  __shared__ __align__(8) uint64_t bars[6];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int dead;
  uint64_t *popFull = &bars[0], *mmaDone = &bars[1], *accFree = &bars[3];    // mmaDone[2], accFree[2]
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int r0 = blockIdx.x * kScRows;
  if (r0 >= a.R) return;
  const int rows = min(kScRows, a.R - r0);
  const int nb_all = (a.pos0 + r0 + rows) / 4;            // blocks visible to the last row of the tile
  if (nb_all <= CR_SEL_BLOCKS) return;
  const int nb_hi = RANGED ? min(nb_all, P.b_hi) : nb_all;   // RANGED: the scored range [b_lo, b_hi) of a rank
  const int tile_lo = RANGED ? P.b_lo / kScBlocks : 0, tiles = (nb_hi + kScBlocks - 1) / kScBlocks - tile_lo;
  if (tiles <= 0) return;
  const int t0 = tile_lo + (int)((long long)tiles * blockIdx.y / gridDim.y), t1 = tile_lo + (int)((long long)tiles * (blockIdx.y + 1) / gridDim.y);
  if (t0 >= t1) return;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;

  if (t == 0) {
    umma::mbar_init(popFull, 8);                          // one arrival per staging warp
    umma::mbar_init(&mmaDone[0], 1);
    umma::mbar_init(&mmaDone[1], 1);
    umma::mbar_init(&accFree[0], 4);                      // one arrival per epilogue warp
    umma::mbar_init(&accFree[1], 4);
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == 12) umma::tmem_alloc(&tmem_slot, 512);
  // query panel: rows r0 .. r0+63 of the four indexer heads, split and stored K-major
  for (int i = t; i < 4 * 16 * kScRows; i += kScThreads) {
    const int row = i % kScRows, dc = (i / kScRows) % 16, h = i / (kScRows * 16);
    float x[8];
    if (row < rows) {
      const float4* src = reinterpret_cast<const float4*>(a.idx + (size_t)(r0 + row) * 640 + h * 128 + dc * 8);
      const float4 u = src[0], v = src[1];
      x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w; x[4] = v.x; x[5] = v.y; x[6] = v.z; x[7] = v.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = 0.f;
    }
    uint4 hi, lo;
    split8(x, hi, lo);
    *reinterpret_cast<uint4*>(Qop + ((size_t)(dc * 4 + h) * kScRows + row) * 16) = hi;
    *reinterpret_cast<uint4*>(Qop + kQopBytes / 2 + ((size_t)(dc * 4 + h) * kScRows + row) * 16) = lo;
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  bool gave_up = false;
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (gave_up) return;
    if (!umma::mbar_wait_timed(bar, parity, &dead)) { gave_up = true; dead = 1; g_qsa_score_status = 1; }
  };

  if (w == 12) {
    // ------------------------------------------------------------------ issuer
    if (l == 0) {
      // One MMA covers the four heads: N = 4 x 64 (head, row) columns, so the pool tile is read once per k-step and
      // product instead of once per head (an MMA of N = 64 is bound by its 6 KB of shared-memory reads).
      constexpr uint32_t idesc = idesc_f16(kScBlocks, 4 * kScRows);
      const uint64_t dPh = umma::smem_desc(Pop, kScBlocks * 16, 128), dPl = umma::smem_desc(Pop + kPopBytes / 2, kScBlocks * 16, 128);
      const uint64_t dQh = umma::smem_desc(Qop, 4 * kScRows * 16, 128), dQl = umma::smem_desc(Qop + kQopBytes / 2, 4 * kScRows * 16, 128);
      for (int i = 0; i < t1 - t0; ++i) {
        const int buf = i & 1;
        wait(popFull, i & 1);
        if (i >= 2) wait(&accFree[buf], ((i >> 1) - 1) & 1);
        if (gave_up || dead) break;                        // no more tensor-core work once any wait has run out
        umma::fence_after_sync();
        const uint32_t d = tm + buf * 256;
        // a step of 16 along K is two 16-byte planes: 2 x 128 units of the pool tile, 2 x 256 of the query panel
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) mma_f16_ss(d, dPh + (uint64_t)(ks * 256), dQh + (uint64_t)(ks * 512), idesc, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) mma_f16_ss(d, dPh + (uint64_t)(ks * 256), dQl + (uint64_t)(ks * 512), idesc, 1u);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) mma_f16_ss(d, dPl + (uint64_t)(ks * 256), dQh + (uint64_t)(ks * 512), idesc, 1u);
        umma::commit(&mmaDone[buf]);
      }
    }
  } else if (w >= 4) {
    // ------------------------------------------------------------------ staging warps: pool tile -> K-major fp16 head + remainder
    const int sw = w - 4, sb = sw & 3, dc0 = (sw >> 2) * 8;        // 32-block sub-tile, first of its 8 dim chunks
    const int blk = sb * 32 + l;
    for (int i = 0; i < t1 - t0; ++i) {
      const int tile = t0 + i;
      const bool live = tile * kScBlocks + sb * 32 < nb_hi;         // the pool is allocated in whole 32-block tiles
      const float* src = a.c.ik_pool + ((size_t)tile * 4 + sb) * 4096 + l;
      float x[8][8];
#pragma unroll
      for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int j = 0; j < 8; ++j) x[c][j] = live ? __ldg(src + ((dc0 + c) * 8 + j) * 32) : 0.f;
      if (i > 0) {                                                  // the MMAs that read the previous tile are done
        if (l == 0) wait(&mmaDone[(i - 1) & 1], ((i - 1) >> 1) & 1);
        __syncwarp();
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 hi, lo;
        split8(x[c], hi, lo);
        *reinterpret_cast<uint4*>(Pop + ((size_t)(dc0 + c) * kScBlocks + blk) * 16) = hi;
        *reinterpret_cast<uint4*>(Pop + kPopBytes / 2 + ((size_t)(dc0 + c) * kScBlocks + blk) * 16) = lo;
      }
      umma::fence_async_smem();
      __syncwarp();
      if (l == 0) umma::mbar_arrive_relaxed(popFull);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps: thread = TMEM lane = block of the tile
    for (int i = 0; i < t1 - t0; ++i) {
      const int buf = i & 1, b = (t0 + i) * kScBlocks + t;
      if (l == 0) wait(&mmaDone[buf], (i >> 1) & 1);
      __syncwarp();
      umma::fence_after_sync();
      float s[kScRows];
#pragma unroll
      for (int c = 0; c < kScRows; ++c) s[c] = 0.f;
#pragma unroll
      for (int h = 0; h < 4; ++h)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float p[32];
          umma::tmem_ld32(umma::tmem_addr(tm, w, buf * 256 + h * 64 + half * 32), p);
#pragma unroll
          for (int c = 0; c < 32; ++c) s[half * 32 + c] += fmaxf(p[c], 0.f);
        }
      umma::fence_before_sync();
      __syncwarp();
      if (l == 0) umma::mbar_arrive_relaxed(&accFree[buf]);
      if (b < nb_hi && (!RANGED || b >= P.b_lo)) {
        float* dst = a.scores + (size_t)r0 * a.sstride + b;
#pragma unroll
        for (int c = 0; c < kScRows; ++c)
          if (c < rows) dst[(size_t)c * a.sstride] = s[c] * kInvSqrt128;
      }
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (w == 12) umma::tmem_dealloc(tm, 512);
}

cr_status qsa_score_tc_launch(const QsaParams& P, int Rmax, int n, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (cr_status st = once_per_device(configured, [] {
        CR_CUDA(cudaFuncSetAttribute(qsa_score_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScoreSmem));
        CR_CUDA(cudaFuncSetAttribute(qsa_score_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScoreSmem));
        return CR_OK;
      })) return st;
  const int row_tiles = (Rmax + kScRows - 1) / kScRows;
  int sm_count = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  // One CTA per SM (192 KB of shared memory, all of TMEM).  The pool tiles of a row tile are dealt to `splits` CTAs;
  // with w waves of CTAs the kernel lasts about w / splits of one row tile's work: take the best of 1 to 3 waves.
  int splits = 1;
  double best = 1e30;
  for (int wv = 1; wv <= 3; ++wv) {
    int sp = wv * sm_count / (row_tiles * n);
    sp = sp < 1 ? 1 : (sp > 64 ? 64 : sp);
    const int waves = (row_tiles * n * sp + sm_count - 1) / sm_count;
    const double cost = (double)waves / sp;
    if (cost < best - 1e-9) { best = cost; splits = sp; }
  }
  if (P.b_lo > 0 || P.b_hi < INT_MAX) qsa_score_tc_kernel<true><<<dim3(row_tiles, splits, n), kScThreads, kScoreSmem, stream>>>(P);
  else qsa_score_tc_kernel<false><<<dim3(row_tiles, splits, n), kScThreads, kScoreSmem, stream>>>(P);
  CR_LAUNCH_CHECK("qsa_score_tc_kernel");
  return CR_OK;
}

}  // namespace cr
