// QSA attention over the attended positions for sm_100a (decode, verify, and the row-wise prefill path).
//
// Split-KV gather (QsaGqaSplitKernel, engine/layers/qsa_long.h:399-456): one CTA of four warps per (split, row,
// KV head).  The query heads of the KV group are the M rows of a tensor-core tile (8..12 heads padded to 16), so
// every K/V row fetched is used by all heads at once:
//   S[16 x 32] = Q[16 x 256] K^T      mma.sync m16n8k16 f16, warp w owns positions 8w .. 8w+7 of the tile
//   O[16 x 256] += P[16 x 32] V       warp w owns channels 64w .. 64w+63
// K and V are fp16 in the cache.  Q and P are fp32 values: each is split into an fp16 head and an fp16 remainder
// and multiplied twice, which keeps the products at fp32 accuracy (the remainder carries the bits fp16 drops).
// Tiles of 32 positions are gathered with cp.async (zero fill for masked positions) into two shared-memory
// stages, the next tile in flight while the current one is multiplied; row maxima and sums cross the four warps
// through shared memory.  Each CTA writes the partial (m, l, acc[256]) of its heads; the merge kernel
// (QsaMergeKernel, qsa_long.h:458-499) combines them by log-sum-exp, applies the sigmoid gate and the output
// transform.  No CTA waits on another CTA.
#include <climits>
#include "qsa.cuh"

namespace cr {

constexpr int kTile = 32;            // positions per shared-memory tile
constexpr int kRowH = 264;           // padded row of 256 halves: 528 B keeps ldmatrix conflict-free
constexpr int kPRowH = 40;           // padded row of the 16 x 32 probability tile (80 B)
constexpr int kMaxSplitPos = 576;    // positions listed in shared memory at a time (18 tiles); a longer split walks its list in chunks

// STAGES = 2: the next tile is gathered while the current one is multiplied (a step: few CTAs, latency counts).
// STAGES = 1: 55 KB per CTA, four CTAs per SM keep more gathers in flight (a prefill part: thousands of CTAs).
template <int STAGES>
struct SplitSmem {
  __half q[2][16][kRowH];            // head and remainder of the query rows
  __half k[STAGES][kTile][kRowH];
  __half v[STAGES][kTile][kRowH];
  __half p[2][16][kPRowH];           // head and remainder of the probabilities
  float red[2][4][16];               // per-warp row maxima / row sums
  int pos[kMaxSplitPos];             // cache position of every attended index of this split, -1 = masked
};

__device__ __forceinline__ int qsa_position(const int* sel, int t, int ns, int nb) {
  return ns < 0 ? t : (t < ns * 4 ? sel[t >> 2] * 4 + (t & 3) : nb * 4 + t - ns * 4);
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((unsigned)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (splits, Rmax * Hkv, spans), or (Rmax * Hkv, splits, spans) for STAGES == 1; 128 threads.
template <int STAGES>
__global__ void __launch_bounds__(128) qsa_attn_split_kernel(const __grid_constant__ QsaParams P, float* partials,
                                                             int splits, int p0, int p1) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  SplitSmem<STAGES>& sm = *reinterpret_cast<SplitSmem<STAGES>*>(smem_raw);
  pdl_release();
  pdl_wait();
  const cr_qsa_args& a = P.span[blockIdx.z];
  // STAGES == 1 (many rows): grid (rows x KV heads, splits), the split being the slow index.  Split s of every row
  // covers about the s-th part of the context (attended positions ascend), so the CTAs in flight at any time read one
  // region of the cache, which L2 can hold.  STAGES == 2 (steps): grid (splits, rows x KV heads).
  const int rg = STAGES == 1 ? blockIdx.x : blockIdx.y;
  const int r = rg / P.Hkv, g = rg % P.Hkv;
  if (r >= a.R || qsa_row_is_tiled(P, r)) return;
  const int gqa = P.Hq / P.Hkv;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int split = STAGES == 1 ? blockIdx.y : blockIdx.x;
  const int p = a.pos0 + r, ns = a.nsel[r], nb = (p + 1) / 4;
  const int n = ns < 0 ? p + 1 : ns * 4 + (p + 1) % 4;
  const int* sel = a.sel + (size_t)r * CR_SEL_BLOCKS;
  // Attended indices run through ascending positions (selected blocks, then the tail), so the positions inside a rank's
  // window [p0, p1) are one contiguous range [t_lo, t_hi) of them: only that range is split and visited.
  int t_lo = 0, t_hi = n;
  if (p0 > 0 || p1 <= p) {
    if (ns < 0) { t_lo = min(p0, n); t_hi = min(p1, n); }
    else {
      auto first_block_at_least = [&](int blk) {          // index of the first selected block >= blk
        int lo = 0, hi = ns;
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (sel[mid] < blk) lo = mid + 1; else hi = mid; }
        return lo;
      };
      t_lo = 4 * first_block_at_least((p0 + 3) / 4);
      t_hi = 4 * first_block_at_least(p1 / 4 + (p1 % 4 ? 1 : 0));
      if (nb * 4 >= p0 && nb * 4 < p1) t_hi = n;          // the tail tokens 4 nb .. p
      else if (nb * 4 < p0) t_lo = t_hi;                  // a window past every attended position
    }
  }
  const int n_win = max(t_hi - t_lo, 0);
  // tiles of 32 attended indices are dealt evenly: the first (tiles % splits) splits take one more
  const int tiles = (n_win + kTile - 1) / kTile, tb = tiles / splits, trem = tiles % splits;
  const int begin = t_lo + (split * tb + min(split, trem)) * kTile, end = min(begin + (tb + (split < trem ? 1 : 0)) * kTile, t_hi);
  const int total = max(end - begin, 0);                  // positions of this split, walked in chunks of at most kMaxSplitPos
  int cnt = 0, chunk0 = 0;
  auto list_chunk = [&]() {                               // attended positions [begin + chunk0, + cnt) into shared memory
    cnt = min(total - chunk0, kMaxSplitPos);
    for (int i = t; i < cnt; i += 128) {
      int pos = qsa_position(sel, begin + chunk0 + i, ns, nb);
      if (pos < p0 || pos >= p1) pos = -1;
      sm.pos[i] = pos;
    }
    __syncthreads();
  };
  list_chunk();

  const __half* kc = reinterpret_cast<const __half*>(a.c.k);
  const __half* vc = reinterpret_cast<const __half*>(a.c.v);
  auto stage = [&](int tile, int buf) {   // 32 positions x (32 K + 32 V) 16-byte pieces
    for (int piece = t; piece < kTile * 64; piece += 128) {
      const int j = piece >> 6, c = piece & 63, idx = tile * kTile + j;
      const int pos = idx < cnt ? sm.pos[idx] : -1;
      const bool valid = pos >= 0;
      const size_t off = valid ? ((size_t)pos * P.Hkv + g) * 256 + (c & 31) * 8 : 0;
      cp_async_16(c < 32 ? &sm.k[buf][j][(c & 31) * 8] : &sm.v[buf][j][(c & 31) * 8], (c < 32 ? kc : vc) + off, valid);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };

  int ntiles = (cnt + kTile - 1) / kTile;
  const int row0 = l >> 2, cq = (l & 3) * 2;              // this thread's rows row0, row0 + 8; columns cq, cq + 1 of an n-tile
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float O[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) O[i][0] = O[i][1] = O[i][2] = O[i][3] = 0.f;
  if (STAGES == 2 && ntiles > 0) stage(0, 0);
  // the query rows are split into fp16 head + remainder while the first tile is in flight
  for (int i = t; i < 16 * 64; i += 128) {
    const int row = i >> 6, c = (i & 63) * 4;
    float4 qv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row < gqa) qv = *reinterpret_cast<const float4*>(a.q + ((size_t)r * P.Hq + g * gqa + row) * 512 + c);
    const __half2 h0 = __floats2half2_rn(qv.x, qv.y), h1 = __floats2half2_rn(qv.z, qv.w);
    const float2 b0 = __half22float2(h0), b1 = __half22float2(h1);
    *reinterpret_cast<__half2*>(&sm.q[0][row][c]) = h0;
    *reinterpret_cast<__half2*>(&sm.q[0][row][c + 2]) = h1;
    *reinterpret_cast<__half2*>(&sm.q[1][row][c]) = __floats2half2_rn(qv.x - b0.x, qv.y - b0.y);
    *reinterpret_cast<__half2*>(&sm.q[1][row][c + 2]) = __floats2half2_rn(qv.z - b1.x, qv.w - b1.y);
  }
  for (;;) {
  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = STAGES == 2 ? (tile & 1) : 0;
    if (STAGES == 1) {
      __syncthreads();                                    // every warp is done with the previous tile (and q is visible)
      stage(tile, 0);
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();                                      // tile visible; every warp is done with the previous one
    if (STAGES == 2 && tile + 1 < ntiles) stage(tile + 1, buf ^ 1);
    // ---- S = Q K^T for positions 8w .. 8w+7
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int ks = 0; ks < 16; ks += 2) {                  // two k-steps of 16 channels per K fragment load
      unsigned kb[4];
      ldsm_x4(kb, &sm.k[buf][8 * w + (l & 7)][ks * 16 + (l >> 3) * 8]);
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        unsigned ah[4], al[4];
        ldsm_x4(ah, &sm.q[0][l & 15][(ks + kk) * 16 + (l >> 4) * 8]);
        ldsm_x4(al, &sm.q[1][l & 15][(ks + kk) * 16 + (l >> 4) * 8]);
        mma_f16(s, ah, kb[2 * kk], kb[2 * kk + 1]);
        mma_f16(s, al, kb[2 * kk], kb[2 * kk + 1]);
      }
    }
    const int pi = tile * kTile + 8 * w + cq;
    const bool v0 = pi < cnt && sm.pos[pi] >= 0, v1 = pi + 1 < cnt && sm.pos[pi + 1] >= 0;
    s[0] = v0 ? s[0] * 0.0625f : -INFINITY; s[1] = v1 ? s[1] * 0.0625f : -INFINITY;
    s[2] = v0 ? s[2] * 0.0625f : -INFINITY; s[3] = v1 ? s[3] * 0.0625f : -INFINITY;
    float mx0 = fmaxf(s[0], s[1]), mx1 = fmaxf(s[2], s[3]);
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if ((l & 3) == 0) { sm.red[0][w][row0] = mx0; sm.red[0][w][row0 + 8] = mx1; }
    __syncthreads();
    float mn[2], corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + 8 * i;
      const float tm = fmaxf(fmaxf(sm.red[0][0][row], sm.red[0][1][row]), fmaxf(sm.red[0][2][row], sm.red[0][3][row]));
      mn[i] = fmaxf(m_run[i], tm);
      corr[i] = m_run[i] > -INFINITY ? __expf(m_run[i] - mn[i]) : 0.f;   // nothing accumulated yet: factor irrelevant
    }
    float e[4];
    e[0] = s[0] > -INFINITY ? __expf(s[0] - mn[0]) : 0.f; e[1] = s[1] > -INFINITY ? __expf(s[1] - mn[0]) : 0.f;
    e[2] = s[2] > -INFINITY ? __expf(s[2] - mn[1]) : 0.f; e[3] = s[3] > -INFINITY ? __expf(s[3] - mn[1]) : 0.f;
    float su0 = e[0] + e[1], su1 = e[2] + e[3];
    su0 += __shfl_xor_sync(0xffffffffu, su0, 1); su1 += __shfl_xor_sync(0xffffffffu, su1, 1);
    su0 += __shfl_xor_sync(0xffffffffu, su0, 2); su1 += __shfl_xor_sync(0xffffffffu, su1, 2);
    if ((l & 3) == 0) { sm.red[1][w][row0] = su0; sm.red[1][w][row0 + 8] = su1; }
#pragma unroll
    for (int i = 0; i < 2; ++i) {                          // probabilities as fp16 head + remainder
      const __half2 hi = __floats2half2_rn(e[2 * i], e[2 * i + 1]);
      const float2 back = __half22float2(hi);
      *reinterpret_cast<__half2*>(&sm.p[0][row0 + 8 * i][8 * w + cq]) = hi;
      *reinterpret_cast<__half2*>(&sm.p[1][row0 + 8 * i][8 * w + cq]) = __floats2half2_rn(e[2 * i] - back.x, e[2 * i + 1] - back.y);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = row0 + 8 * i;
      l_run[i] = l_run[i] * corr[i] + (sm.red[1][0][row] + sm.red[1][1][row]) + (sm.red[1][2][row] + sm.red[1][3][row]);
      m_run[i] = mn[i];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) { O[nt][0] *= corr[0]; O[nt][1] *= corr[0]; O[nt][2] *= corr[1]; O[nt][3] *= corr[1]; }
    // ---- O += P V for channels 64w .. 64w+63
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {                      // 16 positions per k-step
      unsigned ph[4], pl[4];
      ldsm_x4(ph, &sm.p[0][l & 15][kk * 16 + (l >> 4) * 8]);
      ldsm_x4(pl, &sm.p[1][l & 15][kk * 16 + (l >> 4) * 8]);
#pragma unroll
      for (int nt = 0; nt < 8; nt += 2) {                 // two n-tiles of 8 channels per V fragment load
        unsigned vb[4];
        ldsm_x4_trans(vb, &sm.v[buf][kk * 16 + (l & 7) + ((l >> 3) & 1) * 8][64 * w + nt * 8 + (l >> 4) * 8]);
        mma_f16(O[nt], ph, vb[0], vb[1]);
        mma_f16(O[nt], pl, vb[0], vb[1]);
        mma_f16(O[nt + 1], ph, vb[2], vb[3]);
        mma_f16(O[nt + 1], pl, vb[2], vb[3]);
      }
    }
  }
    chunk0 += kMaxSplitPos;                               // a split longer than one chunk (few splits over a long list)
    if (chunk0 >= total) break;
    __syncthreads();                                      // every warp is done with the chunk's positions and tiles
    list_chunk();
    ntiles = (cnt + kTile - 1) / kTile;
    if (STAGES == 2) stage(0, 0);
  }
  // partial records of this split: rows row0 and row0 + 8 are heads g * gqa + row
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + 8 * i;
    if (row >= gqa) continue;
    float* dst = partials + (((size_t)(P.base[blockIdx.z] + r) * P.Hq + g * gqa + row) * splits + split) * CR_QSA_PART;
    if (w == 0 && (l & 3) == 0) { dst[0] = m_run[i]; dst[1] = l_run[i]; }
    // records are 8-byte aligned (258 floats): store pairs
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
      *reinterpret_cast<float2*>(dst + 2 + 64 * w + nt * 8 + cq) = make_float2(O[nt][2 * i], O[nt][2 * i + 1]);
  }
}

// grid (Hq, Rmax, spans), 256 threads: thread d = output channel.
// Partial p of (row, head) is at partials[(part_major ? (p * rows_total + row) * Hq + h : (row * Hq + h) * nparts + p) * 258].
__global__ void __launch_bounds__(256) qsa_merge_kernel(const __grid_constant__ QsaParams P, const float* partials, int nparts,
                                                        int part_major, int rows_total, float* partial_out, int fmt) {
  pdl_release();
  pdl_wait();
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int h = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
  if (r >= a.R || qsa_row_is_tiled(P, r)) return;
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
  if (nparts == 32) {   // the decode case: all 32 loads in flight at once
    float v[32];
#pragma unroll
    for (int p = 0; p < 32; ++p) v[p] = __ldcg(rec(p) + 2 + d);
#pragma unroll
    for (int p = 0; p < 32; ++p) o = fmaf(v[p], fs[p], o);
  } else {
#pragma unroll 8
    for (int p = 0; p < nparts; ++p) o = fmaf(rec(p)[2 + d], fs[p], o);
  }
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
                          int p0, int p1, cudaStream_t stream, const QsaTileSplit* tiles) {
  use_stream(stream);
  CR_REQUIRE(splits >= 1 && splits <= 32, "qsa attention: %d KV splits unsupported (1..32)", splits);
  int row_base = 0;
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    for (int s = 0; s < n; ++s) P.base[s] += row_base;
    if (tiles) { P.tile_count = tiles->count; P.tile_rows = tiles->rows; P.tile_max = tiles->max; }
    const int Rmax = qsa_max_rows(spans + s0, n);
    static PerDeviceOnce configured;
    if (cr_status st = once_per_device(configured, [] {
          CR_CUDA(cudaFuncSetAttribute(qsa_attn_split_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SplitSmem<1>)));
          CR_CUDA(cudaFuncSetAttribute(qsa_attn_split_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(SplitSmem<2>)));
          return CR_OK;
        })) return st;
    const dim3 grid(splits, Rmax * g->kv_heads, n);
    if ((long long)grid.x * grid.y * grid.z > 600)          // more than two waves of the two-stage kernel (2 CTAs per SM)
      CR_CUDA(launch_pdl(qsa_attn_split_kernel<1>, dim3(grid.y, grid.x, grid.z), dim3(128), sizeof(SplitSmem<1>), stream, P, partials, splits, p0, p1));
    else
      CR_CUDA(launch_pdl(qsa_attn_split_kernel<2>, grid, dim3(128), sizeof(SplitSmem<2>), stream, P, partials, splits, p0, p1));
    CR_LAUNCH_CHECK("qsa_attn_split_kernel");
    for (int s = 0; s < n; ++s) row_base += spans[s0 + s].R;
  }
  return CR_OK;
}

cr_status qsa_merge_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, const float* partials, int nparts,
                           bool part_major, float* partial_out, cr_out_format fmt, cudaStream_t stream, const QsaTileSplit* tiles) {
  use_stream(stream);
  CR_REQUIRE(nparts >= 1 && nparts <= 32, "qsa merge: %d partial records per (row, head) unsupported (1..32)", nparts);
  int rows_total = 0, row_base = 0;
  for (int s = 0; s < n_spans; ++s) rows_total += spans[s].R;
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    for (int s = 0; s < n; ++s) P.base[s] += row_base;
    if (tiles) { P.tile_count = tiles->count; P.tile_rows = tiles->rows; P.tile_max = tiles->max; }
    const int Rmax = qsa_max_rows(spans + s0, n);
    CR_CUDA(launch_pdl(qsa_merge_kernel, dim3(g->q_heads, Rmax, n), dim3(256), 0, stream, P, partials, nparts, part_major ? 1 : 0, rows_total, partial_out, (int)fmt));
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

// KV splits per (row, KV head) of a decode / verify pass: 32 for a few rows (latency: many short CTAs), fewer when the
// pass holds many rows, so that the grid stays near two waves of CTAs and the per-CTA work (query staging, a partial
// record per head) is shared by more positions.  A power of two between 4 and 32.
constexpr long long kStepCtas = 1200;   // 600 and 2,400 measured 20 % and 6 % slower on 72 rows
static int step_splits(const cr_geometry* g, const cr_qsa_args* spans, int n_spans) {
  const long long units = (long long)cr::total_rows(spans, n_spans) * g->kv_heads;
  int splits = CR_QSA_SPLITS;
  while (splits > 4 && units * splits > kStepCtas) splits >>= 1;
  return splits;
}

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
  const int splits = step_splits(g, spans, n_spans);
  if (cr_status s = qsa_attn_launch(g, spans, n_spans, (float*)scratch, splits, 0, INT_MAX, (cudaStream_t)stream)) return s;
  return qsa_merge_launch(g, spans, n_spans, (const float*)scratch, splits, false, nullptr, fmt, (cudaStream_t)stream);
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
  const int splits = step_splits(g, spans, n_spans);
  if (cr_status s = qsa_attn_launch(g, spans, n_spans, (float*)scratch, splits, 0, INT_MAX, st)) return s;
  return qsa_merge_launch(g, spans, n_spans, (const float*)scratch, splits, false, nullptr, fmt, st);
}

extern "C" cr_status cr_qsa_shard_attn(const cr_geometry* g, const cr_qsa_args* a, int p0, int p1, float* partials, void* scratch,
                                       size_t scratch_bytes, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_shard_attn", 0)) return s;
  CR_REQUIRE(partials && p0 >= 0 && p1 >= p0, "cr_qsa_shard_attn: bad position window or null output");
  // A part's rows take up to 4 splits each; a window that holds a fraction of the cache holds about that fraction of a
  // row's 2,051 attended positions, so it takes fewer (a split whose list is longer than expected walks it in chunks).
  const long long cache = (long long)a->pos0 + a->R, window = (p1 < cache ? p1 : cache) - p0;
  const int part_splits = window <= 0 ? 1 : (int)((4 * window + cache - 1) / cache);
  const int splits = a->R <= CR_MAX_STEP_ROWS ? CR_QSA_SPLITS : (part_splits < 1 ? 1 : part_splits > 4 ? 4 : part_splits);
  const size_t need = (size_t)a->R * g->q_heads * splits * CR_QSA_PART * sizeof(float);
  CR_REQUIRE(scratch && scratch_bytes >= need, "cr_qsa_shard_attn: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
  if (cr_status s = qsa_attn_launch(g, a, 1, (float*)scratch, splits, p0, p1, (cudaStream_t)stream)) return s;
  return qsa_merge_launch(g, a, 1, (const float*)scratch, splits, false, partials, CR_OUT_RAW_F32, (cudaStream_t)stream);
}

extern "C" cr_status cr_qsa_merge_partials(const cr_geometry* g, const cr_qsa_args* a, int ranks, const float* partials,
                                           cr_out_format fmt, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_merge_partials", 0)) return s;
  if (cr_status s = check_out(a, 1, fmt, "cr_qsa_merge_partials")) return s;
  CR_REQUIRE(partials && ranks >= 1 && ranks <= 32, "cr_qsa_merge_partials: need gathered partials of 1..32 ranks");
  return qsa_merge_launch(g, a, 1, partials, ranks, true, nullptr, fmt, (cudaStream_t)stream);
}
