// QSA prefill attention over row tiles on tcgen05 tensor cores (sm_100a): the job of QsaUnionBuildKernel +
// QsaUnionStageKernel (engine/layers/kernels/prefill_qsa_union.h:25-68, :519-742).
//
// A tile is RT = 128 / gqa consecutive query rows (16 at 8 query heads per KV head, 10 at 12).  The rows of a tile
// share one key list, the union of their attended blocks, so every K/V row is fetched once per tile, and the tile's
// rows x heads are the 128 M rows of the tensor-core products.  A per-block row mask keeps every row's own selection
// exact, and the causal rule (key position <= row position) cuts the tail block.
//
// qsa_union_build_kernel (one CTA per tile): every row contributes a sorted list (its selected blocks, or all
// complete blocks when dense, plus its open tail block).  The union is formed by ranking: an element finds, by binary
// search in the other rows' lists, which rows hold the same block (its mask), whether a lower row already owns it,
// and how many owned blocks of every row precede it (its place in the output).  No array over the context is
// needed, so the context length does not limit it (the reference keeps a byte per block in 64 KB of LDS and falls
// back to row-wise attention past about 196K positions, engine/layers/qsa_union_lds.h:7-11).
//
// qsa_flash_tc_kernel (one CTA per (tile, KV head), 9 warps, 64 keys per step):
//   loader warps (4)   gather the K and V rows of 16 blocks per step with 16-byte cp.async into two stages.  Both
//                      tiles land as 16-byte units at (piece * 64 + key) * 16: for K that is the K-major operand
//                      [key][channel], for V the MN-major operand [key][channel] (channels contiguous), so neither
//                      is transposed anywhere.  Two warps serve the even steps and two the odd steps.
//   issuer warp        S = Q K^T (16 tcgen05.mma kind::f16, M 128 x N 64 x K 16) into one of two TMEM accumulators,
//                      one step ahead of the softmax; O += P V (4 MMAs, N 256) once the probabilities are written.
//   softmax warps (4)  thread = TMEM lane = (row, head): reads S, applies mask and causality, keeps a running
//                      reference maximum that moves only when a logit exceeds it by more than 2^8 (the accumulator is
//                      rescaled in TMEM then, which is rare after the first steps), writes P as fp16 into a K-major
//                      shared-memory tile, sums it.
//   epilogue           O / sum, optional un-gated context, sigmoid gate, output format.
// q and P are fp16 with fp32 accumulation, the reference's prefill numerics (prefill_qsa_union.h:680-684).
// Every wait is bounded; a wait that gives up raises the status word and the CTA runs to its end.
#include <climits>
#include "qsa.cuh"
#include "umma.cuh"

namespace cr {

CR_DEFINE_STATUS_WORD(qsa_flash)

constexpr int kFlKeys = 64;                         // keys per step
constexpr int kFlBlocks = kFlKeys / 4;              // union entries per step
constexpr int kFlThreads = 32 * 9;
constexpr int kFlQBytes = 128 * 256 * 2;            // [32 channel pieces][128 rows][8 halves]
constexpr int kFlKBytes = kFlKeys * 256 * 2;        // [32 channel pieces][64 keys][8 halves]
constexpr int kFlPBytes = 128 * kFlKeys * 2;        // [8 key pieces][128 rows][8 halves]
constexpr size_t kFlashSmem = kFlQBytes + 4 * kFlKBytes + 2 * kFlPBytes + 128;
constexpr uint32_t kColO = 0, kColS = 256;          // TMEM columns: O 0-255, S of step j at 256 + 64 (j & 1)
constexpr int kUbLen = 520;                         // list slots per row in the union builder (512 + tail + sentinel)
constexpr int kUbThreads = 1024;

struct FlashParams {
  cr_qsa_args a;          // the output rows (pos0 = position of row 0)
  const __half* q_hi;     // [R][Hq][256]
  const int2* list;       // [tiles][cap] (block, row mask), ascending blocks
  const int* count;       // [tiles]
  float* gated;           // gated fp32 [R][Hq * 256] when the output transform runs as a second kernel, else null
  int cap, RT, Hq, Hkv, fmt;
};

int qsa_union_rows(const cr_geometry* g) {
  const int most = 128 / (g->q_heads / g->kv_heads);
  const int want = options().qsa_union_rows;
  return want > 0 && want < most ? want : most;
}
int qsa_union_cap(int RT) { return (RT * 513 + 15) / 16 * 16; }

// ---- union lists -------------------------------------------------------------------------------------------
__device__ __forceinline__ int lower_bound_i(const int* a, int n, int v) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] < v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(kUbThreads) qsa_union_build_kernel(cr_qsa_args a, int2* list, int* count, int cap, int RT) {
  extern __shared__ __align__(16) int ub[];
  int* L = ub;                          // [RT][kUbLen] sorted block ids of every row
  int* M = L + 16 * kUbLen;             // [RT][kUbLen] row mask of the elements that own their block, else 0
  int* Pre = M + 16 * kUbLen;           // [RT][kUbLen] owned elements before index i (entry len = the row's total)
  __shared__ int len[16];
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int tile = blockIdx.x, row0 = tile * RT;
  if (w < 16) {
    int n = 0;
    const int gr = row0 + w;
    if (w < RT && gr < a.R) {
      const int p = a.pos0 + gr, nb = (p + 1) / 4, ns = a.nsel[gr];
      n = ns < 0 ? nb : CR_SEL_BLOCKS;
      const int* sel = a.sel + (size_t)gr * CR_SEL_BLOCKS;
      for (int i = l; i < n; i += 32) L[w * kUbLen + i] = ns < 0 ? i : sel[i];
      if ((p + 1) % 4 != 0) { if (l == 0) L[w * kUbLen + n] = nb; ++n; }      // the open block holds the tail tokens
    }
    if (l == 0) len[w] = n;
  }
  __syncthreads();
  for (int e = t; e < RT * kUbLen; e += kUbThreads) {
    const int r = e / kUbLen, i = e % kUbLen;
    int mask = 0;
    if (i < len[r]) {
      const int b = L[e];
      bool own = true;
      mask = 1 << r;
      for (int r2 = 0; r2 < RT; ++r2) {
        if (r2 == r || len[r2] == 0) continue;
        const int at = lower_bound_i(L + r2 * kUbLen, len[r2], b);
        if (at < len[r2] && L[r2 * kUbLen + at] == b) { mask |= 1 << r2; if (r2 < r) own = false; }
      }
      if (!own) mask = 0;
    }
    M[e] = mask;
  }
  __syncthreads();
  if (w < RT) {                          // one warp per row: running count of owned elements
    int run = 0;
    for (int i0 = 0; i0 <= len[w]; i0 += 32) {
      const int i = i0 + l;
      const unsigned own = __ballot_sync(0xffffffffu, i < len[w] && M[w * kUbLen + i] != 0);
      if (i <= len[w]) Pre[w * kUbLen + i] = run + __popc(own & ((1u << l) - 1u));
      run += __popc(own);
    }
  }
  __syncthreads();
  int2* out = list + (size_t)tile * cap;
  for (int e = t; e < RT * kUbLen; e += kUbThreads) {
    const int mask = M[e];
    if (!mask) continue;
    const int b = L[e];
    int rank = 0;
    for (int r2 = 0; r2 < RT; ++r2)
      if (len[r2]) rank += Pre[r2 * kUbLen + lower_bound_i(L + r2 * kUbLen, len[r2], b)];
    out[rank] = make_int2(b, mask);
  }
  if (t == 0) {
    int total = 0;
    for (int r = 0; r < RT; ++r) total += Pre[r * kUbLen + len[r]];
    count[tile] = total;
  }
}

// ---- flash ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ void fl_cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void fl_mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_u32(bar)) : "memory");
}

// grid (tiles, Hkv).
__global__ void __launch_bounds__(kFlThreads, 1) qsa_flash_tc_kernel(const __grid_constant__ FlashParams P) {
  extern __shared__ __align__(128) unsigned char sm[];
  unsigned char* Qs = sm;
  unsigned char* Ks = Qs + kFlQBytes;                    // two stages
  unsigned char* Vs = Ks + 2 * kFlKBytes;                // two stages
  unsigned char* Ps = Vs + 2 * kFlKBytes;                // two buffers
  __shared__ __align__(8) uint64_t bars[8];
  __shared__ int blk_s[2][kFlBlocks], mask_s[2][kFlBlocks];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int dead;
  uint64_t *kvFull = &bars[0], *sFull = &bars[2], *pFull = &bars[4], *pvDone = &bars[6];
  const cr_qsa_args& a = P.a;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int tile = blockIdx.x, g = blockIdx.y, row0 = tile * P.RT;
  const int gqa = P.Hq / P.Hkv;
  const int cnt = P.count[tile];
  const int n = (cnt + kFlBlocks - 1) / kFlBlocks;
  if (n == 0) return;                                    // a tile without rows
  const int last_pos = a.pos0 + a.R - 1;                 // newest position the cache holds

  if (t == 0) {
    for (int i = 0; i < 2; ++i) {
      umma::mbar_init(&kvFull[i], 2);                    // the two loader warps of the stage
      umma::mbar_init(&sFull[i], 1);
      umma::mbar_init(&pFull[i], 4);                     // one arrival per softmax warp
      umma::mbar_init(&pvDone[i], 1);
    }
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == 8) umma::tmem_alloc(&tmem_slot, 512);
  // query tile: M row m = (row m / gqa of the tile, head m % gqa of the group), fp16, K-major
  for (int u = t; u < 128 * 32; u += kFlThreads) {
    const int piece = u & 31, m = u >> 5, r = m / gqa, hq = m % gqa;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < P.RT && row0 + r < a.R)
      v = *reinterpret_cast<const uint4*>(P.q_hi + ((size_t)(row0 + r) * P.Hq + g * gqa + hq) * 256 + piece * 8);
    *reinterpret_cast<uint4*>(Qs + ((size_t)piece * 128 + m) * 16) = v;
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  bool gave_up = false;
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (gave_up) return;
    if (!umma::mbar_wait_timed(bar, parity, &dead)) { gave_up = true; dead = 1; g_qsa_flash_status = 1; }
  };
  auto warp_wait = [&](uint64_t* bar, uint32_t parity) {   // lane 0 polls for the warp
    if (l == 0) wait(bar, parity);
    __syncwarp();
  };

  if (w == 8) {
    // ------------------------------------------------------------------ issuer
    if (l == 0) {
      constexpr uint32_t idS = umma::idesc_f16(128, kFlKeys, false, false), idO = umma::idesc_f16(128, 256, false, true);
      const uint64_t dQ = umma::smem_desc(Qs, 128 * 16, 128);
      auto issue_S = [&](int j) {
        const int s = j & 1;
        const uint64_t dK = umma::smem_desc(Ks + s * kFlKBytes, kFlKeys * 16, 128);
#pragma unroll
        for (int ks = 0; ks < 16; ++ks)                  // 16 channels per MMA = two 16-byte pieces of every row
          umma::mma_f16_ss(tm + kColS + 64 * s, dQ + (uint64_t)(ks * 2 * 128), dK + (uint64_t)(ks * 2 * kFlKeys), idS, ks > 0);
        umma::commit(&sFull[s]);
      };
      wait(&kvFull[0], 0);
      umma::fence_after_sync();
      if (!gave_up) issue_S(0);
      for (int j = 0; j < n; ++j) {
        const int s = j & 1;
        if (j + 1 < n) {
          wait(&kvFull[(j + 1) & 1], ((j + 1) >> 1) & 1);
          if (gave_up || dead) break;
          umma::fence_after_sync();
          issue_S(j + 1);                                 // its accumulator was read by the softmax of step j - 1
        }
        wait(&pFull[s], (j >> 1) & 1);
        if (gave_up || dead) break;
        umma::fence_after_sync();
        const uint64_t dP = umma::smem_desc(Ps + s * kFlPBytes, 128 * 16, 128);
        const uint64_t dV = umma::smem_desc(Vs + s * kFlKBytes, 128, kFlKeys * 16);   // MN-major: step along keys 128 B, along channels 1 KB
#pragma unroll
        for (int kk = 0; kk < kFlKeys / 16; ++kk)
          umma::mma_f16_ss(tm + kColO, dP + (uint64_t)(kk * 2 * 128), dV + (uint64_t)(kk * 16), idO, (j > 0 || kk > 0) ? 1u : 0u);
        umma::commit(&pvDone[s]);
      }
    }
  } else if (w >= 4) {
    // ------------------------------------------------------------------ loaders: warps 4,5 even steps, warps 6,7 odd steps
    const int s = (w - 4) >> 1, lw = (w - 4) & 1;
    const __half* kc = reinterpret_cast<const __half*>(a.c.k);
    const __half* vc = reinterpret_cast<const __half*>(a.c.v);
    const int2* lst = P.list + (size_t)tile * P.cap;
    for (int j = s; j < n; j += 2) {
      if (j >= 2) warp_wait(&pvDone[s], ((j - 2) >> 1) & 1);          // the MMAs of step j - 2 have read the stage
      if (dead) break;
      int blk[4];
#pragma unroll
      for (int kq = 0; kq < 4; ++kq) {
        const int idx = j * kFlBlocks + kq * 4 + (l >> 3);
        blk[kq] = idx < cnt ? lst[idx].x : 0;
      }
      if (lw == 0 && l < kFlBlocks) {
        const int idx = j * kFlBlocks + l;
        const int2 e = idx < cnt ? lst[idx] : make_int2(0, 0);
        blk_s[s][l] = e.x;
        mask_s[s][l] = e.y;
      }
      unsigned char* kd = Ks + s * kFlKBytes;
      unsigned char* vd = Vs + s * kFlKBytes;
#pragma unroll 8
      for (int it = 0; it < 32; ++it) {
        const int kg = it & 3, pp = lw * 8 + (it >> 2);
        const int key = kg * 16 + (l >> 1), piece = 2 * pp + (l & 1);
        const int pos = blk[kg] * 4 + (key & 3);
        const bool valid = pos <= last_pos;
        const size_t src = valid ? ((size_t)pos * P.Hkv + g) * 256 + piece * 8 : 0;
        const size_t dst = ((size_t)piece * kFlKeys + key) * 16;
        fl_cp_async16(kd + dst, kc + src, valid);
        fl_cp_async16(vd + dst, vc + src, valid);
      }
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      umma::fence_async_smem();
      __syncwarp();
      if (l == 0) fl_mbar_arrive(&kvFull[s]);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = TMEM lane m
    const int m = t, r = m / gqa, hq = m % gqa;
    const bool rowok = r < P.RT && row0 + r < a.R;
    const int prow = a.pos0 + row0 + r;
    constexpr float kScale = 0.0625f * 1.4426950408889634f;            // logits / 16, in powers of two
    float m_ref = -INFINITY, lsum = 0.f;
    for (int j = 0; j < n; ++j) {
      const int s = j & 1;
      warp_wait(&kvFull[s], (j >> 1) & 1);                             // block ids and masks of the step are visible
      warp_wait(&sFull[s], (j >> 1) & 1);
      umma::fence_after_sync();
      float sv[kFlKeys];
      {
        float half_[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, kColS + 64 * s), half_);
#pragma unroll
        for (int c = 0; c < 32; ++c) sv[c] = half_[c];
        umma::tmem_ld32(umma::tmem_addr(tm, w, kColS + 64 * s + 32), half_);
#pragma unroll
        for (int c = 0; c < 32; ++c) sv[32 + c] = half_[c];
      }
      float tmax = -INFINITY;
#pragma unroll
      for (int b = 0; b < kFlBlocks; ++b) {
        const int base = blk_s[s][b] * 4;
        const bool mine = rowok && ((mask_s[s][b] >> r) & 1);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int c = 4 * b + k;
          const bool vis = mine && base + k <= prow;
          sv[c] = vis ? sv[c] * kScale : -INFINITY;
          tmax = fmaxf(tmax, sv[c]);
        }
      }
      const bool move = tmax > m_ref + 8.f;                             // also the first visible key (m_ref = -inf)
      if (__any_sync(0xffffffffu, move)) {
        const float nref = move ? tmax : m_ref;
        const float factor = move ? exp2f(m_ref - nref) : 1.f;          // 0 when nothing was accumulated yet
        lsum *= factor;
        m_ref = nref;
        if (j > 0) {                                                    // O holds the steps before this one
          warp_wait(&pvDone[(j - 1) & 1], ((j - 1) >> 1) & 1);
          umma::fence_after_sync();
#pragma unroll 1
          for (int c8 = 0; c8 < 8; ++c8) {
            float o[32];
            umma::tmem_ld32(umma::tmem_addr(tm, w, kColO + 32 * c8), o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] *= factor;
            umma::tmem_st32(umma::tmem_addr(tm, w, kColO + 32 * c8), o);
          }
          umma::tmem_st_wait();
        }
      }
      if (j >= 2) warp_wait(&pvDone[s], ((j - 2) >> 1) & 1);            // the MMAs of step j - 2 have read this P buffer
      unsigned char* pd = Ps + s * kFlPBytes;
      float add = 0.f;
#pragma unroll
      for (int kc8 = 0; kc8 < kFlKeys / 8; ++kc8) {
        unsigned pk[4];
#pragma unroll
        for (int q2 = 0; q2 < 4; ++q2) {
          const float s0 = sv[kc8 * 8 + 2 * q2], s1 = sv[kc8 * 8 + 2 * q2 + 1];
          const float p0 = s0 > -INFINITY ? exp2f(s0 - m_ref) : 0.f, p1 = s1 > -INFINITY ? exp2f(s1 - m_ref) : 0.f;
          add += p0 + p1;
          const __half2 h = __floats2half2_rn(p0, p1);
          pk[q2] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(pd + ((size_t)kc8 * 128 + m) * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      lsum += add;
      umma::fence_async_smem();
      umma::fence_before_sync();
      __syncwarp();
      if (l == 0) fl_mbar_arrive(&pFull[s]);
    }
    // ---------------------------------------------------------------- epilogue
    warp_wait(&pvDone[(n - 1) & 1], ((n - 1) >> 1) & 1);
    umma::fence_after_sync();
    const bool ok = rowok && lsum > 0.f && !dead;
    const float inv = ok ? 1.f / lsum : 0.f;
    const int gr = row0 + r, h = g * gqa + hq;
    const size_t W = (size_t)P.Hq * 256;
    const float* gate = a.q + ((size_t)gr * P.Hq + h) * 512 + 256;
#pragma unroll 1
    for (int c8 = 0; c8 < 8; ++c8) {
      float o[32];
      umma::tmem_ld32(umma::tmem_addr(tm, w, kColO + 32 * c8), o);     // warp-collective: every lane takes part
      if (!ok) continue;
#pragma unroll
      for (int c = 0; c < 32; ++c) o[c] *= inv;
      if (a.context) {
        float4* cx = reinterpret_cast<float4*>(a.context + ((size_t)gr * P.Hq + h) * 256 + 32 * c8);
#pragma unroll
        for (int c = 0; c < 8; ++c) cx[c] = make_float4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float4 gv = *reinterpret_cast<const float4*>(gate + 32 * c8 + 4 * c);
        o[4 * c] *= sigmoidf_(gv.x); o[4 * c + 1] *= sigmoidf_(gv.y); o[4 * c + 2] *= sigmoidf_(gv.z); o[4 * c + 3] *= sigmoidf_(gv.w);
      }
      const size_t at = (size_t)gr * W + h * 256 + 32 * c8;
      if (P.gated) {
        float4* dst = reinterpret_cast<float4*>(P.gated + at);
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[c] = make_float4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
      } else if (P.fmt == CR_OUT_RAW_F32) {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + at);
#pragma unroll
        for (int c = 0; c < 8; ++c) dst[c] = make_float4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
      } else {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + at);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          unsigned pk[4];
#pragma unroll
          for (int q2 = 0; q2 < 4; ++q2) {
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(o[8 * c + 2 * q2], o[8 * c + 2 * q2 + 1]);
            pk[q2] = *reinterpret_cast<const unsigned*>(&b2);
          }
          dst[c] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
      }
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (w == 8) umma::tmem_dealloc(tm, 512);
}

// The reference's out-projection input from gated fp32 rows: fp16(WHT128(RoundH(RoundH(o) * suh)) / sqrt(128))
// (engine/layers/qsa_long.h:476-489).  grid (Hq, R), 64 threads: a warp per 128-channel group.
__global__ void __launch_bounds__(64) qsa_out_transform_kernel(cr_qsa_args a, const float* gated, int Hq) {
  const int h = blockIdx.x, r = blockIdx.y, half = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = Hq * 256, c0 = h * 256 + half * 128 + lane * 4;
  const float4 o = *reinterpret_cast<const float4*>(gated + (size_t)r * W + c0);
  const __half* suh = reinterpret_cast<const __half*>(a.suh_o) + c0;
  float v[4] = {round_h(round_h(o.x) * __half2float(suh[0])), round_h(round_h(o.y) * __half2float(suh[1])),
                round_h(round_h(o.z) * __half2float(suh[2])), round_h(round_h(o.w) * __half2float(suh[3]))};
  wht128(v);
  __half* dst = reinterpret_cast<__half*>(a.out);
#pragma unroll
  for (int i = 0; i < 4; ++i) dst[out_index(r, c0 + i, W, a.pack_rows, a.pack_off)] = __float2half(v[i] * kHadNorm);
}

cr_status qsa_union_build_launch(const cr_geometry* g, const cr_qsa_args& a, int2* list, int* count, cudaStream_t stream) {
  static PerDeviceOnce configured;
  constexpr int smem = 3 * 16 * kUbLen * (int)sizeof(int);
  if (cr_status st = once_per_device(configured, [] {
        CR_CUDA(cudaFuncSetAttribute(qsa_union_build_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        return CR_OK;
      })) return st;
  const int RT = qsa_union_rows(g), tiles = (a.R + RT - 1) / RT;
  use_stream(stream);
  qsa_union_build_kernel<<<tiles, kUbThreads, smem, stream>>>(a, list, count, qsa_union_cap(RT), RT);
  CR_LAUNCH_CHECK("qsa_union_build_kernel");
  return CR_OK;
}

// Attention of the rows of `a` over the union lists; `gated` (rows x Hq x 256 floats) is needed for CR_OUT_EXL3_WHT.
cr_status qsa_flash_launch(const cr_geometry* g, const cr_qsa_args& a, const __half* q_hi, const int2* list, const int* count,
                           float* gated, cr_out_format fmt, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (cr_status st = once_per_device(configured, [] {
        CR_CUDA(cudaFuncSetAttribute(qsa_flash_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFlashSmem));
        return CR_OK;
      })) return st;
  FlashParams P;
  P.a = a; P.q_hi = q_hi; P.list = list; P.count = count;
  P.RT = qsa_union_rows(g); P.cap = qsa_union_cap(P.RT);
  P.Hq = g->q_heads; P.Hkv = g->kv_heads; P.fmt = (int)fmt;
  P.gated = fmt == CR_OUT_EXL3_WHT ? gated : nullptr;
  CR_REQUIRE(fmt != CR_OUT_EXL3_WHT || gated, "qsa flash: the EXL3 output needs the gated fp32 scratch");
  const int tiles = (a.R + P.RT - 1) / P.RT;
  use_stream(stream);
  qsa_flash_tc_kernel<<<dim3(tiles, g->kv_heads), kFlThreads, kFlashSmem, stream>>>(P);
  CR_LAUNCH_CHECK("qsa_flash_tc_kernel");
  if (fmt == CR_OUT_EXL3_WHT) {
    qsa_out_transform_kernel<<<dim3(g->q_heads, a.R), 64, 0, stream>>>(a, gated, g->q_heads);
    CR_LAUNCH_CHECK("qsa_out_transform_kernel");
  }
  return CR_OK;
}

}  // namespace cr
