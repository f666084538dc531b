// QSA prefill attention over row tiles on tcgen05 tensor cores (sm_100a): the job of QsaUnionBuildKernel +
// QsaUnionStageKernel (engine/layers/kernels/prefill_qsa_union.h:25-68, :519-742).
//
// A tile is RT = 128 / gqa consecutive query rows (16 at 8 query heads per KV head, 10 at 12).  The rows of a tile
// share one key list, the union of their attended blocks, so every K/V row is fetched once per tile, and the tile's
// rows x heads are the 128 M rows of the tensor-core products.  A per-block row mask keeps every row's own selection
// exact, and the causal rule (key position <= row position) cuts the tail block.
//
// qsa_union_build_kernel (one CTA per tile): every row contributes its selected blocks (or all complete blocks when
// dense) plus its open tail block as keys (block, row); sorting the keys puts the rows of a block side by side, and
// the first key of every run emits (block, OR of the row bits).  No array over the context is needed, so the context
// length does not limit it (the reference keeps a byte per block in 64 KB of LDS and falls back to row-wise
// attention past about 196K positions, engine/layers/qsa_union_lds.h:7-11).
//
// qsa_flash_tc_kernel (one CTA per (tile, KV head), 15 warps, 64 keys per step):
//   loader warps (6)   gather the K and V rows of 16 blocks per step with 16-byte cp.async into three stages, two
//                      warps per stage.  Both tiles land as 16-byte units at (piece * 64 + key) * 16: for K that is
//                      the K-major operand [key][channel], for V the MN-major operand [key][channel] (channels
//                      contiguous), so neither is transposed anywhere.
//   issuer warp        S = Q K^T (16 tcgen05.mma kind::f16, M 128 x N 64 x K 16, the query tile being the A operand
//                      in tensor memory, which leaves the shared memory to the K/V stages) into one of two TMEM
//                      accumulators, one step ahead of the softmax; O += P V (4 MMAs, N 256) once the probabilities
//                      are written.  An event loop issues whichever is ready.
//   softmax warps (8)  two warps per TMEM lane quarter, thread = (row, head) x half of the step's 64 keys: reads S,
//                      applies mask and causality (a 32-bit visibility word per step), keeps a running reference
//                      maximum that moves only when a logit exceeds it by more than 2^8 (the accumulator is rescaled
//                      in TMEM then, which is rare after the first steps; the two halves agree on the row maximum
//                      through shared memory and a 64-thread named barrier), writes P as fp16 into a K-major
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
constexpr int kFlStages = 3;                        // K/V stages in flight
constexpr int kFlSoftmax = 8;                       // softmax warps: two per TMEM lane quarter, 32 keys of a step each
constexpr int kFlThreads = 32 * (kFlSoftmax + 2 * kFlStages + 1);   // + 2 loader warps per stage + 1 issuer warp
constexpr int kFlIssuer = kFlSoftmax + 2 * kFlStages;
constexpr int kFlKBytes = kFlKeys * 256 * 2;        // [32 channel pieces][64 keys][8 halves]
constexpr int kFlPBytes = 128 * kFlKeys * 2;        // [8 key pieces][128 rows][8 halves]
constexpr size_t kFlashSmem = 2 * kFlStages * kFlKBytes + 2 * kFlPBytes + 128;
// TMEM columns: O 0-255, S of step j at 256 + 64 (j & 1), the query tile (two fp16 channels per column) at 384-511
constexpr uint32_t kColO = 0, kColS = 256, kColQ = 384;
constexpr int kUbThreads = 1024;

struct FlashParams {
  cr_qsa_args a;          // the output rows (pos0 = position of row 0)
  const __half* q_hi;     // [R][Hq][256]
  const int2* list;       // [tiles][cap] (block, row mask), ascending blocks
  const int* count;       // [tiles]
  float* gated;           // gated fp32 [R][Hq * 256] when the output transform runs as a second kernel, else null
  int cap, RT, Hq, Hkv, fmt;
  int flash_max;          // tiles whose union list is longer are left to the row-wise kernels
};

int qsa_union_rows(const cr_geometry* g) {
  const int most = 128 / (g->q_heads / g->kv_heads);
  const int want = options().qsa_union_rows;
  return want > 0 && want < most ? want : most;
}
int qsa_union_cap(int RT) { return (RT * 513 + 15) / 16 * 16; }

// ---- union lists -------------------------------------------------------------------------------------------
// One CTA per tile.  Every (block, row) pair of the tile becomes a 32-bit key block * 16 + row; the keys are sorted
// in shared memory (bitonic network), which puts the rows of one block side by side.  The first key of every block
// gathers the row bits of its run (at most 16 keys) and takes its place in the output from a prefix sum over the
// run heads.
__global__ void __launch_bounds__(kUbThreads) qsa_union_build_kernel(cr_qsa_args a, int2* list, int* count, int cap, int RT, int n_pad) {
  extern __shared__ __align__(16) unsigned ukeys[];      // n_pad keys (a power of two >= RT * 513)
  __shared__ unsigned red[33];
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int tile = blockIdx.x, row0 = tile * RT;
  constexpr unsigned kNone = 0xFFFFFFFFu;                // padding: sorts last
  for (int i = t; i < n_pad; i += kUbThreads) ukeys[i] = kNone;
  __syncthreads();
  if (w < RT && row0 + w < a.R) {                         // one warp per row: slots [513 w, 513 w + 513)
    const int gr = row0 + w, p = a.pos0 + gr, nb = (p + 1) / 4, ns = a.nsel[gr];
    const int n = ns < 0 ? nb : CR_SEL_BLOCKS;           // dense rows attend every complete block (at most 512 of them)
    const int* sel = a.sel + (size_t)gr * CR_SEL_BLOCKS;
    unsigned* mine = ukeys + w * 513;
    for (int i = l; i < n; i += 32) mine[i] = ((unsigned)(ns < 0 ? i : sel[i]) << 4) | (unsigned)w;
    if ((p + 1) % 4 != 0 && l == 0) mine[n] = ((unsigned)nb << 4) | (unsigned)w;   // the open block holds the tail tokens
  }
  // ascending bitonic sort
  for (int k = 2; k <= n_pad; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      __syncthreads();
      for (int q = t; q < (n_pad >> 1); q += kUbThreads) {
        const int i = ((q & ~(j - 1)) << 1) | (q & (j - 1));
        const unsigned x = ukeys[i], y = ukeys[i + j];
        const bool up = (i & k) == 0;
        if ((x > y) == up) { ukeys[i] = y; ukeys[i + j] = x; }
      }
    }
  }
  __syncthreads();
  // run heads: thread t owns the keys [t * per, (t + 1) * per)
  const int per = n_pad / kUbThreads;
  int heads = 0;
  for (int i = t * per; i < (t + 1) * per; ++i) {
    const unsigned k = ukeys[i];
    heads += k != kNone && (i == 0 || (ukeys[i - 1] >> 4) != (k >> 4));
  }
  // exclusive prefix sum of `heads` over the block
  unsigned inc = (unsigned)heads;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const unsigned o = __shfl_up_sync(0xffffffffu, inc, s);
    if (l >= s) inc += o;
  }
  if (l == 31) red[w] = inc;
  __syncthreads();
  if (w == 0) {
    const unsigned mine = red[l];
    unsigned winc = mine;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const unsigned o = __shfl_up_sync(0xffffffffu, winc, s);
      if (l >= s) winc += o;
    }
    red[l] = winc - mine;
    if (l == 31) red[32] = winc;
  }
  __syncthreads();
  int at = (int)(red[w] + inc) - heads;
  int2* out = list + (size_t)tile * cap;
  for (int i = t * per; i < (t + 1) * per; ++i) {
    const unsigned k = ukeys[i];
    if (k == kNone || (i != 0 && (ukeys[i - 1] >> 4) == (k >> 4))) continue;
    int mask = 0;
    for (int e = i; e < n_pad && (ukeys[e] >> 4) == (k >> 4); ++e) mask |= 1 << (ukeys[e] & 15u);
    out[at++] = make_int2((int)(k >> 4), mask);
  }
  if (t == 0) count[tile] = (int)red[32];
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
  unsigned char* Ks = sm;                                // kFlStages stages
  unsigned char* Vs = Ks + kFlStages * kFlKBytes;        // kFlStages stages
  unsigned char* Ps = Vs + kFlStages * kFlKBytes;        // two buffers
  __shared__ __align__(8) uint64_t bars[2 * kFlStages + 4];
  __shared__ unsigned seen_s[kFlStages][16][2];          // per stage and row of the tile: which of the step's 64 keys the row sees
  __shared__ float half_max[2][2][128];                  // [step parity][half][lane]: exchange between the two warps of a TMEM lane quarter
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int dead;
  uint64_t *kvFull = &bars[0], *pvDone = &bars[kFlStages], *sFull = &bars[2 * kFlStages], *pFull = &bars[2 * kFlStages + 2];
  const cr_qsa_args& a = P.a;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int tile = blockIdx.x, g = blockIdx.y, row0 = tile * P.RT;
  const int gqa = P.Hq / P.Hkv;
  const int cnt = P.count[tile];
  const int n = (cnt + kFlBlocks - 1) / kFlBlocks;
  if (n == 0 || cnt > P.flash_max) return;               // a tile without rows, or one the row-wise kernels serve
  const int last_pos = a.pos0 + a.R - 1;                 // newest position the cache holds

  if (t == 0) {
    for (int i = 0; i < kFlStages; ++i) {
      umma::mbar_init(&kvFull[i], 2);                    // the two loader warps of the stage
      umma::mbar_init(&pvDone[i], 1);                    // every MMA that read the stage has completed
    }
    for (int i = 0; i < 2; ++i) {
      umma::mbar_init(&sFull[i], 1);
      umma::mbar_init(&pFull[i], kFlSoftmax);            // one arrival per softmax warp
    }
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == kFlIssuer) umma::tmem_alloc(&tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  // Query tile into tensor memory: M row m = (row m / gqa of the tile, head m % gqa of the group) = TMEM lane m, the
  // 256 fp16 channels of the row as 128 columns (the A operand of S = Q K^T is read from tensor memory).
  if (w < 4) {
    const int m = t, r = m / gqa, hq = m % gqa;
    const bool have = r < P.RT && row0 + r < a.R;
    const uint4* src = reinterpret_cast<const uint4*>(P.q_hi + ((size_t)(have ? row0 + r : 0) * P.Hq + g * gqa + hq) * 256);
#pragma unroll 1
    for (int c8 = 0; c8 < 4; ++c8) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 x = have ? src[c8 * 8 + i] : make_uint4(0u, 0u, 0u, 0u);
        v[4 * i] = __uint_as_float(x.x); v[4 * i + 1] = __uint_as_float(x.y); v[4 * i + 2] = __uint_as_float(x.z); v[4 * i + 3] = __uint_as_float(x.w);
      }
      umma::tmem_st32(umma::tmem_addr(tm, w, kColQ + 32 * c8), v);
    }
    umma::tmem_st_wait();
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  bool gave_up = false;
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (gave_up) return;
    if (!umma::mbar_wait_timed(bar, parity, &dead)) { gave_up = true; dead = 1; g_qsa_flash_status = 1; }
  };
  auto warp_wait = [&](uint64_t* bar, uint32_t parity) {   // lane 0 polls for the warp
    if (l == 0) wait(bar, parity);
    __syncwarp();
  };

  if (w == kFlIssuer) {
    // ------------------------------------------------------------------ issuer
    if (l == 0) {
      constexpr uint32_t idS = umma::idesc_f16(128, kFlKeys, false, false), idO = umma::idesc_f16(128, 256, false, true);
      auto issue_S = [&](int j) {
        const uint64_t dK = umma::smem_desc(Ks + (j % kFlStages) * kFlKBytes, kFlKeys * 16, 128);
#pragma unroll
        for (int ks = 0; ks < 16; ++ks)                  // 16 channels per MMA: 8 columns of Q, two 16-byte pieces of every key
          umma::mma_f16_ts(tm + kColS + 64 * (j & 1), tm + kColQ + 8 * ks, dK + (uint64_t)(ks * 2 * kFlKeys), idS, ks > 0);
        umma::commit(&sFull[j & 1]);
      };
      // Event loop: S of step ns (one step ahead of the softmax at most, its accumulator being free once the
      // probabilities of step ns - 2 are written) as soon as its tiles have landed, O += P V of step np as soon as its
      // probabilities are written; neither waits for the other's barrier.
      auto ready = [&](uint64_t* bar, uint32_t parity) { return umma::mbar_try(umma::smem_u32(bar), parity); };
      auto now_ns = [] { uint64_t v; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v)); return v; };
      int ns = 0, np = 0, idle = 0;
      uint64_t t_idle = 0;
      while (np < n) {
        if (ns < n && ns <= np + 1 && ready(&kvFull[ns % kFlStages], (ns / kFlStages) & 1)) {
          umma::fence_after_sync();
          issue_S(ns);
          ++ns; idle = 0;
        } else if (np < ns && ready(&pFull[np & 1], (np >> 1) & 1)) {
          const int st = np % kFlStages;
          umma::fence_after_sync();
          const uint64_t dP = umma::smem_desc(Ps + (np & 1) * kFlPBytes, 128 * 16, 128);
          const uint64_t dV = umma::smem_desc(Vs + st * kFlKBytes, 128, kFlKeys * 16);   // MN-major: step along keys 128 B, along channels 1 KB
#pragma unroll
          for (int kk = 0; kk < kFlKeys / 16; ++kk)
            umma::mma_f16_ss(tm + kColO, dP + (uint64_t)(kk * 2 * 128), dV + (uint64_t)(kk * 16), idO, (np > 0 || kk > 0) ? 1u : 0u);
          umma::commit(&pvDone[st]);
          ++np; idle = 0;
        } else if ((++idle & 63) == 0) {                  // nothing ready: look at the clock now and then
          const uint64_t t1 = now_ns();
          if (idle == 64) t_idle = t1;
          if (dead || t1 - t_idle > 2000000000ull) { dead = 1; g_qsa_flash_status = 1; break; }
        }
      }
    }
  } else if (w >= kFlSoftmax) {
    // ------------------------------------------------------------------ loaders: two warps per stage
    const int st = (w - kFlSoftmax) >> 1, lw = (w - kFlSoftmax) & 1;
    const __half* kc = reinterpret_cast<const __half*>(a.c.k) + (size_t)g * 256 + (l & 1) * 8;
    const __half* vc = reinterpret_cast<const __half*>(a.c.v) + (size_t)g * 256 + (l & 1) * 8;
    const int2* lst = P.list + (size_t)tile * P.cap;
    const size_t row_halves = (size_t)P.Hkv * 256;
    unsigned char* kd = Ks + st * kFlKBytes;
    unsigned char* vd = Vs + st * kFlKBytes;
    for (int j = st; j < n; j += kFlStages) {
      if (j >= kFlStages) warp_wait(&pvDone[st], ((j - kFlStages) / kFlStages) & 1);   // the MMAs of the stage's last step are done
      if (dead) break;
      if (lw == 0) {
        // Lane b < 16 holds entry b of the step; lane r < 16 then builds the word of row r: bit 4 b + k is set when the
        // row's bit of block b's mask is set and token k of the block is not in the row's future (only the open tail
        // block of a row can hold such tokens).  The softmax threads read one word per step.
        const int idx = j * kFlBlocks + (l & 15);
        const int2 e = idx < cnt ? lst[idx] : make_int2(0, 0);
        const int prow = a.pos0 + row0 + (l & 15);
        const bool rowok = (l & 15) < P.RT && row0 + (l & 15) < a.R;
        unsigned lo_w = 0u, hi_w = 0u;
#pragma unroll
        for (int b = 0; b < kFlBlocks; ++b) {
          const int blk = __shfl_sync(0xffffffffu, e.x, b), msk = __shfl_sync(0xffffffffu, e.y, b);
          const int lim = prow - blk * 4;                             // tokens 0 .. lim of the block are visible
          const unsigned nib = (rowok && ((msk >> (l & 15)) & 1)) ? (lim >= 3 ? 0xFu : (lim < 0 ? 0u : (2u << lim) - 1u)) : 0u;
          if (b < 8) lo_w |= nib << (4 * b); else hi_w |= nib << (4 * (b - 8));
        }
        if (l < 16) { seen_s[st][l][0] = lo_w; seen_s[st][l][1] = hi_w; }
      }
      // lane l serves key 16 kg + l / 2 (kg = 0..3) and the channel pieces 2 pp + l % 2, pp = 8 lw .. 8 lw + 7
#pragma unroll
      for (int kg = 0; kg < 4; ++kg) {
        const int key = kg * 16 + (l >> 1), idx = j * kFlBlocks + (key >> 2);
        const int pos = (idx < cnt ? lst[idx].x : 0) * 4 + (key & 3);
        const bool valid = pos <= last_pos;
        const size_t src = valid ? (size_t)pos * row_halves : 0;
        const size_t dst = ((size_t)(l & 1) * kFlKeys + key) * 16;
#pragma unroll
        for (int p8 = 0; p8 < 8; ++p8) {
          const int pp = lw * 8 + p8;
          fl_cp_async16(kd + dst + (size_t)pp * (2 * kFlKeys * 16), kc + src + pp * 16, valid);
          fl_cp_async16(vd + dst + (size_t)pp * (2 * kFlKeys * 16), vc + src + pp * 16, valid);
        }
      }
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
      umma::fence_async_smem();
      __syncwarp();
      if (l == 0) fl_mbar_arrive(&kvFull[st]);
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = (TMEM lane m, half of the step's keys)
    // Warps w and w + 4 share the lanes 32 (w % 4) .. +31; warp w takes the keys 0-31 of a step, warp w + 4 the keys 32-63.
    const int m = t & 127, hf = t >> 7, r = m / gqa, hq = m % gqa;
    const bool rowok = r < P.RT && row0 + r < a.R;
    const int pair_bar = 1 + (w & 3);                                   // named barrier of the two warps of a lane quarter
    auto pair_sync = [&] { asm volatile("bar.sync %0, 64;\n" ::"r"(pair_bar) : "memory"); };
    constexpr float kScale = 0.0625f * 1.4426950408889634f;            // logits / 16, in powers of two
    float m_ref = -INFINITY, lsum = 0.f;
    for (int j = 0; j < n; ++j) {
      const int s = j & 1, st = j % kFlStages;
      warp_wait(&kvFull[st], (j / kFlStages) & 1);                     // block ids and masks of the step are visible
      const unsigned seen = r < 16 ? seen_s[st][r][hf] : 0u;             // which of this thread's 32 keys its row sees
      warp_wait(&sFull[s], (j >> 1) & 1);
      umma::fence_after_sync();
      float sv[32];
      umma::tmem_ld32(umma::tmem_addr(tm, w, kColS + 64 * s + 32 * hf), sv);
      float tmax = -INFINITY;
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        sv[c] = (seen >> c) & 1u ? sv[c] * kScale : -INFINITY;
        tmax = fmaxf(tmax, sv[c]);
      }
      half_max[s][hf][m] = tmax;                                        // (parity: the partner may still be reading the step before)
      pair_sync();
      tmax = fmaxf(tmax, half_max[s][hf ^ 1][m]);                       // the row's maximum over all 64 keys of the step
      const bool move = tmax > m_ref + 8.f;                             // also the first visible key (m_ref = -inf)
      if (__any_sync(0xffffffffu, move)) {
        const float nref = move ? tmax : m_ref;
        const float factor = move ? exp2f(m_ref - nref) : 1.f;          // 0 when nothing was accumulated yet
        lsum *= factor;
        m_ref = nref;
        if (j > 0) {                                                    // O holds the steps before this one; each warp rescales half of it
          warp_wait(&pvDone[(j - 1) % kFlStages], ((j - 1) / kFlStages) & 1);
          umma::fence_after_sync();
#pragma unroll 1
          for (int c8 = 4 * hf; c8 < 4 * hf + 4; ++c8) {
            float o[32];
            umma::tmem_ld32(umma::tmem_addr(tm, w, kColO + 32 * c8), o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] *= factor;
            umma::tmem_st32(umma::tmem_addr(tm, w, kColO + 32 * c8), o);
          }
          umma::tmem_st_wait();
        }
      }
      if (j >= 2) warp_wait(&pvDone[(j - 2) % kFlStages], ((j - 2) / kFlStages) & 1);   // the MMAs of step j - 2 have read this P buffer
      unsigned char* pd = Ps + s * kFlPBytes;
      float add = 0.f;
#pragma unroll
      for (int kc8 = 0; kc8 < 4; ++kc8) {
        unsigned pk[4];
#pragma unroll
        for (int q2 = 0; q2 < 4; ++q2) {
          float p0, p1;                                                // 2^(-inf) = 0: keys the row does not see drop out
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(sv[kc8 * 8 + 2 * q2] - m_ref));
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(sv[kc8 * 8 + 2 * q2 + 1] - m_ref));
          if (m_ref == -INFINITY) p0 = p1 = 0.f;                       // -inf - -inf: nothing visible yet
          add += p0 + p1;
          const __half2 h = __floats2half2_rn(p0, p1);
          pk[q2] = *reinterpret_cast<const unsigned*>(&h);
        }
        *reinterpret_cast<uint4*>(pd + ((size_t)(4 * hf + kc8) * 128 + m) * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      lsum += add;
      umma::fence_async_smem();
      umma::fence_before_sync();
      __syncwarp();
      if (l == 0) fl_mbar_arrive(&pFull[s]);
    }
    // ---------------------------------------------------------------- epilogue: each warp of a pair writes half of the channels
    float* half_sum = &half_max[n & 1][0][0];                           // the buffer the last step did not use
    if (hf == 1) half_sum[m] = lsum;
    pair_sync();
    if (hf == 0) { lsum += half_sum[m]; half_sum[128 + m] = lsum; }
    pair_sync();
    lsum = half_sum[128 + m];
    warp_wait(&pvDone[(n - 1) % kFlStages], ((n - 1) / kFlStages) & 1);
    umma::fence_after_sync();
    const bool ok = rowok && lsum > 0.f && !dead;
    const float inv = ok ? 1.f / lsum : 0.f;
    const int gr = row0 + r, h = g * gqa + hq;
    const size_t W = (size_t)P.Hq * 256;
    const float* gate = a.q + ((size_t)gr * P.Hq + h) * 512 + 256;
#pragma unroll 1
    for (int c8 = 4 * hf; c8 < 4 * hf + 4; ++c8) {
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
  if (w == kFlIssuer) umma::tmem_dealloc(tm, 512);
}

// The reference's out-projection input from gated fp32 rows: fp16(WHT128(RoundH(RoundH(o) * suh)) / sqrt(128))
// (engine/layers/qsa_long.h:476-489).  grid (Hq, R), 64 threads: a warp per 128-channel group.
__global__ void __launch_bounds__(64) qsa_out_transform_kernel(cr_qsa_args a, const float* gated, int Hq, const int* tile_count, int RT, int flash_max) {
  const int h = blockIdx.x, r = blockIdx.y, half = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (tile_count[r / RT] > flash_max) return;             // a row of the row-wise kernels, which transform their own output
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
  if (cr_status st = once_per_device(configured, [] {
        CR_CUDA(cudaFuncSetAttribute(qsa_union_build_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * (int)sizeof(unsigned)));
        return CR_OK;
      })) return st;
  const int RT = qsa_union_rows(g), tiles = (a.R + RT - 1) / RT;
  int n_pad = kUbThreads;
  while (n_pad < RT * 513) n_pad <<= 1;
  use_stream(stream);
  qsa_union_build_kernel<<<tiles, kUbThreads, (size_t)n_pad * sizeof(unsigned), stream>>>(a, list, count, qsa_union_cap(RT), RT, n_pad);
  CR_LAUNCH_CHECK("qsa_union_build_kernel");
  return CR_OK;
}

// Attention of the rows of `a` over the union lists; `gated` (rows x Hq x 256 floats) is needed for CR_OUT_EXL3_WHT.
cr_status qsa_flash_launch(const cr_geometry* g, const cr_qsa_args& a, const __half* q_hi, const int2* list, const int* count,
                           float* gated, cr_out_format fmt, int flash_max, cudaStream_t stream) {
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
  P.flash_max = flash_max;
  CR_REQUIRE(fmt != CR_OUT_EXL3_WHT || gated, "qsa flash: the EXL3 output needs the gated fp32 scratch");
  const int tiles = (a.R + P.RT - 1) / P.RT;
  use_stream(stream);
  qsa_flash_tc_kernel<<<dim3(tiles, g->kv_heads), kFlThreads, kFlashSmem, stream>>>(P);
  CR_LAUNCH_CHECK("qsa_flash_tc_kernel");
  if (fmt == CR_OUT_EXL3_WHT) {
    qsa_out_transform_kernel<<<dim3(g->q_heads, a.R), 64, 0, stream>>>(a, gated, g->q_heads, count, P.RT, flash_max);
    CR_LAUNCH_CHECK("qsa_out_transform_kernel");
  }
  return CR_OK;
}

}  // namespace cr
