// Exact top-512 of a row of indexer scores for sm_100a (the job of LaunchQsaTop, engine/layers/qsa_long.h:111-380):
// the 512 best blocks in the total order (score descending, block id ascending), emitted in ascending block id.
//
// Method: group maxima, pivot, filter, bisect, mark, compact.  One CTA of 1024 threads per row.
//   1. Scores are >= +0, so their fp32 bit patterns order like unsigned integers (key = pattern + 1; 0 = no element).
//      Thread t reads the elements t, t + 1024, ... (its group) and keeps their maximum.
//   2. The pivot is the 512th largest of the 1024 group maxima, found by bisection over the key bits: 31 block-wide
//      counts, no sorting and no atomics.  At least 512 elements are >= the pivot (those maxima themselves), so every
//      element that can be among the best 512, ties included, is >= the pivot; with unrelated scores about 700 are.
//   3. A second pass gathers the elements >= the pivot into a shared-memory list (warp-aggregated appends).
//   4. The 512th largest key of the list is found by the same bisection; keys above it are taken, and of the keys
//      equal to it the lowest indices (counted among the ties).
//   5. The taken elements set their bit in a bitmap over the row, which is compacted in index order: a prefix sum over
//      word popcounts gives every thread its output offset.
//   Rows of at most 4096 elements skip 1-3: every element goes into the list.
//   When more than 4096 elements pass the pivot (long runs of equal scores), the row takes the slow exact path: the
//   same bisection over the whole row, counting with plain reductions, then the values above the 512th best pattern
//   plus its first ties in index order from a second bitmap.
// The same routine serves a whole row, a rank's block range (candidates with their scores, for split-KV across
// devices, engine/layers/qsa_long.h:228-234) and the merge of gathered candidates.
#include <climits>
#include <cooperative_groups.h>
#include "qsa.cuh"

namespace cg = cooperative_groups;

namespace cr {

constexpr int kSelThreads = 1024;
constexpr int kMaxSelectCount = 262144;   // elements of one selection: the tie bitmap of the slow path shares the 32 KB of the candidate list
constexpr int kSortCap = 4096;            // entries of the candidate list (32 KB)

// ---- element sources ---------------------------------------------------------------------------------------
// A source maps an element index i in [0, count) to (bit pattern, block id, valid).  Index order is block-id order.
struct RowSource {                         // scores[i], block id = id_base + i
  const float* scores;
  int id_base;
  __device__ __forceinline__ bool get(int i, unsigned& bits) const { bits = __float_as_uint(scores[i]); return true; }
  __device__ __forceinline__ int id(int i) const { return id_base + i; }
};
struct GatheredSource {                    // candidates of several ranks: element i = rank i / 512, slot i % 512
  const float* scores;
  const int* ids;
  size_t rank_stride;                      // elements between the lists of consecutive ranks
  __device__ __forceinline__ size_t at(int i) const { return (size_t)(i >> 9) * rank_stride + (i & 511); }
  __device__ __forceinline__ bool get(int i, unsigned& bits) const {
    const size_t a = at(i);
    if (ids[a] < 0) { bits = 0u; return false; }
    bits = __float_as_uint(scores[a]);
    return true;
  }
  __device__ __forceinline__ int id(int i) const { return ids[at(i)]; }
};

// ---- block-wide helpers ------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned block_sum_u32(unsigned v, unsigned* red) {   // red: 33 words
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned t = red[threadIdx.x];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(0xffffffffu, t, m);
    if (threadIdx.x == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
// Exclusive prefix sum of one value per thread over the block (1024 threads); *total receives the sum.
__device__ __forceinline__ unsigned block_exclusive_scan(unsigned v, unsigned* red, unsigned* total) {
  const int l = threadIdx.x & 31, w = threadIdx.x >> 5;
  unsigned inc = v;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const unsigned o = __shfl_up_sync(0xffffffffu, inc, s);
    if (l >= s) inc += o;
  }
  __syncthreads();
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
    red[l] = winc - mine;                    // exclusive over warps
    if (l == 31) red[32] = winc;
  }
  __syncthreads();
  *total = red[32];
  return red[w] + inc - v;
}
// Shared memory of one CTA: candidate list (32 KB), bitmap over the row's elements (count bits), small arrays.
struct SelectSmem {
  uint2* cand;                 // kSortCap (key, index) pairs; the slow path keeps its tie bitmap here instead
  unsigned* bitmap;            // ceil(count / 32) words
  unsigned* red;               // 33 words
  unsigned* counter;           // 1 word
};

constexpr int kBatch = 8;      // loads a thread issues before it uses any of them

// Calls f(i, key) for the elements i = t, t + 1024, ... < count of this thread, key = bit pattern + 1 (0: no element).
// Loads are issued kBatch at a time.  WARP_UNIFORM: f is also called with key 0 for indices past the end, so that all
// lanes of a warp make the same number of calls (f may use warp-collective operations).
template <bool WARP_UNIFORM, typename Src, typename F>
__device__ __forceinline__ void for_each_key(const Src& src, int count, F&& f) {
  const int lane = threadIdx.x & 31;
  for (int i0 = threadIdx.x; i0 - lane < count; i0 += kSelThreads * kBatch) {   // the same trip count for a whole warp
    unsigned key[kBatch];
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int i = i0 + k * kSelThreads;
      unsigned bits = 0u;
      key[k] = (i < count && src.get(i, bits)) ? bits + 1u : 0u;
    }
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
      const int i = i0 + k * kSelThreads;
      if (WARP_UNIFORM ? (i - lane < count) : (i < count)) f(i, key[k]);
    }
  }
}

// The largest T with at least `want` keys >= T, over keys spread one per thread (mine; 0 = none).
__device__ __forceinline__ unsigned bisect_one_per_thread(unsigned mine, int want) {
  unsigned T = 0u;
  for (int bit = 30; bit >= 0; --bit) {
    const unsigned trial = T | (1u << bit);
    if (__syncthreads_count(mine >= trial) >= want) T = trial;
  }
  return T;
}
// The same over the candidate list: thread t holds the list entries t, t + 1024, ... (at most 4).  Every key lies in
// [lo, hi]: the bits above the first bit in which lo and hi differ are settled, and the search starts below them.
__device__ __forceinline__ unsigned bisect_list(const uint2* cand, int m, int want, unsigned lo, unsigned hi) {
  unsigned k[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) { const int i = threadIdx.x + q * kSelThreads; k[q] = i < m ? cand[i].x : 0u; }
  if (lo >= hi) return lo;
  const int top = 31 - __clz(lo ^ hi);                             // the first differing bit
  unsigned T = lo & ~((2u << top) - 1u);
  for (int bit = top; bit >= 0; --bit) {
    const unsigned trial = T | (1u << bit);
    const int c = (k[0] >= trial) + (k[1] >= trial) + (k[2] >= trial) + (k[3] >= trial);
    int total;
    if (m <= kSelThreads) total = __syncthreads_count(c);
    else total = __syncthreads_count(c & 1) + 2 * __syncthreads_count(c & 2) + 4 * __syncthreads_count(c & 4);
    if (total >= want) T = trial;
  }
  return T;
}

// The list sm.cand[0, m) holds (key, index) pairs that include the `want` best elements of the row (want <= m <= kSortCap):
// marks those in sm.bitmap.  The want-th largest key by bisection; keys above it are taken, and of the keys equal to it
// the lowest indices (counted among the ties).
__device__ __forceinline__ void select_from_list(int m, int want, const SelectSmem& sm, unsigned lo = 0u, unsigned hi = 0x7FFFFFFFu) {
  const int t = threadIdx.x;
  const unsigned T = bisect_list(sm.cand, m, want, lo, hi);
  int gt = 0, eq = 0;
  for (int i = t; i < m; i += kSelThreads) { const unsigned k = sm.cand[i].x; gt += k > T; eq += k == T; }
  const int n_gt = (int)block_sum_u32((unsigned)gt, sm.red), n_eq = (int)block_sum_u32((unsigned)eq, sm.red);
  const int need = want - n_gt;                                    // ties to take: 1 <= need <= n_eq
  for (int i = t; i < m; i += kSelThreads) {
    const uint2 c = sm.cand[i];
    bool take = c.x > T;
    if (c.x == T) {
      if (need >= n_eq) take = true;
      else {                                                       // rank among the ties by index
        int before = 0;
        for (int j = 0; j < m; ++j) { const uint2 o = sm.cand[j]; before += (o.x == T && o.y < c.y); }
        take = before < need;
      }
    }
    if (take) atomicOr(&sm.bitmap[c.y >> 5], 1u << (c.y & 31));
  }
  __syncthreads();
}

template <typename Src>
__device__ __forceinline__ void select_slow(const Src& src, int count, int want, const SelectSmem& sm);

// Marks the `want` best elements of [0, count) in sm.bitmap (bit i = element i selected).  want <= valid elements.
template <typename Src>
__device__ __forceinline__ void select_mark(const Src& src, int count, int want, const SelectSmem& sm) {
  const int t = threadIdx.x, l = t & 31;
  const int words = (count + 31) >> 5;
  for (int i = t; i < words; i += kSelThreads) sm.bitmap[i] = 0u;
  if (t == 0) *sm.counter = 0u;
  unsigned pivot = 1u;                                             // every element passes
  if (count > kSortCap) {
    unsigned mine = 0u;
    for_each_key<false>(src, count, [&](int, unsigned key) { mine = key > mine ? key : mine; });
    pivot = bisect_one_per_thread(mine, want);                     // 0 when fewer than `want` groups hold an element
    if (pivot == 0u) pivot = 1u;
  }
  __syncthreads();
  // ---- the elements >= pivot, as (key, index) pairs
  for_each_key<true>(src, count, [&](int i, unsigned key) {
    const bool pass = key >= pivot;
    const unsigned m = __ballot_sync(0xffffffffu, pass);
    if (m) {
      unsigned base = 0u;
      if (l == 0) base = atomicAdd(sm.counter, (unsigned)__popc(m));
      base = __shfl_sync(0xffffffffu, base, 0);
      const unsigned at = base + __popc(m & ((1u << l) - 1u));
      if (pass && at < (unsigned)kSortCap) sm.cand[at] = make_uint2(key, (unsigned)i);
    }
  });
  __syncthreads();
  const int m = (int)*sm.counter;
  if (m >= want && m <= kSortCap) { select_from_list(m, want, sm, pivot); return; }
  select_slow(src, count, want, sm);
}

// The slow exact path over the whole row; sm.bitmap zero on entry.
template <typename Src>
__device__ __forceinline__ void select_slow(const Src& src, int count, int want, const SelectSmem& sm) {
  const int t = threadIdx.x, l = t & 31;
  const int words = (count + 31) >> 5;
  // ---- slow exact path: T = the largest key with at least `want` elements >= T
  unsigned T = 0u;
  for (int bit = 30; bit >= 0; --bit) {
    const unsigned trial = T | (1u << bit);
    unsigned c = 0u;
    for_each_key<false>(src, count, [&](int, unsigned key) { c += key >= trial; });
    if (block_sum_u32(c, sm.red) >= (unsigned)want) T = trial;
  }
  unsigned* ties = reinterpret_cast<unsigned*>(sm.cand);           // bitmap of the elements equal to T (<= 32 KB)
  unsigned above = 0u;
  for_each_key<true>(src, count, [&](int i, unsigned key) {        // a warp covers one bitmap word per call
    const unsigned gt = __ballot_sync(0xffffffffu, key > T), eq = __ballot_sync(0xffffffffu, key == T);
    if (l == 0 && (i >> 5) < words) { sm.bitmap[i >> 5] = gt; ties[i >> 5] = eq; above += __popc(gt); }
  });
  const unsigned n_above = block_sum_u32(above, sm.red);
  const unsigned need = (unsigned)want - n_above;                  // ties to take, lowest indices first
  // every thread owns a run of consecutive words: ties before the run decide how many of its own it takes
  const int per = (words + kSelThreads - 1) / kSelThreads, w0 = t * per, w1 = min(w0 + per, words);
  unsigned mine = 0u;
  for (int w = w0; w < w1; ++w) mine += __popc(ties[w]);
  unsigned total = 0u;
  unsigned before = block_exclusive_scan(mine, sm.red, &total);
  for (int w = w0; w < w1 && before < need; ++w) {
    unsigned e = ties[w];
    const unsigned c = __popc(e);
    if (before + c > need) {                                       // keep only the lowest (need - before) set bits
      unsigned keep = 0u;
      for (unsigned k = need - before; k > 0; --k) { const unsigned low = e & (0u - e); keep |= low; e ^= low; }
      e = keep;
    }
    sm.bitmap[w] |= e;
    before += c;
  }
  __syncthreads();
}

// Writes the marked elements in index order: out_ids (and out_scores) get `want` entries.
template <typename Src>
__device__ __forceinline__ void select_emit(const Src& src, int count, const SelectSmem& sm, int* out_ids, float* out_scores) {
  const int t = threadIdx.x;
  const int words = (count + 31) >> 5;
  const int per = (words + kSelThreads - 1) / kSelThreads, w0 = t * per, w1 = min(w0 + per, words);
  unsigned mine = 0u;
  for (int w = w0; w < w1; ++w) mine += __popc(sm.bitmap[w]);
  unsigned total = 0u;
  unsigned at = block_exclusive_scan(mine, sm.red, &total);
  for (int w = w0; w < w1; ++w) {
    unsigned m = sm.bitmap[w];
    while (m) {
      const int i = (w << 5) + __ffs(m) - 1;
      m &= m - 1;
      out_ids[at] = src.id(i);
      if (out_scores) { unsigned bits; src.get(i, bits); out_scores[at] = __uint_as_float(bits); }
      ++at;
    }
  }
}

__device__ __forceinline__ SelectSmem carve(unsigned char* raw, int max_count) {
  SelectSmem sm;
  sm.cand = reinterpret_cast<uint2*>(raw);
  sm.bitmap = reinterpret_cast<unsigned*>(raw + (size_t)kSortCap * 8);
  sm.red = sm.bitmap + ((max_count + 31) >> 5);
  sm.counter = sm.red + 33;
  return sm;
}
static size_t select_smem_bytes(int max_count) { return (size_t)kSortCap * 8 + (size_t)((max_count + 31) / 32) * 4 + 34 * 4 + 16; }

// grid (rows, spans): the selection of one row.
__global__ void __launch_bounds__(kSelThreads) qsa_topk_kernel(const __grid_constant__ QsaParams P, int max_count) {
  extern __shared__ __align__(16) unsigned char raw[];
  pdl_release();
  pdl_wait();
  const cr_qsa_args& a = P.span[blockIdx.y];
  const int r = blockIdx.x;
  if (r >= a.R) return;
  const int nb = (a.pos0 + r + 1) / 4;
  if (nb <= CR_SEL_BLOCKS) { if (threadIdx.x == 0) a.nsel[r] = -1; return; }
  const SelectSmem sm = carve(raw, max_count);
  const RowSource src{a.scores + (size_t)r * a.sstride, 0};
  select_mark(src, nb, CR_SEL_BLOCKS, sm);
  select_emit(src, nb, sm, a.sel + (size_t)r * CR_SEL_BLOCKS, nullptr);
  if (threadIdx.x == 0) a.nsel[r] = CR_SEL_BLOCKS;
}

// Sorts the 32 values of a warp (one per lane) so that lane 0 holds the largest: a bitonic network of shuffles.
__device__ __forceinline__ unsigned warp_sort_desc(unsigned v) {
  const int l = threadIdx.x & 31;
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const unsigned o = __shfl_xor_sync(0xffffffffu, v, j);
      const bool down = (l & k) == 0, low_lane = (l & j) == 0;       // in a descending run the lower lane keeps the larger value
      v = (low_lane == down) ? (v > o ? v : o) : (v < o ? v : o);
    }
  }
  return v;
}
// Descending bitonic sort of 128 values in shared memory by one warp.
__device__ __forceinline__ void warp_sort128_desc(unsigned* a) {
  const int l = threadIdx.x & 31;
  for (int k = 2; k <= 128; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      __syncwarp();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int q = l + 32 * h, i = ((q & ~(j - 1)) << 1) | (q & (j - 1));
        const unsigned x = a[i], y = a[i + j];
        if ((x < y) == ((i & k) == 0)) { a[i] = y; a[i + j] = x; }
      }
    }
  __syncwarp();
}

// The selection of one row by a cluster of 8 CTAs, for launches of few rows (decode and verify steps), where the time
// of one row is what counts: every CTA keeps an eighth of the row in registers (one read of the row, spread over 8
// SMs).  Pivot: every warp sorts its threads' maxima and lists the best four, a CTA offers the 64th largest of its 128
// listed values (64 of its elements are >= it; usually it is the CTA's 64th largest element), the cluster takes the
// smallest offer of its CTAs (512 elements are >= it; about 600 of 65,536 unrelated scores are).  Every CTA lists
// its elements >= the pivot in its own shared memory; CTA 0 collects the lists through distributed shared memory and
// finishes as the single-CTA kernel does.  grid (8 x rows, spans).
template <int PT>
__global__ void __cluster_dims__(8, 1, 1) __launch_bounds__(kSelThreads, 1) qsa_topk_cluster_kernel(const __grid_constant__ QsaParams P, int max_count) {
  extern __shared__ __align__(16) unsigned char raw[];
  __shared__ unsigned offer_s, max_s, count_s;                     // read by the other CTAs of the cluster
  __shared__ unsigned top4[128];
  pdl_release();
  pdl_wait();
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const cr_qsa_args& a = P.span[blockIdx.y];
  const int r = blockIdx.x / 8, t = threadIdx.x, l = t & 31;
  if (r >= a.R) return;                                            // the same for the whole cluster
  const int nb = (a.pos0 + r + 1) / 4;
  if (nb <= CR_SEL_BLOCKS) { if (rank == 0 && t == 0) a.nsel[r] = -1; return; }
  const SelectSmem sm = carve(raw, max_count);
  const float* sc = a.scores + (size_t)r * a.sstride;
  const int chunk = (((nb + 7) / 8) + kSelThreads - 1) / kSelThreads * kSelThreads;   // elements per CTA, a multiple of 1024
  const int base = rank * chunk;
  unsigned u[PT];
  unsigned mine = 0u;
#pragma unroll
  for (int k = 0; k < PT; ++k) {
    const int i = base + k * kSelThreads + t;
    u[k] = (k * kSelThreads < chunk && i < nb) ? __float_as_uint(sc[i]) + 1u : 0u;
    mine = u[k] > mine ? u[k] : mine;
  }
  const int words = (nb + 31) >> 5;
  if (rank == 0) for (int i = t; i < words; i += kSelThreads) sm.bitmap[i] = 0u;
  if (t == 0) *sm.counter = 0u;
  const unsigned sorted = warp_sort_desc(mine);
  if (l < 4) top4[(t >> 5) * 4 + l] = sorted;
  __syncthreads();
  if (t < 32) {
    warp_sort128_desc(top4);
    if (t == 0) { offer_s = top4[63]; max_s = top4[0]; }
  }
  cluster.sync();
  if (t < 8) {                                                     // eight threads fetch the offers of the eight CTAs
    unsigned x = *cluster.map_shared_rank(&offer_s, t), y = *cluster.map_shared_rank(&max_s, t);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const unsigned xo = __shfl_xor_sync(0xffu, x, o), yo = __shfl_xor_sync(0xffu, y, o);
      x = xo < x ? xo : x;
      y = yo > y ? yo : y;
    }
    if (t == 0) { sm.red[0] = x; sm.red[1] = y; }
  }
  __syncthreads();
  unsigned pivot = sm.red[0];
  const unsigned largest = sm.red[1];
  if (pivot == 0u) pivot = 1u;                                     // a CTA with fewer than 64 threads that hold an element: everything passes
#pragma unroll
  for (int k = 0; k < PT; ++k) {
    const bool pass = u[k] >= pivot && u[k] != 0u;
    const unsigned m = __ballot_sync(0xffffffffu, pass);
    if (m) {
      unsigned at = 0u;
      if (l == 0) at = atomicAdd(sm.counter, (unsigned)__popc(m));
      at = __shfl_sync(0xffffffffu, at, 0) + __popc(m & ((1u << l) - 1u));
      if (pass && at < (unsigned)kSortCap) sm.cand[at] = make_uint2(u[k], (unsigned)(base + k * kSelThreads + t));
    }
  }
  __syncthreads();
  if (t == 0) count_s = *sm.counter;
  cluster.sync();
  if (rank == 0) {
    int total = 0, first[9];
#pragma unroll
    for (int c = 0; c < 8; ++c) { first[c] = total; total += (int)*cluster.map_shared_rank(&count_s, c); }
    first[8] = total;
    if (total <= kSortCap) {
      for (int c = 1; c < 8; ++c) {
        const uint2* theirs = cluster.map_shared_rank(sm.cand, c);
        for (int i = t; i < first[c + 1] - first[c]; i += kSelThreads) sm.cand[first[c] + i] = theirs[i];
      }
    }
    __syncthreads();
    const RowSource src{sc, 0};
    if (total >= CR_SEL_BLOCKS && total <= kSortCap) select_from_list(total, CR_SEL_BLOCKS, sm, pivot, largest);
    else select_slow(src, nb, CR_SEL_BLOCKS, sm);
    select_emit(src, nb, sm, a.sel + (size_t)r * CR_SEL_BLOCKS, nullptr);
    if (t == 0) a.nsel[r] = CR_SEL_BLOCKS;
  }
  cluster.sync();                                                  // the lists stay until CTA 0 has copied them
}

// A rank's candidates among blocks [b0, b1): its best 512 (score, id), ascending id, unused slots -1.
__global__ void __launch_bounds__(kSelThreads) qsa_candidates_kernel(const __grid_constant__ QsaParams P, int b0, int b1, float* cand_scores,
                                                                     int* cand_ids, int max_count) {
  extern __shared__ __align__(16) unsigned char raw[];
  const cr_qsa_args& a = P.span[0];
  const int r = blockIdx.x, t = threadIdx.x;
  const int nb = (a.pos0 + r + 1) / 4;
  float* cs = cand_scores + (size_t)r * CR_SEL_BLOCKS;
  int* ci = cand_ids + (size_t)r * CR_SEL_BLOCKS;
  const int count = min(nb, b1) - b0;
  if (nb <= CR_SEL_BLOCKS || count <= CR_SEL_BLOCKS) {              // dense row, or the rank owns at most 512 blocks: all of them
    if (t < CR_SEL_BLOCKS) {
      const bool have = nb > CR_SEL_BLOCKS && t < count;
      cs[t] = have ? a.scores[(size_t)r * a.sstride + b0 + t] : -1.f;
      ci[t] = have ? b0 + t : -1;
    }
    return;
  }
  const SelectSmem sm = carve(raw, max_count);
  const RowSource src{a.scores + (size_t)r * a.sstride + b0, b0};
  select_mark(src, count, CR_SEL_BLOCKS, sm);
  select_emit(src, count, sm, ci, cs);
}

// Global selection from the gathered candidates [ranks][rows][512] of all ranks (ranks own ascending block ranges).
__global__ void __launch_bounds__(kSelThreads) qsa_merge_candidates_kernel(const __grid_constant__ QsaParams P, int ranks, const float* cand_scores,
                                                                           const int* cand_ids, int max_count) {
  extern __shared__ __align__(16) unsigned char raw[];
  const cr_qsa_args& a = P.span[0];
  const int r = blockIdx.x;
  const int nb = (a.pos0 + r + 1) / 4;
  if (nb <= CR_SEL_BLOCKS) { if (threadIdx.x == 0) a.nsel[r] = -1; return; }
  const SelectSmem sm = carve(raw, max_count);
  const size_t off = (size_t)r * CR_SEL_BLOCKS;
  const GatheredSource src{cand_scores + off, cand_ids + off, (size_t)a.R * CR_SEL_BLOCKS};
  select_mark(src, ranks * CR_SEL_BLOCKS, CR_SEL_BLOCKS, sm);
  select_emit(src, ranks * CR_SEL_BLOCKS, sm, a.sel + off, nullptr);
  if (threadIdx.x == 0) a.nsel[r] = CR_SEL_BLOCKS;
}

static cr_status select_configure() {
  static PerDeviceOnce configured;
  return once_per_device(configured, [] {
    const int most = (int)select_smem_bytes(kMaxSelectCount);
    CR_CUDA(cudaFuncSetAttribute(qsa_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    CR_CUDA(cudaFuncSetAttribute(qsa_topk_cluster_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    CR_CUDA(cudaFuncSetAttribute(qsa_topk_cluster_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    CR_CUDA(cudaFuncSetAttribute(qsa_candidates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    CR_CUDA(cudaFuncSetAttribute(qsa_merge_candidates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most));
    return CR_OK;
  });
}

cr_status qsa_topk_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream) {
  use_stream(stream);
  if (cr_status st = select_configure()) return st;
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    const int Rmax = qsa_max_rows(spans + s0, n);
    int nb_max = 0;
    for (int s = 0; s < n; ++s) nb_max = max(nb_max, (spans[s0 + s].pos0 + spans[s0 + s].R) / 4);
    CR_REQUIRE(nb_max <= kMaxSelectCount, "qsa select: %d blocks exceed the selectable range of %d", nb_max, kMaxSelectCount);
    if ((long long)Rmax * n <= 64 && nb_max >= 16384) {             // few long rows: 8 SMs per row
      if (nb_max <= 65536) CR_CUDA(launch_pdl(qsa_topk_cluster_kernel<8>, dim3(8 * Rmax, n), dim3(kSelThreads), select_smem_bytes(nb_max), stream, P, nb_max));
      else CR_CUDA(launch_pdl(qsa_topk_cluster_kernel<32>, dim3(8 * Rmax, n), dim3(kSelThreads), select_smem_bytes(nb_max), stream, P, nb_max));
      CR_LAUNCH_CHECK("qsa_topk_cluster_kernel");
      continue;
    }
    CR_CUDA(launch_pdl(qsa_topk_kernel, dim3(Rmax, n), dim3(kSelThreads), select_smem_bytes(nb_max), stream, P, nb_max));
    CR_LAUNCH_CHECK("qsa_topk_kernel");
  }
  return CR_OK;
}

}  // namespace cr

extern "C" cr_status cr_qsa_shard_candidates(const cr_geometry* g, const cr_qsa_args* a, int b0, int b1, float* cand_scores,
                                             int* cand_ids, void* stream) {
  using namespace cr;
  CR_REQUIRE(a && b0 >= 0 && b1 >= b0, "cr_qsa_shard_candidates: bad block range");
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_shard_candidates", (b1 < (a->pos0 + a->R) / 4 ? b1 : (a->pos0 + a->R) / 4) - b0)) return s;
  CR_REQUIRE(cand_scores && cand_ids && b0 >= 0 && b1 >= b0 && b1 - b0 <= kMaxSelectCount, "cr_qsa_shard_candidates: bad block range or null output");
  if (cr_status st = select_configure()) return st;
  QsaParams P;
  qsa_fill_params(P, g, a, 1);
  use_stream((cudaStream_t)stream);
  const int most = b1 - b0 > 1 ? b1 - b0 : 1;
  qsa_candidates_kernel<<<a->R, kSelThreads, select_smem_bytes(most), (cudaStream_t)stream>>>(P, b0, b1, cand_scores, cand_ids, most);
  CR_LAUNCH_CHECK("qsa_candidates_kernel");
  return CR_OK;
}

extern "C" cr_status cr_qsa_shard_select(const cr_geometry* g, const cr_qsa_args* a, int b0, int b1, float* cand_scores, int* cand_ids,
                                         void* stream) {
  using namespace cr;
  CR_REQUIRE(a && b0 >= 0 && b1 >= b0, "cr_qsa_shard_select: bad block range");
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_shard_select", (b1 < (a->pos0 + a->R) / 4 ? b1 : (a->pos0 + a->R) / 4) - b0)) return s;
  CR_REQUIRE(cand_scores && cand_ids && b0 >= 0 && b1 >= b0 && b1 - b0 <= kMaxSelectCount, "cr_qsa_shard_select: bad block range or null output");
  if (cr_status s = qsa_score_launch(g, a, 1, (cudaStream_t)stream, b0, b1)) return s;
  return cr_qsa_shard_candidates(g, a, b0, b1, cand_scores, cand_ids, stream);
}

extern "C" cr_status cr_qsa_merge_candidates(const cr_geometry* g, const cr_qsa_args* a, int ranks, const float* cand_scores,
                                             const int* cand_ids, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_merge_candidates", 0)) return s;
  CR_REQUIRE(cand_scores && cand_ids && ranks >= 1 && ranks <= 16, "cr_qsa_merge_candidates: need 1..16 ranks and candidate buffers");
  if (cr_status st = select_configure()) return st;
  QsaParams P;
  qsa_fill_params(P, g, a, 1);
  use_stream((cudaStream_t)stream);
  const int most = ranks * CR_SEL_BLOCKS;
  qsa_merge_candidates_kernel<<<a->R, kSelThreads, select_smem_bytes(most), (cudaStream_t)stream>>>(P, ranks, cand_scores, cand_ids, most);
  CR_LAUNCH_CHECK("qsa_merge_candidates_kernel");
  return CR_OK;
}
