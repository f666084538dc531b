// Exact top-512 of a row of indexer scores for sm_100a (the job of LaunchQsaTop, engine/layers/qsa_long.h:111-380):
// the 512 best blocks in the total order (score descending, block id ascending), emitted in ascending block id.
//
// Method: sample, filter, sort, mark, compact.  One CTA of 1024 threads per row.
//   1. Scores are >= +0, so their fp32 bit patterns order like unsigned integers.  A strided sample of S values
//      (2048..8192, at least one in 32) is sorted in shared memory; the value at a rank a few standard deviations
//      below where the 512th best is expected becomes a cut.
//   2. One pass over the row gathers every value strictly above the cut (typically 700 to 1500 of them) into a
//      shared-memory list, packed as 64-bit keys (bit pattern, inverted index) whose descending order is the total
//      order.  If at least 512 and at most 4096 values passed, the best 512 of the row are among them: exact, whatever
//      the sample was.
//   3. The list is sorted (bitonic network), its first 512 entries set their bit in a bitmap over the row, and the
//      bitmap is compacted in index order: a prefix sum over word popcounts gives every thread its output offset.
//   Rows of at most 4096 values skip 1 and 2: everything is sorted.
//   When the cut fails (fewer than 512 above it: ties at the cut or an unlucky sample; or more than 4096), the row
//   takes the slow exact path: a binary search over the 31 value bits for the 512th best bit pattern, counting with
//   plain reductions (no atomics, so a row of identical scores costs the same as any other), then the values above
//   it plus the first ties in index order.
// The same routine serves a whole row, a rank's block range (candidates with their scores, for split-KV across
// devices, engine/layers/qsa_long.h:228-234) and the merge of gathered candidates.
#include <climits>
#include "qsa.cuh"

namespace cr {

constexpr int kSelThreads = 1024;
constexpr int kMaxSelectCount = 262144;   // elements of one selection: the tie bitmap of the slow path shares the 32 KB sort buffer
constexpr int kSortCap = 4096;            // 64-bit keys in the sort buffer (32 KB); also 8192 32-bit sample values

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
// Descending bitonic sort of n (a power of two, n >= 2) keys in shared memory by the whole block.
template <typename K>
__device__ __forceinline__ void bitonic_sort_desc(K* a, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      __syncthreads();
      for (int p = threadIdx.x; p < (n >> 1); p += kSelThreads) {
        const int i = ((p & ~(j - 1)) << 1) | (p & (j - 1));     // pair (i, i + j)
        const K x = a[i], y = a[i + j];
        const bool down = (i & k) == 0;                           // this run sorts descending
        if ((x < y) == down) { a[i] = y; a[i + j] = x; }
      }
    }
  }
  __syncthreads();
}
__device__ __forceinline__ int pow2_at_least(int n) {
  int p = 2;
  while (p < n) p <<= 1;
  return p;
}
__device__ __forceinline__ unsigned long long pack_key(unsigned bits, int i) {
  return ((unsigned long long)bits << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
}
__device__ __forceinline__ int key_index(unsigned long long k) { return (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull)); }

// Shared memory of one CTA: sort buffer (32 KB), bitmap over the row's elements (count bits), small arrays.
struct SelectSmem {
  unsigned long long* keys;    // kSortCap 64-bit keys; also the sample (32-bit values) and the slow path's tie bitmap
  unsigned* bitmap;            // ceil(count / 32) words
  unsigned* red;               // 33 words
  unsigned* counter;           // 1 word
};

// Marks the `want` best elements of [0, count) in sm.bitmap (bit i = element i selected).  want <= count.
template <typename Src>
__device__ __forceinline__ void select_mark(const Src& src, int count, int want, const SelectSmem& sm) {
  const int t = threadIdx.x, l = t & 31;
  const int words = (count + 31) >> 5;
  for (int i = t; i < words; i += kSelThreads) sm.bitmap[i] = 0u;
  auto mark_sorted_prefix = [&](int n_sorted) {                   // the first `want` keys of the sorted buffer
    (void)n_sorted;
    __syncthreads();
    for (int i = t; i < want; i += kSelThreads) {
      const int e = key_index(sm.keys[i]);
      atomicOr(&sm.bitmap[e >> 5], 1u << (e & 31));
    }
    __syncthreads();
  };
  if (count <= kSortCap) {
    // ---- everything fits: sort it all
    const int n = pow2_at_least(count);
    for (int i = t; i < n; i += kSelThreads) {
      unsigned bits = 0u;
      const bool ok = i < count && src.get(i, bits);
      sm.keys[i] = ok ? pack_key(bits, i) : 0ull;                  // padding sorts last (a real key is never 0)
    }
    bitonic_sort_desc(sm.keys, n);
    mark_sorted_prefix(n);
    return;
  }
  // ---- 1. sample and cut
  int S = pow2_at_least((count + 31) / 32);
  S = S < 2048 ? 2048 : (S > 2 * kSortCap ? 2 * kSortCap : S);
  unsigned* sample = reinterpret_cast<unsigned*>(sm.keys);
  for (int s = t; s < S; s += kSelThreads) {
    const int i = (int)(((long long)s * count) / S);
    unsigned bits = 0u;
    if (!src.get(i, bits)) bits = 0u;
    sample[s] = bits;
  }
  bitonic_sort_desc(sample, S);
  const float expect = (float)want * (float)S / (float)count;     // sample rank where the want-th best is expected
  int rho = (int)ceilf(expect + 5.5f * sqrtf(expect) + 2.f);
  rho = rho > S ? S : rho;
  const unsigned cut = sample[rho - 1];
  __syncthreads();                                                 // the sample is dead: the buffer becomes the list
  if (t == 0) *sm.counter = 0u;
  __syncthreads();
  // ---- 2. gather everything strictly above the cut
  for (int i0 = 0; i0 < count; i0 += kSelThreads) {
    const int i = i0 + t;
    unsigned bits = 0u;
    const bool pass = i < count && src.get(i, bits) && bits > cut;
    const unsigned m = __ballot_sync(0xffffffffu, pass);
    if (m) {
      unsigned base = 0u;
      if (l == 0) base = atomicAdd(sm.counter, (unsigned)__popc(m));
      base = __shfl_sync(0xffffffffu, base, 0);
      const unsigned at = base + __popc(m & ((1u << l) - 1u));
      if (pass && at < (unsigned)kSortCap) sm.keys[at] = pack_key(bits, i);
    }
  }
  __syncthreads();
  const int got = (int)*sm.counter;
  if (got >= want && got <= kSortCap) {
    // ---- 3. the best `want` are all in the list
    const int n = pow2_at_least(got);
    for (int i = got + t; i < n; i += kSelThreads) sm.keys[i] = 0ull;
    bitonic_sort_desc(sm.keys, n);
    mark_sorted_prefix(n);
    return;
  }
  // ---- slow exact path: T = the largest bit pattern with at least `want` elements >= T
  unsigned T = 0u;
  for (int bit = 30; bit >= 0; --bit) {
    const unsigned trial = T | (1u << bit);
    unsigned c = 0u;
    for (int i = t; i < count; i += kSelThreads) {
      unsigned bits;
      if (src.get(i, bits) && bits >= trial) ++c;
    }
    if (block_sum_u32(c, sm.red) >= (unsigned)want) T = trial;
  }
  unsigned* ties = reinterpret_cast<unsigned*>(sm.keys);           // bitmap of the elements equal to T (<= 32 KB)
  unsigned above = 0u;
  for (int i0 = 0; i0 < words * 32; i0 += kSelThreads) {           // a warp covers one bitmap word per iteration
    const int i = i0 + t;
    unsigned bits = 0u;
    const bool ok = i < count && src.get(i, bits);
    const unsigned gt = __ballot_sync(0xffffffffu, ok && bits > T), eq = __ballot_sync(0xffffffffu, ok && bits == T);
    if (l == 0 && (i >> 5) < words) { sm.bitmap[i >> 5] = gt; ties[i >> 5] = eq; above += __popc(gt); }
  }
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
  sm.keys = reinterpret_cast<unsigned long long*>(raw);
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
    CR_CUDA(launch_pdl(qsa_topk_kernel, dim3(Rmax, n), dim3(kSelThreads), select_smem_bytes(nb_max), stream, P, nb_max));
    CR_LAUNCH_CHECK("qsa_topk_kernel");
  }
  return CR_OK;
}

}  // namespace cr

extern "C" cr_status cr_qsa_shard_candidates(const cr_geometry* g, const cr_qsa_args* a, int b0, int b1, float* cand_scores,
                                             int* cand_ids, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_shard_candidates")) return s;
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
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_shard_select")) return s;
  CR_REQUIRE(cand_scores && cand_ids && b0 >= 0 && b1 >= b0 && b1 - b0 <= kMaxSelectCount, "cr_qsa_shard_select: bad block range or null output");
  if (cr_status s = qsa_score_launch(g, a, 1, (cudaStream_t)stream, b0, b1)) return s;
  return cr_qsa_shard_candidates(g, a, b0, b1, cand_scores, cand_ids, stream);
}

extern "C" cr_status cr_qsa_merge_candidates(const cr_geometry* g, const cr_qsa_args* a, int ranks, const float* cand_scores,
                                             const int* cand_ids, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_merge_candidates")) return s;
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
