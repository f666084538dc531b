// QSA row preparation for sm_100a: CN-RMSNorm + partial RoPE of the query / key / indexer-query heads, K/V
// rows to the fp16 cache, raw indexer keys, pooled indexer keys of completed 4-token blocks, RoPE table.
// Follows QsaPrepKernel / QsaPoolKernel / QsaRetainRawKernel / QsaPrefillQueryKernel
// (engine/layers/ops.h:561-645; engine/layers/kernels/prefill_qsa.h:35-51, :220-242).
#include "qsa.cuh"

namespace cr {

__global__ void rope_table_kernel(float* table) {
  const int j = threadIdx.x;
  if (j < 32) table[j] = powf(10000000.f, -2.f * j / 64.f);
  else if (j < CR_ROPE_TABLE_FLOATS) table[j] = j == 32 ? 1.f : 0.f;
}

// Split-half RoPE of x[0..63] (shared memory) at cache position p by threads 0..31; two barriers.  With a table of
// multimodal positions (mrope [capacity][4]: t, h, w of every cache position; engine/layers/ops.h:515-541) frequency j
// turns with the h position when j % 3 == 1, with the w position when j % 3 == 2 and j < 30, else with t (interleaved
// sections [11, 11, 10]); equal axes give the text rotation exactly.
__device__ __forceinline__ void rope64_smem(float* x, const float* rope, const int* mrope, int p) {
  const int j = threadIdx.x;
  float c = 0.f, s = 0.f, a = 0.f, b = 0.f;
  if (j < 32) {
    int pj = p;
    if (mrope) pj = j % 3 == 1 ? mrope[4 * (size_t)p + 1] : (j % 3 == 2 && j < 30 ? mrope[4 * (size_t)p + 2] : mrope[4 * (size_t)p]);
    rope_cs(rope, j, pj, c, s);
    a = x[j];
    b = x[j + 32];
  }
  __syncthreads();
  if (j < 32) {
    x[j] = a * c - b * s;
    x[j + 32] = b * c + a * s;
  }
  __syncthreads();
}

// CN-RMSNorm of n (128 or 256) values in shared memory, one per thread.
__device__ __forceinline__ void cnorm_smem(float* x, int n, const float* w1, float* red) {
  const int j = threadIdx.x;
  const float v = j < n ? x[j] : 0.f;
  const float ss = block_sum<256>(v * v, red);
  if (j < n) x[j] = v * rsqrtf(ss / n + kEps) * w1[j];
  __syncthreads();
}

__device__ __forceinline__ bool raw_uses_chunk(int slots, int rows) { return slots != 0 && rows > 8; }

__device__ __forceinline__ void pool_block(const cr_qsa_args& a, int b, float* x, float* red);

// grid (units + pool_units, Rmax, spans), 256 threads.  Blocks x >= units (row 0 only) pool completed blocks.  Units: [0,Hq) query heads, [Hq,Hq+Hkv) key heads,
// [Hq+Hkv, Hq+2Hkv) value heads, then 4 indexer-query heads, then the raw indexer key.
// u0 skips leading units (u0 = Hq runs the cache units only).  q_hi (optional): fp16 copy of the prepared
// queries [R][Hq][256] for the prefill attention kernels; rows < q_skip are not written to q_hi.
// queries_only: the key, value and raw-key units and the pooling do nothing (a rank of a split-KV group that does not own
// the rows' positions still normalises the queries).
__global__ void __launch_bounds__(256) qsa_prep_kernel(const __grid_constant__ QsaParams P, int u0, __half* q_hi, int q_skip, int units, int queries_only) {
  const cr_qsa_args& a = P.span[blockIdx.z];
  const int r = blockIdx.y;
  if (r >= a.R) return;
  __shared__ float x[256], red[8];
  if (queries_only) {
    const int u = (int)blockIdx.x + u0;
    if ((int)blockIdx.x >= units || (u >= P.Hq && u < P.Hq + 2 * P.Hkv) || u >= P.Hq + 2 * P.Hkv + 4) return;
  }
  if ((int)blockIdx.x >= units) {
    const int b = a.pos0 / 4 + ((int)blockIdx.x - units);
    if (r == 0 && b < (a.pos0 + a.R) / 4) pool_block(a, b, x, red);
    return;
  }
  const int u = blockIdx.x + u0, j = threadIdx.x, p = a.pos0 + r;
  const int Hq = P.Hq, Hkv = P.Hkv;
  if (u < Hq) {
    float* q = a.q + ((size_t)r * Hq + u) * 512;
    x[j] = q[j];
    __syncthreads();
    cnorm_smem(x, 256, a.q_norm1, red);
    rope64_smem(x, a.rope, a.mrope, p);
    q[j] = x[j];
    if (q_hi && r >= q_skip) q_hi[((size_t)r * Hq + u) * 256 + j] = __float2half(x[j]);
  } else if (u < Hq + Hkv) {
    const int g = u - Hq;
    x[j] = a.k[(size_t)r * Hkv * 256 + g * 256 + j];
    __syncthreads();
    cnorm_smem(x, 256, a.k_norm1, red);
    rope64_smem(x, a.rope, a.mrope, p);
    reinterpret_cast<__half*>(a.c.k)[((size_t)p * Hkv + g) * 256 + j] = __float2half(x[j]);
  } else if (u < Hq + 2 * Hkv) {
    const int g = u - Hq - Hkv;
    reinterpret_cast<__half*>(a.c.v)[((size_t)p * Hkv + g) * 256 + j] = __float2half(a.v[(size_t)r * Hkv * 256 + g * 256 + j]);
  } else if (u < Hq + 2 * Hkv + 4) {
    float* iq = a.idx + (size_t)r * 640 + (u - Hq - 2 * Hkv) * 128;
    if (j < 128) x[j] = iq[j];
    __syncthreads();
    cnorm_smem(x, 128, a.iq_norm1, red);
    rope64_smem(x, a.rope, a.mrope, p);
    if (j < 128) iq[j] = x[j];
  } else if (j < 128 && !raw_uses_chunk(a.c.raw_slots, a.R)) {
    a.c.ik_raw[raw_offset(a.c.raw_slots, p, j)] = a.idx[(size_t)r * 640 + 512 + j];
  }
}

// Pooled key of block b (complete within rows pos0..pos0+R-1 or earlier): mean of 4 raw keys -> fp16 round ->
// CN-RMSNorm -> RoPE at the block start.  Raw keys of this call's rows are read from the input rows, older ones
// from the cache, so the result does not depend on the prep units having run.
__device__ __forceinline__ void pool_block(const cr_qsa_args& a, int b, float* x, float* red) {
  const int j = threadIdx.x;
  if (j < 128) {
    float m = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int pos = b * 4 + t;
      m += pos >= a.pos0 ? a.idx[(size_t)(pos - a.pos0) * 640 + 512 + j] : a.c.ik_raw[raw_offset(a.c.raw_slots, pos, j)];
    }
    x[j] = round_h(m * 0.25f);
  }
  __syncthreads();
  cnorm_smem(x, 128, a.ik_norm1, red);
  rope64_smem(x, a.rope, a.mrope, b * 4);
  if (j < 128) a.c.ik_pool[pool_offset(b, j)] = x[j];
}

// Block b = pos0/4 + blockIdx.x of span blockIdx.y, if these rows complete it (bulk rows; steps pool inside prep).
__global__ void __launch_bounds__(256) qsa_pool_kernel(const __grid_constant__ QsaParams P) {
  const cr_qsa_args& a = P.span[blockIdx.y];
  __shared__ float x[256], red[8];
  const int b = a.pos0 / 4 + blockIdx.x;
  if (b >= (a.pos0 + a.R) / 4) return;
  pool_block(a, b, x, red);
}

// Bulk rows with a raw ring: keep the newest min(R, slots) raw keys (after every pool has read the old tail).
__global__ void qsa_retain_raw_kernel(const __grid_constant__ QsaParams P) {
  const cr_qsa_args& a = P.span[blockIdx.y];
  if (!raw_uses_chunk(a.c.raw_slots, a.R)) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int keep = min(a.R, a.c.raw_slots);
  if (i >= keep * 128) return;
  const int row = a.R - keep + i / 128, dim = i % 128;
  a.c.ik_raw[raw_offset(a.c.raw_slots, a.pos0 + row, dim)] = a.idx[(size_t)row * 640 + 512 + dim];
}

cr_status qsa_validate(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, int max_rows, const char* who, int score_blocks) {
  if (cr_status s = check_geometry(g)) return s;
  CR_REQUIRE(spans && n_spans >= 1, "%s: no spans", who);
  for (int s = 0; s < n_spans; ++s) {
    const cr_qsa_args& a = spans[s];
    CR_REQUIRE(a.R >= 1 && a.R <= max_rows, "%s: span %d has R=%d, need 1..%d", who, s, a.R, max_rows);
    CR_REQUIRE(a.pos0 >= 0, "%s: span %d has negative pos0", who, s);
    const int need_stride = score_blocks >= 0 ? score_blocks : (a.pos0 + a.R) / 4;   // entries that score a block range need that range only
    CR_REQUIRE(a.sstride >= need_stride, "%s: span %d score stride %d < %d blocks", who, s, a.sstride, need_stride);
    CR_REQUIRE(a.q && a.k && a.v && a.idx && a.q_norm1 && a.k_norm1 && a.iq_norm1 && a.ik_norm1 && a.c.k && a.c.v &&
               a.c.ik_raw && a.c.ik_pool && a.sel && a.nsel && a.rope, "%s: span %d has a null buffer", who, s);
    CR_REQUIRE(a.scores || (a.pos0 + a.R) / 4 <= CR_SEL_BLOCKS, "%s: span %d needs a score buffer", who, s);
    CR_REQUIRE(a.c.raw_slots == 0 || a.c.raw_slots >= 16, "%s: span %d raw ring of %d slots is too small", who, s, a.c.raw_slots);
  }
  return CR_OK;
}

int qsa_max_rows(const cr_qsa_args* spans, int n) {
  int m = 0;
  for (int s = 0; s < n; ++s) m = spans[s].R > m ? spans[s].R : m;
  return m;
}

void qsa_fill_params(QsaParams& P, const cr_geometry* g, const cr_qsa_args* spans, int n) {
  for (int s = 0; s < n; ++s) P.span[s] = spans[s];
  int base = 0;
  for (int s = 0; s < n; ++s) { P.base[s] = base; base += spans[s].R; }
  P.Hq = g->q_heads; P.Hkv = g->kv_heads; P.n = n;
  P.b_lo = 0; P.b_hi = INT_MAX;
  P.tile_count = nullptr; P.tile_rows = 1; P.tile_max = 0;
}

cr_status qsa_prep_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, int u0, __half* q_hi, int q_skip,
                          cudaStream_t stream, bool queries_only) {
  use_stream(stream);
  for (int s0 = 0; s0 < n_spans; s0 += kMaxSpans) {
    const int n = n_spans - s0 < kMaxSpans ? n_spans - s0 : kMaxSpans;
    QsaParams P;
    qsa_fill_params(P, g, spans + s0, n);
    const int Rmax = qsa_max_rows(spans + s0, n);
    const int units = g->q_heads + 2 * g->kv_heads + 5 - u0;
    int completed = 0, keep = 0;
    bool ring = false;
    for (int s = 0; s < n; ++s) {
      const cr_qsa_args& a = spans[s0 + s];
      const int c = (a.pos0 + a.R) / 4 - a.pos0 / 4;
      completed = c > completed ? c : completed;
      ring = ring || (a.c.raw_slots != 0 && a.R > 8);
      keep = a.c.raw_slots > keep ? a.c.raw_slots : keep;
    }
    const bool fused_pool = Rmax <= 16;            // steps: pooling rides in the prep launch
    qsa_prep_kernel<<<dim3(units + (fused_pool && !queries_only ? completed : 0), Rmax, n), 256, 0, stream>>>(P, u0, q_hi, q_skip, units, queries_only ? 1 : 0);
    CR_LAUNCH_CHECK("qsa_prep_kernel");
    if (queries_only) continue;
    if (completed && !fused_pool) {
      qsa_pool_kernel<<<dim3(completed, n), 256, 0, stream>>>(P);
      CR_LAUNCH_CHECK("qsa_pool_kernel");
    }
    if (ring) {
      qsa_retain_raw_kernel<<<dim3((keep * 128 + 255) / 256, n), 256, 0, stream>>>(P);
      CR_LAUNCH_CHECK("qsa_retain_raw_kernel");
    }
  }
  return CR_OK;
}

}  // namespace cr

extern "C" cr_status cr_rope_table_fill(float* table, void* stream) {
  using namespace cr;
  CR_REQUIRE(table, "cr_rope_table_fill: null table");
  use_stream((cudaStream_t)stream);
  rope_table_kernel<<<1, CR_ROPE_TABLE_FLOATS, 0, (cudaStream_t)stream>>>(table);
  CR_LAUNCH_CHECK("rope_table_kernel");
  return CR_OK;
}

// YaRN table for a context of factor x 262,144 positions (the rows of engine/layers/rope_tables.h; Hugging Face
// "yarn" rope scaling with original context 262,144, beta_fast 32, beta_slow 1, rotary dim 64, theta 1e7): frequencies
// that turn more than 32 times over the original context are kept, those that turn less than once are divided by the
// factor, a linear ramp in between; the cos/sin multiplier is 0.1 ln(factor) + 1.
extern "C" cr_status cr_rope_table_fill_yarn(float* table, int factor, void* stream) {
  using namespace cr;
  CR_REQUIRE(table, "cr_rope_table_fill_yarn: null table");
  CR_REQUIRE(factor >= 1 && factor <= 64, "cr_rope_table_fill_yarn: factor %d outside 1..64", factor);
  if (factor == 1) return cr_rope_table_fill(table, stream);
  constexpr double kDim = 64.0, kBase = 1e7, kOrig = 262144.0, kPi = 3.14159265358979323846;
  auto turns_dim = [&](double turns) { return kDim * log(kOrig / (turns * 2.0 * kPi)) / (2.0 * log(kBase)); };
  double low = floor(turns_dim(32.0)), high = ceil(turns_dim(1.0));
  low = low < 0 ? 0 : low;
  high = high > kDim - 1 ? kDim - 1 : high;
  if (low == high) high += 0.001;
  float host[CR_ROPE_TABLE_FLOATS] = {};
  for (int j = 0; j < 32; ++j) {
    const float extrap = 1.0f / powf(10000000.f, (float)(2 * j) / 64.f), interp = extrap / (float)factor;
    float ramp = ((float)j - (float)low) / ((float)high - (float)low);
    ramp = ramp < 0.f ? 0.f : (ramp > 1.f ? 1.f : ramp);
    const float keep = 1.f - ramp;                        // share of the original frequency
    host[j] = interp * (1.f - keep) + extrap * keep;
  }
  host[32] = (float)(0.1 * log((double)factor) + 1.0);
  CR_CUDA(cudaMemcpyAsync(table, host, sizeof(host), cudaMemcpyHostToDevice, (cudaStream_t)stream));   // pageable source: staged before the call returns
  return CR_OK;
}

// The query units of cr_qsa_prep alone: q heads and indexer-query heads normalised + roped in place; no cache row, raw
// key or pooled key is written.  For the ranks of a split-KV group that do not own the rows' positions.  No counterpart
// in the single-device reference.
extern "C" cr_status cr_qsa_prep_queries(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, spans, n_spans, CR_MAX_PREFILL_ROWS, "cr_qsa_prep_queries", 0)) return s;
  return qsa_prep_launch(g, spans, n_spans, 0, nullptr, 0, (cudaStream_t)stream, true);
}

extern "C" cr_status cr_qsa_prep(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, spans, n_spans, CR_MAX_STEP_ROWS, "cr_qsa_prep")) return s;
  return qsa_prep_launch(g, spans, n_spans, 0, nullptr, 0, (cudaStream_t)stream);
}

extern "C" cr_status cr_qsa_prefill_cache(const cr_geometry* g, const cr_qsa_args* a, void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, a, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_prefill_cache")) return s;
  return qsa_prep_launch(g, a, 1, g->q_heads, nullptr, 0, (cudaStream_t)stream);
}

extern "C" size_t cr_qsa_pool_floats(int ctx) { return (size_t)((ctx + 127) / 128) * 4096; }

extern "C" cr_status cr_qsa_cache_bytes(const cr_geometry* g, int ctx, int bounded, size_t out_bytes[4]) {
  using namespace cr;
  if (cr_status s = check_geometry(g)) return s;
  CR_REQUIRE(out_bytes, "cr_qsa_cache_bytes: null output");
  CR_REQUIRE(ctx >= 1 && ctx <= 1048576, "cr_qsa_cache_bytes: context %d is out of range", ctx);
  out_bytes[0] = out_bytes[1] = (size_t)ctx * g->kv_heads * 256 * 2;
  out_bytes[2] = (size_t)(bounded ? 16 : ctx) * 128 * sizeof(float);
  out_bytes[3] = cr_qsa_pool_floats(ctx) * sizeof(float);
  return CR_OK;
}
