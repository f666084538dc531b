// Gated DeltaNet prefill for sm_100a: row preparation, the exact fp32 token-serial scan, the gated readout
// and the raw-row ring.  The chunk-64 tensor-core scan lives in gdn_chunk.cu and shares prep/gate/ring.
//
// Pipeline of one call (rows pos0..pos0+R-1 of one layer, engine/layers/kernels/prefill_gdn.h:1206-1279):
//   gdn_prep   conv(4)+SiLU on the raw projection, L2 norms of q/k per key head, g = -exp(A_log)softplus(a+dt),
//              beta = sigmoid(b)                                   -> workspace (qn, kn, vn, glog, beta)
//   scan       delta rule over the rows from the carried state     -> raw readout y, new state
//   gdn_gate   y * rsqrt(mean y^2 + eps) * gamma * sigmoid(z), output transform
//   gdn_ring   last 16 raw rows -> hist ring (GdnPrefillHistoryKernel, prefill_gdn.h:274-282)
#include "common.cuh"
#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>
#include "gdn_prefill.cuh"

namespace cr {

// ---- gdn_prep ----------------------------------------------------------------------------------------
// grid (ceil(R/16), Hk + Hv/2 + 1), 256 threads.  Unit u < Hk: key head u (threads 0..127 the q channels,
// 128..255 the k channels).  Hk <= u < Hk + Hv/2: value heads 2(u-Hk), 2(u-Hk)+1.  Last unit: g and beta.
// Each thread slides a 4-row window down its channel over the 16 rows of the tile.
template <bool BF16>
__global__ void __launch_bounds__(256) gdn_prep_kernel(GdnPrefillParams P) {
  const cr_gdn_args& a = P.a;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int r0 = blockIdx.x * 16, u = blockIdx.y;
  const int KW = P.Hk * 128, VW = P.Hv * 128, C = 2 * KW + VW;
  const int rows = min(16, a.R - r0);
  if (u == P.Hk + P.Hv / 2) {
    // g / beta for rows r0.. and all value heads
    for (int i = t; i < rows * P.Hv; i += 256) {
      const int r = r0 + i / P.Hv, h = i % P.Hv;
      const float av = load_in<BF16>(P.ab_logits, (size_t)r * 2 * P.Hv + h);
      const float bv = load_in<BF16>(P.ab_logits, (size_t)r * 2 * P.Hv + P.Hv + h);
      const float sp = av + a.dt_bias[h];
      const float softplus = sp > 20.f ? sp : log1pf(expf(sp));
      P.glog[(size_t)r * P.Hv + h] = -expf(a.A_log[h]) * softplus;
      P.beta[(size_t)r * P.Hv + h] = sigmoidf_(bv);
    }
    return;
  }
  const bool is_qk = u < P.Hk;
  const int ch = is_qk ? (t < 128 ? u * 128 + t : KW + u * 128 + (t - 128)) : 2 * KW + (u - P.Hk) * 256 + t;
  const float4 wv = *reinterpret_cast<const float4*>(a.conv + (size_t)ch * 4);
  auto raw = [&](int r) -> float {   // raw projection value of this channel at call row r (may be negative)
    if (r >= 0 || P.halo_in) return load_in<BF16>(a.qkv, (long long)r * C + ch);
    const int p = a.pos0 + r;
    return p < 0 ? 0.f : a.hist[(size_t)(p & 15) * C + ch];
  };
  float x0 = raw(r0 - 3), x1 = raw(r0 - 2), x2 = raw(r0 - 1);
  float val[16];
  __shared__ float red[16][8];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float c = 0.f;
    if (i < rows) {
      const float x3 = raw(r0 + i);
      c = wv.x * x0;
      c = fmaf(wv.y, x1, c); c = fmaf(wv.z, x2, c); c = fmaf(wv.w, x3, c);
      c = siluf_(c);
      x0 = x1; x1 = x2; x2 = x3;
    }
    val[i] = c;
    if (is_qk) {
      const float s = warp_sum(c * c);
      if (l == 0) red[i][w] = s;
    }
  }
  if (is_qk) {
    __syncthreads();
    const int part = t >> 7, j = t & 127;
    float* dst = part ? P.kn : P.qn;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i >= rows) break;
      const float ss = red[i][part * 4] + red[i][part * 4 + 1] + red[i][part * 4 + 2] + red[i][part * 4 + 3];
      const float sc = rsqrtf(ss + kEps) * (part ? 1.f : kInvSqrt128);
      float o = val[i] * sc;
      if (P.tf32) o = tf32r(o);
      dst[((size_t)(r0 + i) * P.Hk + u) * 128 + j] = o;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i >= rows) break;
      P.vn[(size_t)(r0 + i) * VW + (u - P.Hk) * 256 + t] = val[i];
    }
  }
}

// ---- exact fp32 serial scan --------------------------------------------------------------------------
// grid Hv*4 CTAs x 256 threads.  CTA (h, slice) owns 32 value columns; warp w owns 4 of them; the 8 lanes
// that share a column hold 16 key rows each in registers, so one token costs two 3-step shuffle reductions
// and no block barrier.  Inputs of the next token are fetched while the current one is computed.
__global__ void __launch_bounds__(256) gdn_scan_serial_kernel(GdnPrefillParams P) {
  const cr_gdn_args& a = P.a;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int h = blockIdx.x >> 2, slice = blockIdx.x & 3;
  const int rep = P.Hv / P.Hk, kh = h / rep, VW = P.Hv * 128;
  const int col = slice * 32 + w * 4 + (l >> 3), sub = l & 7;
  float S[16];
  float* st = a.state + (size_t)h * 16384 + col;
#pragma unroll
  for (int i = 0; i < 16; ++i) S[i] = st[(size_t)(sub * 16 + i) * 128];

  auto fetch = [&](int r, float4 (&k4)[4], float4 (&q4)[4], float& v, float& g, float& b) {
    const float4* kp = reinterpret_cast<const float4*>(P.kn + ((size_t)r * P.Hk + kh) * 128 + sub * 16);
    const float4* qp = reinterpret_cast<const float4*>(P.qn + ((size_t)r * P.Hk + kh) * 128 + sub * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) { k4[i] = kp[i]; q4[i] = qp[i]; }
    v = P.vn[(size_t)r * VW + h * 128 + col];
    g = P.glog[(size_t)r * P.Hv + h];
    b = P.beta[(size_t)r * P.Hv + h];
  };
  float4 kc[4], qc[4], kn_[4], qn_[4];
  float vc, gc, bc, vn_ = 0.f, gn_ = 0.f, bn_ = 0.f;
  fetch(0, kc, qc, vc, gc, bc);
  for (int r = 0; r < a.R; ++r) {
    if (r + 1 < a.R) fetch(r + 1, kn_, qn_, vn_, gn_, bn_);
    const float decay = expf(gc);
    const float* k = reinterpret_cast<const float*>(kc);
    const float* q = reinterpret_cast<const float*>(qc);
    float m0 = 0.f, m1 = 0.f, m2 = 0.f, m3 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      m0 = fmaf(S[i], k[i], m0); m1 = fmaf(S[i + 1], k[i + 1], m1);
      m2 = fmaf(S[i + 2], k[i + 2], m2); m3 = fmaf(S[i + 3], k[i + 3], m3);
    }
    float mem = (m0 + m1) + (m2 + m3);
    mem += __shfl_xor_sync(0xffffffffu, mem, 1);
    mem += __shfl_xor_sync(0xffffffffu, mem, 2);
    mem += __shfl_xor_sync(0xffffffffu, mem, 4);
    const float delta = bc * (vc - decay * mem);
    float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      S[i] = fmaf(k[i], delta, decay * S[i]);             y0 = fmaf(S[i], q[i], y0);
      S[i + 1] = fmaf(k[i + 1], delta, decay * S[i + 1]); y1 = fmaf(S[i + 1], q[i + 1], y1);
      S[i + 2] = fmaf(k[i + 2], delta, decay * S[i + 2]); y2 = fmaf(S[i + 2], q[i + 2], y2);
      S[i + 3] = fmaf(k[i + 3], delta, decay * S[i + 3]); y3 = fmaf(S[i + 3], q[i + 3], y3);
    }
    float y = (y0 + y1) + (y2 + y3);
    y += __shfl_xor_sync(0xffffffffu, y, 1);
    y += __shfl_xor_sync(0xffffffffu, y, 2);
    y += __shfl_xor_sync(0xffffffffu, y, 4);
    if (sub == 0) P.yraw[(size_t)r * VW + h * 128 + col] = y;
#pragma unroll
    for (int i = 0; i < 4; ++i) { kc[i] = kn_[i]; qc[i] = qn_[i]; }
    vc = vn_; gc = gn_; bc = bn_;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) st[(size_t)(sub * 16 + i) * 128] = S[i];
}

// ---- gated readout -----------------------------------------------------------------------------------
// One warp per four consecutive (row, head) units; lane l holds columns 4l..4l+3 of each (the WHT layout).  All
// loads of the four units are issued before anything is consumed: the kernel is a stream, and bytes in flight per
// thread are what its bandwidth depends on.
constexpr int kGateUnits = 4;
template <bool BF16>
__global__ void __launch_bounds__(256) gdn_gate_kernel(GdnPrefillParams P) {
  const cr_gdn_args& a = P.a;
  const int VW = P.Hv * 128, l = threadIdx.x & 31;
  const long long total = (long long)a.R * P.Hv;
  const long long unit0 = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * kGateUnits;
  if (unit0 >= total) return;
  float4 y4[kGateUnits], z4[kGateUnits];
#pragma unroll
  for (int u = 0; u < kGateUnits; ++u) {
    y4[u] = z4[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (unit0 + u < total) {
      const size_t base = (size_t)(unit0 + u) * 128 + l * 4;   // (row, head) units are contiguous: r * VW + h * 128
      y4[u] = *reinterpret_cast<const float4*>(P.yraw + base);
      if constexpr (BF16) {
        const uint2 zz = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.z) + base);
        const float2 z0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&zz.x));
        const float2 z1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&zz.y));
        z4[u] = make_float4(z0.x, z0.y, z1.x, z1.y);
      } else {
        z4[u] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.z) + base);
      }
    }
  }
  const float4 gm = *reinterpret_cast<const float4*>(a.gamma + l * 4);
#pragma unroll
  for (int u = 0; u < kGateUnits; ++u) {
    if (unit0 + u >= total) break;                          // warp uniform
    const int r = (int)((unit0 + u) / P.Hv), h = (int)((unit0 + u) % P.Hv);
    const size_t base = (size_t)r * VW + h * 128 + l * 4;
    const float y[4] = {y4[u].x, y4[u].y, y4[u].z, y4[u].w};
    const float z[4] = {z4[u].x, z4[u].y, z4[u].z, z4[u].w};
    const float g4[4] = {gm.x, gm.y, gm.z, gm.w};
    const float ss = warp_sum(y[0] * y[0] + y[1] * y[1] + y[2] * y[2] + y[3] * y[3]);
    const float rs = rsqrtf(ss * (1.f / 128.f) + kEps);
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = y[i] * rs * g4[i] * sigmoidf_(z[i]);
    if (P.fmt == CR_OUT_RAW_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + base) = make_float4(o[0], o[1], o[2], o[3]);
    } else if (P.fmt == CR_OUT_RAW_BF16) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<const unsigned*>(&lo); pk.y = *reinterpret_cast<const unsigned*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + base) = pk;
    } else {
      const __half* suh = reinterpret_cast<const __half*>(a.suh_out) + h * 128 + l * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = round_h(round_h(o[i]) * __half2float(suh[i]));
      wht128(o);
      __half* dst = reinterpret_cast<__half*>(a.out);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        dst[out_index(r, h * 128 + l * 4 + i, VW, a.pack_rows, a.pack_off)] = __float2half(o[i] * kHadNorm);
    }
  }
}

// ---- raw-row ring --------------------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(256) gdn_ring_kernel(GdnPrefillParams P) {
  const cr_gdn_args& a = P.a;
  const int C = 2 * P.Hk * 128 + P.Hv * 128;
  const int keep = min(a.R, 16);
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= (long long)keep * C) return;
  const int r = a.R - keep + (int)(i / C), ch = (int)(i % C);
  a.hist[(size_t)((a.pos0 + r) & 15) * C + ch] = load_in<BF16>(a.qkv, (size_t)r * C + ch);
}

// ---- materialize -----------------------------------------------------------------------------------------
struct GdnStates { float* layer[64]; int Hv; };
__global__ void __launch_bounds__(1024) gdn_materialize_kernel(GdnStates s) {
  float* const state = s.layer[blockIdx.y];
  float* const slot = state + (size_t)s.Hv * 16384 + blockIdx.x;
  const float c = *slot;
  if (c == 0.f || c == 1.f) return;
  float* const x = state + (size_t)blockIdx.x * 16384;
  for (int i = threadIdx.x; i < 16384; i += blockDim.x) x[i] *= c;
  __syncthreads();
  if (threadIdx.x == 0) *slot = 1.f;
}

size_t gdn_workspace_layout(const cr_geometry* g, int rows, GdnPrefillParams* P, char* base) {
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
  const size_t R = (size_t)rows, Hk = g->gdn_kheads, Hv = g->gdn_vheads;
  const size_t o_qn = take(R * Hk * 128 * 4), o_kn = take(R * Hk * 128 * 4), o_vn = take(R * Hv * 128 * 4);
  const size_t o_g = take(R * Hv * 4), o_b = take(R * Hv * 4), o_y = take(R * Hv * 128 * 4);
  const size_t o_chunk = take(gdn_chunk_workspace_bytes(g, rows));
  if (P) {
    P->qn = (float*)(base + o_qn); P->kn = (float*)(base + o_kn); P->vn = (float*)(base + o_vn);
    P->glog = (float*)(base + o_g); P->beta = (float*)(base + o_b); P->yraw = (float*)(base + o_y);
    P->chunk_ws = base + o_chunk;
  }
  return off;
}

int gdn_part_rows() { return options().gdn_part_chunks * 64; }

// Row ranges of the parts of a pipelined call.  The first local kernel and the last scan run with nothing beside
// them, so the first part is short and the parts at the end halve (each scan then ends soon after the local
// kernel that follows it): [32 chunks] [equal parts of at most P chunks] [P/2] [P/4] ... [>= 16 chunks].
static std::vector<std::pair<int, int>> part_schedule(int R, int part_rows) {
  std::vector<int> rows;
  const int chunks = (R + 63) / 64, P = part_rows / 64;
  std::vector<int> tail;
  int left = chunks;
  const int first = chunks > 2 * P ? std::min(32, P) : 0;   // never longer than the part a workspace is sized for
  left -= first;
  for (int t = P / 2; t >= 16 && left - t >= P; t /= 2) { tail.push_back(t); left -= t; }
  const int mid = (left + P - 1) / P;
  if (first) rows.push_back(first);
  for (int i = 0; i < mid; ++i) rows.push_back(left / mid + (i < left % mid ? 1 : 0));
  for (int t : tail) rows.push_back(t);
  std::vector<std::pair<int, int>> out;
  int p0 = 0;
  for (int c : rows) {
    const int n = std::min(c * 64, R - p0);
    if (n > 0) out.push_back({p0, n});
    p0 += n;
  }
  return out;
}

// Internal streams and events of the part pipeline, one set per device, created on first use.  Calls on one
// device are serialised while they enqueue (the events are shared).
struct PipeStreams {
  cudaStream_t hi = nullptr, lo = nullptr, mid = nullptr;
  cudaEvent_t scan_done[2] = {nullptr, nullptr};
  cudaEvent_t fork = nullptr, local_done[2] = {nullptr, nullptr}, part_done[2] = {nullptr, nullptr};
  std::mutex mu;
};
static PipeStreams* pipe_streams() {
  static std::mutex mu;
  static PipeStreams* per_dev[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!per_dev[dev]) {
    PipeStreams* ps = new PipeStreams();
    int lo_pri = 0, hi_pri = 0;
    bool ok = cudaDeviceGetStreamPriorityRange(&lo_pri, &hi_pri) == cudaSuccess;
    ok = ok && cudaStreamCreateWithPriority(&ps->hi, cudaStreamNonBlocking, hi_pri) == cudaSuccess;
    ok = ok && cudaStreamCreateWithPriority(&ps->lo, cudaStreamNonBlocking, lo_pri) == cudaSuccess;
    ok = ok && cudaStreamCreateWithPriority(&ps->mid, cudaStreamNonBlocking, lo_pri) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&ps->fork, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < 2 && ok; ++i) {
      ok = ok && cudaEventCreateWithFlags(&ps->local_done[i], cudaEventDisableTiming) == cudaSuccess;
      ok = ok && cudaEventCreateWithFlags(&ps->part_done[i], cudaEventDisableTiming) == cudaSuccess;
      ok = ok && cudaEventCreateWithFlags(&ps->scan_done[i], cudaEventDisableTiming) == cudaSuccess;
    }
    if (!ok) { delete ps; return nullptr; }
    per_dev[dev] = ps;
  }
  return per_dev[dev];
}

}  // namespace cr

extern "C" size_t cr_gdn_prefill_workspace_bytes(const cr_geometry* g, int rows) {
  if (!g || rows < 1) return 0;
  const size_t part = cr::gdn_workspace_layout(g, rows < cr::gdn_part_rows() ? rows : cr::gdn_part_rows(), nullptr, nullptr);
  return rows > cr::gdn_part_rows() ? 2 * part : part;   // a call of several parts works on two workspaces in turn
}

extern "C" int cr_gdn_prefill_parts(int rows, int* first_row, int* n_rows, int max_parts) {
  if (rows < 1) return 0;
  std::vector<std::pair<int, int>> parts;
  if (rows > cr::gdn_part_rows()) parts = cr::part_schedule(rows, cr::gdn_part_rows());
  else parts.push_back({0, rows});
  for (int i = 0; i < (int)parts.size() && i < max_parts; ++i) {
    if (first_row) first_row[i] = parts[i].first;
    if (n_rows) n_rows[i] = parts[i].second;
  }
  return (int)parts.size();
}

extern "C" int cr_gdn_algo_available(cr_gdn_algo algo) {
  return algo == CR_GDN_SERIAL_F32 || (algo == CR_GDN_CHUNK_TC && cr::gdn_chunk_available());
}

extern "C" cr_status cr_gdn_prefill(const cr_geometry* g, const cr_gdn_prefill_args* args, cr_gdn_algo algo,
                                    cr_out_format fmt, void* stream_) {
  using namespace cr;
  if (cr_status s = check_geometry(g)) return s;
  CR_REQUIRE(args, "cr_gdn_prefill: null args");
  const cr_gdn_args& a = args->input;
  cudaStream_t stream = (cudaStream_t)stream_;
  use_stream(stream);
  CR_REQUIRE(a.R >= 1 && a.pos0 >= 0, "cr_gdn_prefill: need R >= 1 and pos0 >= 0 (R=%d pos0=%d)", a.R, a.pos0);
  CR_REQUIRE(a.replay == 0 && a.commit == a.R, "cr_gdn_prefill: prefill rows are all committed (replay=0, commit=R)");
  CR_REQUIRE(a.qkv && a.z && a.conv && a.A_log && a.dt_bias && a.gamma && a.hist && a.state && a.out && args->ab_logits,
             "cr_gdn_prefill: null buffer");
  CR_REQUIRE(args->in_dtype == CR_IN_F32 || args->in_dtype == CR_IN_BF16, "cr_gdn_prefill: bad in_dtype");
  CR_REQUIRE(fmt == CR_OUT_RAW_F32 || fmt == CR_OUT_RAW_BF16 || fmt == CR_OUT_EXL3_WHT, "cr_gdn_prefill: bad output format");
  CR_REQUIRE(fmt != CR_OUT_EXL3_WHT || a.suh_out, "cr_gdn_prefill: suh_out needed for the EXL3 output");
  CR_REQUIRE(fmt == CR_OUT_EXL3_WHT || a.pack_rows == 0, "cr_gdn_prefill: packed layout only with the EXL3 output");
  CR_REQUIRE(algo == CR_GDN_SERIAL_F32 || algo == CR_GDN_CHUNK_TC, "cr_gdn_prefill: unknown algorithm");
  if (algo == CR_GDN_CHUNK_TC && g->gdn_vheads / g->gdn_kheads > 3) {   // the chunk-local kernel keeps gate tables for 3 value heads per key head
    set_error("cr_gdn_prefill: the chunked scan serves up to 3 value heads per key head (%d / %d given); use CR_GDN_SERIAL_F32",
              g->gdn_vheads, g->gdn_kheads);
    return CR_ERR_UNSUPPORTED;
  }
  const int part_rows = a.R < gdn_part_rows() ? a.R : gdn_part_rows();
  const size_t part_bytes = gdn_workspace_layout(g, part_rows, nullptr, nullptr);
  const size_t need = a.R > gdn_part_rows() ? 2 * part_bytes : part_bytes;
  CR_REQUIRE(args->workspace && args->workspace_bytes >= need, "cr_gdn_prefill: workspace of %zu bytes needed, %zu given",
             need, args->workspace_bytes);
  CR_REQUIRE(((uintptr_t)args->workspace & 255) == 0, "cr_gdn_prefill: workspace must be 256-byte aligned");

  const bool bf = args->in_dtype == CR_IN_BF16;
  const size_t in_elt = bf ? 2 : 4, out_elt = fmt == CR_OUT_RAW_F32 ? 4 : 2;
  const size_t Cw = 2 * (size_t)g->gdn_kheads * 128 + (size_t)g->gdn_vheads * 128, VWs = (size_t)g->gdn_vheads * 128;
  GdnPrefillParams P;
  // The call runs in parts of gdn_part_rows() rows; the state carries from part to part.
  auto part_params = [&](int p0, int buf, int rows = 0) {
    P.a = a;
    P.a.qkv = (const char*)a.qkv + (size_t)p0 * Cw * in_elt;
    P.a.z = (const char*)a.z + (size_t)p0 * VWs * in_elt;
    if (a.pack_rows) P.a.pack_off = a.pack_off + p0; else P.a.out = (char*)a.out + (size_t)p0 * VWs * out_elt;
    P.a.pos0 = a.pos0 + p0;
    P.a.R = rows ? rows : (a.R - p0 < gdn_part_rows() ? a.R - p0 : gdn_part_rows());
    P.a.commit = P.a.R;
    P.ab_logits = (const char*)args->ab_logits + (size_t)p0 * 2 * g->gdn_vheads * in_elt;
    P.Hv = g->gdn_vheads; P.Hk = g->gdn_kheads; P.fmt = (int)fmt;
    P.tf32 = 0;
    P.halo_in = p0 > 0;


    gdn_workspace_layout(g, part_rows, &P, (char*)args->workspace + (size_t)buf * part_bytes);
    if (args->raw_y) P.yraw = args->raw_y + (size_t)p0 * VWs;
  };
  auto gate = [&](cudaStream_t st) -> cr_status {
    const unsigned gg = (unsigned)(((long long)P.a.R * g->gdn_vheads + 8 * kGateUnits - 1) / (8 * kGateUnits));
    if (bf) gdn_gate_kernel<true><<<gg, 256, 0, st>>>(P); else gdn_gate_kernel<false><<<gg, 256, 0, st>>>(P);
    CR_LAUNCH_CHECK("gdn_gate_kernel");
    return CR_OK;
  };
  if (algo == CR_GDN_CHUNK_TC && a.R > gdn_part_rows() && !profiling()) {
    // Pipeline over parts on two internal streams that fork from the caller's stream and join it again.  The
    // scan of part p is enqueued before the local kernel of part p + 1 and on the stream of higher priority, so
    // that its CTAs (one whole SM each) are placed while the SMs are empty; the local kernel then fills the rest.
    PipeStreams* ps = pipe_streams();
    CR_REQUIRE(ps, "cr_gdn_prefill: cannot create the internal streams");
    const std::vector<std::pair<int, int>> parts = part_schedule(a.R, gdn_part_rows());
    const int np = (int)parts.size();
    for (const auto& pr : parts) CR_REQUIRE(pr.second <= part_rows, "cr_gdn_prefill: internal part of %d rows exceeds the workspace part of %d", pr.second, part_rows);
    std::lock_guard<std::mutex> lock(ps->mu);
    CR_CUDA(cudaEventRecord(ps->fork, stream));
    CR_CUDA(cudaStreamWaitEvent(ps->hi, ps->fork, 0));
    CR_CUDA(cudaStreamWaitEvent(ps->lo, ps->fork, 0));
    CR_CUDA(cudaStreamWaitEvent(ps->mid, ps->fork, 0));
    auto enqueue = [&]() -> cr_status {
      part_params(parts[0].first, 0, parts[0].second);
      if (cr_status s = gdn_chunk_local_only(g, P, bf, ps->lo)) return s;
      CR_CUDA(cudaEventRecord(ps->local_done[0], ps->lo));
      for (int pi = 0; pi < np; ++pi) {
        const int buf = pi & 1;
        part_params(parts[pi].first, buf, parts[pi].second);
        CR_CUDA(cudaStreamWaitEvent(ps->hi, ps->local_done[buf], 0));
        if (cr_status s = gdn_chunk_scan_only(g, P, ps->hi)) return s;
        // the gated readout runs on a third stream, so the next scan does not queue behind it
        CR_CUDA(cudaEventRecord(ps->scan_done[buf], ps->hi));
        CR_CUDA(cudaStreamWaitEvent(ps->mid, ps->scan_done[buf], 0));
        if (cr_status s = gate(ps->mid)) return s;
        CR_CUDA(cudaEventRecord(ps->part_done[buf], ps->mid));
        if (pi + 1 < np) {   // local kernel of the next part, into the other workspace
          // Its workspace was last read by the scan and the gate of part pi - 1.  Waiting for the gate (which runs
          // late, behind the local kernel of part pi) also delays this launch just long enough for the scan of part
          // pi to take its SMs while they are empty; waiting for the scan alone measured 7 % slower.
          if (pi >= 1) CR_CUDA(cudaStreamWaitEvent(ps->lo, ps->part_done[buf ^ 1], 0));
          part_params(parts[pi + 1].first, buf ^ 1, parts[pi + 1].second);
          if (cr_status s = gdn_chunk_local_only(g, P, bf, ps->lo)) return s;
          CR_CUDA(cudaEventRecord(ps->local_done[buf ^ 1], ps->lo));
        }
      }
      return CR_OK;
    };
    const cr_status enq = enqueue();
    // Join: whatever was enqueued on the three internal streams (all of it, or the part before an error) is waited
    // for by the caller's stream, so the streams never stay forked (a capture would otherwise be left unjoined).
    cudaEvent_t join[3] = {ps->local_done[0], ps->scan_done[0], ps->part_done[0]};
    cudaStream_t internal[3] = {ps->lo, ps->hi, ps->mid};
    for (int i = 0; i < 3; ++i) {
      const cudaError_t e1 = cudaEventRecord(join[i], internal[i]);
      const cudaError_t e2 = e1 == cudaSuccess ? cudaStreamWaitEvent(stream, join[i], 0) : e1;
      if (e2 != cudaSuccess && enq == CR_OK) return cuda_fail(e2, "cr_gdn_prefill: joining the internal streams");
    }
    if (enq) return enq;
  } else {
    int pi = 0;
    for (int p0 = 0; p0 < a.R; p0 += gdn_part_rows(), ++pi) {
      part_params(p0, a.R > gdn_part_rows() ? (pi & 1) : 0);
      if (algo == CR_GDN_SERIAL_F32) {
        const dim3 pg((P.a.R + 15) / 16, g->gdn_kheads + g->gdn_vheads / 2 + 1);
        if (bf) gdn_prep_kernel<true><<<pg, 256, 0, stream>>>(P); else gdn_prep_kernel<false><<<pg, 256, 0, stream>>>(P);
        CR_LAUNCH_CHECK("gdn_prep_kernel");
        gdn_scan_serial_kernel<<<g->gdn_vheads * 4, 256, 0, stream>>>(P);
        CR_LAUNCH_CHECK("gdn_scan_serial_kernel");
      } else {   // the chunked scan prepares its rows itself
        if (cr_status s = gdn_chunk_scan(g, P, bf, stream)) return s;
      }
      if (cr_status s = gate(stream)) return s;
    }
  }
  P.a = a;
  const int C = 2 * g->gdn_kheads * 128 + g->gdn_vheads * 128;
  const unsigned rg = (unsigned)(((long long)(a.R < 16 ? a.R : 16) * C + 255) / 256);
  if (bf) gdn_ring_kernel<true><<<rg, 256, 0, stream>>>(P); else gdn_ring_kernel<false><<<rg, 256, 0, stream>>>(P);
  CR_LAUNCH_CHECK("gdn_ring_kernel");
  return CR_OK;
}

extern "C" cr_status cr_gdn_materialize(const cr_geometry* g, float* const* states, int n_states, void* stream) {
  using namespace cr;
  if (cr_status s = check_geometry(g)) return s;
  CR_REQUIRE(states && n_states >= 0, "cr_gdn_materialize: null states");
  use_stream((cudaStream_t)stream);
  for (int i = 0; i < n_states; i += 64) {
    GdnStates s{};
    const int n = n_states - i < 64 ? n_states - i : 64;
    for (int j = 0; j < n; ++j) {
      CR_REQUIRE(states[i + j], "cr_gdn_materialize: null state %d", i + j);
      s.layer[j] = states[i + j];
    }
    s.Hv = g->gdn_vheads;
    gdn_materialize_kernel<<<dim3(g->gdn_vheads, n), 1024, 0, (cudaStream_t)stream>>>(s);
    CR_LAUNCH_CHECK("gdn_materialize_kernel");
  }
  return CR_OK;
}
