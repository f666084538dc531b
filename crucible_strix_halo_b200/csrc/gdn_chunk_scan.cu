// gdn_chunk_scan_kernel: the sequential part of the chunk-64 WY scan.  One CTA per (value head, NC-column
// slice of the state); the slice stays in accumulator registers (fp32) for the whole call; the operands of the
// next chunk are streamed with cp.async while the current chunk is multiplied.  Warps 0-3 run the recurrence
// chain (W S, U, K^T U), warps 4-7 the readout (Q S, QKd U), so the readout is off the critical path.
#include <cstdlib>
#include "gdn_chunk.cuh"

namespace cr {

template <int NC>
struct ScanSmem {
  static constexpr int kLdS = NC + 8;       // stride % 32 == 8
  static constexpr size_t kFloats = 2 * 64 * kLdK /* W, Q */ + 64 * kLdS /* Ut */ + 64 /* G */ + 64 * kLdX /* K */ +
                                    64 * kLdM /* QKd */ + 128 * kLdS /* S operand */ + 2 * 64 * kLdS /* U, U' */;
  static constexpr size_t kBytes = kFloats * sizeof(float);
};

template <int NC>
__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(GdnPrefillParams P, ChunkWs ws) {
  constexpr int kLdS = ScanSmem<NC>::kLdS, NT = NC / 8, SL = 128 / NC;
  extern __shared__ __align__(16) float sm[];
  float* Wsm = sm;                       // [64][132]
  float* Qsm = Wsm + 64 * kLdK;          // [64][132]
  float* Utsm = Qsm + 64 * kLdK;         // [64][NC+8]
  float* Gsm = Utsm + 64 * kLdS;         // [64]
  float* Ksm = Gsm + 64;                 // [64][136]  khat, read transposed
  float* QKsm = Ksm + 64 * kLdX;         // [64][68]
  float* Sop = QKsm + 64 * kLdM;         // [128][NC+8]  tf32 copy of the state slice
  float* Usm = Sop + 128 * kLdS;         // [64][NC+8]
  float* Upsm = Usm + 64 * kLdS;         // [64][NC+8]   e^{G_end - G} U
  const int t = threadIdx.x, w = t >> 5, l = t & 31, g = l >> 2, tq = l & 3;
  const int h = blockIdx.x / SL, col0 = (blockIdx.x % SL) * NC;
  const int rep = P.Hv / P.Hk, kh = h / rep, VW = P.Hv * 128, R = P.a.R;
  const int nch = ws.chunks;

  auto load_a = [&](int c) {   // W, Q, Ut slice, G of chunk c
    const size_t unit = (size_t)h * nch + c;
    const int r0 = c * kChunk;
    const float* Wg = ws.W + unit * 64 * 128;
    for (int i = t; i < 64 * 32; i += 256) {
      const int row = i >> 5, c4 = (i & 31) * 4;
      cp_async16(Wsm + row * kLdK + c4, Wg + row * 128 + c4, true);
      const bool ok = r0 + row < R;
      cp_async16(Qsm + row * kLdK + c4, P.qn + ((size_t)(ok ? r0 + row : 0) * P.Hk + kh) * 128 + c4, ok);
    }
    const float* Ug = ws.Ut + unit * 64 * 128 + col0;
    for (int i = t; i < 64 * (NC / 4); i += 256) {
      const int row = i / (NC / 4), c4 = (i % (NC / 4)) * 4;
      cp_async16(Utsm + row * kLdS + c4, Ug + row * 128 + c4, true);
    }
    if (t < 16) cp_async16(Gsm + t * 4, ws.G + unit * 64 + t * 4, true);
  };
  auto load_b = [&](int c) {   // K, QKd of chunk c
    const size_t unit = (size_t)h * nch + c;
    const int r0 = c * kChunk;
    for (int i = t; i < 64 * 32; i += 256) {
      const int row = i >> 5, c4 = (i & 31) * 4;
      const bool ok = r0 + row < R;
      cp_async16(Ksm + row * kLdX + c4, P.kn + ((size_t)(ok ? r0 + row : 0) * P.Hk + kh) * 128 + c4, ok);
    }
    const float* Qg = ws.QKd + unit * 64 * 64;
    for (int i = t; i < 64 * 16; i += 256) {
      const int row = i >> 4, c4 = (i & 15) * 4;
      cp_async16(QKsm + row * kLdM + c4, Qg + row * 64 + c4, true);
    }
  };

  // state slice: warp w < 4 owns key rows [32w, 32w+32) x NC columns as two 16-row accumulator tiles
  float S[2][NT][4];
  float* st = P.a.state + (size_t)h * 16384 + col0;
  if (w < 4) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int row = 32 * w + 16 * mi + g, col = 8 * n + 2 * tq;
        const float2 lo = *reinterpret_cast<const float2*>(st + (size_t)row * 128 + col);
        const float2 hi = *reinterpret_cast<const float2*>(st + (size_t)(row + 8) * 128 + col);
        S[mi][n][0] = lo.x; S[mi][n][1] = lo.y; S[mi][n][2] = hi.x; S[mi][n][3] = hi.y;
        *reinterpret_cast<float2*>(Sop + row * kLdS + col) = make_float2(tf32r(lo.x), tf32r(lo.y));
        *reinterpret_cast<float2*>(Sop + (row + 8) * kLdS + col) = make_float2(tf32r(hi.x), tf32r(hi.y));
      }
  }
  load_a(0);
  cp_async_commit();

  for (int c = 0; c < nch; ++c) {
    cp_async_wait_all();
    __syncthreads();                       // group A of chunk c and the state operand are visible
    load_b(c);
    cp_async_commit();
    const int mt = w & 3;
    const float Gend = Gsm[63];
    const float Glo = Gsm[mt * 16 + g], Ghi = Gsm[mt * 16 + g + 8];
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    warp_gemm<NT, 16, false, false>(acc, (w < 4 ? Wsm : Qsm) + mt * 16 * kLdK, kLdK, Sop, kLdS);
    if (w < 4) {   // U = Ut - W S; keep U (tf32) and U' = e^{G_end - G} U for the state update
      const float slo = __expf(Gend - Glo), shi = __expf(Gend - Ghi);
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int col = 8 * n + 2 * tq;
        const float2 ulo = *reinterpret_cast<const float2*>(Utsm + (mt * 16 + g) * kLdS + col);
        const float2 uhi = *reinterpret_cast<const float2*>(Utsm + (mt * 16 + g + 8) * kLdS + col);
        const float u0 = ulo.x - acc[n][0], u1 = ulo.y - acc[n][1], u2 = uhi.x - acc[n][2], u3 = uhi.y - acc[n][3];
        *reinterpret_cast<float2*>(Usm + (mt * 16 + g) * kLdS + col) = make_float2(tf32r(u0), tf32r(u1));
        *reinterpret_cast<float2*>(Usm + (mt * 16 + g + 8) * kLdS + col) = make_float2(tf32r(u2), tf32r(u3));
        *reinterpret_cast<float2*>(Upsm + (mt * 16 + g) * kLdS + col) = make_float2(tf32r(slo * u0), tf32r(slo * u1));
        *reinterpret_cast<float2*>(Upsm + (mt * 16 + g + 8) * kLdS + col) = make_float2(tf32r(shi * u2), tf32r(shi * u3));
      }
    } else {       // readout part 1: e^G (Q S)
      const float elo = __expf(Glo), ehi = __expf(Ghi);
#pragma unroll
      for (int n = 0; n < NT; ++n) { acc[n][0] *= elo; acc[n][1] *= elo; acc[n][2] *= ehi; acc[n][3] *= ehi; }
    }
    cp_async_wait_all();
    __syncthreads();                       // U, U' and group B visible; W / Q / Ut / G free
    if (c + 1 < nch) load_a(c + 1);
    cp_async_commit();
    if (w < 4) {   // S <- e^{G_end} S + K^T U'
      const float eend = __expf(Gend);
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
        for (int n = 0; n < NT; ++n) { S[mi][n][0] *= eend; S[mi][n][1] *= eend; S[mi][n][2] *= eend; S[mi][n][3] *= eend; }
        warp_gemm<NT, 8, true, false>(S[mi], Ksm + 32 * w + 16 * mi, kLdX, Upsm, kLdS);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const int row = 32 * w + 16 * mi + g, col = 8 * n + 2 * tq;
          *reinterpret_cast<float2*>(Sop + row * kLdS + col) = make_float2(tf32r(S[mi][n][0]), tf32r(S[mi][n][1]));
          *reinterpret_cast<float2*>(Sop + (row + 8) * kLdS + col) = make_float2(tf32r(S[mi][n][2]), tf32r(S[mi][n][3]));
        }
      }
    } else {       // readout part 2: + QKd U, then store
      warp_gemm<NT, 8, false, false>(acc, QKsm + mt * 16 * kLdM, kLdM, Usm, kLdS);
      const int r_lo = c * kChunk + mt * 16 + g, r_hi = r_lo + 8;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int col = h * 128 + col0 + 8 * n + 2 * tq;
        if (r_lo < R) *reinterpret_cast<float2*>(P.yraw + (size_t)r_lo * VW + col) = make_float2(acc[n][0], acc[n][1]);
        if (r_hi < R) *reinterpret_cast<float2*>(P.yraw + (size_t)r_hi * VW + col) = make_float2(acc[n][2], acc[n][3]);
      }
    }
    // the barrier at the top of the next iteration orders: S operand written / K, QKd, U, U' free
  }
  cp_async_wait_all();
  if (w < 4) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int row = 32 * w + 16 * mi + g, col = 8 * n + 2 * tq;
        *reinterpret_cast<float2*>(st + (size_t)row * 128 + col) = make_float2(S[mi][n][0], S[mi][n][1]);
        *reinterpret_cast<float2*>(st + (size_t)(row + 8) * 128 + col) = make_float2(S[mi][n][2], S[mi][n][3]);
      }
  }
}

// slice width: CR_GDN_SCAN_NC=32|64 overrides (for experiments).  32 is the default: twice the CTAs on a chain
// that is latency-bound measured faster (1.8 ms against 2.6 ms for 32768 tokens) than halving the operand re-reads.
cr_status gdn_chunk_scan_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, cudaStream_t stream) {
  static const int nc = [] { const char* e = getenv("CR_GDN_SCAN_NC"); return (e && atoi(e) == 64) ? 64 : 32; }();
  static PerDeviceOnce configured;
  if (first_use_on_device(configured)) {
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_scan_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ScanSmem<32>::kBytes));
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_scan_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ScanSmem<64>::kBytes));
  }
  if (nc == 32) gdn_chunk_scan_kernel<32><<<g->gdn_vheads * 4, 256, ScanSmem<32>::kBytes, stream>>>(P, ws);
  else gdn_chunk_scan_kernel<64><<<g->gdn_vheads * 2, 256, ScanSmem<64>::kBytes, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_scan_kernel");
  return CR_OK;
}

}  // namespace cr
