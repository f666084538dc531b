// gdn_chunk_scan_tc_kernel: the sequential part of the chunk-64 WY scan on tcgen05 tensor cores.
//
// One CTA per (value head, 32-column slice of the state): four compute warps (128 threads = the 128 lanes of
// tensor memory) and one issuer warp whose elected thread feeds the tensor core and the bulk-copy engine.
// Accumulators live in tensor memory; operands are K-major un-swizzled tiles in shared memory
// (float[K/4][rows][4], see umma.cuh).  The local kernel writes W, Qt = e^G Q, K^T and QKd in exactly that
// layout, so each arrives with one bulk copy (TMA, mbarrier transaction count) into a buffer that is re-filled
// for the next chunk as soon as the MMA that read it has completed.  S^T, U^T and U'^T are written by the compute
// warps themselves (transposed, double-buffered), so every operand is K-major.  Per chunk:
//   D1a[64 x 32]  = W  S        (tokens on lanes 0..15 of each warp, M = 64)  -> U = Ut - D1a, U' = e^{G_end-G} U
//   D2 [128 x 32] = K^T U'      (keys on lanes, M = 128)                      -> S = e^{G_end} S + D2 (fp32 registers)
//   D1b[64 x 32]  = Qt S + QKd U  (readout; issued one chunk late so it never sits between D1a and D2)  -> Y
// The warps synchronise only through mbarriers (no block barrier inside the loop).  Every wait is bounded: a wait
// that gives up raises a status word, after which no thread waits again; the kernel runs to its end, frees its
// tensor memory and returns.
#include "gdn_chunk.cuh"
#include "umma.cuh"

namespace cr {

__device__ int g_gdn_scan_status = 0;

constexpr int kNC = 32, kNCP = kNC + 1;    // slice width; padded plane (conflict-free transposed stores)
struct TcSmem {
  static constexpr int kW = 0, kQ = 8192, kK = 16384, kQK = 24576, kS = 28672;      // float offsets
  static constexpr int kSsz = 32 * kNCP * 4, kUsz = 16 * kNCP * 4;
  static constexpr int kU = kS + 2 * kSsz, kUp = kU + 2 * kUsz, kEnd = kUp + 2 * kUsz;
  static constexpr size_t kBytes = (size_t)kEnd * sizeof(float) + 128;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(160) gdn_chunk_scan_tc_kernel(GdnPrefillParams P, ChunkWs ws) {
  using L = TcSmem;
  constexpr int NC = kNC, NCP = kNCP;
  constexpr uint32_t kTmemCols = 128;
  extern __shared__ __align__(128) float sm[];
  float* Wsm = sm + L::kW;       // [32][64][4]   W, K-major over keys
  float* Qsm = sm + L::kQ;       // [32][64][4]   e^G Q
  float* Ksm = sm + L::kK;       // [16][128][4]  K^T, K-major over tokens
  float* QKsm = sm + L::kQK;     // [16][64][4]   QKd
  float* Ssm = sm + L::kS;       // 2 x [32][33][4] S^T, K-major over keys
  float* Usm = sm + L::kU;       // 2 x [16][33][4] U^T, K-major over tokens
  float* Upsm = sm + L::kUp;     // 2 x [16][33][4] U'^T
  __shared__ __align__(8) uint64_t bars[9];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int dead;
  uint64_t *fullW = &bars[0], *fullQ = &bars[1], *fullK = &bars[2], *fullQK = &bars[3];
  uint64_t *d1a = &bars[4], *d2 = &bars[5], *d3 = &bars[6], *uReady = &bars[7], *sReady = &bars[8];
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  const int h = blockIdx.x >> 2, col0 = (blockIdx.x & 3) * NC;
  const int rep = P.Hv / P.Hk, kh = h / rep, VW = P.Hv * 128, R = P.a.R;
  const int nch = ws.chunks;

  if (t == 0) {
#pragma unroll
    for (int i = 0; i < 7; ++i) umma::mbar_init(&bars[i], 1);
    umma::mbar_init(uReady, 128);
    umma::mbar_init(sReady, 128);
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == 4) umma::tmem_alloc(&tmem_slot, kTmemCols);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (dead) return;
    if (!umma::mbar_wait(bar, parity)) { dead = 1; g_gdn_scan_status = 1; }
  };

  if (w == 4) {
    // ------------------------------------------------------------------ issuer: loads and tensor-core work
    if (l == 0) {
      auto load_w = [&](int c) { umma::mbar_expect_tx(fullW, 32768); umma::bulk_load(Wsm, ws.W + ((size_t)h * nch + c) * 8192, 32768, fullW); };
      auto load_q = [&](int c) { umma::mbar_expect_tx(fullQ, 32768); umma::bulk_load(Qsm, ws.Qt + ((size_t)h * nch + c) * 8192, 32768, fullQ); };
      auto load_k = [&](int c) { umma::mbar_expect_tx(fullK, 32768); umma::bulk_load(Ksm, ws.Kt + ((size_t)kh * nch + c) * 8192, 32768, fullK); };
      auto load_qk = [&](int c) { umma::mbar_expect_tx(fullQK, 16384); umma::bulk_load(QKsm, ws.QKd + ((size_t)h * nch + c) * 4096, 16384, fullQK); };
      load_w(0); load_k(0); load_q(0); load_qk(0);
      constexpr uint32_t idesc64 = umma::idesc_tf32(64, NC, false, false), idesc128 = umma::idesc_tf32(128, NC, false, false);
      // descriptors of the first K step; a step of 8 along K advances the start address by 2 planes (16-byte units)
      const uint64_t dW = umma::desc_kmajor(Wsm, 64, 0), dQ = umma::desc_kmajor(Qsm, 64, 0), dK = umma::desc_kmajor(Ksm, 128, 0);
      const uint64_t dQK = umma::desc_kmajor(QKsm, 64, 0);
      uint64_t dS[2], dU[2], dUp[2];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        dS[b] = umma::desc_kmajor_padded(Ssm + b * L::kSsz, NCP, 0);
        dU[b] = umma::desc_kmajor_padded(Usm + b * L::kUsz, NCP, 0);
        dUp[b] = umma::desc_kmajor_padded(Upsm + b * L::kUsz, NCP, 0);
      }
      auto readout = [&](int c) {     // D1b(c) = Qt S^T(c) + QKd U^T(c)
        const int b = c & 1;
        wait(fullQ, b);
#pragma unroll
        for (int s8 = 0; s8 < 16; ++s8) umma::mma_tf32_ss(tm + NC, dQ + (uint64_t)(s8 * 128), dS[b] + (uint64_t)(s8 * 2 * NCP), idesc64, s8 > 0);
        wait(fullQK, b);
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ss(tm + NC, dQK + (uint64_t)(s8 * 128), dU[b] + (uint64_t)(s8 * 2 * NCP), idesc64, 1u);
        umma::commit(d3);
      };
      for (int c = 0; c < nch; ++c) {
        const int b = c & 1;
        wait(sReady, b);
        wait(fullW, b);
        umma::fence_after_sync();
#pragma unroll
        for (int s8 = 0; s8 < 16; ++s8) umma::mma_tf32_ss(tm, dW + (uint64_t)(s8 * 128), dS[b] + (uint64_t)(s8 * 2 * NCP), idesc64, s8 > 0);
        umma::commit(d1a);
        if (c > 0) readout(c - 1);                       // runs on the tensor core while the warps compute U(c)
        wait(uReady, b);
        wait(fullK, b);
        umma::fence_after_sync();
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ss(tm + 2 * NC, dK + (uint64_t)(s8 * 256), dUp[b] + (uint64_t)(s8 * 2 * NCP), idesc128, s8 > 0);
        umma::commit(d2);
        // refill the buffers whose readers have completed
        wait(d1a, b);
        if (c + 1 < nch) load_w(c + 1);
        if (c > 0) { wait(d3, (c - 1) & 1); load_q(c); load_qk(c); }
        wait(d2, b);
        if (c + 1 < nch) load_k(c + 1);
      }
      readout(nch - 1);
    }
  } else {
    // ------------------------------------------------------------------ compute warps (thread = TMEM lane)
    const bool tokth = l < 16;                             // M = 64 accumulators: rows on lanes 0..15 of each warp
    const int tk = 16 * w + l;
    float S[NC];                                           // state row of key t: fp32 master
    float* st = P.a.state + (size_t)h * 16384 + (size_t)t * 128 + col0;
#pragma unroll
    for (int j = 0; j < NC; j += 4) {
      const float4 v = *reinterpret_cast<const float4*>(st + j);
      S[j] = v.x; S[j + 1] = v.y; S[j + 2] = v.z; S[j + 3] = v.w;
    }
#pragma unroll
    for (int j = 0; j < NC; ++j) Ssm[((t >> 2) * NCP + j) * 4 + (t & 3)] = tf32r(S[j]);
    umma::fence_async_smem();
    mbar_arrive(sReady);

    float ut[NC];                                          // Ut row of this thread's token
    float Gtok = 0.f, Gend = 0.f;
    auto fetch_rows = [&](int c) {
      const size_t unit = (size_t)h * nch + c;
      Gend = ws.G[unit * 64 + 63];
      if (tokth) {
        Gtok = ws.G[unit * 64 + tk];
        const float* up = ws.Ut + (unit * 64 + tk) * 128 + col0;
#pragma unroll
        for (int j = 0; j < NC; j += 4) {
          const float4 v = *reinterpret_cast<const float4*>(up + j);
          ut[j] = v.x; ut[j + 1] = v.y; ut[j + 2] = v.z; ut[j + 3] = v.w;
        }
      }
    };
    auto store_y = [&](int c) {     // Y(c) = e^G (Q S) + QKd U, after the readout MMAs of chunk c
      wait(d3, c & 1);
      umma::fence_after_sync();
      float p[32];
      umma::tmem_ld32(umma::tmem_addr(tm, w, NC), p);
      const int row = c * kChunk + tk;
      if (tokth && row < R) {
        float* dst = P.yraw + (size_t)row * VW + h * 128 + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(p[j], p[j + 1], p[j + 2], p[j + 3]);
      }
      umma::fence_before_sync();
    };
    fetch_rows(0);
    for (int c = 0; c < nch; ++c) {
      const int b = c & 1;
      float* Ub = Usm + b * L::kUsz;
      float* Upb = Upsm + b * L::kUsz;
      const float gt = Gtok, ge = Gend;
      wait(d1a, b);
      umma::fence_after_sync();
      {   // U = Ut - W S, transposed into shared memory (tf32), and U' = e^{G_end - G} U
        const float sc = __expf(ge - gt);
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, 0), p);
        if (tokth) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float u = ut[j] - p[j];
            const int at = ((tk >> 2) * NCP + j) * 4 + (tk & 3);
            Ub[at] = tf32r(u);
            Upb[at] = tf32r(sc * u);
          }
        }
      }
      umma::fence_async_smem();
      umma::fence_before_sync();
      mbar_arrive(uReady);
      if (c + 1 < nch) fetch_rows(c + 1);                  // global loads fly while the tensor core works
      if (c > 0) store_y(c - 1);
      wait(d2, b);
      umma::fence_after_sync();
      {   // S <- e^{G_end} S + K^T U'; the transposed tf32 copy goes to the other buffer
        const float eend = __expf(ge);
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, 2 * NC), p);
        float* Sb = Ssm + ((c + 1) & 1) * L::kSsz;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          S[j] = fmaf(eend, S[j], p[j]);
          Sb[((t >> 2) * NCP + j) * 4 + (t & 3)] = tf32r(S[j]);
        }
      }
      umma::fence_async_smem();
      umma::fence_before_sync();
      mbar_arrive(sReady);
    }
    store_y(nch - 1);
#pragma unroll
    for (int j = 0; j < NC; j += 4) *reinterpret_cast<float4*>(st + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (w == 4) umma::tmem_dealloc(tm, kTmemCols);
}

cr_status gdn_chunk_scan_tc_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem::kBytes));
    configured = true;
  }
  gdn_chunk_scan_tc_kernel<<<g->gdn_vheads * 4, 160, TcSmem::kBytes, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_scan_tc_kernel");
  return CR_OK;
}

int gdn_scan_status_read() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gdn_scan_status, sizeof(int));
  return v;
}

}  // namespace cr
