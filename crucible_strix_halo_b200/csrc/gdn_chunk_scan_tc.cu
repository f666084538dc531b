// gdn_chunk_scan_tc_kernel: the sequential part of the chunk-64 WY scan on tcgen05 tensor cores.
//
// One CTA (128 threads) per (value head, NC-column slice of the state).  Accumulators live in tensor memory,
// operands in shared memory as K-major un-swizzled tiles (float[K/4][rows][4], see umma.cuh); the local kernel
// writes W, Qt = e^G Q, K^T and QKd in exactly that layout, so each arrives with one bulk copy (TMA, mbarrier
// transaction count) into a buffer that is re-filled for the next chunk as soon as its MMA has completed.
// Per chunk (S^T, U^T, U'^T are written by the threads themselves, transposed so that every operand is K-major):
//   D1a[64 x NC]  = W  S        (tokens on TMEM lanes, M = 64)        -> U = Ut - D1a, U' = e^{G_end-G} U
//   D1b[64 x NC]  = Qt S  (+ QKd U, accumulated by D3)               -> Y
//   D2 [128 x NC] = K^T U'      (keys on TMEM lanes, M = 128)         -> S = e^{G_end} S + D2 (fp32 registers)
// Every wait is bounded; a wait that gives up raises a status word and the kernel runs to its end without
// waiting again, frees its tensor memory and returns.
#include "gdn_chunk.cuh"
#include "umma.cuh"

namespace cr {

__device__ int g_gdn_scan_status = 0;
__device__ long long g_prof[16];
#define PROF(i) do { if (blockIdx.x == 0 && t == 32) { long long now_ = clock64(); g_prof[i] += now_ - last_; last_ = now_; } } while (0)

template <int NC>
struct TcSmem {
  static constexpr int NCP = NC + 1;                       // padded plane: conflict-free transposed stores
  static constexpr int kW = 0, kQ = 8192, kK = 16384, kQK = 24576, kS = 28672;
  static constexpr int kU = kS + 32 * NCP * 4, kUp = kU + 16 * NCP * 4, kEnd = kUp + 16 * NCP * 4;
  static constexpr size_t kBytes = (size_t)kEnd * sizeof(float) + 128;
};

template <int NC>
__global__ void __launch_bounds__(128) gdn_chunk_scan_tc_kernel(GdnPrefillParams P, ChunkWs ws) {
  using L = TcSmem<NC>;
  constexpr int NCP = L::NCP;
  constexpr uint32_t kTmemCols = NC == 64 ? 256 : 128;
  extern __shared__ __align__(128) float sm[];
  float* Wsm = sm + L::kW;       // [32][64][4]   W, K-major over keys
  float* Qsm = sm + L::kQ;       // [32][64][4]   e^G Q
  float* Ksm = sm + L::kK;       // [16][128][4]  K^T, K-major over tokens
  float* QKsm = sm + L::kQK;     // [16][64][4]   QKd
  float* Ssm = sm + L::kS;       // [32][NC+1][4] S^T, K-major over keys
  float* Usm = sm + L::kU;       // [16][NC+1][4] U^T, K-major over tokens
  float* Upsm = sm + L::kUp;     // [16][NC+1][4] U'^T
  __shared__ __align__(8) uint64_t bars[7];                // full W, Q, K, QK; done D1a, D2, D3
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int dead;
  uint64_t *fullW = &bars[0], *fullQ = &bars[1], *fullK = &bars[2], *fullQK = &bars[3];
  uint64_t *d1a = &bars[4], *d2 = &bars[5], *d3 = &bars[6];
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  constexpr int SL = 128 / NC;
  const int h = blockIdx.x / SL, col0 = (blockIdx.x % SL) * NC;
  const int rep = P.Hv / P.Hk, kh = h / rep, VW = P.Hv * 128, R = P.a.R;
  const int nch = ws.chunks;
  const bool tokth = l < 16;                               // M = 64 accumulators: rows on lanes 0..15 of each warp
  const int tk = 16 * w + l;

  if (t == 0) {
#pragma unroll
    for (int i = 0; i < 7; ++i) umma::mbar_init(&bars[i], 1);
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == 0) umma::tmem_alloc(&tmem_slot, kTmemCols);
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (dead) return;
    if (!umma::mbar_wait(bar, parity)) { dead = 1; g_gdn_scan_status = 1; }
  };
  auto load_w = [&](int c) { umma::mbar_expect_tx(fullW, 32768); umma::bulk_load(Wsm, ws.W + ((size_t)h * nch + c) * 8192, 32768, fullW); };
  auto load_q = [&](int c) { umma::mbar_expect_tx(fullQ, 32768); umma::bulk_load(Qsm, ws.Qt + ((size_t)h * nch + c) * 8192, 32768, fullQ); };
  auto load_k = [&](int c) { umma::mbar_expect_tx(fullK, 32768); umma::bulk_load(Ksm, ws.Kt + ((size_t)kh * nch + c) * 8192, 32768, fullK); };
  auto load_qk = [&](int c) { umma::mbar_expect_tx(fullQK, 16384); umma::bulk_load(QKsm, ws.QKd + ((size_t)h * nch + c) * 4096, 16384, fullQK); };

  // state row of key t: fp32 master in registers, tf32 copy transposed into shared memory
  float S[NC];
  float* st = P.a.state + (size_t)h * 16384 + (size_t)t * 128 + col0;
#pragma unroll
  for (int j = 0; j < NC; j += 4) {
    const float4 v = *reinterpret_cast<const float4*>(st + j);
    S[j] = v.x; S[j + 1] = v.y; S[j + 2] = v.z; S[j + 3] = v.w;
  }
#pragma unroll
  for (int j = 0; j < NC; ++j) Ssm[((t >> 2) * NCP + j) * 4 + (t & 3)] = tf32r(S[j]);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  if (t == 0) { load_w(0); load_q(0); load_k(0); load_qk(0); }

  constexpr uint32_t idesc64 = umma::idesc_tf32(64, NC, false, false), idesc128 = umma::idesc_tf32(128, NC, false, false);
  // descriptors of the first K step; a step of 8 along K advances the start address by 2 planes (16-byte units)
  const uint64_t dW = umma::desc_kmajor(Wsm, 64, 0), dQ = umma::desc_kmajor(Qsm, 64, 0), dK = umma::desc_kmajor(Ksm, 128, 0);
  const uint64_t dQK = umma::desc_kmajor(QKsm, 64, 0), dS = umma::desc_kmajor_padded(Ssm, NCP, 0);
  const uint64_t dU = umma::desc_kmajor_padded(Usm, NCP, 0), dUp = umma::desc_kmajor_padded(Upsm, NCP, 0);
  float ut[NC];                                           // Ut row of this thread's token
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
  fetch_rows(0);

  long long last_ = clock64();
  for (int c = 0; c < nch; ++c) {
    const uint32_t ph = c & 1;
    PROF(0);
    if (t == 0) {
      wait(fullW, ph);
      umma::fence_after_sync();
#pragma unroll
      for (int s8 = 0; s8 < 16; ++s8) umma::mma_tf32_ss(tm, dW + (uint64_t)(s8 * 128), dS + (uint64_t)(s8 * 2 * NCP), idesc64, s8 > 0);
      umma::commit(d1a);
    }
    wait(d1a, ph);
    umma::fence_after_sync();
    PROF(1);
    if (t == 0 && c + 1 < nch) load_w(c + 1);
    const float gt = Gtok, ge = Gend;
    {   // U = Ut - W S, transposed into shared memory (tf32), and U' = e^{G_end - G} U
      const float sc = __expf(ge - gt);
#pragma unroll
      for (int j0 = 0; j0 < NC; j0 += 32) {
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, j0), p);
        if (tokth) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float u = ut[j0 + j] - p[j];
            const int at = ((tk >> 2) * NCP + j0 + j) * 4 + (tk & 3);
            Usm[at] = tf32r(u);
            Upsm[at] = tf32r(sc * u);
          }
        }
      }
    }
    PROF(2);
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    PROF(3);
    if (t == 0) {
      wait(fullK, ph);
#pragma unroll
      for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ss(tm + 2 * NC, dK + (uint64_t)(s8 * 256), dUp + (uint64_t)(s8 * 2 * NCP), idesc128, s8 > 0);
      umma::commit(d2);
      // the readout products are off the chain: Qt S^T (S^T stays untouched until d3), then + QKd U^T
      wait(fullQ, ph);
#pragma unroll
      for (int s8 = 0; s8 < 16; ++s8) umma::mma_tf32_ss(tm + NC, dQ + (uint64_t)(s8 * 128), dS + (uint64_t)(s8 * 2 * NCP), idesc64, s8 > 0);
      wait(fullQK, ph);
#pragma unroll
      for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ss(tm + NC, dQK + (uint64_t)(s8 * 128), dU + (uint64_t)(s8 * 2 * NCP), idesc64, 1u);
      umma::commit(d3);
    }
    if (c + 1 < nch) fetch_rows(c + 1);                    // global loads fly while the tensor core works
    PROF(4);
    wait(d2, ph);
    umma::fence_after_sync();
    PROF(5);
    if (t == 0 && c + 1 < nch) load_k(c + 1);
    {   // S <- e^{G_end} S + K^T U' (registers; the transposed copy is rewritten after d3)
      const float eend = __expf(ge);
#pragma unroll
      for (int j0 = 0; j0 < NC; j0 += 32) {
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, 2 * NC + j0), p);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          S[j0 + j] = fmaf(eend, S[j0 + j], p[j]);
        }
      }
    }
    PROF(6);
    wait(d3, ph);
    umma::fence_after_sync();
    PROF(7);
    if (t == 0 && c + 1 < nch) { load_q(c + 1); load_qk(c + 1); }
#pragma unroll
    for (int j = 0; j < NC; ++j) Ssm[((t >> 2) * NCP + j) * 4 + (t & 3)] = tf32r(S[j]);   // Qt S^T has completed
    {   // Y = e^G (Q S) + QKd U
      const int row = c * kChunk + tk;
#pragma unroll
      for (int j0 = 0; j0 < NC; j0 += 32) {
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, NC + j0), p);
        if (tokth && row < R) {
          float* dst = P.yraw + (size_t)row * VW + h * 128 + col0 + j0;
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(p[j], p[j + 1], p[j + 2], p[j + 3]);
        }
      }
    }
    PROF(8);
    umma::fence_async_smem();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    PROF(9);
  }
#pragma unroll
  for (int j = 0; j < NC; j += 4) *reinterpret_cast<float4*>(st + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
  umma::fence_before_sync();
  __syncthreads();
  if (w == 0) umma::tmem_dealloc(tm, kTmemCols);
}

cr_status gdn_chunk_scan_tc_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_scan_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem<32>::kBytes));
    configured = true;
  }
  gdn_chunk_scan_tc_kernel<32><<<g->gdn_vheads * 4, 128, TcSmem<32>::kBytes, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_scan_tc_kernel");
  return CR_OK;
}

extern "C" void cr_debug_prof(long long* out) { cudaMemcpyFromSymbol(out, g_prof, sizeof(long long) * 16); long long z[16] = {0}; cudaMemcpyToSymbol(g_prof, z, sizeof(z)); }
int gdn_scan_status_read() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gdn_scan_status, sizeof(int));
  return v;
}

}  // namespace cr
