// gdn_chunk_scan_tc_kernel: the sequential part of the chunk-64 WY scan on tcgen05 tensor cores.
//
// One CTA per (value head, 64-column slice of the state): two compute warpgroups (each 128 threads = the 128 lanes
// of tensor memory, 32 accumulator columns per warpgroup) and one issuer warp whose elected thread feeds the
// tensor core and the bulk-copy engine.
// Accumulators live in tensor memory; operands are K-major un-swizzled tiles in shared memory
// (float[K/4][rows][4], see umma.cuh).  The local kernel writes them in exactly that layout, so each arrives
// with one bulk copy (TMA, mbarrier transaction count) into a buffer that is re-filled for the next chunk as soon
// as the MMAs that read it have completed.  S^T, U^T and U'^T are written by the compute warps themselves
// (transposed; one buffer each is enough, because every writer waits on a commit that follows the last MMA
// reading the old contents).  Per chunk, three MMA groups (32 tcgen05.mma of K = 8, N = 64):
//   D1[128 x 64] = [W ; e^G Q] S^T   lanes 0-63: W S (tokens)        -> U = Ut - W S, U' = e^{G_end-G} U   (token warps)
//                                    lanes 64-127: e^G Q S
//   D2[128 x 64] = K^T U'            lanes = keys                    -> S = e^{G_end} S + D2 (fp32 registers, all warps)
//   D1 += [0 ; QKd] U                lanes 64-127 become Y           -> readout stored by the other warps, off the chain
// D1 alternates between two accumulators, so the readout of chunk c overlaps D1 of chunk c+1.  The warps
// synchronise only through mbarriers.  Every wait is bounded: a wait that gives up raises a status word, after
// which no thread waits again; the kernel runs to its end, frees its tensor memory and returns.
#include "gdn_chunk.cuh"
#include "umma.cuh"

namespace cr {

__device__ int g_gdn_scan_status = 0;

constexpr int kWG = 2;                      // compute warpgroups per CTA, 32 state columns each
constexpr int kNC = 32 * kWG, kNCP = kNC + 1;    // slice width; padded plane (conflict-free transposed stores)
struct TcSmem {
  static constexpr int kA1 = 0, kK = 16384, kQK = 24576, kS = 32768;      // float offsets
  static constexpr int kSsz = 32 * kNCP * 4, kUsz = 16 * kNCP * 4;
  static constexpr int kU = kS + kSsz, kUp = kU + kUsz, kEnd = kUp + kUsz;
  static constexpr size_t kBytes = (size_t)kEnd * sizeof(float) + 128;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(128 * kWG + 32) gdn_chunk_scan_tc_kernel(GdnPrefillParams P, ChunkWs ws) {
  using L = TcSmem;
  constexpr int NC = kNC, NCP = kNCP;
  constexpr uint32_t kTmemCols = kWG == 1 ? 128 : 256;   // D1 x 2 (NC columns each), D2 (NC)
  constexpr int kIssuer = 4 * kWG;              // index of the issuer warp
  extern __shared__ __align__(128) float sm[];
  float* A1sm = sm + L::kA1;     // [32][128][4]  rows 0-63 W, rows 64-127 e^G Q; K-major over keys
  float* Ksm = sm + L::kK;       // [16][128][4]  K^T, K-major over tokens
  float* QKsm = sm + L::kQK;     // [16][128][4]  rows 0-63 zero, rows 64-127 QKd
  float* Ssm = sm + L::kS;       // [32][NC+1][4] S^T, K-major over keys
  float* Usm = sm + L::kU;       // [16][NC+1][4] U^T, K-major over tokens
  float* Upsm = sm + L::kUp;     // [16][NC+1][4] U'^T
  __shared__ __align__(8) uint64_t bars[8];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int dead;
  uint64_t *fullA = &bars[0], *fullK = &bars[1], *fullQK = &bars[2];
  uint64_t *d1 = &bars[3], *d2 = &bars[4], *d3 = &bars[5], *uReady = &bars[6], *sReady = &bars[7];
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  constexpr int SL = 128 / NC;
  const int h = blockIdx.x / SL, col0 = (blockIdx.x % SL) * NC;
  const int rep = P.Hv / P.Hk, kh = h / rep, VW = P.Hv * 128, R = P.a.R;
  const int nch = ws.chunks;

  if (t == 0) {
#pragma unroll
    for (int i = 0; i < 6; ++i) umma::mbar_init(&bars[i], 1);
    umma::mbar_init(uReady, 64 * kWG);
    umma::mbar_init(sReady, 128 * kWG);
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == kIssuer) umma::tmem_alloc(&tmem_slot, kTmemCols);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (dead) return;
    if (!umma::mbar_wait(bar, parity)) { dead = 1; g_gdn_scan_status = 1; }
  };

  if (w == kIssuer) {
    // ------------------------------------------------------------------ issuer: loads and tensor-core work
    if (l == 0) {
      auto load_a = [&](int c) { umma::mbar_expect_tx(fullA, 65536); umma::bulk_load(A1sm, ws.WQ + ((size_t)h * nch + c) * 16384, 65536, fullA); };
      auto load_k = [&](int c) { umma::mbar_expect_tx(fullK, 32768); umma::bulk_load(Ksm, ws.Kt + ((size_t)kh * nch + c) * 8192, 32768, fullK); };
      auto load_qk = [&](int c) { umma::mbar_expect_tx(fullQK, 32768); umma::bulk_load(QKsm, ws.QKp + ((size_t)h * nch + c) * 8192, 32768, fullQK); };
      load_a(0); load_k(0); load_qk(0);
      constexpr uint32_t idesc = umma::idesc_tf32(128, NC, false, false);
      // descriptors of the first K step; a step of 8 along K advances the start address by 2 planes (16-byte units)
      const uint64_t dA = umma::desc_kmajor(A1sm, 128, 0), dK = umma::desc_kmajor(Ksm, 128, 0), dQK = umma::desc_kmajor(QKsm, 128, 0);
      const uint64_t dS = umma::desc_kmajor_padded(Ssm, NCP, 0), dU = umma::desc_kmajor_padded(Usm, NCP, 0);
      const uint64_t dUp = umma::desc_kmajor_padded(Upsm, NCP, 0);
      for (int c = 0; c < nch; ++c) {
        const int b = c & 1;
        const uint32_t acc1 = tm + b * NC;
        wait(sReady, b);
        wait(fullA, b);
        umma::fence_after_sync();
#pragma unroll
        for (int s8 = 0; s8 < 16; ++s8) umma::mma_tf32_ss(acc1, dA + (uint64_t)(s8 * 256), dS + (uint64_t)(s8 * 2 * NCP), idesc, s8 > 0);
        umma::commit(d1);
        wait(uReady, b);
        wait(fullK, b);
        umma::fence_after_sync();
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ss(tm + 2 * NC, dK + (uint64_t)(s8 * 256), dUp + (uint64_t)(s8 * 2 * NCP), idesc, s8 > 0);
        umma::commit(d2);
        wait(fullQK, b);
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ss(acc1, dQK + (uint64_t)(s8 * 256), dU + (uint64_t)(s8 * 2 * NCP), idesc, 1u);
        umma::commit(d3);
        // refill the buffers whose readers have completed
        if (c + 1 < nch) {
          wait(d1, b); load_a(c + 1);
          wait(d2, b); load_k(c + 1);
          wait(d3, b); load_qk(c + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps (thread = TMEM lane)
    const int wg = w >> 2, key = t & 127, cw = 32 * wg;    // warpgroup wg owns columns [cw, cw + 32) of every accumulator
    const bool tokw = (w & 3) < 2;                         // lanes 0-63 of D1 = W S (tokens); lanes 64-127 = readout
    const int tk = key & 63;
    float S[32];                                           // state row of this key, this warpgroup's columns: fp32 master
    float* st = P.a.state + (size_t)h * 16384 + (size_t)key * 128 + col0 + cw;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 v = *reinterpret_cast<const float4*>(st + j);
      S[j] = v.x; S[j + 1] = v.y; S[j + 2] = v.z; S[j + 3] = v.w;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) Ssm[((key >> 2) * NCP + cw + j) * 4 + (key & 3)] = tf32r(S[j]);
    umma::fence_async_smem();
    mbar_arrive(sReady);

    float ut[32];                                          // Ut row of this thread's token (token warps)
    float Gtok = 0.f, Gend = 0.f;
    auto fetch_rows = [&](int c) {
      const size_t unit = (size_t)h * nch + c;
      Gend = ws.G[unit * 64 + 63];
      if (tokw) {
        Gtok = ws.G[unit * 64 + tk];
        const float* up = ws.Ut + (unit * 64 + tk) * 128 + col0 + cw;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 v = *reinterpret_cast<const float4*>(up + j);
          ut[j] = v.x; ut[j + 1] = v.y; ut[j + 2] = v.z; ut[j + 3] = v.w;
        }
      }
    };
    fetch_rows(0);
    for (int c = 0; c < nch; ++c) {
      const int b = c & 1;
      const float ge = Gend;
      if (tokw) {   // U = Ut - W S, transposed into shared memory (tf32), and U' = e^{G_end - G} U
        const float sc = __expf(ge - Gtok);
        wait(d1, b);
        umma::fence_after_sync();
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, b * NC + cw), p);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float u = ut[j] - p[j];
          const int at = ((tk >> 2) * NCP + cw + j) * 4 + (tk & 3);
          Usm[at] = tf32r(u);
          Upsm[at] = tf32r(sc * u);
        }
        umma::fence_async_smem();
        umma::fence_before_sync();
        mbar_arrive(uReady);
      }
      if (c + 1 < nch) fetch_rows(c + 1);                  // global loads fly while the tensor core works
      wait(d2, b);
      umma::fence_after_sync();
      {   // S <- e^{G_end} S + K^T U'; D1 of this chunk, the only reader of S^T, completed before U
        const float eend = __expf(ge);
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, 2 * NC + cw), p);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          S[j] = fmaf(eend, S[j], p[j]);
          Ssm[((key >> 2) * NCP + cw + j) * 4 + (key & 3)] = tf32r(S[j]);
        }
      }
      umma::fence_async_smem();
      umma::fence_before_sync();
      mbar_arrive(sReady);
      if (!tokw) {   // Y(c) = e^G (Q S) + QKd U on lanes 64-127 of D1; overlaps D1 of the next chunk
        wait(d3, b);
        umma::fence_after_sync();
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, b * NC + cw), p);
        const int row = c * kChunk + tk;
        if (row < R) {
          float* dst = P.yraw + (size_t)row * VW + h * 128 + col0 + cw;
#pragma unroll
          for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(p[j], p[j + 1], p[j + 2], p[j + 3]);
        }
        umma::fence_before_sync();
      }
    }
#pragma unroll
    for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(st + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
  }
  umma::fence_before_sync();
  __syncthreads();
  if (w == kIssuer) umma::tmem_dealloc(tm, kTmemCols);
}

cr_status gdn_chunk_scan_tc_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    CR_CUDA(cudaFuncSetAttribute(gdn_chunk_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem::kBytes));
    configured = true;
  }
  gdn_chunk_scan_tc_kernel<<<g->gdn_vheads * (128 / kNC), 128 * kWG + 32, TcSmem::kBytes, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_scan_tc_kernel");
  return CR_OK;
}

int gdn_scan_status_read() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_gdn_scan_status, sizeof(int));
  return v;
}

}  // namespace cr
