// gdn_chunk_scan_tc_kernel: the sequential part of the chunk-64 WY scan on tcgen05 tensor cores, with the
// recurrent operands resident in tensor memory.
//
// One CTA per value head.  Everything is kept transposed, so that a lane of tensor memory is one value column
// v of the state and the 128 lanes are the 128 columns of the head:
//   S^T [v][key]   tf32 copy of the state         TMEM columns   0-127   A operand of D1
//   D2  [v][key]   (K'^T U)^T                     TMEM columns 128-255
//   D1  [v][r]     r < 64: (W S)^T, r >= 64: Y^T  TMEM columns 256-383 (even chunks), 384-511 (odd chunks)
//   U^T [v][token] overwrites (W S)^T in place    A operand of D2 and D3
// Per chunk (32 tcgen05.mma of K = 8, A from tensor memory, B a K-major tile in shared memory that the local
// kernel wrote in exactly that layout and one bulk copy brings in):
//   D1 = S^T [W ; e^G Q]^T  (N = 128)   ->  U = Ut - W S, written back to TMEM
//   D2 = U^T K'             (N = 128)   ->  S = e^{G_end} S + D2   (fp32 master in registers, tf32 copy to TMEM)
//        K' = e^{G_end - G} K: the local kernel folds the decay towards the chunk end into the key tile
//   D1[:, 64:] += U^T QKd^T (N = 64)    ->  Y, stored to global memory
// Because an accumulator row and an A-operand row are both "lane v", no epilogue transposes anything and nothing
// recurrent passes through shared memory.  Four compute warpgroups split the columns of every accumulator
// (warp w reaches lanes 32 (w % 4) .. +31, so each warpgroup covers all lanes); the fp32 master state is spread
// the same way (thread = column v, 32 keys).  One issuer warp feeds the tensor core, one loader warp keeps two
// chunks of operand tiles in flight (224 KB of shared memory, two stages).  Warps synchronise only through
// mbarriers.  Every wait is bounded: a wait that gives up raises a status word, after which no thread waits
// again; the kernel runs to its end, frees its tensor memory and returns.
#include "gdn_chunk.cuh"
#include "umma.cuh"

namespace cr {

CR_DEFINE_STATUS_WORD(gdn_scan)

constexpr int kWG = 4;                                    // compute warpgroups
constexpr int kScanThreads = 128 * kWG + 64;              // + issuer warp + loader warp
constexpr int kStageFloats = 16384 + 8192 + 4096;         // [W ; e^G Q] 64 KB, K^T 32 KB, QKd 16 KB
constexpr size_t kScanSmem = (size_t)2 * kStageFloats * sizeof(float) + 128;
constexpr uint32_t kColS = 0, kColD2 = 128, kColD1 = 256;   // D1 of chunk c at kColD1 + 128 (c & 1)

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(kScanThreads, 1) gdn_chunk_scan_tc_kernel(GdnPrefillParams P, ChunkWs ws) {
  extern __shared__ __align__(128) float sm[];
  __shared__ __align__(8) uint64_t bars[12];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int dead;
  uint64_t* full = &bars[0];                               // one per stage: all three tiles of a chunk
  uint64_t *d1 = &bars[4], *d2 = &bars[5], *d3 = &bars[6];
  uint64_t *uReady = &bars[8], *sReady = &bars[9];
  uint64_t* empty = &bars[10];                             // one per stage: every MMA that read the stage has completed
  uint64_t* yDone = &bars[2];                              // one per D1 accumulator
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  constexpr int kIssuer = 4 * kWG, kLoader = kIssuer + 1;
  const int h = blockIdx.x, VW = P.Hv * 128, R = P.a.R;
  const int nch = ws.chunks;

  if (t == 0) {
    umma::mbar_init(&full[0], 1);
    umma::mbar_init(&full[1], 1);
    umma::mbar_init(d1, 1);
    umma::mbar_init(d2, 1);
    umma::mbar_init(d3, 1);
    umma::mbar_init(&empty[0], 1);
    umma::mbar_init(&empty[1], 1);
    umma::mbar_init(uReady, 4 * kWG);                      // one arrival per compute warp
    umma::mbar_init(sReady, 4 * kWG);
    umma::mbar_init(&yDone[0], 4 * kWG);
    umma::mbar_init(&yDone[1], 4 * kWG);
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == kIssuer) umma::tmem_alloc(&tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  bool gave_up = false;                                    // a thread that gave up once does not wait again
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (gave_up) return;
    if (!umma::mbar_wait_timed(bar, parity, &dead)) { gave_up = true; dead = 1; g_gdn_scan_status = 1; }
  };
  // Compute warps: lane 0 polls and lane 0 arrives, both relaxed: what the warps exchange lives in tensor memory
  // and is ordered by tcgen05.wait / tcgen05.fence, while an acquiring wait or a releasing arrive would also wait
  // for the thread's prefetches of the next chunk and for its stores of Y, and did (1000 to 2500 cycles a chunk).
  auto warp_wait = [&](uint64_t* bar, uint32_t parity) {
    if (l == 0 && !gave_up && !umma::mbar_wait_timed<true>(bar, parity, &dead)) { gave_up = true; dead = 1; g_gdn_scan_status = 1; }
    __syncwarp();
    umma::fence_after_sync();
  };
  auto warp_arrive = [&](uint64_t* bar) {
    umma::fence_before_sync();
    __syncwarp();
    if (l == 0) umma::mbar_arrive_relaxed(bar);
  };

  if (w == kLoader) {
    // ------------------------------------------------------------------ loader: two chunks of tiles in flight
    if (l == 0) {
      auto load = [&](int c) {
        const int s = c & 1;
        float* A1s = sm + s * kStageFloats;
        const float* a = ws.WQ + ((size_t)h * nch + c) * 16384;
        umma::mbar_expect_tx(&full[s], kStageFloats * 4);
        umma::bulk_load(A1s, a, 32768, &full[s]);
        umma::bulk_load(A1s + 8192, a + 8192, 32768, &full[s]);
        umma::bulk_load(A1s + 16384, ws.Kt + ((size_t)h * nch + c) * 8192, 32768, &full[s]);
        umma::bulk_load(A1s + 24576, ws.QKp + ((size_t)h * nch + c) * 4096, 16384, &full[s]);
      };
      // The tiles of a chunk are asked into L2 kLead chunks before their copy to shared memory is issued, and the
      // rows of Ut that the compute threads read themselves one chunk before they are read.
      constexpr int kLead = 2;
      auto prefetch = [&](int c) {
        if (c >= nch) return;
        const size_t unit = (size_t)h * nch + c;
        umma::bulk_prefetch_l2(ws.WQ + unit * 16384, 65536);
        umma::bulk_prefetch_l2(ws.Kt + unit * 8192, 32768);
        umma::bulk_prefetch_l2(ws.QKp + unit * 4096, 16384);
        umma::bulk_prefetch_l2(ws.Ut + unit * 8192, 32768);
      };
      for (int c = 0; c < 2 + kLead; ++c) prefetch(c);
      load(0);
      if (nch > 1) load(1);
      // The stage of chunk c is free once every MMA of chunk c has completed.  Each stage has its own barrier, which
      // completes once per use of the stage and cannot complete again before this warp has refilled the stage: a
      // loader that falls behind never sees a phase it was not waiting for.
      for (int c = 0; c + 2 < nch; ++c) {
        wait(&empty[c & 1], (c >> 1) & 1);
        if (gave_up || dead) break;                        // no more copies once any wait has run out
        load(c + 2);
        prefetch(c + 2 + kLead);
      }
    }
  } else if (w == kIssuer) {
    // ------------------------------------------------------------------ issuer: tensor-core work
    if (l == 0) {
      constexpr uint32_t idesc128 = umma::idesc_tf32(128, 128, false, false), idesc64 = umma::idesc_tf32(128, 64, false, false);
      for (int c = 0; c < nch; ++c) {
        const int b = c & 1, s = c & 1, ph = (c >> 1) & 1;
        const float* A1s = sm + s * kStageFloats;
        // a step of 8 along K advances a descriptor's start address by two planes (16-byte units)
        const uint64_t dA = umma::desc_kmajor(A1s, 128, 0), dK = umma::desc_kmajor(A1s + 16384, 128, 0);
        const uint64_t dQK = umma::desc_kmajor(A1s + 24576, 64, 0);
        const uint32_t cD1 = kColD1 + 128 * b;
        if (c == 0) wait(&full[s], ph);                    // later chunks: waited for at the end of the previous one
        wait(sReady, b);
        if (gave_up || dead) break;                        // no more tensor-core work once any wait has run out
        umma::fence_after_sync();
#pragma unroll
        for (int s8 = 0; s8 < 16; ++s8) umma::mma_tf32_ts(tm + cD1, tm + kColS + 8 * s8, dA + (uint64_t)(s8 * 256), idesc128, s8 > 0);
        umma::commit(d1);
        wait(uReady, b);
        if (gave_up || dead) break;
        umma::fence_after_sync();
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ts(tm + kColD2, tm + cD1 + 8 * s8, dK + (uint64_t)(s8 * 256), idesc128, s8 > 0);
        umma::commit(d2);
#pragma unroll
        for (int s8 = 0; s8 < 8; ++s8) umma::mma_tf32_ts(tm + cD1 + 64, tm + cD1 + 8 * s8, dQK + (uint64_t)(s8 * 128), idesc64, 1u);
        umma::commit(d3);
        umma::commit(&empty[s]);
        if (c + 1 < nch) {   // off the chain: the next tiles arrive early, and Y of chunk c - 1 left its accumulator long ago
          wait(&full[(c + 1) & 1], ((c + 1) >> 1) & 1);
          if (c > 0) wait(&yDone[(c + 1) & 1], (((c + 1) >> 1) - 1) & 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps (thread = TMEM lane = column v)
    const int wg = w >> 2, v = t & 127;
    float S[32];                                           // state column v, keys 32 wg .. +31: fp32 master
    float* st = P.a.state + (size_t)h * 16384 + (size_t)(32 * wg) * 128 + v;
#pragma unroll
    for (int j = 0; j < 32; ++j) S[j] = st[j * 128];
    {
      float r[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = tf32r(S[j]);
      umma::tmem_st32(umma::tmem_addr(tm, w, kColS + 32 * wg), r);
      umma::tmem_st_wait();
    }
    warp_arrive(sReady);

    float ut[16];                                          // Ut of column v, tokens 16 wg .. +15
    float Gend = 0.f;
    auto fetch_rows = [&](int c) {
      const size_t unit = (size_t)h * nch + c;
      Gend = ws.G[unit * 64 + 63];
      const float* up = ws.Ut + unit * 8192 + (size_t)wg * 2048 + v * 4;   // [token / 16][(token % 16) / 4][v][token % 4]
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 x = *reinterpret_cast<const float4*>(up + j * 128);
        ut[j] = x.x; ut[j + 1] = x.y; ut[j + 2] = x.z; ut[j + 3] = x.w;
      }
    };
    fetch_rows(0);
    for (int c = 0; c < nch; ++c) {
      const int b = c & 1;
      const uint32_t cD1 = kColD1 + 128 * b;
      const float ge = Gend;
      warp_wait(d1, b);
      {   // U = Ut - W S, written over W S in tensor memory: the A operand of D2 and D3
        float p[16];
        umma::tmem_ld16(umma::tmem_addr(tm, w, cD1 + 16 * wg), p);
#pragma unroll
        for (int j = 0; j < 16; ++j) p[j] = tf32r(ut[j] - p[j]);
        umma::tmem_st16(umma::tmem_addr(tm, w, cD1 + 16 * wg), p);
        umma::tmem_st_wait();
      }
      warp_arrive(uReady);
      if (c + 1 < nch) fetch_rows(c + 1);                  // global loads fly while the tensor core works
      warp_wait(d2, b);
      {   // S <- e^{G_end} S + K^T U'; every MMA that read the old S^T completed before D2 did
        const float eend = __expf(ge);
        float p[32];
        umma::tmem_ld32(umma::tmem_addr(tm, w, kColD2 + 32 * wg), p);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          S[j] = fmaf(eend, S[j], p[j]);
          p[j] = tf32r(S[j]);
        }
        umma::tmem_st32(umma::tmem_addr(tm, w, kColS + 32 * wg), p);
        umma::tmem_st_wait();
      }
      warp_arrive(sReady);                                 // S^T is current
      warp_wait(d3, b);
      {   // Y^T of tokens 16 wg .. +15: a warp stores 32 consecutive columns of one row
        float p[16];
        umma::tmem_ld16(umma::tmem_addr(tm, w, cD1 + 64 + 16 * wg), p);
        float* dst = P.yraw + (size_t)(c * kChunk + 16 * wg) * VW + h * 128 + v;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c * kChunk + 16 * wg + j < R) dst[(size_t)j * VW] = p[j];
      }
      warp_arrive(&yDone[b]);                                  // this D1 accumulator may be overwritten (by chunk c + 2)
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) st[j * 128] = S[j];
  }
  umma::fence_before_sync();
  __syncthreads();
  if (w == kIssuer) umma::tmem_dealloc(tm, 512);
}

cr_status gdn_chunk_scan_tc_launch(const cr_geometry* g, const GdnPrefillParams& P, const ChunkWs& ws, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (cr_status st = once_per_device(configured, [] {
        CR_CUDA(cudaFuncSetAttribute(gdn_chunk_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScanSmem));
        return CR_OK;
      })) return st;
  gdn_chunk_scan_tc_kernel<<<g->gdn_vheads, kScanThreads, kScanSmem, stream>>>(P, ws);
  CR_LAUNCH_CHECK("gdn_chunk_scan_tc_kernel");
  return CR_OK;
}

}  // namespace cr
