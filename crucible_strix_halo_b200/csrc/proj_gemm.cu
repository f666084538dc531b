// Projection GEMM either side of the attention core for sm_100a: Y[R][N] = X[R][K] W[N][K]^T with bf16 operands and
// fp32 accumulation, the columns of Y scattered straight into the buffers the core reads (qkv / z / gate logits of a
// GDN layer, q / k / v / idx of a QSA layer) or, on the way out, the hidden rows.  The role of the input and output
// GEMM groups of a prefill layer (PrefillLayer::input / ::output, engine/runtime/prefill_engine.inc:261-270, :362)
// for plain bf16 weights; the reference's EXL3 trellis decoding is not part of this path.
//
// One persistent CTA per SM, six warps:
//   warp 0    TMA producer: per 64-channel K step one 128 x 64 box of X and one 256 x 64 box of W into a four-stage
//             ring of 128-byte-swizzled tiles (48 KB per stage), one mbarrier per stage;
//   warp 1    issuer: four tcgen05.mma kind::f16 (M 128, N 256, K 16) per stage into one of two 256-column TMEM
//             accumulators; a commit frees the stage, a last commit hands the accumulator to the epilogue;
//   warps 2-5 epilogue: tcgen05.ld of the warp's 32 lanes, conversion, row stores into the output that owns the
//             32-column chunk; the other accumulator is filled meanwhile.
// Tiles are walked in bands of sixteen 256-column tiles, rows fastest, so a wave of CTAs shares sixteen W tiles and about
// nine X tiles through L2.  Rows and columns past the matrix are zero-filled by the copy engine and masked in the
// epilogue.  Every wait is bounded; a wait that gives up raises bit 4 of the device status word.
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace cr {

CR_DEFINE_STATUS_WORD(proj_gemm)

constexpr int kGM = 128, kGN = 256, kGK = 64, kGStages = 4, kGBand = 16;   // bands of 4 and 8 column tiles measured 4 % and 1.5 % slower
constexpr int kGABytes = kGM * kGK * 2, kGBBytes = kGN * kGK * 2, kGStageBytes = kGABytes + kGBBytes;
constexpr int kGThreads = 192;
constexpr size_t kGSmem = (size_t)kGStages * kGStageBytes + (2 * kGStages + 4) * 8 + 16;
constexpr int kMaxOuts = 6;

struct ProjParams {
  int R, K, N, n_outs;
  void* ptr[kMaxOuts];
  int col0[kMaxOuts], cols[kMaxOuts], ld[kMaxOuts], f32[kMaxOuts];
};

__device__ __forceinline__ void load_box_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                   umma::smem_u32(dst)),
               "l"(map), "r"(c0), "r"(c1), "r"(umma::smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void gemm_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_u32(bar)) : "memory");
}
// Instruction descriptor for kind::f16 with bf16 operands (format 1), fp32 accumulation, both operands K-major.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__global__ void __launch_bounds__(kGThreads, 1) proj_gemm_kernel(const __grid_constant__ ProjParams P, const __grid_constant__ CUtensorMap xmap,
                                                                 const __grid_constant__ CUtensorMap wmap) {
  extern __shared__ __align__(1024) unsigned char sm[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kGStages * kGStageBytes);
  uint64_t *full = bars, *empty = bars + kGStages, *accFull = bars + 2 * kGStages, *accEmpty = bars + 2 * kGStages + 2;
  uint32_t& tmem_slot = *reinterpret_cast<uint32_t*>(bars + 2 * kGStages + 4);
  volatile int& dead = *reinterpret_cast<volatile int*>(&tmem_slot + 1);
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  if ((umma::smem_u32(sm) & 1023u) != 0) {
    if (t == 0) g_proj_gemm_status = 1;
    return;
  }
  const int mt = (P.R + kGM - 1) / kGM, nt = (P.N + kGN - 1) / kGN, kb_n = P.K / kGK;
  const int tiles = mt * nt;
  // tile index -> (row tile, column tile): bands of kGBand column tiles, rows fastest inside a band
  auto tile_at = [&](int i, int& m0, int& n0) {
    const int per_band = mt * kGBand, band = i / per_band, in = i - band * per_band;
    const int width = min(kGBand, nt - band * kGBand);
    m0 = (in / width) * kGM;
    n0 = (band * kGBand + in % width) * kGN;
  };
  if (t == 0) {
    for (int i = 0; i < kGStages; ++i) { umma::mbar_init(&full[i], 1); umma::mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { umma::mbar_init(&accFull[i], 1); umma::mbar_init(&accEmpty[i], 4); }
    umma::mbar_fence_init();
    dead = 0;
  }
  if (w == 1) umma::tmem_alloc(&tmem_slot, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tm = tmem_slot;
  bool gave_up = false;
  auto wait = [&](uint64_t* bar, uint32_t parity) {
    if (gave_up) return;
    if (!umma::mbar_wait_timed(bar, parity, &dead)) { gave_up = true; dead = 1; g_proj_gemm_status = 1; }
  };

  if (w == 0) {
    // ---------------------------------------------------------------- producer
    if (l == 0) {
      int it = 0;
      for (int i = blockIdx.x; i < tiles && !gave_up; i += gridDim.x) {
        int m0, n0;
        tile_at(i, m0, n0);
        for (int kb = 0; kb < kb_n; ++kb, ++it) {
          const int s = it % kGStages;
          if (it >= kGStages) wait(&empty[s], ((it - kGStages) / kGStages) & 1);
          if (gave_up) break;
          unsigned char* st = sm + s * kGStageBytes;
          umma::mbar_expect_tx(&full[s], kGStageBytes);
          load_box_2d(st, &xmap, kb * kGK, m0, &full[s]);
          load_box_2d(st + kGABytes, &wmap, kb * kGK, n0, &full[s]);
        }
      }
    }
  } else if (w == 1) {
    // ---------------------------------------------------------------- issuer
    if (l == 0) {
      constexpr uint32_t idesc = idesc_bf16(kGM, kGN);
      int it = 0, local = 0;
      for (int i = blockIdx.x; i < tiles && !gave_up; i += gridDim.x, ++local) {
        const int acc = local & 1;
        if (local >= 2) wait(&accEmpty[acc], ((local - 2) >> 1) & 1);      // the epilogue has read this accumulator
        umma::fence_after_sync();
        for (int kb = 0; kb < kb_n && !gave_up; ++kb, ++it) {
          const int s = it % kGStages;
          wait(&full[s], (it / kGStages) & 1);
          if (gave_up) break;
          umma::fence_after_sync();
          const unsigned char* st = sm + s * kGStageBytes;
#pragma unroll
          for (int ks = 0; ks < kGK / 16; ++ks)
            umma::mma_f16_ss(tm + acc * kGN, tma::desc_sw128(st + ks * 32, 16, 1024), tma::desc_sw128(st + kGABytes + ks * 32, 16, 1024), idesc,
                             (kb > 0 || ks > 0) ? 1u : 0u);
          umma::commit(&empty[s]);                                          // the stage is free once these MMAs have read it
        }
        if (!gave_up) umma::commit(&accFull[acc]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: warp w owns TMEM lanes 32 (w % 4) .. +31
    const int q = w & 3;
    int local = 0;
    for (int i = blockIdx.x; i < tiles; i += gridDim.x, ++local) {
      int m0, n0;
      tile_at(i, m0, n0);
      const int acc = local & 1;
      if (l == 0) wait(&accFull[acc], (local >> 1) & 1);
      __syncwarp();
      if (dead) break;
      umma::fence_after_sync();
      const int row = m0 + 32 * q + l;
#pragma unroll 1
      for (int c = 0; c < kGN / 32; ++c) {
        float v[32];
        umma::tmem_ld32(umma::tmem_addr(tm, q, acc * kGN + 32 * c), v);     // warp-collective
        const int col = n0 + 32 * c;
        if (row >= P.R || col >= P.N) continue;
        int o = 0;
        while (o < P.n_outs - 1 && col >= P.col0[o] + P.cols[o]) ++o;       // outputs are ordered by column; chunks do not straddle them
        const size_t at = (size_t)row * P.ld[o] + (col - P.col0[o]);
        if (P.f32[o]) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(P.ptr[o]) + at);
#pragma unroll
          for (int k = 0; k < 8; ++k) dst[k] = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(P.ptr[o]) + at);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            unsigned pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[8 * k + 2 * j], v[8 * k + 2 * j + 1]);
              pk[j] = *reinterpret_cast<const unsigned*>(&b2);
            }
            dst[k] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      }
      umma::fence_before_sync();
      __syncwarp();
      if (l == 0) gemm_arrive(&accEmpty[acc]);
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (w == 1) umma::tmem_dealloc(tm, 512);
}

// Row-major bf16 matrix [rows][K] as a tensor map with boxes of box_rows x 64 channels, 128-byte swizzle.
static cr_status map_rows_bf16(CUtensorMap* map, const void* base, long long rows, int K, int box_rows) {
  tma::EncodeFn enc;
  if (cr_status s = tma::encoder(&enc)) return s;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kGK, (cuuint32_t)box_rows}, unit[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, unit, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return CR_ERR_CUDA;
  }
  return CR_OK;
}
}  // namespace cr

extern "C" cr_status cr_proj_gemm(const void* x, const void* w, int R, int K, int N, const cr_proj_out* outs, int n_outs, void* stream_) {
  using namespace cr;
  CR_REQUIRE(x && w && outs, "cr_proj_gemm: null buffer");
  CR_REQUIRE(R >= 1 && N >= 32 && K >= kGK && K % kGK == 0, "cr_proj_gemm: R >= 1, N >= 32, K a multiple of 64 (got R=%d K=%d N=%d)", R, K, N);
  CR_REQUIRE(n_outs >= 1 && n_outs <= kMaxOuts, "cr_proj_gemm: 1..%d outputs", kMaxOuts);
  CR_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0, "cr_proj_gemm: operands must be 16-byte aligned");
  ProjParams P;
  P.R = R; P.K = K; P.N = N; P.n_outs = n_outs;
  int next = 0;
  for (int i = 0; i < n_outs; ++i) {
    const cr_proj_out& o = outs[i];
    CR_REQUIRE(o.ptr && o.col0 == next && o.cols >= 32 && o.cols % 32 == 0, "cr_proj_gemm: output %d must start at column %d and hold a multiple of 32 columns", i, next);
    CR_REQUIRE(o.ld >= o.cols && (o.ld * (o.f32 ? 4 : 2)) % 16 == 0 && ((uintptr_t)o.ptr & 15) == 0, "cr_proj_gemm: output %d: row pitch and base must keep 16-byte alignment", i);
    P.ptr[i] = o.ptr; P.col0[i] = o.col0; P.cols[i] = o.cols; P.ld[i] = o.ld; P.f32[i] = o.f32 ? 1 : 0;
    next += o.cols;
  }
  CR_REQUIRE(next == N, "cr_proj_gemm: the outputs cover %d columns, the product has %d", next, N);
  static PerDeviceOnce configured;
  if (cr_status st = once_per_device(configured, [] {
        CR_CUDA(cudaFuncSetAttribute(proj_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGSmem));
        return CR_OK;
      })) return st;
  CUtensorMap xmap, wmap;
  if (cr_status st = map_rows_bf16(&xmap, x, R, K, kGM)) return st;
  if (cr_status st = map_rows_bf16(&wmap, w, N, K, kGN)) return st;
  int dev = 0, sms = 0;
  CR_CUDA(cudaGetDevice(&dev));
  CR_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int tiles = ((R + kGM - 1) / kGM) * ((N + kGN - 1) / kGN);
  cudaStream_t stream = (cudaStream_t)stream_;
  use_stream(stream);
  proj_gemm_kernel<<<tiles < sms ? tiles : sms, kGThreads, kGSmem, stream>>>(P, xmap, wmap);
  CR_LAUNCH_CHECK("proj_gemm_kernel");
  return CR_OK;
}
