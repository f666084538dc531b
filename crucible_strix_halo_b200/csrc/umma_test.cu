// Self-check of the tcgen05 primitives in umma.cuh: D[128][N] = A B^T with tf32 operands on one CTA, both
// operands K-major.  Exposed as cr_debug_umma_gemm so the GPU tests pin the descriptor conventions the
// production kernels rely on.  (For tf32 the MN-major operand form returns zeros on this hardware, so the
// production kernels write every operand K-major and this check covers that form only.)
#include "common.cuh"
#include "umma.cuh"
#include "tma.cuh"

namespace cr {

// A: [128][K], B: [N][K], D: [128][N].
__global__ void __launch_bounds__(128) umma_test_kernel(const float* A, const float* B, float* D, int K, int N, int* status) {
  extern __shared__ __align__(128) float sm[];
  float* As = sm;
  float* Bs = sm + 128 * K;
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int t = threadIdx.x, w = t >> 5;
  auto stage = [&](float* dst, const float* src, int rows) {   // src [rows][K] -> [K/4][rows][4]
    for (int u = t; u < rows * K / 4; u += 128) {
      const int r = u % rows, kc = u / rows;
      const float4 v = *reinterpret_cast<const float4*>(src + (size_t)r * K + kc * 4);
      *reinterpret_cast<float4*>(dst + (size_t)(kc * rows + r) * 4) = make_float4(tf32r(v.x), tf32r(v.y), tf32r(v.z), tf32r(v.w));
    }
  };
  stage(As, A, 128);
  stage(Bs, B, N);
  if (t == 0) { umma::mbar_init(&bar, 1); umma::mbar_fence_init(); }
  if (w == 0) umma::tmem_alloc(&tmem_slot, 128);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (t == 0) {
    const uint32_t idesc = umma::idesc_tf32(128, N, false, false);
    for (int k0 = 0; k0 < K; k0 += 8) umma::mma_tf32_ss(tmem, umma::desc_kmajor(As, 128, k0), umma::desc_kmajor(Bs, N, k0), idesc, k0 > 0);
    umma::commit(&bar);
  }
  const bool ok = umma::mbar_wait(&bar, 0);
  umma::fence_after_sync();
  for (int c0 = 0; c0 < N; c0 += 32) {
    float v[32];
    umma::tmem_ld32(umma::tmem_addr(tmem, w, c0), v);
    if (ok) {
#pragma unroll
      for (int i = 0; i < 32; ++i) D[(size_t)t * N + c0 + i] = v[i];
    }
  }
  if (!ok && t == 0) *status = 1;          // the wait gave up: report instead of hanging
  umma::fence_before_sync();
  __syncthreads();
  if (w == 0) umma::tmem_dealloc(tmem, 128);
}

// D[128][N] = A[128][K] B[K][N] with fp16 operands (kind::f16): A K-major, B as it lies in memory when the N index
// is contiguous (MN-major: the layout of a V tile, keys x channels).  Shared-memory images, no swizzle, 16-byte units:
//   A: unit (k / 8, row)      at ((k / 8) * 128 + row) * 16
//   B: unit (n / 8, k)        at ((n / 8) * K + k) * 16      core matrix = 8 k x 8 n, n contiguous
// variant 0: B descriptor with LBO = step between core matrices along N, SBO = step along K; variant 1: swapped.
__global__ void __launch_bounds__(128) umma_f16_test_kernel(const __half* A, const __half* B, float* D, int K, int N, int variant, int* status) {
  extern __shared__ __align__(128) unsigned char smb[];
  unsigned char* As = smb;
  unsigned char* Bs = smb + (size_t)128 * K * 2;
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const int t = threadIdx.x, w = t >> 5;
  for (int u = t; u < 128 * K / 8; u += 128) {
    const int row = u % 128, kc = u / 128;
    *reinterpret_cast<uint4*>(As + ((size_t)kc * 128 + row) * 16) = *reinterpret_cast<const uint4*>(A + (size_t)row * K + kc * 8);
  }
  for (int u = t; u < K * N / 8; u += 128) {
    const int nc = u % (N / 8), k = u / (N / 8);
    *reinterpret_cast<uint4*>(Bs + ((size_t)nc * K + k) * 16) = *reinterpret_cast<const uint4*>(B + (size_t)k * N + nc * 8);
  }
  if (t == 0) { umma::mbar_init(&bar, 1); umma::mbar_fence_init(); }
  if (w == 0) umma::tmem_alloc(&tmem_slot, 512);
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const bool a_tmem = (variant & 2) != 0;
  if (a_tmem) {   // A from tensor memory: lane = row, column c of the operand holds elements 2c (low half) and 2c + 1
    for (int c0 = 0; c0 < K / 2; c0 += 16) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i)
        v[i] = c0 + i < K / 2 ? __uint_as_float(*reinterpret_cast<const unsigned*>(A + (size_t)t * K + 2 * (c0 + i))) : 0.f;
      umma::tmem_st16(umma::tmem_addr(tmem, w, 256 + c0), v);
    }
    umma::tmem_st_wait();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
  }
  if (t == 0) {
    const uint32_t idesc = umma::idesc_f16(128, N, false, true);
    const uint32_t step_n = (uint32_t)K * 16u, step_k = 128u;
    for (int k0 = 0; k0 < K; k0 += 16) {
      const uint64_t da = umma::smem_desc(As + (size_t)(k0 / 8) * 128 * 16, 128 * 16, 128);
      const uint64_t db = (variant & 1) == 0 ? umma::smem_desc(Bs + (size_t)k0 * 16, step_n, step_k) : umma::smem_desc(Bs + (size_t)k0 * 16, step_k, step_n);
      if (a_tmem) umma::mma_f16_ts(tmem, tmem + 256 + k0 / 2, db, idesc, k0 > 0);
      else umma::mma_f16_ss(tmem, da, db, idesc, k0 > 0);
    }
    umma::commit(&bar);
  }
  const bool ok = umma::mbar_wait(&bar, 0);
  umma::fence_after_sync();
  for (int c0 = 0; c0 < N; c0 += 32) {
    float v[32];
    umma::tmem_ld32(umma::tmem_addr(tmem, w, c0), v);
    if (ok) {
#pragma unroll
      for (int i = 0; i < 32; ++i) D[(size_t)t * N + c0 + i] = v[i];
    }
  }
  if (!ok && t == 0) *status = 1;
  umma::fence_before_sync();
  __syncthreads();
  if (w == 0) umma::tmem_dealloc(tmem, 512);
}

// One step of the tiled prefill attention without its softmax, as a check of the tensor-map copies and of the
// swizzled descriptors: the K and V rows of 16 four-token blocks arrive through cr::tma::load_box in [4 channel
// groups][64 keys][128 bytes] tiles; S[128][64] = Q K^T reads the K tile K-major with the query tile in tensor
// memory, O[128][256] = Pm V reads the V tile MN-major with Pm[128][64] as an un-swizzled K-major operand.
__global__ void __launch_bounds__(128) umma_kv_step_test_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                                                                int head, const int* blocks, const __half* Q, const __half* Pm, float* S, float* O,
                                                                int* status) {
  extern __shared__ __align__(1024) unsigned char smk[];
  unsigned char* Kt = smk;
  unsigned char* Vt = smk + tma::kTileBytes;
  unsigned char* Ps = smk + 2 * tma::kTileBytes;
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ uint32_t tmem_slot;
  const int t = threadIdx.x, w = t >> 5, l = t & 31;
  if ((umma::smem_u32(smk) & 1023u) != 0) {          // tiles must start on a swizzle-atom boundary
    if (t == 0) *status = 2;
    return;
  }
  if (t == 0) { umma::mbar_init(&bars[0], 1); umma::mbar_init(&bars[1], 1); umma::mbar_fence_init(); }
  if (w == 0) umma::tmem_alloc(&tmem_slot, 512);
  for (int u = t; u < 128 * 8; u += 128) {           // Pm [128][64] -> K-major units (k / 8, row)
    const int row = u % 128, kc = u / 128;
    *reinterpret_cast<uint4*>(Ps + ((size_t)kc * 128 + row) * 16) = *reinterpret_cast<const uint4*>(Pm + (size_t)row * 64 + kc * 8);
  }
  umma::fence_async_smem();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  {   // query tile: lane = row, column c holds channels 2c and 2c + 1
    const uint4* src = reinterpret_cast<const uint4*>(Q + (size_t)t * 256);
#pragma unroll 1
    for (int c8 = 0; c8 < 4; ++c8) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 x = src[c8 * 8 + i];
        v[4 * i] = __uint_as_float(x.x); v[4 * i + 1] = __uint_as_float(x.y); v[4 * i + 2] = __uint_as_float(x.z); v[4 * i + 3] = __uint_as_float(x.w);
      }
      umma::tmem_st32(umma::tmem_addr(tmem, w, 384 + 32 * c8), v);
    }
    umma::tmem_st_wait();
  }
  if (w == 0) {                                      // lane = (entry, K or V): four boxes each
    if (l == 0) umma::mbar_expect_tx(&bars[0], 2 * tma::kTileBytes);
    __syncwarp();
    const int e = l >> 1, blk = blocks[e];
    unsigned char* tile = (l & 1) ? Vt : Kt;
    for (int cg = 0; cg < 4; ++cg) tma::load_box(tile + cg * tma::kGroupBytes + e * 512, (l & 1) ? &vmap : &kmap, cg * 64, head, blk * 4, &bars[0]);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  bool ok = umma::mbar_wait(&bars[0], 0);
  if (t == 0 && ok) {
    constexpr uint32_t idS = umma::idesc_f16(128, 64, false, false), idO = umma::idesc_f16(128, 256, false, true);
    for (int ks = 0; ks < 16; ++ks)
      umma::mma_f16_ts(tmem + 256, tmem + 384 + 8 * ks, tma::desc_sw128(Kt + (ks >> 2) * tma::kGroupBytes + (ks & 3) * 32, 16, 1024), idS, ks > 0);
    for (int kk = 0; kk < 4; ++kk)
      umma::mma_f16_ss(tmem, umma::smem_desc(Ps + (size_t)kk * 2 * 128 * 16, 128 * 16, 128), tma::desc_sw128(Vt + kk * 2048, tma::kGroupBytes, 1024), idO, kk > 0);
    umma::commit(&bars[1]);
  }
  ok = ok && umma::mbar_wait(&bars[1], 0);
  umma::fence_after_sync();
  for (int c0 = 0; c0 < 320; c0 += 32) {
    float v[32];
    umma::tmem_ld32(umma::tmem_addr(tmem, w, c0), v);
    if (ok) {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (c0 < 256) O[(size_t)t * 256 + c0 + i] = v[i];
        else S[(size_t)t * 64 + c0 - 256 + i] = v[i];
      }
    }
  }
  if (!ok && t == 0) *status = 1;
  umma::fence_before_sync();
  __syncthreads();
  if (w == 0) umma::tmem_dealloc(tmem, 512);
}

CR_DEFINE_STATUS_WORD(debug_wait)

// One CTA of 32 threads: lane 0 waits on an mbarrier that nothing completes.  No copy and no tensor-core work is
// pending, so when the wait runs out the kernel simply reports and ends.
__global__ void __launch_bounds__(32) debug_wait_kernel(int* status, unsigned long long max_ns) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) { umma::mbar_init(&bar, 1); umma::mbar_fence_init(); }
  __syncwarp();
  if (threadIdx.x == 0 && !umma::mbar_wait_timed(&bar, 0, nullptr, max_ns)) {
    *status = 1;
    g_debug_wait_status = 1;
  }
}

}  // namespace cr

extern "C" cr_status cr_debug_wait_timeout(int* status, unsigned max_us, void* stream) {
  using namespace cr;
  CR_REQUIRE(status && max_us >= 1 && max_us <= 100000, "cr_debug_wait_timeout: need a status word and 1..100000 us");
  use_stream((cudaStream_t)stream);
  debug_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (unsigned long long)max_us * 1000ull);
  CR_LAUNCH_CHECK("debug_wait_kernel");
  return CR_OK;
}

extern "C" cr_status cr_debug_umma_f16_gemm(const uint16_t* A, const uint16_t* B, float* D, int K, int N, int variant, int* status, void* stream) {
  using namespace cr;
  CR_REQUIRE(A && B && D && status, "cr_debug_umma_f16_gemm: null buffer");
  CR_REQUIRE(K >= 16 && K % 16 == 0 && K <= 128 && N >= 32 && N % 32 == 0 && N <= 256, "cr_debug_umma_f16_gemm: K in 16..128 step 16, N in 32..256 step 32");
  CR_REQUIRE(variant >= 0 && variant <= 3, "cr_debug_umma_f16_gemm: variant 0..3");
  const size_t smem = (size_t)(128 + N) * K * 2;
  CR_CUDA(cudaFuncSetAttribute(umma_f16_test_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  use_stream((cudaStream_t)stream);
  umma_f16_test_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(reinterpret_cast<const __half*>(A), reinterpret_cast<const __half*>(B), D, K, N, variant, status);
  CR_LAUNCH_CHECK("umma_f16_test_kernel");
  return CR_OK;
}

extern "C" cr_status cr_debug_umma_kv_step(const uint16_t* k_cache, const uint16_t* v_cache, int kv_heads, int rows, int head, const int* blocks,
                                           const uint16_t* Q, const uint16_t* Pm, float* S, float* O, int* status, void* stream) {
  using namespace cr;
  CR_REQUIRE(k_cache && v_cache && blocks && Q && Pm && S && O && status, "cr_debug_umma_kv_step: null buffer");
  CR_REQUIRE(kv_heads >= 1 && head >= 0 && head < kv_heads && rows >= 1, "cr_debug_umma_kv_step: bad head or row count");
  CUtensorMap kmap, vmap;
  if (cr_status s = tma::kv_map(&kmap, k_cache, kv_heads, rows)) return s;
  if (cr_status s = tma::kv_map(&vmap, v_cache, kv_heads, rows)) return s;
  const size_t smem = 2 * tma::kTileBytes + 128 * 64 * 2;
  CR_CUDA(cudaFuncSetAttribute(umma_kv_step_test_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  use_stream((cudaStream_t)stream);
  umma_kv_step_test_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(kmap, vmap, head, blocks, reinterpret_cast<const __half*>(Q),
                                                                   reinterpret_cast<const __half*>(Pm), S, O, status);
  CR_LAUNCH_CHECK("umma_kv_step_test_kernel");
  return CR_OK;
}

extern "C" cr_status cr_debug_umma_gemm(const float* A, const float* B, float* D, int K, int N, int* status, void* stream) {
  using namespace cr;
  CR_REQUIRE(A && B && D && status, "cr_debug_umma_gemm: null buffer");
  CR_REQUIRE(K >= 8 && K % 8 == 0 && K <= 128 && N >= 32 && N % 32 == 0 && N <= 128, "cr_debug_umma_gemm: K in 8..128 step 8, N in 32..128 step 32");
  const size_t smem = (size_t)(128 + N) * K * sizeof(float);
  CR_CUDA(cudaFuncSetAttribute(umma_test_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  use_stream((cudaStream_t)stream);
  umma_test_kernel<<<1, 128, smem, (cudaStream_t)stream>>>(A, B, D, K, N, status);
  CR_LAUNCH_CHECK("umma_test_kernel");
  return CR_OK;
}
