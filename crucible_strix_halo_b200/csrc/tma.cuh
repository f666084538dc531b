// Tensor-map (TMA) copies of K / V cache rows into 128-byte-swizzled shared-memory tiles that tcgen05.mma reads
// directly.  A cache is fp16 [position][kv head][256]; a box is (64 channels, 1 head, 4 positions) = one 4-token
// block of one 64-channel group = four 128-byte rows, which land as rows 4 e .. 4 e + 3 of a [64 keys][128 bytes]
// tile (entry e of a 16-entry step).  The 128-byte swizzle is a function of the shared-memory address, so a box
// written at a 512-byte offset fills the upper half of an 8-row swizzle atom correctly; tiles are 1,024-byte
// aligned.  The same image is the K-major operand [key][channel] of S = Q K^T and the MN-major operand of O += P V.
// Positions past the tensor's extent are filled with zeros by the copy engine.  No multicast anywhere.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "common.cuh"
#include "umma.cuh"

namespace cr {
namespace tma {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up once (the library does not link libcuda).
inline cr_status encoder(EncodeFn* out) {
  static EncodeFn fn = nullptr;
  static std::mutex lock;
  std::lock_guard<std::mutex> guard(lock);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res;
    CR_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res));
    if (res != cudaDriverEntryPointSuccess || !p) {
      set_error("the driver has no cuTensorMapEncodeTiled");
      return CR_ERR_UNSUPPORTED;
    }
    fn = reinterpret_cast<EncodeFn>(p);
  }
  *out = fn;
  return CR_OK;
}

// Map of a K or V cache holding `rows` positions: dims (256 channels, kv heads, positions), box (64, 1, 4),
// 128-byte swizzle.
inline cr_status kv_map(CUtensorMap* map, const void* cache, int kv_heads, long long rows) {
  EncodeFn enc;
  if (cr_status s = encoder(&enc)) return s;
  const cuuint64_t dims[3] = {256, (cuuint64_t)kv_heads, (cuuint64_t)rows};
  const cuuint64_t strides[2] = {512, (cuuint64_t)kv_heads * 512};
  const cuuint32_t box[3] = {64, 1, 4}, unit[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(cache), dims, strides, box, unit,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d", (int)r);
    return CR_ERR_CUDA;
  }
  return CR_OK;
}

// One box of the map to shared memory; completes 512 bytes on the mbarrier.  c0 (channels) is a multiple of 64.
__device__ __forceinline__ void load_box(void* dst, const CUtensorMap* map, int c0, int head, int pos, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
                   umma::smem_u32(dst)),
               "l"(map), "r"(c0), "r"(head), "r"(pos), "r"(umma::smem_u32(bar))
               : "memory");
}

// Shared-memory descriptor of a 128-byte-swizzled tile (rows of 128 bytes, atoms of 8 rows = 1,024 bytes).
// K-major use: sbo = step between 8-row atoms, lbo unused.  MN-major use: lbo = step between 64-element groups
// along the contiguous index, sbo = step between 8-row atoms along K.
__device__ __forceinline__ uint64_t desc_sw128(const void* base, uint32_t lbo, uint32_t sbo) {
  return umma::smem_desc(base, lbo, sbo) | ((uint64_t)2 << 61);
}

constexpr int kTileBytes = 64 * 256 * 2;       // K or V of one 64-key step: [4 channel groups][64 keys][128 bytes]
constexpr int kGroupBytes = 64 * 128;          // one channel group of the tile

}  // namespace tma
}  // namespace cr
