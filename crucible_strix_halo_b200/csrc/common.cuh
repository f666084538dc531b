// Shared device/host helpers of the sm_100a attention kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include "../../include/crucible_attn.h"

#include <atomic>
#include <mutex>
#include <utility>
#include <cstdlib>

namespace cr {

// ---- programmatic dependent launch ---------------------------------------------------------------------------
// A kernel launched with launch_pdl may be scheduled while the kernel before it on the stream is still running;
// it calls pdl_wait() before it touches anything that kernel (or any earlier one) wrote, which returns once the
// earlier grid has completed and its writes are visible.  Every kernel of a chain calls pdl_release() at its top so
// that its successor's launch latency and CTA placement overlap its own execution.  Both are no-ops in a kernel
// launched the plain way.  cr_options.pdl = 0 turns the launch attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
// Work that belongs to a device rather than to the process (function attributes such as the dynamic shared-memory
// limit): `fn` runs once per device, under a lock, and the device is marked done only after it returned CR_OK, so a
// second host thread cannot launch before the attributes are set and a failed attempt is retried by the next call.
struct PerDeviceOnce {
  std::mutex mu;
  std::atomic<bool> done[64] = {};
};
template <class F>
inline cr_status once_per_device(PerDeviceOnce& f, F&& fn) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fn();
  if (f.done[dev].load(std::memory_order_acquire)) return CR_OK;
  std::lock_guard<std::mutex> lock(f.mu);
  if (f.done[dev].load(std::memory_order_relaxed)) return CR_OK;
  const cr_status s = fn();
  if (s == CR_OK) f.done[dev].store(true, std::memory_order_release);
  return s;
}
// Process-wide tuning options (cr_get_options / cr_set_options); nothing is read from the environment.
const cr_options& options();
inline bool pdl_enabled() { return options().pdl != 0; }
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}


constexpr float kEps = 1e-6f;                         // every norm epsilon
constexpr float kInvSqrt128 = 0.08838834764831845f;   // 1/sqrt(128)
constexpr float kHadNorm = 0.088388347648f;           // ExLlamaV3's 1/sqrt(128) constant
constexpr int kGdnPartChunksDefault = 111;               // chunks per internal part of a long GDN prefill call
constexpr int kMaxSpans = 32;                         // spans per launch (they travel as kernel parameters: 4 KB in all)

// ---- host-side error plumbing -------------------------------------------------------------------
void set_error(const char* fmt, ...);
cr_status cuda_fail(cudaError_t e, const char* what);
void count_launch(const char* name);
bool profiling();                        // stage timing is on: launchers keep everything on one stream
void use_stream(cudaStream_t stream);   // the stream the following launches go to (for stage timing)
#define CR_CUDA(call)                                                          \
  do {                                                                         \
    cudaError_t e_ = (call);                                                   \
    if (e_ != cudaSuccess) return ::cr::cuda_fail(e_, #call);                  \
  } while (0)
#define CR_REQUIRE(cond, ...)                                                  \
  do {                                                                         \
    if (!(cond)) { ::cr::set_error(__VA_ARGS__); return CR_ERR_INVALID; }      \
  } while (0)
#define CR_LAUNCH_CHECK(name)                                                  \
  do {                                                                         \
    cudaError_t e_ = cudaGetLastError();                                       \
    if (e_ != cudaSuccess) return ::cr::cuda_fail(e_, name);                   \
    ::cr::count_launch(name);                                                  \
  } while (0)

cr_status check_geometry(const cr_geometry* g);

// A device status word of one translation unit with its host-side reader and clearer (both synchronise).  A bounded
// wait that gives up stores 1 in it; api.cu assembles the words of all units into cr_device_status().
#define CR_DEFINE_STATUS_WORD(name)                                                                        \
  __device__ int g_##name##_status = 0;                                                                    \
  int name##_status_read() { int v = 0; cudaMemcpyFromSymbol(&v, g_##name##_status, sizeof(int)); return v; } \
  void name##_status_clear() { const int v = 0; cudaMemcpyToSymbol(g_##name##_status, &v, sizeof(int)); }
int gdn_scan_status_read();   void gdn_scan_status_clear();
int qsa_score_status_read();  void qsa_score_status_clear();
int qsa_flash_status_read();  void qsa_flash_status_clear();
int debug_wait_status_read(); void debug_wait_status_clear();
int proj_gemm_status_read();  void proj_gemm_status_clear();

// ---- device math ---------------------------------------------------------------------------------
__device__ __forceinline__ float round_h(float v) { return __half2float(__float2half_rn(v)); }
// __fdividef: reciprocal + multiply (2 ulp), instead of the IEEE division sequence; the denominators lie in [1, inf].
__device__ __forceinline__ float sigmoidf_(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }
__device__ __forceinline__ float siluf_(float v) { return __fdividef(v, 1.f + __expf(-v)); }
__device__ __forceinline__ float bf16_bits_to_float(uint16_t u) { return __uint_as_float((uint32_t)u << 16); }

// Round to tf32 (10-bit mantissa, nearest, ties away): the tensor-core unit ignores the low 13 bits of an
// fp32 operand, so operands are rounded when they are written.  Integer add + mask gives the same bits as
// cvt.rna.tf32.f32 for every finite value (and keeps infinities); the cvt instruction itself issues at the
// rate of the special-function unit (about one warp instruction per 7 cycles per scheduler, measured), which
// made it the longest part of every epilogue that used it.
__device__ __forceinline__ float tf32r(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}

// Sum over a block of NT threads; red holds NT/32 floats; every thread gets the same fixed-order result.
template <int NT>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NT / 32; ++i) t += red[i];
  return t;
}

// In-warp natural-order Sylvester-Hadamard of 128 values, lane l holding elements 4l..4l+3; unnormalised.
__device__ __forceinline__ void wht128(float v[4]) {
  const int lane = threadIdx.x & 31;
  const float a0 = v[0] + v[1], a1 = v[0] - v[1], a2 = v[2] + v[3], a3 = v[2] - v[3];
  v[0] = a0 + a2; v[1] = a1 + a3; v[2] = a0 - a2; v[3] = a1 - a3;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? (o - v[i]) : (v[i] + o);
    }
  }
}

// Out-projection input index: row-major [R][width], or (pack_rows > 0) the packed GEMM layout
// [width/16][pack_rows][16] at row pack_off + r.
__host__ __device__ __forceinline__ size_t out_index(int r, int c, int width, int pack_rows, int pack_off) {
  return pack_rows ? ((size_t)(c >> 4) * pack_rows + pack_off + r) * 16 + (c & 15) : (size_t)r * width + c;
}

// Loads element i of a row buffer that is fp32 or bf16.
template <bool BF16>
__device__ __forceinline__ float load_in(const void* p, long long i) {
  if constexpr (BF16) return bf16_bits_to_float(reinterpret_cast<const uint16_t*>(p)[i]);
  else return reinterpret_cast<const float*>(p)[i];
}

// Split-half partial RoPE angle terms for pair j (< 32) at position p with a 64-float table.
__device__ __forceinline__ void rope_cs(const float* rope, int j, int p, float& c, float& s) {
  const float ang = (float)p * rope[j], m = rope[32];
  c = cosf(ang) * m;
  s = sinf(ang) * m;
}

__host__ __device__ __forceinline__ size_t pool_offset(int b, int d) {
  return (size_t)(b >> 5) * 4096 + (size_t)d * 32 + (b & 31);
}
__host__ __device__ __forceinline__ size_t raw_offset(int slots, int position, int dim) {
  return (size_t)(slots ? position % slots : position) * 128 + dim;
}

}  // namespace cr
