// cr_qsa_attn_static: the decode / verify attention of cr_qsa_attn for callers that cannot hand over scratch
// memory.  Some hosts of this library run where device allocation is off the table once the engine is up: a
// serving process that has already given every spare byte of HBM to KV caches and must not fragment or fail on a
// late cudaMalloc, a plugin loaded into someone else's process without access to that process's allocator, or
// code running while a stream capture is open on another thread, where an allocation would invalidate the
// capture.  For them the split-KV partials live in a fixed array that is part of the library image.
//
// Limits and sharing: the array holds CR_STATIC_ATTN_MAX_ROW_HEADS (row, head) pairs x 32 splits x 258 floats
// (8.45 MB) and every GPU that loads the library keeps it until the process exits.  All calls on a device share
// it, so two calls whose kernels can overlap on the GPU (different streams, no ordering between them) race.
// Nothing in it needs to start at zero: every split record a merge reads is written by the same call first.
// The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that first call
// before any stream capture begins.
#include <climits>
#include <mutex>
#include "qsa.cuh"

namespace cr {

constexpr size_t kStaticFloats = (size_t)CR_STATIC_ATTN_MAX_ROW_HEADS * CR_QSA_SPLITS * CR_QSA_PART;
static __device__ __align__(256) float g_static_partials[kStaticFloats];

constexpr int kMaxDevices = 64;
static float* g_static_ptr[kMaxDevices];     // device address of g_static_partials, per device
static std::mutex g_static_mutex;

// Host code cannot use g_static_partials as a pointer: the name is a host-side stand-in.  The address a kernel
// needs comes from cudaGetSymbolAddress, once per device, with that device current.
static cr_status static_partials(float** out) {
  int dev = -1;
  CR_CUDA(cudaGetDevice(&dev));
  CR_REQUIRE(dev >= 0 && dev < kMaxDevices, "cr_qsa_attn_static: device ordinal %d is beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    CR_CUDA(cudaGetSymbolAddress(&p, g_static_partials));
    g_static_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_static_ptr[dev];
  return CR_OK;
}

}  // namespace cr

extern "C" cr_status cr_qsa_attn_static(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cr_out_format fmt,
                                        void* stream) {
  using namespace cr;
  if (cr_status s = qsa_validate(g, spans, n_spans, CR_MAX_STEP_ROWS, "cr_qsa_attn_static")) return s;
  CR_REQUIRE(fmt == CR_OUT_RAW_F32 || fmt == CR_OUT_RAW_BF16 || fmt == CR_OUT_EXL3_WHT, "cr_qsa_attn_static: bad output format");
  size_t rows = 0;
  for (int s = 0; s < n_spans; ++s) {
    CR_REQUIRE(spans[s].out, "cr_qsa_attn_static: span %d has no output buffer", s);
    CR_REQUIRE(fmt != CR_OUT_EXL3_WHT || spans[s].suh_o, "cr_qsa_attn_static: span %d needs suh_o for the EXL3 output", s);
    CR_REQUIRE(fmt == CR_OUT_EXL3_WHT || spans[s].pack_rows == 0, "cr_qsa_attn_static: packed layout only with the EXL3 output");
    rows += (size_t)spans[s].R;
  }
  CR_REQUIRE(rows * (size_t)g->q_heads <= (size_t)CR_STATIC_ATTN_MAX_ROW_HEADS,
             "cr_qsa_attn_static: %zu rows x %d heads exceed the built-in scratch of %d (row, head) pairs; use cr_qsa_attn with caller scratch",
             rows, g->q_heads, CR_STATIC_ATTN_MAX_ROW_HEADS);
  float* partials = nullptr;
  if (cr_status s = static_partials(&partials)) return s;
  if (cr_status s = qsa_attn_launch(g, spans, n_spans, partials, CR_QSA_SPLITS, 0, INT_MAX, (cudaStream_t)stream)) return s;
  return qsa_merge_launch(g, spans, n_spans, partials, CR_QSA_SPLITS, false, nullptr, fmt, (cudaStream_t)stream);
}
