// Snapshot / restore of a sequence's device state: the spans a host lists (fixed GDN state, conv rings, pending rows,
// compact raw rings, the open pool tile; or a whole conversation snapshot) are copied to or from one contiguous buffer
// in span order by ONE kernel per 96 spans, instead of one copy call per span
// (SlotCheckpointIO::Save / Restore, engine/runtime/slot_checkpoint_io.h:49-73; CopySnapshotSpans,
// engine/runtime/snapshot_bytes.h:692-704).  The copy is a grid-stride walk over 16 KB pieces of all spans together, so
// 133 spans of a 48-layer model between 2 KB and 2 MiB fill every SM evenly; each thread issues its four 128-bit
// loads before the first store.  HBM-bound: bytes read + bytes written = 2 x the spans' bytes.
#include "common.cuh"

namespace cr {

constexpr int kCopySpans = 96;                 // spans per launch (the table travels as a kernel parameter)
constexpr int kPieceBytes = 16384;             // 256 threads x 4 x 16 bytes

struct CopyTable {
  const char* src[kCopySpans];
  char* dst[kCopySpans];
  unsigned first[kCopySpans + 1];              // first piece of span i; first[n] = pieces in all
  unsigned bytes16[kCopySpans];                // span length in 16-byte units
  int n;
};

__global__ void __launch_bounds__(256) state_copy_kernel(const __grid_constant__ CopyTable T) {
  __shared__ unsigned first_s[kCopySpans + 1];
  for (int i = threadIdx.x; i <= T.n; i += 256) first_s[i] = T.first[i];
  __syncthreads();
  const unsigned total = first_s[T.n];
  for (unsigned piece = blockIdx.x; piece < total; piece += gridDim.x) {
    int lo = 0, hi = T.n - 1;                  // the span that holds this piece: last i with first[i] <= piece
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (first_s[mid] <= piece) lo = mid; else hi = mid - 1;
    }
    const unsigned unit0 = (piece - first_s[lo]) * (kPieceBytes / 16), units = T.bytes16[lo];
    const uint4* s = reinterpret_cast<const uint4*>(T.src[lo]) + unit0;
    uint4* d = reinterpret_cast<uint4*>(T.dst[lo]) + unit0;
    uint4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const unsigned u = threadIdx.x + 256 * k;
      if (unit0 + u < units) v[k] = __ldcs(s + u);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const unsigned u = threadIdx.x + 256 * k;
      if (unit0 + u < units) __stcs(d + u, v[k]);
    }
  }
}

static cr_status copy_spans(const cr_span* spans, int n, char* buffer, size_t buffer_bytes, bool save, cudaStream_t stream,
                            const char* who) {
  CR_REQUIRE(n >= 0 && (n == 0 || spans), "%s: null span list", who);
  CR_REQUIRE(n == 0 || buffer, "%s: null buffer", who);
  CR_REQUIRE(((uintptr_t)buffer & 15) == 0, "%s: the buffer must be 16-byte aligned", who);
  size_t total = 0;
  for (int i = 0; i < n; ++i) {
    CR_REQUIRE(spans[i].ptr || spans[i].bytes == 0, "%s: span %d is null", who, i);
    CR_REQUIRE(((uintptr_t)spans[i].ptr & 15) == 0 && spans[i].bytes % 16 == 0, "%s: span %d is not a multiple of 16 bytes at a 16-byte boundary",
               who, i);
    CR_REQUIRE(spans[i].bytes / 16 <= 0xffffffffull, "%s: span %d is too long", who, i);
    total += spans[i].bytes;
  }
  CR_REQUIRE(total <= buffer_bytes, "%s: the spans hold %zu bytes, the buffer %zu", who, total, buffer_bytes);
  int sms = 0, dev = 0;
  CR_CUDA(cudaGetDevice(&dev));
  CR_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  size_t offset = 0;
  for (int i0 = 0; i0 < n; i0 += kCopySpans) {
    CopyTable T;
    T.n = 0;
    unsigned pieces = 0;
    for (int i = i0; i < n && T.n < kCopySpans; ++i) {
      if (spans[i].bytes == 0) continue;
      char* flat = buffer + offset;
      T.src[T.n] = save ? static_cast<const char*>(spans[i].ptr) : flat;
      T.dst[T.n] = save ? flat : static_cast<char*>(spans[i].ptr);
      T.first[T.n] = pieces;
      T.bytes16[T.n] = (unsigned)(spans[i].bytes / 16);
      pieces += (unsigned)((spans[i].bytes + kPieceBytes - 1) / kPieceBytes);
      offset += spans[i].bytes;
      ++T.n;
    }
    if (T.n == 0) continue;
    T.first[T.n] = pieces;
    const unsigned grid = pieces < (unsigned)(sms * 8) ? pieces : (unsigned)(sms * 8);
    state_copy_kernel<<<grid, 256, 0, stream>>>(T);
    CR_LAUNCH_CHECK("state_copy_kernel");
  }
  return CR_OK;
}
}  // namespace cr

extern "C" size_t cr_spans_bytes(const cr_span* spans, int n) {
  size_t total = 0;
  for (int i = 0; spans && i < n; ++i) total += spans[i].bytes;
  return total;
}

extern "C" cr_status cr_state_save(const cr_span* spans, int n, void* buffer, size_t buffer_bytes, void* stream) {
  return cr::copy_spans(spans, n, static_cast<char*>(buffer), buffer_bytes, true, (cudaStream_t)stream, "cr_state_save");
}

extern "C" cr_status cr_state_restore(const cr_span* spans, int n, const void* buffer, size_t buffer_bytes, void* stream) {
  return cr::copy_spans(spans, n, const_cast<char*>(static_cast<const char*>(buffer)), buffer_bytes, false, (cudaStream_t)stream,
                        "cr_state_restore");
}
