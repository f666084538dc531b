// Chunk-64 WY Gated DeltaNet scan: workspace layout and launch order (kernels in gdn_chunk_local.cu,
// and gdn_chunk_scan_tc.cu).
#include "gdn_chunk.cuh"

namespace cr {

bool gdn_chunk_available() { return true; }

size_t gdn_chunk_layout(const cr_geometry* g, int rows, ChunkWs* ws, char* base) {
  const size_t chunks = (size_t)(rows + kChunk - 1) / kChunk, Hv = g->gdn_vheads;
  size_t off = 0;
  auto take = [&](size_t bytes) { const size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
  const size_t oU = take(Hv * chunks * 64 * 128 * 4), oG = take(Hv * chunks * 64 * 4);
  const size_t oWQ = take(Hv * chunks * 16384 * 4), oQKp = take(Hv * chunks * 4096 * 4);
  const size_t oKt = take(Hv * chunks * 8192 * 4);
  if (ws) {
    ws->Ut = (float*)(base + oU); ws->G = (float*)(base + oG);
    ws->WQ = (float*)(base + oWQ); ws->QKp = (float*)(base + oQKp); ws->Kt = (float*)(base + oKt);
    ws->chunks = (int)chunks;
  }
  return off;
}

size_t gdn_chunk_workspace_bytes(const cr_geometry* g, int rows) { return gdn_chunk_layout(g, rows, nullptr, nullptr); }

cr_status gdn_chunk_scan(const cr_geometry* g, const GdnPrefillParams& P, bool bf16_in, cudaStream_t stream) {
  ChunkWs ws;
  gdn_chunk_layout(g, P.a.R, &ws, P.chunk_ws);
  if (cr_status s = gdn_chunk_local_launch(g, P, ws, bf16_in, stream)) return s;
  return gdn_chunk_scan_tc_launch(g, P, ws, stream);
}

cr_status gdn_chunk_local_only(const cr_geometry* g, const GdnPrefillParams& P, bool bf16_in, cudaStream_t stream) {
  ChunkWs ws;
  gdn_chunk_layout(g, P.a.R, &ws, P.chunk_ws);
  return gdn_chunk_local_launch(g, P, ws, bf16_in, stream);
}

cr_status gdn_chunk_scan_only(const cr_geometry* g, const GdnPrefillParams& P, cudaStream_t stream) {
  ChunkWs ws;
  gdn_chunk_layout(g, P.a.R, &ws, P.chunk_ws);
  return gdn_chunk_scan_tc_launch(g, P, ws, stream);
}

}  // namespace cr

