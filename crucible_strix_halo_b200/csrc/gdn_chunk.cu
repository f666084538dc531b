// Chunk-64 WY Gated DeltaNet scan on tensor cores (placeholder until the kernels land).
#include "gdn_prefill.cuh"

namespace cr {
size_t gdn_chunk_workspace_bytes(const cr_geometry*, int) { return 0; }
cr_status gdn_chunk_scan(const cr_geometry*, const GdnPrefillParams&, cudaStream_t) {
  set_error("cr_gdn_prefill: CR_GDN_CHUNK_TC is not built yet");
  return CR_ERR_UNSUPPORTED;
}
bool gdn_chunk_available() { return false; }
}  // namespace cr
