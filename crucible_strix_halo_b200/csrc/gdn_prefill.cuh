// Shared declarations of the GDN prefill kernels (gdn_prefill.cu, gdn_chunk.cu).
#pragma once
#include "common.cuh"

namespace cr {

// Rows per internal part: 111 chunks.  A long call runs as a pipeline over parts: the chunk-local kernel of part
// p + 1 runs beside the scan of part p (the scan holds one SM per value head, the local kernel takes the rest), on
// two workspaces used in turn.  The scan pays a fixed cost per launch (state load and store, pipeline fill, 15 to
// 40 us measured), which argues for long parts; the first local kernel and the last scan have nothing to run
// beside, which argues for short ones.  A part's intermediates take about 72 KB per row.
int gdn_part_rows();   // 64 x cr_options.gdn_part_chunks (kGdnPartRowsDefault unless a host changed it)

struct GdnPrefillParams {
  cr_gdn_args a;
  const void* ab_logits;   // [R][2Hv]
  float *qn, *kn;          // [R][Hk][128] normalised q (already / sqrt(128)) and k
  float* vn;               // [R][Hv][128] conv + SiLU values
  float *glog, *beta;      // [R][Hv]
  float* yraw;             // [R][Hv][128] un-gated readout
  char* chunk_ws;          // workspace of the chunked scan
  int Hv, Hk, fmt;
  int halo_in;             // 1: rows before this part's first row are read from the input (a later part of one call)
  int tf32;                // 1: prep rounds q/k to tf32 (operands of the tensor-core scan)
};

bool gdn_chunk_available();
size_t gdn_chunk_workspace_bytes(const cr_geometry* g, int rows);
cr_status gdn_chunk_scan(const cr_geometry* g, const GdnPrefillParams& P, bool bf16_in, cudaStream_t stream);
// The two halves of gdn_chunk_scan with the tcgen05 layouts, for callers that run them on different streams.
cr_status gdn_chunk_local_only(const cr_geometry* g, const GdnPrefillParams& P, bool bf16_in, cudaStream_t stream);
cr_status gdn_chunk_scan_only(const cr_geometry* g, const GdnPrefillParams& P, cudaStream_t stream);

}  // namespace cr
