// Shared declarations of the GDN prefill kernels (gdn_prefill.cu, gdn_chunk.cu).
#pragma once
#include "common.cuh"

namespace cr {

// Rows per internal part: 148 chunks.  The scan pays a fixed cost per launch (state load and store, pipeline
// fill, about 40 us measured), so parts are long; 148 chunks x 16 key heads = 2368 local CTAs = eight full waves
// of 2 CTAs on 148 SMs, and the part's intermediates (about 72 KB per row) take 0.7 GB.
constexpr int kGdnPartRows = 148 * 64;

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
cr_status gdn_chunk_scan(const cr_geometry* g, const GdnPrefillParams& P, bool bf16_in, bool tcgen05, cudaStream_t stream);

}  // namespace cr
