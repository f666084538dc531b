// QSA prefill part (1..2048 rows against the growing cache) for sm_100a: cache rows, query prep, scores,
// selection, attention with the fused gate.  Entry point of a part, in the role of LaunchQsaPrefillUnion /
// LaunchQsaPrefill (engine/layers/kernels/prefill_qsa_union.h:782-807; prefill_qsa.h:274-299).
// This path attends row by row with the split-KV gather kernel (4 splits per row); rows of a part are
// independent once the cache and the pool hold the part, so causality inside the part falls out of pos0 + r.
#include <climits>
#include "qsa.cuh"

namespace cr {
constexpr int kPrefillSplits = 4;
CR_DEFINE_STATUS_WORD(qsa_flash)
}

extern "C" size_t cr_qsa_prefill_scratch_bytes(const cr_geometry* g, int rows) {
  if (!g || rows < 1) return 0;
  return (size_t)rows * g->q_heads * cr::kPrefillSplits * CR_QSA_PART * sizeof(float);
}

extern "C" cr_status cr_qsa_prefill(const cr_geometry* g, const cr_qsa_prefill_args* args, int skip, cr_out_format fmt, void* stream_) {
  using namespace cr;
  CR_REQUIRE(args, "cr_qsa_prefill: null args");
  cr_qsa_args q = args->input;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (cr_status s = qsa_validate(g, &q, 1, CR_MAX_PREFILL_ROWS, "cr_qsa_prefill")) return s;
  CR_REQUIRE(skip >= 0 && skip < q.R && skip % 16 == 0, "cr_qsa_prefill: skip=%d must be a multiple of 16 below R=%d", skip, q.R);
  CR_REQUIRE(fmt == CR_OUT_RAW_F32 || fmt == CR_OUT_RAW_BF16 || fmt == CR_OUT_EXL3_WHT, "cr_qsa_prefill: bad output format");
  CR_REQUIRE(q.out && (fmt != CR_OUT_EXL3_WHT || q.suh_o), "cr_qsa_prefill: output buffer (and suh_o for the EXL3 output) needed");
  CR_REQUIRE(fmt == CR_OUT_EXL3_WHT || q.pack_rows == 0, "cr_qsa_prefill: packed layout only with the EXL3 output");
  const size_t need = cr_qsa_prefill_scratch_bytes(g, q.R - skip);
  CR_REQUIRE(args->scratch && args->scratch_bytes >= need, "cr_qsa_prefill: scratch of %zu bytes needed, %zu given", need, args->scratch_bytes);
  // cache rows + query prep for the whole part (rows below skip get cache work only)
  if (cr_status s = qsa_prep_launch(g, &q, 1, 0, reinterpret_cast<__half*>(args->q_hi), skip, stream)) return s;
  // the output rows [skip, R)
  const size_t W = (size_t)g->q_heads * 256;
  q.pos0 += skip; q.R -= skip;
  q.q += (size_t)skip * g->q_heads * 512; q.idx += (size_t)skip * 640;
  if (q.context) q.context += (size_t)skip * W;
  if (q.pack_rows) q.pack_off += skip;
  else q.out = (char*)q.out + (size_t)skip * W * (fmt == CR_OUT_RAW_F32 ? 4 : 2);
  if (cr_status s = qsa_select_launch(g, &q, 1, stream)) return s;
  if (cr_status s = qsa_attn_launch(g, &q, 1, (float*)args->scratch, kPrefillSplits, 0, INT_MAX, stream)) return s;
  return qsa_merge_launch(g, &q, 1, (const float*)args->scratch, kPrefillSplits, false, nullptr, fmt, stream);
}
