// Shared declarations of the QSA kernels (qsa_prep.cu, qsa_select.cu, qsa_attn.cu, qsa_prefill.cu).
#pragma once
#include <climits>
#include "common.cuh"

namespace cr {

// All spans of one launch; base[s] = first row of span s in scratch laid out by row.
struct QsaParams {
  cr_qsa_args span[kMaxSpans];
  int base[kMaxSpans];
  int Hq, Hkv, n;
  int b_lo, b_hi;          // scoring only: the blocks [b_lo, b_hi) are scored (a rank's own blocks; 0, INT_MAX = all)
  // Prefill parts that mix the tiled and the row-wise attention: tile_count[r / tile_rows] is the size of the union
  // list of row r's tile; the row-wise kernels serve the rows whose tile has more than tile_max entries (null: all).
  const int* tile_count;
  int tile_rows, tile_max;
};
__device__ __forceinline__ bool qsa_row_is_tiled(const QsaParams& P, int r) {
  return P.tile_count && P.tile_count[r / P.tile_rows] <= P.tile_max;
}

// score_blocks >= 0: the score stride must cover that many blocks (a rank's own range, or 0 for entries that never touch
// the scores) instead of every block of the rows.
cr_status qsa_validate(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, int max_rows, const char* who, int score_blocks = -1);
int qsa_max_rows(const cr_qsa_args* spans, int n);
void qsa_fill_params(QsaParams& P, const cr_geometry* g, const cr_qsa_args* spans, int n);
cr_status qsa_prep_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, int u0, __half* q_hi, int q_skip,
                          cudaStream_t stream, bool queries_only = false);
cr_status qsa_score_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream, int b_lo = 0, int b_hi = INT_MAX);
// Prefill parts (many rows): the scores as four GEMMs on tcgen05 tensor cores.
cr_status qsa_score_tc_launch(const QsaParams& P, int Rmax, int n, cudaStream_t stream);
// Spans of 3..16 rows (verify passes): the scores as an HBM stream through mma.sync, every block of every row.
cr_status qsa_score_mma_launch(const QsaParams& P, int tiles, int Rmax, int n, cudaStream_t stream);
cr_status qsa_topk_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream);
cr_status qsa_select_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, cudaStream_t stream);
// splits: KV splits per (row, KV head). p0/p1: position window (shard mode) or 0 / INT_MAX.
struct QsaTileSplit { const int* count; int rows, max; };   // see QsaParams::tile_count
cr_status qsa_attn_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, float* partials, int splits,
                          int p0, int p1, cudaStream_t stream, const QsaTileSplit* tiles = nullptr);
// Merges `nparts` partial records per (row, head) found at partials[((part_major ? part*rows_total+row : row) ...)].
cr_status qsa_merge_launch(const cr_geometry* g, const cr_qsa_args* spans, int n_spans, const float* partials, int nparts,
                           bool part_major, float* partial_out, cr_out_format fmt, cudaStream_t stream, const QsaTileSplit* tiles = nullptr);

}  // namespace cr
